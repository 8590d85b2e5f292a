"""In-tree build of the two native libraries.

``lib/libfu_kernels.so``  the sm_100a CUDA kernels behind a C interface (nvcc, no torch headers)
``_C.so``                 the torch operator layer and the group runtime (g++, links the above)

Both are rebuilt only when a source or header is newer than the object, so importing the package
after a build costs nothing. Everything is compiled for ``sm_100a`` only: tcgen05, tensor memory
and TMA need the architecture-specific target.

Parity: CMakeLists.txt and setup.py of the reference build one ``_C`` for sm_80..sm_120; this
library targets one architecture and needs no wheel matrix.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "lib"
KERNEL_LIB = LIB / "libfu_kernels.so"
EXT = PKG / "_C.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "-DFU_BUILDING"]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = Path(cuda_home) / "bin" / "nvcc"
    return str(cand) if cand.exists() else (shutil.which("nvcc") or "nvcc")


def _cxx() -> str:
    """The host compiler. Some images put a wrapper first on PATH whose libstdc++.so link is
    dangling, which makes the linker fall back to a STATIC libstdc++ inside the extension; two C++
    runtimes in one process crash in iostream locale code. The distribution's own g++ is preferred."""
    if os.environ.get("FU_CXX"):
        return os.environ["FU_CXX"]
    candidates = ["/usr/bin/g++", os.environ.get("CXX"), shutil.which("g++")]
    for cand in candidates:
        if not cand or not Path(cand).exists():
            continue
        probe = subprocess.run([cand, "-print-file-name=libstdc++.so"], capture_output=True, text=True)
        if probe.returncode == 0 and Path(probe.stdout.strip()).exists():
            return cand
    return "g++"


def _newest(paths) -> float:
    return max((p.stat().st_mtime for p in paths), default=0.0)


def _stale(target: Path, deps) -> bool:
    return (not target.exists()) or target.stat().st_mtime < _newest(deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"build step failed ({res.returncode}): {' '.join(str(c) for c in cmd)}\n"
                           f"{res.stdout}\n{res.stderr}")
    if verbose and (res.stdout or res.stderr):
        print(res.stdout, res.stderr, flush=True)
    return res


def kernel_sources():
    return sorted((CSRC / "kernels").glob("*.cu"))


def build_kernels(verbose: bool = False, force: bool = False) -> Path:
    """Compile every .cu under csrc/kernels for sm_100a and link libfu_kernels.so."""
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    headers = list((CSRC / "kernels").glob("*.h")) + list((CSRC / "kernels").glob("*.cuh"))
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in kernel_sources():
        obj = OBJ / (src.stem + ".cu.o")
        objs.append(obj)
        if force or _stale(obj, [src, *headers]):
            jobs.append([nvcc, "-ccbin", _cxx(), *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC / "kernels", "-c", src, "-o",
                         obj])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(lambda c: _run(c, verbose), jobs))
    if force or jobs or _stale(KERNEL_LIB, objs):
        _run([nvcc, "-ccbin", _cxx(), *ARCH_FLAGS, "-shared", "-Xcompiler", "-fPIC", "-o", KERNEL_LIB, *objs],
             verbose)
    return KERNEL_LIB


def _torch_flags():
    import torch
    from torch.utils import cpp_extension as ce

    inc = []
    for p in ce.include_paths("cuda"):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    defs = ["-DTORCH_API_INCLUDE_EXTENSION_H", "-DTORCH_EXTENSION_NAME=_C",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-DFU_HAS_WORK_REGISTRY=1"]
    get_abi = getattr(ce, "_get_pybind11_abi_build_flags", None)
    if get_abi is not None:
        defs += list(get_abi())
    torch_lib = Path(torch.__file__).parent / "lib"
    cuda_home = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    link = ["-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-L", cuda_home / "lib64", "-lcudart", "-L", LIB, "-lfu_kernels", "-ldl",
            "-Wl,-rpath,$ORIGIN/lib", f"-Wl,-rpath,{torch_lib}"]
    return inc, defs, link


def ext_sources():
    return sorted((CSRC / "plan").glob("*.cc")) + sorted((CSRC / "runtime").glob("*.cc")) + sorted(
        (CSRC / "ops").glob("*.cc"))


def build_ext(verbose: bool = False, force: bool = False) -> Path:
    """Compile the plan library, the group runtime and the operator layer into _C.so."""
    build_kernels(verbose, force)
    OBJ.mkdir(exist_ok=True)
    headers = [p for d in ("plan", "runtime", "ops", "kernels") for p in (CSRC / d).glob("*.h*")]
    inc, defs, link = _torch_flags()
    cxx = _cxx()
    jobs, objs = [], []
    for src in ext_sources():
        obj = OBJ / (src.parent.name + "_" + src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [src, *headers]):
            jobs.append([cxx, "-std=c++17", "-O2", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-function",
                         *defs, *inc, "-c", src, "-o", obj])
    with ThreadPoolExecutor(max_workers=min(6, max(1, len(jobs)))) as pool:
        list(pool.map(lambda c: _run(c, verbose), jobs))
    if force or jobs or _stale(EXT, [*objs, KERNEL_LIB]):
        _run([cxx, "-shared", "-o", EXT, *objs, *link], verbose)
    import torch

    (OBJ / "build_meta.txt").write_text(
        f"torch={torch.__version__}\ncuda={torch.version.cuda}\n"
        f"python={sys.version_info.major}.{sys.version_info.minor}\narch=sm_100a\n")
    return EXT


def build_all(verbose: bool = False, force: bool = False) -> None:
    build_ext(verbose, force)


if __name__ == "__main__":
    build_all(verbose="-q" not in sys.argv, force="--force" in sys.argv)
    print("built:", KERNEL_LIB, EXT)
