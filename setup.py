"""Builds the native libraries in-tree (nvcc for sm_100a, g++ against the installed torch) as part
of ``pip install -e . --no-build-isolation``. There is no wheel matrix: one architecture, one
toolchain. Parity: setup.py / CMakeLists.txt of the reference drive one multi-arch CMake build."""

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNative(build_py):
    def run(self):
        import importlib.util
        import pathlib

        path = pathlib.Path(__file__).parent / "fast_ulysses_b200" / "_build.py"
        spec = importlib.util.spec_from_file_location("_fu_build", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build_all(verbose=True)
        super().run()


setup(cmdclass={"build_py": BuildNative})
