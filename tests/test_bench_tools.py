"""The benchmark helpers that only read the GPUs' state: run against a fake nvidia-smi on PATH."""

import os
import stat
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def fake_smi(tmp_path, foreign_pids):
    """An `nvidia-smi` that answers the two queries exclusive.py makes."""
    path = tmp_path / "nvidia-smi"
    apps = "\n".join(f"{pid}, GPU-0000" for pid in foreign_pids)
    path.write_text(textwrap.dedent(f"""\
        #!/bin/sh
        case "$*" in
          *query-compute-apps*) printf '%s\\n' "{apps}" ;;
          *query-gpu=clocks.sm*) echo 1755 ;;
          *) echo fake ;;
        esac
        """))
    path.chmod(path.stat().st_mode | stat.S_IEXEC)
    return {**os.environ, "PATH": f"{tmp_path}:{os.environ['PATH']}"}


def run_exclusive(env, *cmd):
    return subprocess.run([sys.executable, os.path.join(ROOT, "benchmarks", "exclusive.py"), "--gpus", "0",
                           "--sample-secs", "0.05", "--", *cmd], env=env, capture_output=True, text=True, timeout=60)


def test_exclusive_run_reports_exclusive_and_the_minimum_clock(tmp_path):
    r = run_exclusive(fake_smi(tmp_path, []), sys.executable, "-c", "import time; time.sleep(0.3)")
    assert r.returncode == 0, r.stdout + r.stderr
    assert "EXCLUSIVE" in r.stdout and "1755 MHz" in r.stdout


def test_exclusive_refuses_to_start_beside_foreign_processes(tmp_path):
    r = run_exclusive(fake_smi(tmp_path, [4242]), sys.executable, "-c", "print('must not run')")
    assert r.returncode == 3 and "CONTENDED before start" in r.stdout and "must not run" not in r.stdout


def test_exclusive_passes_the_command_exit_code_on(tmp_path):
    r = run_exclusive(fake_smi(tmp_path, []), sys.executable, "-c", "import sys; sys.exit(7)")
    assert r.returncode == 7


def test_collect_and_bench_a2a_parse_their_arguments():
    for script, arg in (("collect.py", "--help"), ("bench_a2a.py", "--help")):
        r = subprocess.run([sys.executable, os.path.join(ROOT, "benchmarks", script), arg], capture_output=True,
                           text=True, timeout=120)
        assert r.returncode == 0 and "usage" in r.stdout.lower(), r.stderr[-500:]


def test_preflight_refuses_a_machine_without_gpus_and_explains_itself(tmp_path):
    """preflight.py is the manual release gate; without GPUs it must say so instead of running suites."""
    path = tmp_path / "nvidia-smi"
    path.write_text("#!/bin/sh\nexit 0\n")  # reports no GPU at all
    path.chmod(path.stat().st_mode | stat.S_IEXEC)
    env = {**os.environ, "PATH": f"{tmp_path}:{os.environ['PATH']}"}
    script = os.path.join(ROOT, "benchmarks", "preflight.py")
    r = subprocess.run([sys.executable, script], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 2 and "needs a machine with GPUs" in r.stdout
    h = subprocess.run([sys.executable, script, "--help"], capture_output=True, text=True, timeout=120)
    assert h.returncode == 0 and "exclusive.py" in h.stdout and "doctor" in h.stdout


def test_async_overlap_example_runs_on_two_gloo_ranks():
    """examples/overlap_async.py in its dry-run form: both transports' settings, the staged input,
    a lent window, every result equal to the synchronous call."""
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port),
                        os.path.join(ROOT, "examples", "overlap_async.py"), "--cpu"],
                       capture_output=True, text=True, timeout=240, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("all equal to the synchronous call") == 2
