"""bench.py pieces that need no GPU: the command line, the stage markers and the watchdog of multi-rank runs."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "bench.py")


def test_help_lists_the_contract_flags():
    r = subprocess.run([sys.executable, BENCH, "--help"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--workload"):
        assert flag in r.stdout


def test_watchdog_ends_a_stalled_multi_rank_run_with_a_message():
    code = (
        "import importlib.util, time\n"
        f"spec = importlib.util.spec_from_file_location('bench', {BENCH!r})\n"
        "b = importlib.util.module_from_spec(spec); spec.loader.exec_module(b)\n"
        "b.stage('started')\n"
        "b.start_watchdog(1)\n"   # single GPU: no watchdog
        "b.start_watchdog(2)\n"
        "time.sleep(20)\n"
        "print('not reached')\n")
    env = dict(os.environ, INGOT_BENCH_LIMIT_S="1", RANK="0")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 3
    assert '"error"' in r.stdout and "did not finish within 1 s" in r.stdout and "not reached" not in r.stdout
    assert "[bench rank 0" in r.stderr and "started" in r.stderr and "watchdog" in r.stderr
