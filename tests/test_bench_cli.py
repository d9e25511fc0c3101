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


def _agree_worker(rank, world, port, ret):
    import importlib.util
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    spec = importlib.util.spec_from_file_location("bench", BENCH)
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = (b.all_ranks_agree(True, "cpu"),        # every rank is ready: take the fused path
                     b.all_ranks_agree(rank != 1, "cpu"),   # rank 1 could not set it up: nobody takes it
                     b.worst_status(0, "cpu"),
                     b.worst_status(16 if rank == 1 else 0, "cpu"))  # rank 1's bounded wait ran out: all ranks see it
    finally:
        dist.destroy_process_group()


def test_ranks_take_the_same_gather_path_two_ranks():
    import socket
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_agree_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret.get(0) == (True, False, 0, 16) and ret.get(1) == (True, False, 0, 16)
