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
    assert "[bench rank 0" in r.stderr and "started" in r.stderr and "giving up" in r.stderr


def test_watchdog_reports_a_finished_headline_when_a_later_workload_stalls():
    code = (
        "import importlib.util, time\n"
        f"spec = importlib.util.spec_from_file_location('bench', {BENCH!r})\n"
        "b = importlib.util.module_from_spec(spec); spec.loader.exec_module(b)\n"
        "b._PARTIAL['line'] = {'metric': 'm', 'value': 1.5, 'n_gpus': 2}\n"
        "b._PARTIAL['pending'] = ['prefill', 'c4_batched']\n"
        "b.start_watchdog(2)\n"
        "time.sleep(20)\n")
    env = dict(os.environ, INGOT_BENCH_LIMIT_S="1", RANK="0")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0
    import json
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["value"] == 1.5 and "prefill, c4_batched" in line["incomplete"] and "error" not in line


def _run_snippet(body, **env):
    code = ("import importlib.util, time\n"
            f"spec = importlib.util.spec_from_file_location('bench', {BENCH!r})\n"
            "b = importlib.util.module_from_spec(spec); spec.loader.exec_module(b)\n" + body)
    return subprocess.Popen([sys.executable, "-c", code], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                            env=dict(os.environ, RANK="0", **env))


def test_watchdog_ends_a_run_that_stops_writing_stage_markers():
    p = _run_snippet("b.start_watchdog(2)\nb.stage('one')\ntime.sleep(0.5)\nb.stage('two')\ntime.sleep(30)\n",
                     INGOT_BENCH_LIMIT_S="600", INGOT_BENCH_STALL_S="2")
    out, err = p.communicate(timeout=120)
    assert p.returncode == 3 and "made no progress for 2 s" in out and "two" in err


import pytest  # noqa: E402

# what the main thread is doing when the signal arrives: something Python can interrupt, or a C call that never returns
# (a second lock of a plain pthread mutex: the stand-in for a thread waiting inside a collective)
_WAITS = {"sleep": "time.sleep(60)\n",
          "stuck_in_c": "import ctypes\nlibc = ctypes.CDLL(None)\nm = ctypes.create_string_buffer(128)\n"
                        "libc.pthread_mutex_init(m, None)\nlibc.pthread_mutex_lock(m)\nprint('ready', flush=True)\n"
                        "libc.pthread_mutex_lock(m)\n"}


@pytest.mark.parametrize("wait", ["sleep", "stuck_in_c"])
def test_sigterm_from_the_launcher_still_gets_the_headline_out(wait):
    import json
    import signal
    import time
    p = _run_snippet("b._PARTIAL['line'] = {'metric': 'm', 'value': 2.5}\nb._PARTIAL['pending'] = ['prefill']\n"
                     "b.start_watchdog(2)\n" + ("print('ready', flush=True)\n" if wait == "sleep" else "") + _WAITS[wait])
    assert p.stdout.readline().strip() == "ready"
    time.sleep(0.2)
    p.send_signal(signal.SIGTERM)
    out, err = p.communicate(timeout=120)
    line = json.loads(out.strip().splitlines()[-1])
    assert p.returncode == 0 and line["value"] == 2.5 and "SIGTERM" in line["incomplete"] and "prefill" in line["incomplete"]


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


def _load_bench():
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_under_test", BENCH)
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    return b


def _fake_leg(name, unit):
    def run(args, rank, world, *rest):
        return {"metric": name, "value": 2.0, "unit": unit, "ms_per_step": 0.5, "scaling": "weak", "dtype": "f16",
                "roofline": {"frac": 0.5}, "e2e": {"value": 1.0}, "gpu_launches": 4, "clocks": {"sm_mhz": 1900}}
    return run


def test_main_assembles_one_line_from_the_workloads(monkeypatch, capsys):
    """The order and the keys of bench.py's output line, with every GPU workload replaced by a stand-in."""
    import json
    b = _load_bench()
    monkeypatch.setattr(b, "dist_setup", lambda n: (0, 1, 0))
    monkeypatch.setattr(b, "run_decode", _fake_leg("decode", "GB/s"))
    monkeypatch.setattr(b, "run_prefill", _fake_leg("prefill", "TFLOP/s"))
    monkeypatch.setattr(b, "run_chunked", _fake_leg("chunked", "us"))
    monkeypatch.setattr(b, "run_batched_decode", _fake_leg("batched", "GB/s"))
    monkeypatch.setattr(b, "cpu_decode_sample", lambda n, reps: (5.0, "reference", 16, 0.003))
    monkeypatch.setattr(b, "cpu_prefill_sample", lambda: (0.01, "reference", 16, 48))

    monkeypatch.setattr(sys, "argv", ["bench.py", "--steps", "7", "--warmup", "1"])
    b.main()
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["metric"] == "decode" and line["value"] == 2.0 and line["unit"] == "GB/s" and line["n_gpus"] == 1
    assert line["steps"] == 7 and line["warmup"] == 3 and line["higher_is_better"] is True and line["vs_baseline"] is None
    assert line["roofline"]["frac"] == 0.5 and line["e2e"]["value"] == 1.0 and line["gpu_launches"] == 4
    assert line["cpu_baseline"]["kind"] == "reference" and line["cpu_baseline"]["cores"] == 16
    assert line["prefill"]["metric"] == "prefill" and line["prefill"]["cpu_baseline"]["unit"] == "TFLOP/s"
    assert [k for k in ("c1_prefill128", "c3_chunked", "c4_batched") if k in line] == ["c1_prefill128", "c3_chunked", "c4_batched"]
    assert b._PARTIAL["pending"] == []

    # the prefill shape as the headline: decode rides along; a single named configuration runs alone
    monkeypatch.setattr(sys, "argv", ["bench.py", "--workload", "prefill_c5", "--no-cpu"])
    b.main()
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["metric"] == "prefill" and line["decode"]["metric"] == "decode" and "cpu_baseline" not in line
    monkeypatch.setattr(sys, "argv", ["bench.py", "--workload", "c4_batched"])
    b.main()
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["metric"] == "batched" and "prefill" not in line and "decode" not in line and "c4_batched" not in line


def test_main_at_two_ranks_runs_the_batched_decode_before_the_gathering_prefill(monkeypatch, capsys):
    import json
    import torch.distributed as dist
    b = _load_bench()
    order = []

    def leg(name, unit):
        inner = _fake_leg(name, unit)

        def run(args, rank, world, *rest):
            order.append((name, list(b._PARTIAL["pending"])))
            return inner(args, rank, world)
        return run

    monkeypatch.setattr(b, "dist_setup", lambda n: (0, 2, 0))
    monkeypatch.setattr(b, "start_watchdog", lambda world: None)
    monkeypatch.setattr(b, "run_decode", leg("decode", "GB/s"))
    monkeypatch.setattr(b, "run_prefill", leg("prefill", "TFLOP/s"))
    monkeypatch.setattr(b, "run_batched_decode", leg("batched", "GB/s"))
    monkeypatch.setattr(dist, "barrier", lambda *a, **k: None)
    monkeypatch.setattr(dist, "destroy_process_group", lambda *a, **k: None)
    monkeypatch.setattr(sys, "argv", ["bench.py", "--gpus", "2"])
    b.main()
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    # the headline first (nothing pending yet), then the workload without an exchange, then the one with the fused gather
    assert order == [("decode", []), ("batched", ["c4_batched", "prefill"]), ("prefill", ["prefill"])]
    assert line["n_gpus"] == 2 and "cpu_baseline" not in line and "c1_prefill128" not in line
    assert line["c4_batched"]["metric"] == "batched" and line["prefill"]["metric"] == "prefill"
