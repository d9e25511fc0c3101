#!/usr/bin/env python
"""Benchmark of the B200 attention path: decode KV-cache HBM GB/s and causal-prefill TFLOP/s.

    python bench.py --gpus N --steps K --warmup W [--workload decode_c2|prefill_c5|c1_prefill128|c3_chunked|c4_batched|e2e_model]
                    [--impl reference]

Headline (`metric`/`value`): single-token decode attention at 4096 keys, 24 query / 8 KV heads,
head_dim 128, f16 KV cache, one pass over 28 distinct per-layer caches per step (470 MB, larger than
L2), reported as KV-cache bytes per second with the reference's own `abench` byte formula
(2 * n_layer * (pos+1) * n_head_kv * head_dim * 2, src/main.cpp:446). With N > 1 every rank decodes its
own sequence (sequence sharding, no collective on the data path): weak scaling.

The same JSON line carries, as objects of their own:
  prefill        32768-token causal GQA prefill (bf16 q, f16 K/V) in TFLOP/s counting 4*S^2*H*d/2, sharded by KV head
                 over the N ranks with the gather of the head outputs fused into the kernel (strong scaling);
  c4_batched     64-sequence paged decode, sequences sharded over the N ranks by length (strong scaling);
  c1_prefill128, c3_chunked   the two chunked-prefill configurations (N = 1 only: they are replicas).
Every object has `parity` (max-abs and relative L2 error against the CPU reference on the tensors that were timed,
computed outside the timed region), `roofline`, and where it applies `e2e` (host buffers, copies inside the timed
region) and `clocks` (NVML, sampled while the timed region runs).

Timing: W warm-up steps, then blocks of K steps, each block timed with CUDA events on the launching stream, repeated
back to back between two barriers until at least --min-timed-s (0.5 s) have been timed; `ms_per_step` is the median
block divided by K, `timed_region_s` the sum of the blocks, MAX over ranks.

`--impl reference` times the reference's own CPU attention (oracle/_ref, the reference sources compiled
unmodified; the plain-C restatement if that is absent) on the host cores for the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

_T0 = time.time()

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "inference-agent_b200"))

N_LAYER, H, HKV, D = 28, 24, 8, 128
DECODE_KEYS = 4096
PREFILL_TOKENS = 32768

# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum) from ncu captures of
# the same kernels. decode: captured at the benchmark shape. prefill: reads captured at 8192 tokens (84.0 MB) and
# scaled by the 4x token count (compulsory q/K/V traffic grows in proportion); writes are the 32768 x 24 x 128 f16
# output, 201 MB, which unlike the 8192-token case (50 MB, absorbed by L2 during the capture) cannot stay in L2.
NCU_TRAFFIC = {"attn_decode_kernel": 470275840 + 4313344, "attn_prefill_sm100_kernel": 4 * 83955712 + PREFILL_TOKENS * H * D * 2}
MIN_TIMED_S = 0.5  # the timed region is repeated in blocks of `steps` steps until it is at least this long


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "tflops_burst": d["bf16_tflops"], "tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only) in a thread while GPU work runs."""

    def __init__(self, gpu_index, period_s=0.005):
        self.gpu_index, self.period, self.samples, self.reasons = gpu_index, period_s, [], 0
        self.sm_max, self._stop, self.thread = None, threading.Event(), None

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = int(visible.split(",")[self.gpu_index]) if visible and visible.split(",")[0].isdigit() else self.gpu_index
            h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))

            def loop():
                while not self._stop.is_set():
                    try:
                        self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        self.reasons |= int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                    except pynvml.NVMLError:
                        pass
                    time.sleep(self.period)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self.thread:
            self.thread.join(timeout=2)

    def summary(self):
        bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.sm_max,
                "reasons": [n for n, b in bits.items() if self.reasons & b], "samples": len(self.samples)}


# Rank 0's output line as far as it is complete: "line" is set once the headline workload has been measured, "pending"
# names the remaining workloads. The watchdog of a multi-rank run prints it if a later workload stalls.
_PARTIAL = {"line": None, "pending": []}


_LAST_STAGE = [time.time(), 0]  # when the last stage marker was written, and how many there have been


def stage(msg):
    """Progress marker on stderr (every rank): if a multi-GPU run ever stalls, the log says where."""
    _LAST_STAGE[0], _LAST_STAGE[1] = time.time(), _LAST_STAGE[1] + 1
    print(f"[bench rank {os.environ.get('RANK', '0')} +{time.time() - _T0:6.1f}s] {msg}", file=sys.stderr, flush=True)


_BAIL_LOCK = None


def bail(world, why):
    """Ends this rank of a multi-rank run at once. Rank 0 first prints what it has: the finished headline line with an
    `incomplete` key naming the workloads that did not finish (exit code 0), else an `error` object (exit code 3)."""
    global _BAIL_LOCK
    import threading
    if _BAIL_LOCK is None:
        _BAIL_LOCK = threading.Lock()
    if not _BAIL_LOCK.acquire(blocking=False):  # another thread is already on its way out
        time.sleep(30)
        os._exit(3)
    stage(f"giving up: {why}")
    why = f"bench.py --gpus {world} {why} (see the stage markers on stderr)"
    rank0 = os.environ.get("RANK", "0") == "0"
    done = _PARTIAL.get("line")
    if rank0:
        if done is not None:  # the headline workload was measured in full: report it and say what is missing
            print(json.dumps(dict(done, incomplete=f"{why}; not finished: {', '.join(_PARTIAL['pending'])}")), flush=True)
        else:
            print(json.dumps({"error": why}), flush=True)
    os._exit(0 if done is not None or not rank0 else 3)


def mark(world, msg):
    """stage() for multi-rank runs only (a single-GPU run keeps stderr quiet)."""
    if world > 1:
        stage(msg)


def start_watchdog(world):
    """Keeps a multi-rank run from occupying the GPUs until somebody else's limit (a stalled collective would otherwise wait
    for ever) and from ending without a line. The run ends itself through bail() when it has not finished after
    INGOT_BENCH_LIMIT_S seconds (default 540), when no stage marker has been written for INGOT_BENCH_STALL_S seconds
    (default 180; a healthy stage takes well under a minute; twice that before the first marker), or when the launcher sends SIGTERM (another rank failed, or an
    outer time limit ran out) - the last also while the main thread sits inside a collective, through a wake-up pipe."""
    if world <= 1:
        return
    import signal
    import threading
    limit = float(os.environ.get("INGOT_BENCH_LIMIT_S", "540"))
    stall = float(os.environ.get("INGOT_BENCH_STALL_S", "180"))
    _LAST_STAGE[0], _LAST_STAGE[1] = time.time(), 0

    def watch():
        while True:
            time.sleep(0.25)
            now = time.time()
            if now - _T0 > limit:
                bail(world, f"did not finish within {limit:.0f} s")
            # until the first marker (the process group is up) twice the time: a cold machine pages the libraries in first
            patience = stall if _LAST_STAGE[1] > 0 else 2 * stall
            if now - _LAST_STAGE[0] > patience:
                bail(world, f"made no progress for {patience:.0f} s")

    threading.Thread(target=watch, daemon=True).start()
    if threading.current_thread() is threading.main_thread():
        r, w = os.pipe()
        os.set_blocking(w, False)
        signal.signal(signal.SIGTERM, lambda signum, frame: None)  # the work is done by the thread below, whatever the main thread is in
        signal.set_wakeup_fd(w, warn_on_full_buffer=False)

        def on_signal():
            while True:
                data = os.read(r, 16)
                if not data or signal.SIGTERM in data:
                    bail(world, "was told to stop (SIGTERM)")

        threading.Thread(target=on_signal, daemon=True).start()


def dist_setup(n_gpus):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import datetime
        import torch.distributed as dist
        torch.cuda.set_device(local)
        # NCCL only carries barriers, one-element reductions and the one-time all-gather check here, so in-switch reduction buys
        # nothing; without it no rank's memory is bound to an NVLink multicast object, which matters because the watchdog and the
        # collective time-out below can end ranks at slightly different times. (Set NCCL_NVLS_ENABLE=1 to override.)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        # a collective that a rank never joins ends with an error after this long instead of the default ten minutes (long
        # enough for the slowest rank of a fresh machine to get through its imports)
        limit = datetime.timedelta(seconds=float(os.environ.get("INGOT_BENCH_PG_TIMEOUT_S", "300")))
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=limit)
        stage("process group up")
    else:
        torch.cuda.set_device(0)
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {n_gpus}")
    return rank, world, local


def timed(fn, steps, warmup, world, min_time_s=MIN_TIMED_S, max_blocks=2000):
    """W warm-up calls, then blocks of `steps` calls each, back to back between two barriers, until the region is
    at least min_time_s long. Every block is timed with CUDA events on the launching stream and reduced with MAX
    over the ranks. Returns {"ms": median block (ms for `steps` steps), "ms_best": fastest block, "blocks": B,
    "timed_region_s": sum of the blocks}."""
    import torch
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    # block count from one probe block (the same on every rank)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    probe = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(probe, op=dist.ReduceOp.MAX)
    blocks = int(min(max_blocks, max(1, -(-min_time_s * 1e3 // max(float(probe.item()), 1e-3)))))
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
    marks[0].record()
    for b in range(blocks):
        for _ in range(steps):
            fn()
        marks[b + 1].record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = torch.tensor([marks[b].elapsed_time(marks[b + 1]) for b in range(blocks)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = ms.cpu().tolist()
    return {"ms": statistics.median(ms), "ms_best": min(ms), "blocks": blocks, "timed_region_s": round(sum(ms) * 1e-3, 4)}


def parity(got, want):
    """max-abs and relative L2 error of the attention output against the f32 CPU reference (bounds 2e-3 / 1e-3)."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = got - want
    out = {"max_abs": float(np.abs(d).max()), "rel_l2": float(np.linalg.norm(d) / max(np.linalg.norm(want), 1e-30))}
    out["within_tolerance"] = bool(out["max_abs"] <= 2e-3 and out["rel_l2"] <= 1e-3 and np.isfinite(got).all())
    return out


def oracle_rows(q_rows, k_f16, v_f16, positions, n_head_kv):
    """CPU reference attention (the checker under oracle/) for already-rotated query rows [r,H,d] at `positions`
    over f16 cache rows [n,Hkv,d] widened to the reference's f32 cache. Outside every timed region."""
    from oracle import loader
    lib = loader.load_oracle()
    n = k_f16.shape[0]
    kc = np.ascontiguousarray(k_f16.astype(np.float32).reshape(n, -1))
    vc = np.ascontiguousarray(v_f16.astype(np.float32).reshape(n, -1))
    return loader.attend_rows(lib, q_rows, kc, vc, np.asarray(positions, dtype=np.int32), q_rows.shape[1], n_head_kv,
                              q_rows.shape[2])


# ------------------------------------------------------------------------------------------------
# decode: configs[1]
# ------------------------------------------------------------------------------------------------

def decode_bytes_per_step():
    return 2 * N_LAYER * DECODE_KEYS * HKV * D * 2


def decode_config(world):
    """The workload description both arms (this library and the reference's CPU code) report."""
    return {"workload": "configs[1]: decode @4096 keys, batch 1 per GPU, 28 per-layer caches per step; the 28 layers are "
                        "independent (as in the reference's abench) and share one grid plus one merge launch",
            "n_layer": N_LAYER, "n_keys": DECODE_KEYS, "n_head": H, "n_head_kv": HKV, "head_dim": D,
            "l2": "inputs larger than L2 (470 MB of KV per step, 28 distinct caches)",
            "parallelism": f"sequence sharding x{world} (one sequence per GPU, no collective)"}


def prefill_config(S, world):
    return {"workload": ("configs[4]: 32768-token causal prefill, FLOPs = 4*S^2*H*d/2" if S == PREFILL_TOKENS
                         else f"PROFILING CASE: {S}-token causal prefill (not the benchmark configuration)"), "n_tok": S,
            "n_head": H, "n_head_kv": HKV, "head_dim": D, "l2": "inputs larger than L2 (q+out 400 MB, K/V 134 MB)",
            "parallelism": f"KV-head sharding x{world}"}


def captured(fn):
    """Runs fn once eagerly (the library sizes its scratch on a first call, which cannot happen under capture),
    then captures it into a CUDA graph and returns the replay function."""
    import torch
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g.replay


def run_decode(args, rank, world):
    import torch
    import ingot_b200 as ib
    from ingot_b200 import workloads as W
    torch.manual_seed(1 + rank)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, N_LAYER, HKV, DECODE_KEYS)
    # Layer 0 holds the configs[1] tensors themselves (numpy default_rng(1), draw order q, K, V: the bits the parity
    # tests use); the other 27 caches are N(0,1) generated on the device.
    c2 = W.c2_decode4096()
    q = torch.randn(N_LAYER, 1, H, D, device="cuda")
    q[0].copy_(torch.from_numpy(c2.q))
    for l in range(N_LAYER):
        if l == 0:
            kv.import_f16(0, torch.from_numpy(c2.k[0]).cuda(), torch.from_numpy(c2.v[0]).cuda(), 0)
        else:
            kv.layer_view(l, "k").copy_(torch.randn(HKV, DECODE_KEYS, D, device="cuda").half())
            kv.layer_view(l, "v").copy_(torch.randn(HKV, DECODE_KEYS, D, device="cuda").half())
    out = torch.zeros(N_LAYER, 1, H, D, device="cuda")
    mark(world, "decode: caches ready")

    def launch_layers():
        ib.attn_decode_layers(kv, 0, q, out, max_seq_len=DECODE_KEYS, chunk_keys=args.chunk_keys)

    # The 28 launches of a step are captured once in a CUDA graph (the reference encodes them into one
    # command buffer, src/metal_backend.mm:594-649); a step is one replay.
    step = launch_layers if args.no_graph else captured(launch_layers)

    with ClockSampler(torch.cuda.current_device()) as clk:  # clocks are sampled while the timed region runs
        t = timed(step, args.steps, args.warmup, world, 0.0 if args.no_graph else MIN_TIMED_S)
    ms = t["ms"]
    mark(world, "decode: timed")

    # Parity of what was just timed, outside the timed region: three of the 28 layers against the CPU reference.
    torch.cuda.synchronize()
    errs = []
    for l in (0, N_LAYER // 2, N_LAYER - 1):
        k_l = kv.layer_view(l, "k").permute(1, 0, 2).contiguous().cpu().numpy()  # [keys, Hkv, d]
        v_l = kv.layer_view(l, "v").permute(1, 0, 2).contiguous().cpu().numpy()
        want = oracle_rows(q[l].cpu().numpy(), k_l, v_l, [DECODE_KEYS - 1], HKV)
        errs.append(parity(out[l].cpu().numpy(), want))
    par = {"max_abs": max(e["max_abs"] for e in errs), "rel_l2": max(e["rel_l2"] for e in errs),
           "within_tolerance": all(e["within_tolerance"] for e in errs),
           "checked": "layers 0 (the configs[1] seed-1 tensors), 14 and 27 of the timed call against the CPU reference"}

    launches = args.steps * t["blocks"] * 2  # per step: one grid with every layer's split CTAs, one merge launch
    bytes_step = decode_bytes_per_step()
    value = world * bytes_step * args.steps / (ms * 1e-3) / 1e9
    per_launch_s = ms * 1e-3 / (args.steps * N_LAYER)
    peaks = measured_peaks()
    achieved = bytes_step / N_LAYER / per_launch_s / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": NCU_TRAFFIC["attn_decode_kernel"],
                "kernel": "attn_decode_kernel", "peak_source": f"of {peaks['source']} (STREAM-style copy)",
                "frac_of_nominal_8000": round(achieved / 8000.0, 4),
                "algorithmic_bytes_per_launch": bytes_step, "us_per_launch": round(ms * 1e3 / args.steps, 3),
                "us_per_layer": round(per_launch_s * 1e6, 3),
                "note": "one grid carries the split CTAs of all 28 layers (algorithmic bytes per launch = 28 x 16 777 216); "
                        "us_per_layer is step time / 28. In a forward pass the layers depend on one another: see "
                        "in_backend_us_per_layer"}

    # The same 28 layers the way a forward pass has to run them (its layers depend on one another): one
    # ingot_attn_decode call per layer on one stream, i.e. a split launch and a merge launch per layer.
    if not args.no_graph and not args.no_secondary:
        def per_layer_calls():
            for l in range(N_LAYER):
                ib.attn_decode(kv, l, q[l], out=out[l], max_seq_len=DECODE_KEYS, chunk_keys=args.chunk_keys)

        t2 = timed(captured(per_layer_calls), args.steps, 3, world, min(0.1, MIN_TIMED_S))
        us = t2["ms"] * 1e3 / (args.steps * N_LAYER)
        roofline["in_backend_us_per_layer"] = round(us, 3)
        roofline["in_backend_gbs"] = round(bytes_step / N_LAYER / (us * 1e-6) / 1e9, 1)

    mark(world, "decode: parity and per-layer form done")
    # End to end through the host-buffer C-ABI call: per layer q/k/v rows host->device, RoPE+append,
    # decode at position 4095 (4096 keys), output device->host; one synchronisation per step.
    inv = torch.from_numpy(inv_freq_table()).cuda()
    # q, k and v rows sit in one pinned block (q of all layers, then k, then v): the call then needs one copy in.
    nq, nk = N_LAYER * H * D, N_LAYER * HKV * D
    blk = torch.randn(nq + 2 * nk).pin_memory()
    qh, kh, vh = blk[:nq].view(N_LAYER, 1, H, D), blk[nq:nq + nk].view(N_LAYER, 1, HKV, D), blk[nq + nk:].view(N_LAYER, 1, HKV, D)
    oh = torch.empty(N_LAYER, 1, H, D).pin_memory()

    def step_e2e():
        ib.attn_layers_host(kv, 0, qh, kh, vh, oh, inv, DECODE_KEYS - 1)
        torch.cuda.current_stream().synchronize()

    te = timed(step_e2e, args.steps, args.warmup, world, 0.0 if args.no_graph else min(0.25, MIN_TIMED_S))
    ms_e2e = te["ms"]
    e2e = {"value": round(world * bytes_step * args.steps / (ms_e2e * 1e-3) / 1e9, 1), "unit": "GB/s",
           "h2d_bytes_per_step": int(N_LAYER * (H + 2 * HKV) * D * 4 + 8), "d2h_bytes_per_step": int(N_LAYER * H * D * 4),
           "ms_per_step": round(ms_e2e / args.steps, 4), "gpu_launches_per_step": 3,
           "timed_region_s": te["timed_region_s"]}
    assert kv.status() == 0
    return {"metric": "decode attention KV-cache HBM GB/s (4096 keys, 24q/8kv heads, d128, f16 KV, 28 layers)",
            "value": round(value, 1), "unit": "GB/s", "ms_per_step": round(ms / args.steps, 5), "scaling": "weak",
            "dtype": "f16 KV / f16 MMA operands / f32 accumulate+softmax", "roofline": roofline, "e2e": e2e,
            "gpu_launches": launches, "clocks": clk.summary(), "parity": par, "blocks": t["blocks"],
            "timed_region_s": t["timed_region_s"], "ms_per_step_best_block": round(t["ms_best"] / args.steps, 5),
            "config": decode_config(world)}


def inv_freq_table():
    # src/model.cpp:59-69, iterated f32 multiply.
    out = np.empty(D // 2, dtype=np.float32)
    scale = np.float32(np.power(np.float32(500000.0), np.float32(-2.0 / D), dtype=np.float32))
    f = np.float32(1.0)
    for i in range(D // 2):
        out[i] = f
        f = np.float32(f * scale)
    return out


# ------------------------------------------------------------------------------------------------
# prefill: configs[4]
# ------------------------------------------------------------------------------------------------

def prefill_flops(n_tok=None):
    n_tok = n_tok or PREFILL_TOKENS
    return 4 * n_tok * n_tok * H * D // 2


def all_ranks_agree(ok, device):
    """True only if `ok` is true on every rank (one MIN all-reduce): all ranks then take the same branch."""
    import torch
    import torch.distributed as dist
    t = torch.tensor([1 if ok else 0], device=device, dtype=torch.int32)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(int(t.item()))


def worst_status(status, device):
    """The largest status word over all ranks (0 = no rank reported an error)."""
    import torch
    import torch.distributed as dist
    t = torch.tensor([int(status)], device=device, dtype=torch.int32)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return int(t.item())


def run_prefill(args, rank, world):
    import torch
    import ingot_b200 as ib
    from ingot_b200 import workloads as W
    assert HKV % world == 0
    hkv_l, h_l = HKV // world, H // world
    S = args.prefill_tokens
    # The configs[4] tensors themselves (numpy default_rng(4), draw order q, K, V; q rounded to bf16, K/V to f16),
    # the same on every rank; each rank keeps its KV-head slice.
    c5 = W.c5_prefill32k(n_tok=S)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, hkv_l, S)
    kv.import_f16(0, torch.from_numpy(np.ascontiguousarray(c5.k[:, rank * hkv_l:(rank + 1) * hkv_l])).cuda(),
                  torch.from_numpy(np.ascontiguousarray(c5.v[:, rank * hkv_l:(rank + 1) * hkv_l])).cuda(), 0)
    q = torch.from_numpy(np.ascontiguousarray(c5.q[:, rank * h_l:(rank + 1) * h_l])).cuda().bfloat16()
    out = torch.empty(S, h_l, D, device="cuda", dtype=torch.float16)
    mark(world, "prefill: inputs ready")
    gathered = torch.empty(world * S, h_l, D, device="cuda", dtype=torch.float16) if world > 1 else None  # rank-major
    # N > 1: the gather of head outputs is fused into the kernel's epilogue - every rank stores its rows straight
    # into all ranks' token-major [S][24][128] buffers (symmetric memory, plain peer stores over NVLink) and then
    # signals every peer; a small kernel waits (bounded) for all peers' signals (class GatherSync). If symmetric
    # memory cannot be set up the step falls back to kernel + NCCL all-gather and says so in `config`.
    gather_mode, peer_ptrs, full, gs = "none (single GPU)", None, None, None
    if world > 1:
        import torch.distributed as dist
        gather_mode = "NCCL all_gather_into_tensor after the kernel"
        if not args.no_fused_gather:
            try:
                gs = GatherSync(S, world, rank, args.gather_barrier)
                full, peer_ptrs = gs.full, gs.peer_ptrs
                gather_mode = gs.mode
            except Exception as e:  # noqa: BLE001
                peer_ptrs, gs = None, None
                gather_mode += f" (symmetric memory unavailable: {type(e).__name__}: {e})"
            # Every rank takes the same path: the fused form only if symmetric memory came up on all of them.
            if not all_ranks_agree(peer_ptrs is not None, "cuda") and peer_ptrs is not None:
                peer_ptrs, gs, full = None, None, None
                gather_mode = "NCCL all_gather_into_tensor after the kernel (symmetric memory unavailable on another rank)"
            dist.barrier()  # every rank's signal counters are zero before anyone signals
        stage(f"prefill: gather mode = {gather_mode}")

    def step():
        if peer_ptrs is not None:
            gs.step(kv, q, h_l)
        else:
            ib.attn_prefill(kv, 0, q, 0, out=out, impl=2)
            if world > 1:
                dist.all_gather_into_tensor(gathered, out)

    def step_kernel_only():
        ib.attn_prefill(kv, 0, q, 0, out=out, impl=2)

    gather_checked = None
    if peer_ptrs is not None:  # one-time check of the fused gather against kernel + NCCL all-gather
        step()
        torch.cuda.synchronize()
        # If some rank's bounded wait for the signals ran out, every rank switches to the all-reduce barrier (and says so).
        waited_out = worst_status(kv.status(), "cuda")
        if waited_out != 0 and gs.barrier == "signal":
            gs.barrier = "nccl"
            gs.mode = ("fused: peer stores from the kernel epilogue + 1-element all-reduce barrier "
                       f"(the wait for the in-kernel signals ran out on some rank, status {waited_out})")
            gather_mode = gs.mode
            stage("prefill: signal wait timed out, falling back to the all-reduce barrier")
            step()
            torch.cuda.synchronize()
            kv.status()
        step_kernel_only()
        dist.all_gather_into_tensor(gathered, out)
        torch.cuda.synchronize()
        ref = gathered.view(world, S, h_l, D).permute(1, 0, 2, 3).reshape(S, H, D)
        gather_checked = bool(torch.equal(ref, full))
        if not gather_checked:
            raise SystemExit("fused gather differs from kernel + NCCL all-gather")
        stage("prefill: fused gather verified")

    steps = max(1, min(args.steps, args.prefill_steps))
    with ClockSampler(torch.cuda.current_device()) as clk:
        t = timed(step, steps, args.warmup, world, MIN_TIMED_S)
    ms = t["ms"]
    tk = t if world == 1 else timed(step_kernel_only, steps, 3, world, min(0.1, MIN_TIMED_S))
    ms_kernel = tk["ms"]
    assert kv.status() == 0
    mark(world, "prefill: timed")

    # Parity of the timed call's output, outside the timed region: row 0, the last row and 14 random rows (all 24
    # heads; at N > 1 read from the gathered buffer) against the CPU reference.
    torch.cuda.synchronize()
    rows = np.unique(np.concatenate([[0, S - 1], np.random.default_rng(44).integers(0, S, 14)])).astype(np.int64)
    if world > 1 and peer_ptrs is None:
        torch.cuda.synchronize()
        got = gathered.view(world, S, h_l, D).permute(1, 0, 2, 3).reshape(S, H, D)[rows].float().cpu().numpy()
    else:
        got = (full if world > 1 else out)[torch.from_numpy(rows).cuda()].float().cpu().numpy()
    par = None
    if rank == 0:
        want = oracle_rows(c5.q[rows], c5.k, c5.v, rows, HKV)
        par = parity(got, want)
        par["checked"] = f"{len(rows)} query rows x 24 heads (row 0, the last row, random rows) against the CPU reference"
    del c5

    flops = prefill_flops(S)
    value = flops * steps / (ms * 1e-3) / 1e12
    peaks = measured_peaks()
    per_gpu = flops / world * steps / (ms_kernel * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": round(per_gpu, 1), "peak": peaks["tflops_burst"], "unit": "TFLOP/s",
                "frac": round(per_gpu / peaks["tflops_burst"], 4), "traffic": NCU_TRAFFIC["attn_prefill_sm100_kernel"],
                "kernel": "attn_prefill_sm100_kernel", "peak_source": f"of {peaks['source']} (cuBLAS bf16 burst)",
                "frac_of_sustained": round(per_gpu / peaks["tflops_sustained"], 4),
                "frac_of_nominal_2250": round(per_gpu / 2250.0, 4), "ms_per_launch": round(ms_kernel / steps, 4),
                "best_block_tflops": round(flops / world * steps / (tk["ms_best"] * 1e-3) / 1e12, 1)}

    mark(world, "prefill: parity done")
    # End to end with host buffers through the C ABI (ingot_attn_prefill_host): this rank's q slice in pinned host
    # memory in, its output rows in pinned host memory out; the call cuts the rows into chunks of three CTA waves and overlaps
    # the copy in of the next chunk, the attention of the current one and the copy out of the previous one.
    qh = q.cpu().pin_memory()
    oh = torch.empty(out.shape, dtype=out.dtype).pin_memory()

    def step_e2e():
        ib.attn_prefill_host(kv, 0, qh, 0, oh)
        torch.cuda.current_stream().synchronize()

    te = timed(step_e2e, min(steps, 5), 1, world, min(0.1, MIN_TIMED_S))
    ms_e2e = te["ms"] / min(steps, 5)
    assert kv.status() == 0
    e2e_par = None
    if rank == 0:
        e2e_par = parity(oh[torch.from_numpy(rows)].float().numpy(), want[:, :oh.shape[1]])  # rank 0 owns the first heads
    e2e = {"value": round(flops / (ms_e2e * 1e-3) / 1e12, 1), "unit": "TFLOP/s",
           "h2d_bytes_per_step": int(q.numel() * 2), "d2h_bytes_per_step": int(out.numel() * 2),
           "ms_per_step": round(ms_e2e, 4), "call": "ingot_attn_prefill_host: chunks of three CTA waves, copies overlapped with the kernels",
           "parity": e2e_par}
    return {"metric": f"causal GQA prefill attention TFLOP/s ({S} tokens, 24q/8kv heads, d128, bf16 q, f16 K/V)",
            "value": round(value, 1), "unit": "TFLOP/s", "ms_per_step": round(ms / steps, 4), "steps": steps,
            "ms_kernel": round(ms_kernel / steps, 4), "blocks": t["blocks"], "timed_region_s": t["timed_region_s"],
            "scaling": "strong", "dtype": "f16 MMA operands (bf16 q converted on load) / f32 accumulate+softmax",
            "roofline": roofline, "e2e": e2e, "gpu_launches": steps * t["blocks"] * (1 if world == 1 else 2),
            "clocks": clk.summary(), "parity": par,
            "config": dict(prefill_config(S, world), gather=gather_mode, gather_verified=gather_checked)}


class GatherSync:
    """Destination buffers and completion signalling of the KV-head-sharded prefill at N > 1: one symmetric-memory
    allocation per rank holding the token-major output [S][24][128] f16 and one holding a counter per source rank.
    A step is the fused kernel (peer stores from its epilogue, then one released signal per destination from its
    last CTA) followed by the bounded wait for all N signals on this rank - no collective on the data path.
    --gather-barrier nccl keeps the earlier form, a one-element NCCL all-reduce as the completion barrier."""

    def __init__(self, S, world, rank, barrier="signal"):
        import torch
        import torch.distributed as dist
        # The kernels here use plain peer stores only; no multicast object is wanted on these buffers (a rank that leaves
        # early - the watchdog, a collective time-out - must not leave peers with memory bound to one).
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        self.full = symm.empty((S, H, D), dtype=torch.float16, device="cuda")
        hdl = symm.rendezvous(self.full, dist.group.WORLD)
        self.peer_ptrs = [int(x) for x in hdl.buffer_ptrs]
        self.rank, self.world, self.barrier = rank, world, barrier
        self.token = torch.zeros(1, device="cuda")
        if barrier == "signal":
            self.sig = symm.empty((64,), dtype=torch.int32, device="cuda")
            self.sig.zero_()
            torch.cuda.synchronize()
            sh = symm.rendezvous(self.sig, dist.group.WORLD)
            self.sig_ptrs = [int(x) for x in sh.buffer_ptrs]
            self.mode = "fused: peer stores from the kernel epilogue + released per-source signals, bounded wait kernel"
        else:
            self.mode = "fused: peer stores from the kernel epilogue + 1-element all-reduce barrier"

    def step(self, kv, q, h_l):
        import torch.distributed as dist
        import ingot_b200 as ib
        if self.barrier == "signal":
            ib.attn_prefill_gather_signal(kv, 0, q, 0, self.peer_ptrs, self.sig_ptrs, self.rank, ib.F16, H, self.rank * h_l)
            ib.gather_wait(kv, self.sig, self.world)
        else:
            ib.attn_prefill_gather(kv, 0, q, 0, self.peer_ptrs, ib.F16, H, self.rank * h_l)
            dist.all_reduce(self.token)


# ------------------------------------------------------------------------------------------------
# the other configurations (parity-test shapes; reported for completeness, not headline lines)
# ------------------------------------------------------------------------------------------------

def oracle_chunk(wl):
    """CPU reference output (RoPE + append + per-token attention loop) for a workloads.Prefill with rope=True: the
    reference's own compiled code when oracle/_ref is present (all host threads), else the plain-C restatement."""
    from oracle import loader
    lib, prefix = loader.load_ref(), "ref_"
    if lib is None:
        lib, prefix = loader.load_oracle(), "oracle_"
    n_ctx = wl.pos0 + wl.n_tok
    kc = np.zeros((n_ctx, HKV * D), dtype=np.float32)
    vc = np.zeros((n_ctx, HKV * D), dtype=np.float32)
    if wl.pos0:
        kc[:wl.pos0] = wl.cache_k.astype(np.float32).reshape(wl.pos0, -1)
        vc[:wl.pos0] = wl.cache_v.astype(np.float32).reshape(wl.pos0, -1)
    return loader.attn_forward(lib, prefix, wl.q, wl.k, wl.v, wl.pos0, n_ctx, loader.inv_freq(lib, prefix), kc, vc)[0]


def run_chunked(args, rank, world, wl, label):
    """K1 + K2 per layer for a chunk of new tokens (configs[0] / configs[2]), 28 layers per step, one GPU per rank
    (replicas). Layer 0 carries the configuration's own seeded tensors and is checked against the CPU reference."""
    import torch
    import ingot_b200 as ib
    n_tok, pos0 = wl.n_tok, wl.pos0
    torch.manual_seed(2)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, N_LAYER, HKV, pos0 + n_tok)
    for l in range(N_LAYER):
        kv.layer_view(l, "k").copy_(torch.randn(HKV, pos0 + n_tok, D, device="cuda").half())
        kv.layer_view(l, "v").copy_(torch.randn(HKV, pos0 + n_tok, D, device="cuda").half())
    q = torch.randn(N_LAYER, n_tok, H, D, device="cuda")
    k = torch.randn(N_LAYER, n_tok, HKV, D, device="cuda")
    v = torch.randn(N_LAYER, n_tok, HKV, D, device="cuda")
    q[0].copy_(torch.from_numpy(wl.q)); k[0].copy_(torch.from_numpy(wl.k)); v[0].copy_(torch.from_numpy(wl.v))
    if pos0:
        kv.import_f16(0, torch.from_numpy(wl.cache_k).cuda(), torch.from_numpy(wl.cache_v).cuda(), 0)
    out = torch.empty(N_LAYER, n_tok, H, D, device="cuda")
    inv = torch.from_numpy(inv_freq_table()).cuda()
    want = oracle_chunk(wl) if rank == 0 else None
    res, par = {}, {}
    steps = max(1, min(args.steps, 10))
    names = {0: "auto", 1: "warp_mma", 2: "tcgen05"}
    for impl in (1, 2, 0):
        def launch_layers():
            for l in range(N_LAYER):
                qr = ib.rope_kv_append(kv, l, q[l], k[l], v[l], inv, pos0)
                ib.attn_prefill(kv, l, qr, pos0, out=out[l], impl=impl)
        # One CUDA graph per step (the 28 layers' launches), so that Python launch overhead is not timed.
        step = launch_layers if args.no_graph else captured(launch_layers)
        t = timed(step, steps, args.warmup, world, min(0.1, MIN_TIMED_S))
        res[impl] = t["ms"] / steps / N_LAYER
        torch.cuda.synchronize()
        if rank == 0:
            par[names[impl]] = parity(out[0].cpu().numpy(), want)
    assert kv.status() == 0
    flops = wl.flops
    best = res[0]
    peaks = measured_peaks()
    tf = flops / (best * 1e-3) / 1e12
    return {"metric": f"causal GQA chunked prefill TFLOP/s ({label})", "value": round(world * tf, 2), "unit": "TFLOP/s",
            "ms_per_step": round(best * N_LAYER, 4), "steps": steps, "scaling": "weak",
            "dtype": "f16 MMA operands / f32 accumulate+softmax",
            "roofline": {"bound": "tensor", "achieved": round(tf, 2), "peak": peaks["tflops_burst"], "unit": "TFLOP/s",
                         "frac": round(tf / peaks["tflops_burst"], 4), "traffic": None,
                         "us_per_layer": {names[i]: round(res[i] * 1e3, 2) for i in (0, 1, 2)}},
            "gpu_launches": 2 * N_LAYER * steps, "parity": par,
            "config": {"workload": label, "n_tok": n_tok, "pos0": pos0, "n_layer": N_LAYER, "flops_per_layer": flops,
                       "includes": "RoPE+append (K1) and attention (K2, plus its split merge where used) per layer, 28 layers per CUDA graph replay",
                       "parallelism": f"replicas x{world}"}}


def run_batched_decode(args, rank, world):
    """configs[3]: 64 sequences, lengths U{256..8192}, paged f16 cache with permuted 16-token blocks, bf16 queries;
    sequences sharded over the ranks by length-balanced (LPT) assignment, no collective on the data path."""
    import torch
    import ingot_b200 as ib
    from ingot_b200 import workloads as W
    lens_all = W.c4_lengths()
    mine = W.lpt_assign(lens_all, world)[rank]
    lens = lens_all[mine]
    n_seq = len(lens)
    nb = int(((lens + 15) // 16).sum())
    perm = np.random.default_rng([3, 2, rank]).permutation(nb).astype(np.int32)
    bt_np = W.block_tables(lens, perm)
    bt = torch.from_numpy(bt_np).cuda()
    n_layers = 4  # distinct per-layer pools so that a step streams more than L2 holds
    kv = ib.KVCache(ib.KV_PAGED, n_layers, HKV, nb, max_seqs=n_seq)
    torch.manual_seed(3 + rank)
    for l in range(n_layers):
        kv.layer_view(l, "k").copy_(torch.randn(nb, HKV, 16, D, device="cuda").half())
        kv.layer_view(l, "v").copy_(torch.randn(nb, HKV, 16, D, device="cuda").half())
    q = torch.randn(n_layers, n_seq, H, D, device="cuda").bfloat16()
    out = torch.zeros(n_layers, n_seq, H, D, device="cuda")
    lens_d = torch.from_numpy(lens).cuda()

    def launch():
        ib.attn_decode_layers(kv, 0, q, out, seq_lens=lens_d, max_seq_len=int(lens.max()), block_tables=bt,
                              chunk_keys=args.chunk_keys)

    step = launch if args.no_graph else captured(launch)
    with ClockSampler(torch.cuda.current_device()) as clk:
        t = timed(step, args.steps, args.warmup, world, min(0.25, MIN_TIMED_S))
    ms = t["ms"]
    assert kv.status() == 0
    # Parity outside the timed region: this rank's shortest, longest and one middle sequence of the last layer.
    torch.cuda.synchronize()
    order = np.argsort(lens)
    errs = []
    lyr = n_layers - 1
    for s_i in (int(order[0]), int(order[len(order) // 2]), int(order[-1])):
        n = int(lens[s_i])
        blocks = torch.from_numpy(bt_np[s_i, :(n + 15) // 16].astype(np.int64)).cuda()
        k_s = kv.layer_view(lyr, "k")[blocks].permute(0, 2, 1, 3).reshape(-1, HKV, D)[:n].cpu().numpy()
        v_s = kv.layer_view(lyr, "v")[blocks].permute(0, 2, 1, 3).reshape(-1, HKV, D)[:n].cpu().numpy()
        want = oracle_rows(q[lyr, s_i:s_i + 1].float().cpu().numpy(), k_s, v_s, [n - 1], HKV)
        errs.append(parity(out[lyr, s_i:s_i + 1].cpu().numpy(), want))
    par = torch.tensor([max(e["max_abs"] for e in errs), max(e["rel_l2"] for e in errs)], device="cuda", dtype=torch.float64)
    bytes_rank = int(lens.astype(np.int64).sum()) * HKV * D * 2 * 2 * n_layers
    tot = torch.tensor([float(bytes_rank)], device="cuda", dtype=torch.float64)
    mx = tot.clone()
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(tot)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(par, op=dist.ReduceOp.MAX)
    value = float(tot.item()) * args.steps / (ms * 1e-3) / 1e9
    peaks = measured_peaks()
    per_gpu = float(mx.item()) * args.steps / (ms * 1e-3) / 1e9  # the most loaded rank sets the step time
    return {"metric": "batched paged decode attention KV-cache HBM GB/s (64 sequences, lengths 256..8192)", "value": round(value, 1),
            "unit": "GB/s", "ms_per_step": round(ms / args.steps, 5), "scaling": "strong", "blocks": t["blocks"],
            "timed_region_s": t["timed_region_s"],
            "dtype": "f16 KV / f16 MMA operands (bf16 q converted on load) / f32 accumulate+softmax",
            "roofline": {"bound": "hbm", "achieved": round(per_gpu, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(per_gpu / peaks["hbm_gbs"], 4), "traffic": None, "kernel": "attn_decode_kernel",
                         "note": "per GPU, on the most loaded rank"},
            "gpu_launches": args.steps * t["blocks"] * 2, "clocks": clk.summary(),
            "parity": {"max_abs": float(par[0].item()), "rel_l2": float(par[1].item()),
                       "within_tolerance": bool(par[0].item() <= 2e-3 and par[1].item() <= 1e-3),
                       "checked": "shortest, median and longest sequence of every rank (last layer) against the CPU reference"},
            "config": {"workload": "configs[3]: 64-sequence paged decode, 16-token blocks, random block permutation",
                       "n_seq_this_rank": n_seq, "layers_per_step": n_layers, "kv_bytes_per_layer_this_rank": bytes_rank // n_layers,
                       "load_imbalance_max_over_mean": round(float(mx.item()) * world / float(tot.item()), 4),
                       "parallelism": f"sequence sharding x{world} (LPT length balancing, no collective)"}}


def run_e2e_model(args):
    """`ingot bench -p 128 -n 32` through the reference's own engine glue on a seeded random-init
    Llama-3.2-3B-shaped F16 GGUF: the CUDA backend of this repository against the reference's CpuBackend
    (both inside backend/_build/libingot_engine_cuda.so). Whole-model tokens/s. --no-cpu skips the CpuBackend leg."""
    import ctypes as C
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_random_gguf
    eng = os.path.join(ROOT, "inference-agent_b200", "backend", "_build", "libingot_engine_cuda.so")
    lib = C.CDLL(eng)
    i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
    f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")
    lib.ingot_e2e_bench.argtypes = [C.c_char_p, C.c_char_p, i32p, C.c_int, C.c_int, C.c_int, C.c_int, f64p]
    lib.ingot_e2e_last_error.restype = C.c_char_p
    n_layer, n_vocab = (28, 128256) if not args.small_model else (2, 32064)
    tag = "" if args.wtype == "F16" else f"_{args.wtype}_{args.output_type or args.wtype}"
    path = os.path.join(os.environ.get("INGOT_E2E_DIR", "/tmp"), f"ingot_random_l{n_layer}_v{n_vocab}_s0{tag}.gguf")
    if not os.path.exists(path):
        make_random_gguf.write(path + ".tmp", n_layer, n_vocab, seed=0, wtype=args.wtype, output_type=args.output_type)
        os.replace(path + ".tmp", path)
    # bytes of weights one generated token has to read: every layer matrix and the output matrix (not the embedding table)
    bpw = {"F16": 2.0, "Q8_0": 34 / 32, "Q4_0": 18 / 32, "Q4_1": 20 / 32, "Q6_K": 210 / 256}
    layer_params = n_layer * (3072 * 3072 * 2 + 3072 * 1024 * 2 + 3 * 3072 * 8192)
    weight_bytes = layer_params * bpw[args.wtype] + n_vocab * 3072 * bpw[args.output_type or args.wtype]
    prompt = np.random.default_rng(0).integers(0, n_vocab, size=128).astype(np.int32)
    res = {}
    res["cpu"] = None
    for name, backend, reps in (("cuda", b"metal", 3), ("cpu", b"cpu", 1)):
        if name == "cpu" and args.no_cpu:
            continue
        out = np.zeros(2, dtype=np.float64)
        if lib.ingot_e2e_bench(path.encode(), backend, prompt, 128, 32, 512, reps, out) != 0:
            raise SystemExit(lib.ingot_e2e_last_error().decode())
        res[name] = {"pp128_tok_s": round(float(out[0]), 2), "tg32_tok_s": round(float(out[1]), 2)}
    return {"metric": "whole-model tokens/s, pp128 / tg32 (the reference's `ingot bench` measurement)", "value": res["cuda"]["tg32_tok_s"],
            "unit": "tok/s (tg32)", "n_gpus": 1, "steps": 3, "warmup": 1, "ms_per_step": None, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 weights, f32 activations, f16 KV", "data": "synthetic",
            "config": {"workload": f"random-init Llama-3.2-3B-shaped {args.wtype} GGUF (output matrix {args.output_type or args.wtype}), "
                                   f"{n_layer} layers, vocab {n_vocab}; 128 prompt ids, 32 greedy steps"},
            "cuda_backend": res["cuda"], "cpu_reference_backend": res["cpu"],
            "roofline": {"bound": "hbm", "unit": "GB/s", "peak": measured_peaks()["hbm_gbs"],
                         "achieved": round(weight_bytes * res["cuda"]["tg32_tok_s"] / 1e9, 1),
                         "frac": round(weight_bytes * res["cuda"]["tg32_tok_s"] / 1e9 / measured_peaks()["hbm_gbs"], 4),
                         "traffic": None, "weight_bytes_per_token": int(weight_bytes),
                         "note": "single-token steps are bound by reading every weight once per token"},
            "note": "reference README (Apple M5, Metal, F16): pp128 864 tok/s, tg32 15.6 tok/s"}

# ------------------------------------------------------------------------------------------------
# CPU reference legs
# ------------------------------------------------------------------------------------------------

def cpu_decode_sample(n_layers, reps):
    """Times the reference's CPU attention (f32 cache, all host threads) on the decode workload.

    Returns (GB/s by the same byte formula, kind, cores, seconds per layer)."""
    from oracle import loader
    ref = loader.load_ref()
    rng = np.random.default_rng(1)
    kc = rng.standard_normal((DECODE_KEYS, HKV * D), dtype=np.float32)
    vc = rng.standard_normal((DECODE_KEYS, HKV * D), dtype=np.float32)
    caches = [(kc.copy(), vc.copy()) for _ in range(n_layers)]  # distinct memory per layer, like the GPU leg
    q = rng.standard_normal((H, D), dtype=np.float32)
    out = np.empty((H, D), dtype=np.float32)
    scores = np.empty(H * DECODE_KEYS, dtype=np.float32)
    if ref is not None:
        kind, cores = "reference", ref.ref_thread_count()
        run = lambda k, v: ref.ref_attend(q.reshape(-1), k.reshape(-1), v.reshape(-1), DECODE_KEYS - 1, H, HKV, D,
                                          out.reshape(-1), scores)
    else:
        orc = loader.load_oracle()
        kind, cores = "port", 1
        run = lambda k, v: orc.oracle_attend(q.reshape(-1), k.reshape(-1), v.reshape(-1), DECODE_KEYS - 1, H, HKV, D,
                                             out.reshape(-1), scores)
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        for k, v in caches:
            run(k, v)
        best = min(best, time.perf_counter() - t0)
    per_layer = best / n_layers
    gbs = (decode_bytes_per_step() / N_LAYER) / per_layer / 1e9
    return gbs, kind, cores, per_layer


def cpu_prefill_sample(n_rows=48):
    """Reference CPU attention on a stratified row sample of the 32768-token prefill, extrapolated by FLOPs."""
    from oracle import loader
    ref = loader.load_ref()
    rng = np.random.default_rng(4)
    S = PREFILL_TOKENS
    kc = rng.standard_normal((S, HKV * D), dtype=np.float32)
    vc = rng.standard_normal((S, HKV * D), dtype=np.float32)
    rows = np.unique(np.concatenate([np.arange(8), np.arange(S - 8, S), rng.integers(0, S, n_rows - 16)]))
    q = rng.standard_normal((H, D), dtype=np.float32)
    out = np.empty((H, D), dtype=np.float32)
    scores = np.empty(H * S, dtype=np.float32)
    if ref is not None:
        kind, cores, fn = "reference", ref.ref_thread_count(), ref.ref_attend
    else:
        orc = loader.load_oracle()
        kind, cores, fn = "port", 1, orc.oracle_attend
    t0 = time.perf_counter()
    for r in rows:
        fn(q.reshape(-1), kc.reshape(-1), vc.reshape(-1), int(r), H, HKV, D, out.reshape(-1), scores)
    dt = time.perf_counter() - t0
    flops = sum(4 * H * D * (int(r) + 1) for r in rows)
    return flops / dt / 1e12, kind, cores, len(rows)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    if args.workload == "prefill_c5":
        tf, kind, cores, n = cpu_prefill_sample()
        sample = f"{n} query rows (first 8, last 8, random) x 24 heads of the 32768-token prefill, extrapolated by FLOPs"
        line = {"metric": "causal GQA prefill attention TFLOP/s (32768 tokens, 24q/8kv heads, d128, bf16 q, f16 K/V)",
                "value": round(tf, 5), "unit": "TFLOP/s", "ms_per_step": None, "scaling": "strong",
                "config": prefill_config(PREFILL_TOKENS, args.gpus)}
    else:
        t0 = time.perf_counter()
        for _ in range(args.warmup):
            cpu_decode_sample(4, 1)
        vals = []
        for _ in range(args.steps):
            gbs, kind, cores, per_layer = cpu_decode_sample(N_LAYER, 1)
            vals.append((gbs, per_layer))
            if time.perf_counter() - t0 > 120:
                break
        gbs = statistics.median(v[0] for v in vals)
        per_layer = statistics.median(v[1] for v in vals)
        sample = f"{len(vals)} steps x 28 layers of the full decode workload (f32 cache as the reference keeps it)"
        line = {"metric": "decode attention KV-cache HBM GB/s (4096 keys, 24q/8kv heads, d128, f16 KV, 28 layers)",
                "value": round(gbs, 3), "unit": "GB/s", "ms_per_step": round(per_layer * N_LAYER * 1e3, 3), "scaling": "weak",
                "config": decode_config(args.gpus)}
    line.update({"impl": "reference", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                 "higher_is_better": True, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                 "cpu_baseline": {"value": line["value"], "unit": line["unit"], "cores": cores, "kind": kind, "sample": sample},
                 "e2e": {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    return line


def main():
    global MIN_TIMED_S
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ingot", choices=["ingot", "reference"])
    ap.add_argument("--workload", default="decode_c2", choices=["decode_c2", "prefill_c5", "c1_prefill128", "c3_chunked", "c4_batched", "e2e_model"])
    ap.add_argument("--small-model", action="store_true", help="e2e_model: 2 layers and a 32064-token vocabulary")
    ap.add_argument("--wtype", default="F16", choices=["F16", "Q8_0", "Q4_0", "Q4_1", "Q6_K"], help="e2e_model: weight type of the GGUF")
    ap.add_argument("--output-type", default=None, choices=["F16", "Q8_0", "Q4_0", "Q4_1", "Q6_K"],
                    help="e2e_model: type of the embedding / output matrix (default: --wtype)")
    ap.add_argument("--chunk-keys", type=int, default=0, help="decode split size (0 = library default)")
    ap.add_argument("--prefill-steps", type=int, default=10, help="cap on timed prefill steps (each is ~10 ms)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="prefill length; anything but 32768 is a profiling case, not the benchmark configuration")
    ap.add_argument("--no-secondary", action="store_true", help="skip the non-headline workload")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-fused-gather", action="store_true",
                    help="prefill at N > 1: kernel + NCCL all-gather instead of the fused peer-store epilogue")
    ap.add_argument("--gather-barrier", default="signal", choices=["signal", "nccl"],
                    help="prefill at N > 1: completion of the fused gather by in-kernel signals (default) or a 1-element NCCL all-reduce")
    ap.add_argument("--min-timed-s", type=float, default=MIN_TIMED_S,
                    help="minimum length of the headline timed region; 0 for a profiling run that should launch little")
    ap.add_argument("--no-graph", action="store_true", help="decode: launch the 28 layers from Python instead of replaying a CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    MIN_TIMED_S = args.min_timed_s

    if args.impl == "reference":
        line = run_reference(args)
        if line is not None:
            print(json.dumps(line), flush=True)
        return

    if args.workload == "e2e_model":
        print(json.dumps(run_e2e_model(args)), flush=True)
        return

    start_watchdog(int(os.environ.get("WORLD_SIZE", "1")))  # before the process group comes up: its set-up can stall too
    rank, world, _ = dist_setup(args.gpus)
    from ingot_b200 import workloads as W
    others = {
        "c1_prefill128": lambda a, r, w: run_chunked(a, r, w, W.c1_prefill128(), "configs[0]: 128-token prefill at position 0"),
        "c3_chunked": lambda a, r, w: run_chunked(a, r, w, W.c3_chunked(), "configs[2]: 512-token chunk onto 3584 cached positions"),
        "c4_batched": run_batched_decode,
    }
    if args.workload in others:
        args.no_secondary = args.no_cpu = True
        primary, secondary = others[args.workload], None
    else:
        primary, secondary = (run_decode, run_prefill) if args.workload == "decode_c2" else (run_prefill, run_decode)
    line = primary(args, rank, world)
    out = None
    if rank == 0:
        out = {"metric": line.pop("metric"), "value": line.pop("value"), "unit": line.pop("unit"), "n_gpus": world,
               "steps": line.pop("steps", args.steps), "warmup": args.warmup, "ms_per_step": line.pop("ms_per_step"),
               "higher_is_better": True, "scaling": line.pop("scaling"), "vs_baseline": None, "dtype": line.pop("dtype"),
               "data": "synthetic"}
        line.setdefault("clocks", None)
        line.setdefault("e2e", None)
        out.update(line)
    other_name = "prefill" if args.workload == "decode_c2" else "decode"
    # the remaining configurations ride along as objects of their own: the other headline shape, the two chunked-prefill
    # shapes on one GPU (they are replicas at N > 1) and the sequence-sharded batched decode at every N
    # (at N > 1 the workload without a data-path exchange runs before the one with the fused gather)
    rest = [] if args.no_secondary else ([other_name, "c1_prefill128", "c3_chunked", "c4_batched"] if world == 1 else ["c4_batched", other_name])
    _PARTIAL["pending"] = list(rest)
    _PARTIAL["line"] = out
    if world > 1:
        stage("primary workload done")
    other = None
    for name in rest:
        res = secondary(args, rank, world) if name == other_name else others[name](args, rank, world)
        if name == other_name:
            other = res
        if rank == 0:
            out[name] = res
        _PARTIAL["pending"].remove(name)
        if world > 1:
            stage(f"{name} done")
    if rank == 0:
        if world == 1 and not args.no_cpu:
            if args.workload == "decode_c2":
                gbs, kind, cores, per_layer = cpu_decode_sample(N_LAYER, 3)
                out["cpu_baseline"] = {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": kind,
                                       "sample": "best of 3 passes over the 28 layers of the full decode workload "
                                                 "(f32 cache as the reference keeps it; same byte formula)",
                                       "ms_per_layer": round(per_layer * 1e3, 3)}
                if other is not None:
                    tf, kind, cores, n = cpu_prefill_sample()
                    other["cpu_baseline"] = {"value": round(tf, 5), "unit": "TFLOP/s", "cores": cores, "kind": kind,
                                             "sample": f"{n} query rows x 24 heads of the 32768-token prefill, extrapolated by FLOPs"}
            else:
                tf, kind, cores, n = cpu_prefill_sample()
                out["cpu_baseline"] = {"value": round(tf, 5), "unit": "TFLOP/s", "cores": cores, "kind": kind,
                                       "sample": f"{n} query rows x 24 heads of the 32768-token prefill, extrapolated by FLOPs"}
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except Exception as exc:  # noqa: BLE001
        n_ranks = int(os.environ.get("WORLD_SIZE", "1"))
        if n_ranks <= 1:
            raise
        import traceback
        traceback.print_exc()
        bail(n_ranks, f"stopped with {type(exc).__name__}: {exc}")
