#!/usr/bin/env python
"""Benchmark of the B200 attention path: decode KV-cache HBM GB/s and causal-prefill TFLOP/s.

    python bench.py --gpus N --steps K --warmup W [--workload decode_c2|prefill_c5] [--impl reference]

Headline (`metric`/`value`): single-token decode attention at 4096 keys, 24 query / 8 KV heads,
head_dim 128, f16 KV cache, one pass over 28 distinct per-layer caches per step (470 MB, larger than
L2), reported as KV-cache bytes per second with the reference's own `abench` byte formula
(2 * n_layer * (pos+1) * n_head_kv * head_dim * 2, src/main.cpp:446). With N > 1 every rank decodes its
own sequence (sequence sharding, no collective on the data path): weak scaling.
The same line carries a `prefill` object: 32768-token causal GQA prefill (bf16 q, f16 K/V) in TFLOP/s
counting 4*S^2*H*d/2, sharded by KV head over the N ranks with an NCCL all-gather of the head outputs
inside the timed region (strong scaling). `--workload prefill_c5` makes that the headline instead.

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

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "inference-agent_b200"))

N_LAYER, H, HKV, D = 28, 24, 8, 128
DECODE_KEYS = 4096
PREFILL_TOKENS = 32768

# DRAM bytes per launch of the dominant kernel from an ncu capture of the same kernel
# (dram__bytes_read.sum + dram__bytes_write.sum); see profiles/ for the command and the raw figures.
# decode: captured at the benchmark shape (profiles/attn_decode_c2.md). prefill: captured at 8192 tokens
# (84.0 MB read + 20.8 MB written; profiles/attn_prefill_sm100_8k.md) and scaled by the 4x token count,
# compulsory q/K/V/out traffic growing in proportion.
NCU_TRAFFIC = {"attn_decode_kernel": 16947456, "attn_prefill_sm100_kernel": 4 * (83955712 + 20809472)}


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


def dist_setup(n_gpus):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {n_gpus}")
    return rank, world, local


def timed(fn, steps, warmup, world):
    """W warm-up calls, then `steps` calls timed with CUDA events between barriers; max over ranks (ms)."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


# ------------------------------------------------------------------------------------------------
# decode: configs[1]
# ------------------------------------------------------------------------------------------------

def decode_bytes_per_step():
    return 2 * N_LAYER * DECODE_KEYS * HKV * D * 2


def decode_config(world):
    """The workload description both arms (this library and the reference's CPU code) report."""
    return {"workload": "configs[1]: decode @4096 keys, batch 1 per GPU, 28 per-layer caches per step",
            "n_layer": N_LAYER, "n_keys": DECODE_KEYS, "n_head": H, "n_head_kv": HKV, "head_dim": D,
            "l2": "inputs larger than L2 (470 MB of KV per step, 28 distinct caches)",
            "parallelism": f"sequence sharding x{world} (one sequence per GPU, no collective)"}


def prefill_config(S, world):
    return {"workload": ("configs[4]: 32768-token causal prefill, FLOPs = 4*S^2*H*d/2" if S == PREFILL_TOKENS
                         else f"PROFILING CASE: {S}-token causal prefill (not the benchmark configuration)"), "n_tok": S,
            "n_head": H, "n_head_kv": HKV, "head_dim": D, "l2": "inputs larger than L2 (q+out 400 MB, K/V 134 MB)",
            "parallelism": f"KV-head sharding x{world}"}


def decode_chains(n_layers):
    """Launch chains ingot_attn_decode_layers uses for n_layers (csrc/kv_cache.cu: up to INGOT_DECODE_STREAMS, default 8,
    then as few as give the same number of rounds)."""
    cap = min(max(int(os.environ.get("INGOT_DECODE_STREAMS", "8")), 1), 8, n_layers)
    rounds = -(-n_layers // cap)
    return -(-n_layers // rounds)


def run_decode(args, rank, world):
    import torch
    import ingot_b200 as ib
    torch.manual_seed(1 + rank)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, N_LAYER, HKV, DECODE_KEYS)
    for l in range(N_LAYER):  # synthetic N(0,1) cache, generated on the device
        kv.layer_view(l, "k").copy_(torch.randn(HKV, DECODE_KEYS, D, device="cuda").half())
        kv.layer_view(l, "v").copy_(torch.randn(HKV, DECODE_KEYS, D, device="cuda").half())
    q = torch.randn(N_LAYER, 1, H, D, device="cuda")
    out = torch.empty(N_LAYER, 1, H, D, device="cuda")

    def launch_layers():
        ib.attn_decode_layers(kv, 0, q, out, max_seq_len=DECODE_KEYS, chunk_keys=args.chunk_keys)

    # The 28 launches of a step are captured once in a CUDA graph (the reference encodes them into one
    # command buffer, src/metal_backend.mm:594-649); a step is one replay.
    launch_layers()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        launch_layers()
    step = graph.replay if not args.no_graph else launch_layers

    with ClockSampler(torch.cuda.current_device()) as clk:
        ms = timed(step, args.steps, args.warmup, world)
        # keep the same load running so that the clock samples mean something (skipped with --no-graph,
        # which is the profiling form of the command: a profiler should see the timed launches only)
        t_end = time.perf_counter() + (0.0 if args.no_graph else 0.4)
        while time.perf_counter() < t_end:
            step()
        torch.cuda.synchronize()
    # A step is 28 launches that each carry one layer's splits (and the previous layer's merge) plus
    # one merge-only launch per launch chain that closes it.
    launches = args.steps * (N_LAYER + decode_chains(N_LAYER))
    bytes_step = decode_bytes_per_step()
    value = world * bytes_step * args.steps / (ms * 1e-3) / 1e9
    per_launch_s = ms * 1e-3 / (args.steps * N_LAYER)  # per data-carrying launch (one layer)
    peaks = measured_peaks()
    achieved = bytes_step / N_LAYER / per_launch_s / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": NCU_TRAFFIC["attn_decode_kernel"],
                "kernel": "attn_decode_kernel", "peak_source": f"of {peaks['source']} (STREAM-style copy)",
                "algorithmic_bytes_per_launch": bytes_step // N_LAYER, "us_per_launch": round(per_launch_s * 1e6, 3)}

    # End to end through the host-buffer C-ABI call: per layer q/k/v rows host->device, RoPE+append,
    # decode at position 4095 (4096 keys), output device->host; one synchronisation per step.
    inv = torch.from_numpy(inv_freq_table()).cuda()
    qh = torch.randn(N_LAYER, 1, H, D).pin_memory()
    kh = torch.randn(N_LAYER, 1, HKV, D).pin_memory()
    vh = torch.randn(N_LAYER, 1, HKV, D).pin_memory()
    oh = torch.empty(N_LAYER, 1, H, D).pin_memory()

    def step_e2e():
        ib.attn_layers_host(kv, 0, qh, kh, vh, oh, inv, DECODE_KEYS - 1)
        torch.cuda.current_stream().synchronize()

    ms_e2e = timed(step_e2e, args.steps, args.warmup, world)
    e2e = {"value": round(world * bytes_step * args.steps / (ms_e2e * 1e-3) / 1e9, 1), "unit": "GB/s",
           "h2d_bytes_per_step": int(N_LAYER * (H + 2 * HKV) * D * 4), "d2h_bytes_per_step": int(N_LAYER * H * D * 4),
           "ms_per_step": round(ms_e2e / args.steps, 4), "gpu_launches_per_step": 1 + N_LAYER + decode_chains(N_LAYER)}
    assert kv.status() == 0
    return {"metric": "decode attention KV-cache HBM GB/s (4096 keys, 24q/8kv heads, d128, f16 KV, 28 layers)",
            "value": round(value, 1), "unit": "GB/s", "ms_per_step": round(ms / args.steps, 5), "scaling": "weak",
            "dtype": "f16 KV / f16 MMA operands / f32 accumulate+softmax", "roofline": roofline, "e2e": e2e,
            "gpu_launches": launches, "clocks": clk.summary(),
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


def run_prefill(args, rank, world):
    import torch
    import ingot_b200 as ib
    assert HKV % world == 0
    hkv_l, h_l = HKV // world, H // world
    torch.manual_seed(4)  # same tensors on every rank; each rank keeps its KV-head slice
    S = args.prefill_tokens
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, hkv_l, S)
    g = torch.Generator(device="cuda").manual_seed(4)
    k_all = torch.randn(HKV, S, D, device="cuda", generator=g).half()
    v_all = torch.randn(HKV, S, D, device="cuda", generator=g).half()
    q_all = torch.randn(S, H, D, device="cuda", generator=g).bfloat16()
    kv.layer_view(0, "k").copy_(k_all[rank * hkv_l:(rank + 1) * hkv_l])
    kv.layer_view(0, "v").copy_(v_all[rank * hkv_l:(rank + 1) * hkv_l])
    q = q_all[:, rank * h_l:(rank + 1) * h_l].contiguous()
    del k_all, v_all, q_all
    out = torch.empty(S, h_l, D, device="cuda", dtype=torch.float16)
    gathered = torch.empty(world * S, h_l, D, device="cuda", dtype=torch.float16) if world > 1 else None  # rank-major
    # N > 1: the gather of head outputs is fused into the kernel's epilogue — every rank stores its rows
    # straight into all ranks' token-major [S][24][128] buffers (symmetric memory, plain peer stores over
    # NVLink), followed by a one-element NCCL all-reduce as the cross-rank completion barrier. If symmetric
    # memory cannot be set up the step falls back to kernel + NCCL all-gather and says so in `config`.
    gather_mode, peer_ptrs, full, token = "none (single GPU)", None, None, None
    if world > 1:
        import torch.distributed as dist
        gather_mode = "NCCL all_gather_into_tensor after the kernel"
        if not args.no_fused_gather:
            try:
                import torch.distributed._symmetric_memory as symm
                full = symm.empty((S, H, D), dtype=torch.float16, device="cuda")
                hdl = symm.rendezvous(full, dist.group.WORLD)
                peer_ptrs = [int(x) for x in hdl.buffer_ptrs]
                token = torch.zeros(1, device="cuda")
                gather_mode = "fused: peer stores from the kernel epilogue + 1-element all-reduce barrier"
            except Exception as e:  # noqa: BLE001
                peer_ptrs = None
                gather_mode += f" (symmetric memory unavailable: {type(e).__name__})"

    def step():
        if peer_ptrs is not None:
            ib.attn_prefill_gather(kv, 0, q, 0, peer_ptrs, ib.F16, H, rank * h_l)
            dist.all_reduce(token)
        else:
            ib.attn_prefill(kv, 0, q, 0, out=out, impl=2)
            if world > 1:
                dist.all_gather_into_tensor(gathered, out)

    def step_kernel_only():
        ib.attn_prefill(kv, 0, q, 0, out=out, impl=2)

    gather_checked = None
    if peer_ptrs is not None:  # one-time check of the fused gather against kernel + NCCL all-gather
        step()
        step_kernel_only()
        dist.all_gather_into_tensor(gathered, out)
        torch.cuda.synchronize()
        ref = gathered.view(world, S, h_l, D).permute(1, 0, 2, 3).reshape(S, H, D)
        gather_checked = bool(torch.equal(ref, full))
        if not gather_checked:
            raise SystemExit("fused gather differs from kernel + NCCL all-gather")

    steps = max(1, min(args.steps, args.prefill_steps))
    with ClockSampler(torch.cuda.current_device()) as clk:
        ms = timed(step, steps, args.warmup, world)
    ms_kernel = ms if world == 1 else timed(step_kernel_only, steps, 3, world)
    assert kv.status() == 0
    flops = prefill_flops(S)
    value = flops * steps / (ms * 1e-3) / 1e12
    peaks = measured_peaks()
    per_gpu = flops / world * steps / (ms_kernel * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": round(per_gpu, 1), "peak": peaks["tflops_burst"], "unit": "TFLOP/s",
                "frac": round(per_gpu / peaks["tflops_burst"], 4), "traffic": NCU_TRAFFIC["attn_prefill_sm100_kernel"],
                "kernel": "attn_prefill_sm100_kernel", "peak_source": f"of {peaks['source']} (cuBLAS bf16 burst)",
                "frac_of_sustained": round(per_gpu / peaks["tflops_sustained"], 4),
                "frac_of_nominal_2250": round(per_gpu / 2250.0, 4), "ms_per_launch": round(ms_kernel / steps, 4)}

    # End to end with host buffers: this rank's q slice host->device, prefill, output device->host.
    qh = q.cpu().pin_memory()
    oh = torch.empty(out.shape, dtype=out.dtype).pin_memory()

    def step_e2e():
        q.copy_(qh, non_blocking=True)
        ib.attn_prefill(kv, 0, q, 0, out=out, impl=2)
        oh.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    ms_e2e = timed(step_e2e, steps, 1, world)
    e2e = {"value": round(flops * steps / (ms_e2e * 1e-3) / 1e12, 1), "unit": "TFLOP/s",
           "h2d_bytes_per_step": int(q.numel() * 2), "d2h_bytes_per_step": int(out.numel() * 2),
           "ms_per_step": round(ms_e2e / steps, 4)}
    return {"metric": f"causal GQA prefill attention TFLOP/s ({S} tokens, 24q/8kv heads, d128, bf16 q, f16 K/V)",
            "value": round(value, 1), "unit": "TFLOP/s", "ms_per_step": round(ms / steps, 4), "steps": steps,
            "scaling": "strong", "dtype": "f16 MMA operands (bf16 q converted on load) / f32 accumulate+softmax",
            "roofline": roofline, "e2e": e2e, "gpu_launches": steps, "clocks": clk.summary(),
            "config": dict(prefill_config(S, world), gather=gather_mode, gather_verified=gather_checked)}



# ------------------------------------------------------------------------------------------------
# the other configurations (parity-test shapes; reported for completeness, not headline lines)
# ------------------------------------------------------------------------------------------------

def run_chunked(args, rank, world, n_tok, pos0, label):
    """K1 + K2 of one layer: n_tok new tokens appended at pos0 (configs[0] / configs[2]), one GPU per rank (replicas)."""
    import torch
    import ingot_b200 as ib
    torch.manual_seed(2)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, N_LAYER, HKV, pos0 + n_tok)
    for l in range(N_LAYER):
        kv.layer_view(l, "k").copy_(torch.randn(HKV, pos0 + n_tok, D, device="cuda").half())
        kv.layer_view(l, "v").copy_(torch.randn(HKV, pos0 + n_tok, D, device="cuda").half())
    q = torch.randn(N_LAYER, n_tok, H, D, device="cuda")
    k = torch.randn(N_LAYER, n_tok, HKV, D, device="cuda")
    v = torch.randn(N_LAYER, n_tok, HKV, D, device="cuda")
    out = torch.empty(N_LAYER, n_tok, H, D, device="cuda")
    inv = torch.from_numpy(inv_freq_table()).cuda()
    res = {}
    for impl in (0, 1, 2):
        def launch_layers():
            for l in range(N_LAYER):
                qr = ib.rope_kv_append(kv, l, q[l], k[l], v[l], inv, pos0)
                ib.attn_prefill(kv, l, qr, pos0, out=out[l], impl=impl)
        # One CUDA graph per step (the 28 layers' launches), so that Python launch overhead is not timed.
        launch_layers()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            launch_layers()
        step = launch_layers if args.no_graph else graph.replay
        steps = max(1, min(args.steps, 10))
        ms = timed(step, steps, args.warmup, world)
        res[impl] = ms / steps / N_LAYER
    flops = 4 * H * D * (n_tok * pos0 + n_tok * n_tok // 2)
    best = res[0]
    peaks = measured_peaks()
    tf = flops / (best * 1e-3) / 1e12
    return {"metric": f"causal GQA chunked prefill TFLOP/s ({label})", "value": round(world * tf, 2), "unit": "TFLOP/s",
            "ms_per_step": round(best * N_LAYER, 4), "scaling": "weak", "dtype": "f16 MMA operands / f32 accumulate+softmax",
            "roofline": {"bound": "tensor", "achieved": round(tf, 2), "peak": peaks["tflops_burst"], "unit": "TFLOP/s",
                         "frac": round(tf / peaks["tflops_burst"], 4), "traffic": None,
                         "us_per_layer": {"auto": round(res[0] * 1e3, 2), "warp_mma": round(res[1] * 1e3, 2),
                                          "tcgen05": round(res[2] * 1e3, 2)}},
            "gpu_launches": 2 * N_LAYER * max(1, min(args.steps, 10)),
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
    bt = torch.from_numpy(W.block_tables(lens, perm)).cuda()
    n_layers = 4  # distinct per-layer pools so that a step streams more than L2 holds
    kv = ib.KVCache(ib.KV_PAGED, n_layers, HKV, nb, max_seqs=n_seq)
    torch.manual_seed(3 + rank)
    for l in range(n_layers):
        kv.layer_view(l, "k").copy_(torch.randn(nb, HKV, 16, D, device="cuda").half())
        kv.layer_view(l, "v").copy_(torch.randn(nb, HKV, 16, D, device="cuda").half())
    q = torch.randn(n_layers, n_seq, H, D, device="cuda").bfloat16()
    out = torch.empty(n_layers, n_seq, H, D, device="cuda")
    lens_d = torch.from_numpy(lens).cuda()

    def step():
        ib.attn_decode_layers(kv, 0, q, out, seq_lens=lens_d, max_seq_len=int(lens.max()), block_tables=bt,
                              chunk_keys=args.chunk_keys)

    ms = timed(step, args.steps, args.warmup, world)
    assert kv.status() == 0
    bytes_rank = int(lens.astype(np.int64).sum()) * HKV * D * 2 * 2 * n_layers
    tot = torch.tensor([float(bytes_rank)], device="cuda", dtype=torch.float64)
    mx = tot.clone()
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(tot)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    value = float(tot.item()) * args.steps / (ms * 1e-3) / 1e9
    peaks = measured_peaks()
    per_gpu = bytes_rank * args.steps / (ms * 1e-3) / 1e9
    return {"metric": "batched paged decode attention KV-cache HBM GB/s (64 sequences, lengths 256..8192)", "value": round(value, 1),
            "unit": "GB/s", "ms_per_step": round(ms / args.steps, 5), "scaling": "strong",
            "dtype": "f16 KV / f16 MMA operands (bf16 q converted on load) / f32 accumulate+softmax",
            "roofline": {"bound": "hbm", "achieved": round(per_gpu, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(per_gpu / peaks["hbm_gbs"], 4), "traffic": None},
            "gpu_launches": args.steps * (n_layers + decode_chains(n_layers)),
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
    path = os.path.join(os.environ.get("INGOT_E2E_DIR", "/tmp"), f"ingot_random_l{n_layer}_v{n_vocab}_s0.gguf")
    if not os.path.exists(path):
        make_random_gguf.write(path + ".tmp", n_layer, n_vocab, seed=0)
        os.replace(path + ".tmp", path)
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
            "config": {"workload": f"random-init Llama-3.2-3B-shaped F16 GGUF, {n_layer} layers, vocab {n_vocab}; 128 prompt ids, 32 greedy steps"},
            "cuda_backend": res["cuda"], "cpu_reference_backend": res["cpu"],
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
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ingot", choices=["ingot", "reference"])
    ap.add_argument("--workload", default="decode_c2", choices=["decode_c2", "prefill_c5", "c1_prefill128", "c3_chunked", "c4_batched", "e2e_model"])
    ap.add_argument("--small-model", action="store_true", help="e2e_model: 2 layers and a 32064-token vocabulary")
    ap.add_argument("--chunk-keys", type=int, default=0, help="decode split size (0 = library default)")
    ap.add_argument("--prefill-steps", type=int, default=10, help="cap on timed prefill steps (each is ~10 ms)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="prefill length; anything but 32768 is a profiling case, not the benchmark configuration")
    ap.add_argument("--no-secondary", action="store_true", help="skip the non-headline workload")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-fused-gather", action="store_true",
                    help="prefill at N > 1: kernel + NCCL all-gather instead of the fused peer-store epilogue")
    ap.add_argument("--no-graph", action="store_true", help="decode: launch the 28 layers from Python instead of replaying a CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        line = run_reference(args)
        if line is not None:
            print(json.dumps(line), flush=True)
        return

    if args.workload == "e2e_model":
        print(json.dumps(run_e2e_model(args)), flush=True)
        return

    rank, world, _ = dist_setup(args.gpus)
    if args.workload in ("c1_prefill128", "c3_chunked", "c4_batched"):
        args.no_secondary = args.no_cpu = True
        primary = {"c1_prefill128": lambda a, r, w: run_chunked(a, r, w, 128, 0, "configs[0]: 128-token prefill at position 0"),
                   "c3_chunked": lambda a, r, w: run_chunked(a, r, w, 512, 3584, "configs[2]: 512-token chunk onto 3584 cached positions"),
                   "c4_batched": run_batched_decode}[args.workload]
        secondary = None
    else:
        primary, secondary = (run_decode, run_prefill) if args.workload == "decode_c2" else (run_prefill, run_decode)
    line = primary(args, rank, world)
    other = None if args.no_secondary else secondary(args, rank, world)
    if rank == 0:
        out = {"metric": line.pop("metric"), "value": line.pop("value"), "unit": line.pop("unit"), "n_gpus": world,
               "steps": line.pop("steps", args.steps), "warmup": args.warmup, "ms_per_step": line.pop("ms_per_step"),
               "higher_is_better": True, "scaling": line.pop("scaling"), "vs_baseline": None, "dtype": line.pop("dtype"),
               "data": "synthetic"}
        line.setdefault("clocks", None)
        line.setdefault("e2e", None)
        out.update(line)
        if other is not None:
            out["prefill" if args.workload == "decode_c2" else "decode"] = other
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
    main()
