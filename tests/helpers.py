"""Shared helpers for the parity tests: tolerances, oracle drivers and CUDA-path drivers."""
import numpy as np

from oracle import loader

# Tolerances of the attention output against the f32 CPU reference.
MAX_ABS_TOL = 2e-3
REL_L2_TOL = 1e-3

H, HKV, D = 24, 8, 128

_oracle = None


def oracle():
    global _oracle
    if _oracle is None:
        _oracle = loader.load_oracle()
    return _oracle


def inv_freq(head_dim=D, theta=500000.0):
    return loader.inv_freq(oracle(), "oracle_", head_dim, theta)


def errors(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    diff = got - want
    return float(np.abs(diff).max()), float(np.linalg.norm(diff) / max(np.linalg.norm(want), 1e-30))


def assert_parity(got, want, what=""):
    assert np.isfinite(np.asarray(got, dtype=np.float64)).all(), f"{what}: non-finite output"
    max_abs, rel_l2 = errors(got, want)
    assert max_abs <= MAX_ABS_TOL and rel_l2 <= REL_L2_TOL, f"{what}: max_abs={max_abs:.3e} rel_l2={rel_l2:.3e}"
    return max_abs, rel_l2


def f32_cache(rows_f16, n_ctx=None):
    """[n, Hkv, d] f16 rows -> the reference's f32 cache [n_ctx, Hkv*d] (values widened exactly)."""
    n = rows_f16.shape[0]
    n_ctx = n_ctx or n
    c = np.zeros((n_ctx, rows_f16.shape[1] * rows_f16.shape[2]), dtype=np.float32)
    c[:n] = rows_f16.astype(np.float32).reshape(n, -1)
    return c


def oracle_prefill(wl, rows=None):
    """Reference output for a workloads.Prefill. rows: optional token indices to evaluate (rope=False only)."""
    lib = oracle()
    n, Hq, d = wl.q.shape
    hkv = wl.k.shape[1]
    if wl.rope:
        n_ctx = wl.pos0 + n
        kc = vc = None
        if wl.pos0:
            kc = f32_cache(wl.cache_k, n_ctx)
            vc = f32_cache(wl.cache_v, n_ctx)
        out, q_rot, k_rot, kc, vc = loader.attn_forward(lib, "oracle_", wl.q, wl.k, wl.v, wl.pos0, n_ctx,
                                                        inv_freq(d), kc, vc)
        return out, q_rot, k_rot
    kc = f32_cache(wl.k)
    vc = f32_cache(wl.v)
    rows = np.arange(n) if rows is None else np.asarray(rows)
    out = loader.attend_rows(lib, wl.q[rows], kc, vc, (wl.pos0 + rows).astype(np.int32), Hq, hkv, d)
    return out, None, None


def oracle_decode(wl):
    lib = oracle()
    n_seq, Hq, d = wl.q.shape
    outs = []
    for s in range(n_seq):
        kc = f32_cache(wl.k[s])
        vc = f32_cache(wl.v[s])
        pos = np.array([int(wl.lens[s]) - 1], dtype=np.int32)
        outs.append(loader.attend_rows(lib, wl.q[s:s + 1], kc, vc, pos, Hq, wl.k[s].shape[1], d, 1)[0])
    return np.stack(outs)


# ---- CUDA-path drivers (need a GPU) ----

def to_dev(x, dtype=None):
    """Uploads a numpy array (optionally converted to `dtype`) into a canary-guarded device tensor."""
    import torch
    import ingot_b200 as ib
    src = torch.from_numpy(np.ascontiguousarray(x))
    t = ib.guarded_empty(src.shape, dtype or src.dtype)
    t.copy_(src)
    return t


def gpu_prefill(wl, impl=0, paged=False, out_f16=False, seed=0, extra_ctx=0):
    """Runs a workloads.Prefill through K1 (if rope) / import and K2. Returns (out, q_rot_f16, kv)."""
    import torch
    import ingot_b200 as ib
    n, Hq, d = wl.q.shape
    hkv = wl.k.shape[1]
    n_ctx = wl.pos0 + n + extra_ctx
    bt = None
    if paged:
        nb = (n_ctx + 15) // 16
        perm = np.random.default_rng(seed + 1000).permutation(nb + 3).astype(np.int32)[:nb]
        kv = ib.KVCache(ib.KV_PAGED, 1, hkv, nb + 3)
        bt = to_dev(perm)
    else:
        kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, hkv, n_ctx)
    if wl.pos0:
        kv.import_f16(0, to_dev(wl.cache_k), to_dev(wl.cache_v), 0, bt)
    q_rot = None
    if wl.rope:
        q_rot = ib.rope_kv_append(kv, 0, to_dev(wl.q), to_dev(wl.k), to_dev(wl.v), to_dev(inv_freq(d)), wl.pos0,
                                  block_tables=None if bt is None else bt.view(1, -1))
        q_in = q_rot
    else:
        kv.import_f16(0, to_dev(wl.k), to_dev(wl.v), wl.pos0, bt)
        q_in = to_dev(wl.q, torch.bfloat16 if wl.q_is_bf16 else None)
    out = ib.attn_prefill(kv, 0, q_in, wl.pos0, out_dtype=torch.float16 if out_f16 else torch.float32,
                          block_table=bt, impl=impl)
    torch.cuda.synchronize()
    assert kv.status() == 0
    return out, q_rot, kv


def gpu_decode(wl, paged=False, chunk_keys=0, out_f16=False):
    import torch
    import ingot_b200 as ib
    from ingot_b200 import workloads as W
    n_seq, Hq, d = wl.q.shape
    hkv = wl.k[0].shape[1]
    lens = wl.lens
    q = to_dev(wl.q, torch.bfloat16 if wl.q_is_bf16 else None)
    if paged:
        nb = int(((lens + 15) // 16).sum())
        perm = wl.block_perm if wl.block_perm is not None else np.random.default_rng(7).permutation(nb).astype(np.int32)
        bt_np = W.block_tables(lens, perm)
        kv = ib.KVCache(ib.KV_PAGED, 1, hkv, nb, max_seqs=n_seq)
        bt = to_dev(bt_np)
        for s in range(n_seq):
            kv.import_f16(0, to_dev(wl.k[s]), to_dev(wl.v[s]), 0, bt[s])
        out = ib.attn_decode(kv, 0, q, out_dtype=torch.float16 if out_f16 else torch.float32, seq_lens=to_dev(lens),
                             max_seq_len=int(lens.max()), block_tables=bt, chunk_keys=chunk_keys)
    else:
        assert n_seq == 1
        kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, hkv, int(lens[0]))
        kv.import_f16(0, to_dev(wl.k[0]), to_dev(wl.v[0]), 0)
        out = ib.attn_decode(kv, 0, q, out_dtype=torch.float16 if out_f16 else torch.float32,
                             max_seq_len=int(lens[0]), chunk_keys=chunk_keys)
    torch.cuda.synchronize()
    assert kv.status() == 0
    return out, kv
