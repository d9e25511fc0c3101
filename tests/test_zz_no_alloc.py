"""The allocation-free decode entry point against the regular one.

ingot_attn_decode_noalloc exists for callers that may not allocate device memory (plugins handed
pre-allocated buffers, serving loops where cudaMalloc is banned): it keeps its split scratch in a
fixed array inside the library. It must give the same answer as ingot_attn_decode on the same inputs,
also when called twice in a row (the array keeps the previous call's contents). Collected last on
purpose, so a failure here cannot hide the result of any other test.
"""
import ctypes as C

import numpy as np
import pytest

import helpers
from helpers import D, H, HKV
from ingot_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _noalloc_decode(ib, kv, q, n_keys, out_dtype_code, out, chunk_keys=0):
    import torch
    lib = ib.lib()
    q_code = {torch.float32: ib.F32, torch.float16: ib.F16, torch.bfloat16: ib.BF16}[q.dtype]
    rc = lib.ingot_attn_decode_noalloc(lib.ingot_kv_k_dev(kv.handle, 0), lib.ingot_kv_v_dev(kv.handle, 0), kv.capacity,
                                       kv.n_head_kv, C.c_void_p(q.data_ptr()), q_code, C.c_void_p(out.data_ptr()),
                                       out_dtype_code, q.shape[1], n_keys, chunk_keys,
                                       C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.ingot_last_error()
    return out


def test_noalloc_decode_matches_regular_decode_twice():
    import torch
    import ingot_b200 as ib
    rng = np.random.default_rng(77)
    n_ctx = 4096
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, HKV, n_ctx)
    k = rng.standard_normal((n_ctx, HKV, D), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((n_ctx, HKV, D), dtype=np.float32).astype(np.float16)
    kv.import_f16(0, helpers.to_dev(k), helpers.to_dev(v), 0)
    # two different calls in a row: the second one meets the first one's leftovers in the shared array
    for n_keys, seed in ((4096, 1), (1000, 2)):
        q = helpers.to_dev(np.random.default_rng(seed).standard_normal((1, H, D), dtype=np.float32))
        want = ib.attn_decode(kv, 0, q, max_seq_len=n_keys)
        got = _noalloc_decode(ib, kv, q, n_keys, ib.F32, torch.empty_like(want))
        torch.cuda.synchronize()
        helpers.assert_parity(got.cpu().numpy(), want.cpu().numpy(), f"no-alloc decode n_keys={n_keys}")
        # and against the CPU reference itself, not only against the sibling entry point
        wl = W.Decode(q.cpu().numpy(), [k[:n_keys]], [v[:n_keys]], np.array([n_keys], dtype=np.int32))
        helpers.assert_parity(got.cpu().numpy(), helpers.oracle_decode(wl), f"no-alloc decode vs reference, n_keys={n_keys}")


def test_noalloc_decode_at_its_limits():
    """The largest call the built-in array is sized for: 64 query heads in groups of 8 and 64 split partials
    (1024 keys in splits of 16), once with f32 and once with f16 output, each against the CPU reference; then
    a small call, which must not be disturbed by what the big one left in the array."""
    import torch
    import ingot_b200 as ib
    rng = np.random.default_rng(78)
    n_head, n_keys = 64, 1024
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, HKV, n_keys)
    k = rng.standard_normal((n_keys, HKV, D), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((n_keys, HKV, D), dtype=np.float32).astype(np.float16)
    kv.import_f16(0, helpers.to_dev(k), helpers.to_dev(v), 0)
    q = rng.standard_normal((1, n_head, D), dtype=np.float32)
    want = helpers.oracle_decode(W.Decode(q, [k], [v], np.array([n_keys], dtype=np.int32)))
    qd = helpers.to_dev(q)
    got32 = _noalloc_decode(ib, kv, qd, n_keys, ib.F32, torch.empty(1, n_head, D, device="cuda"), chunk_keys=16)
    got16 = _noalloc_decode(ib, kv, qd, n_keys, ib.F16, torch.empty(1, n_head, D, device="cuda", dtype=torch.float16),
                            chunk_keys=16)
    torch.cuda.synchronize()
    helpers.assert_parity(got32.cpu().numpy(), want, "no-alloc decode, 64 heads x 64 partials, f32 out")
    # f16 output adds half an f16 ulp of |out| < 1 (4.9e-4) to the error budget
    assert np.abs(got16.float().cpu().numpy() - want).max() <= helpers.MAX_ABS_TOL + 4.9e-4
    assert torch.equal(got16, got32.half())
    q2 = rng.standard_normal((1, H, D), dtype=np.float32)
    got2 = _noalloc_decode(ib, kv, helpers.to_dev(q2), 100, ib.F32, torch.empty(1, H, D, device="cuda"))
    torch.cuda.synchronize()
    want2 = helpers.oracle_decode(W.Decode(q2, [k[:100]], [v[:100]], np.array([100], dtype=np.int32)))
    helpers.assert_parity(got2.cpu().numpy(), want2, "no-alloc decode after the large call")


def test_noalloc_decode_rejects_oversize():
    import torch
    import ingot_b200 as ib
    lib = ib.lib()
    buf = torch.zeros(16, device="cuda")
    p = C.c_void_p(buf.data_ptr())
    rc = lib.ingot_attn_decode_noalloc(p, p, 64, 16, p, ib.F32, p, ib.F32, 128, 10, 0, None)  # 128 heads > 64
    assert rc == 1 and b"64 heads" in lib.ingot_last_error()
