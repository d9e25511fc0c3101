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

pytestmark = pytest.mark.gpu


def _noalloc_decode(ib, kv, q, n_keys, out_dtype_code, out):
    import torch
    lib = ib.lib()
    rc = lib.ingot_attn_decode_noalloc(lib.ingot_kv_k_dev(kv.handle, 0), lib.ingot_kv_v_dev(kv.handle, 0), kv.capacity,
                                       kv.n_head_kv, C.c_void_p(q.data_ptr()), ib.F32, C.c_void_p(out.data_ptr()),
                                       out_dtype_code, q.shape[1], n_keys, 0,
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


def test_noalloc_decode_rejects_oversize():
    import torch
    import ingot_b200 as ib
    lib = ib.lib()
    buf = torch.zeros(16, device="cuda")
    p = C.c_void_p(buf.data_ptr())
    rc = lib.ingot_attn_decode_noalloc(p, p, 64, 16, p, ib.F32, p, ib.F32, 128, 10, 0, None)  # 128 heads > 64
    assert rc == 1 and b"64 heads" in lib.ingot_last_error()
