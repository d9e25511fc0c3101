"""The single-process multi-GPU handle (ingot_mg_*): a prefill sharded by KV head over several GPUs with the gather
fused into the kernels and in-kernel completion signals. Needs at least two GPUs with peer access; skipped
otherwise (the one-GPU form of the signalling is covered by tests/test_gpu_prefill.py)."""
import ctypes as C

import numpy as np
import pytest

import helpers
from helpers import D, H, HKV
from ingot_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_dev", [2, 4, 8])
def test_head_sharded_prefill_gathers_every_head_on_every_gpu(n_dev):
    import torch
    import ingot_b200 as ib
    if torch.cuda.device_count() < n_dev:
        pytest.skip(f"needs {n_dev} GPUs")
    lib = ib.lib()
    S = 1024
    wl = W.c5_prefill32k(seed=21, n_tok=S)
    rows = np.array([0, 1, 500, S - 1])
    want, _, _ = helpers.oracle_prefill(wl, rows=rows)
    mg = C.c_void_p()
    assert lib.ingot_mg_create(C.byref(mg), n_dev, 1, H, HKV, S, ib.F16) == 0, lib.ingot_last_error()
    try:
        hkv_l, h_l = HKV // n_dev, H // n_dev
        qs = []
        for d in range(n_dev):
            with torch.cuda.device(d):
                kv = lib.ingot_mg_kv(mg, d)
                k = torch.from_numpy(np.ascontiguousarray(wl.k[:, d * hkv_l:(d + 1) * hkv_l])).cuda()
                v = torch.from_numpy(np.ascontiguousarray(wl.v[:, d * hkv_l:(d + 1) * hkv_l])).cuda()
                assert lib.ingot_kv_import_f16(kv, 0, k.data_ptr(), v.data_ptr(), 0, S, None, None) == 0
                qs.append(torch.from_numpy(np.ascontiguousarray(wl.q[:, d * h_l:(d + 1) * h_l])).cuda().bfloat16())
                torch.cuda.synchronize()
        q_ptrs = (C.c_void_p * n_dev)(*[C.c_void_p(q.data_ptr()) for q in qs])
        for _ in range(2):  # twice: the counters must be back at zero after the first round
            assert lib.ingot_mg_prefill(mg, 0, q_ptrs, ib.BF16, 0, S, 2000) == 0, lib.ingot_last_error()
        outs = []
        for d in range(n_dev):
            with torch.cuda.device(d):
                class A:
                    __cuda_array_interface__ = {"shape": (S, H, D), "typestr": "<f2", "data": (lib.ingot_mg_out(mg, d), False), "version": 2}
                outs.append(torch.as_tensor(A(), device=torch.device("cuda", d)).cpu())
        for d in range(n_dev):
            assert torch.equal(outs[d], outs[0])  # every GPU ends up with the same rows
        helpers.assert_parity(outs[0][torch.from_numpy(rows)].float().numpy(), want, f"head-sharded prefill on {n_dev} GPUs")
    finally:
        lib.ingot_mg_destroy(mg)
