"""GGUF block-quantised weights on the GPU (backend/quant_kernels.cu) against the reference's decoding.

Block decoding is byte/integer work plus one or two f32 multiplies, so it has to be BIT-EXACT against
ops::dequant_row (src/ops.cpp:33-91, 198-200; restated in oracle/quant_oracle.c and pinned to the compiled
reference by tests/test_oracle_quant.py) - for weight-like scales and for arbitrary finite f16 scale bit patterns.
The products built on it (dequantise-in-GEMV for one token, f16 hi/lo planes for the tensor-core GEMM) are held to
an f32 tolerance against a float64 product of the decoded values.
"""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import loader

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENGINE = os.path.join(ROOT, "inference-agent_b200", "backend", "_build", "libingot_engine_cuda.so")
QTYPES = ["Q8_0", "Q4_0", "Q4_1", "Q6_K"]


def _lib():
    if not os.path.exists(ENGINE):
        pytest.skip("libingot_engine_cuda.so not built (needs a reference checkout at build time)")
    lib = C.CDLL(ENGINE)
    P, I, SZ = C.c_void_p, C.c_int, C.c_size_t
    lib.ingot_quant_supported.argtypes = [I, I]
    lib.ingot_quant_planar_bytes.argtypes = [I, I, I]
    lib.ingot_quant_planar_bytes.restype = SZ
    lib.ingot_quant_repack.argtypes = [P, P, I, I, I, P]
    lib.ingot_quant_dequant_rows.argtypes = [P, P, I, I, I, P, I, P, P]
    lib.ingot_quant_dequant_hilo.argtypes = [P, P, P, I, I, I, P]
    lib.ingot_quant_gemv.argtypes = [P, P, I, P, I, I, I, P]
    return lib


def _upload(lib, type_name, raw, n_in, n_out):
    """Raw GGUF rows (uint8 [n_out, row_bytes]) -> repacked device planes."""
    import torch
    t = loader.GGML_TYPES[type_name]
    raw_d = torch.from_numpy(np.ascontiguousarray(raw)).cuda()
    planar = torch.empty(lib.ingot_quant_planar_bytes(t, n_in, n_out), dtype=torch.uint8, device="cuda")
    assert lib.ingot_quant_repack(planar.data_ptr(), raw_d.data_ptr(), t, n_in, n_out, None) == 0
    torch.cuda.synchronize()
    return planar


def _oracle_rows(type_name, raw, n_in):
    orc = loader.load_oracle()
    return np.stack([loader.dequant(orc, "oracle_", type_name, raw[r], n_in) for r in range(raw.shape[0])])


@pytest.mark.parametrize("extreme", [False, True])
@pytest.mark.parametrize("type_name", QTYPES)
def test_block_decode_is_bit_exact(type_name, extreme):
    import torch
    lib = _lib()
    n_in, n_out = 1024, 37
    rng = np.random.default_rng([11, QTYPES.index(type_name), int(extreme)])
    raw = loader.random_blocks(type_name, n_out, n_in, rng, extreme=extreme)
    want = _oracle_rows(type_name, raw, n_in)
    planar = _upload(lib, type_name, raw, n_in, n_out)
    t = loader.GGML_TYPES[type_name]
    out = torch.empty(n_out, n_in, device="cuda")
    assert lib.ingot_quant_dequant_rows(out.data_ptr(), planar.data_ptr(), t, n_in, n_out, None, n_out, None, None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    # gather form (embedding rows): arbitrary row order, repeats, and one index outside the table
    rows = np.array([5, 0, 36, 5, 99, 17], dtype=np.int32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = torch.full((len(rows), n_in), 7.0, device="cuda")
    assert lib.ingot_quant_dequant_rows(got.data_ptr(), planar.data_ptr(), t, n_in, n_out, torch.from_numpy(rows).cuda().data_ptr(),
                                        len(rows), status.data_ptr(), None) == 0
    torch.cuda.synchronize()
    g = got.cpu().numpy()
    for i, r in enumerate(rows):
        if r < n_out:
            assert np.array_equal(g[i].view(np.uint32), want[r].view(np.uint32))
        else:
            assert not g[i].any()
    assert int(status.item()) == 1


@pytest.mark.parametrize("type_name", QTYPES)
def test_hi_lo_planes_add_up_exactly(type_name):
    """hi = f16(w), lo = f16(w - hi): for weight-like magnitudes the two f16 planes reproduce the f32 value exactly."""
    import torch
    lib = _lib()
    n_in, n_out = 512, 64
    rng = np.random.default_rng([12, QTYPES.index(type_name)])
    raw = loader.random_blocks(type_name, n_out, n_in, rng)
    want = _oracle_rows(type_name, raw, n_in)
    planar = _upload(lib, type_name, raw, n_in, n_out)
    hi = torch.empty(n_out, n_in, dtype=torch.float16, device="cuda")
    lo = torch.empty_like(hi)
    assert lib.ingot_quant_dequant_hilo(hi.data_ptr(), lo.data_ptr(), planar.data_ptr(), loader.GGML_TYPES[type_name], n_in, n_out, None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(hi.cpu().numpy(), want.astype(np.float16))
    total = hi.float().cpu().numpy().astype(np.float64) + lo.float().cpu().numpy().astype(np.float64)
    assert np.abs(total - want.astype(np.float64)).max() <= 2.0 ** -25  # f16 subnormal spacing bounds the residual's error
    assert (total == want.astype(np.float64)).mean() > 0.99


@pytest.mark.parametrize("accumulate", [0, 1])
@pytest.mark.parametrize("n_in,n_out", [(3072, 3072), (8192, 3072), (3072, 1024), (256, 9)])
@pytest.mark.parametrize("type_name", QTYPES)
def test_gemv_matches_float64(type_name, n_in, n_out, accumulate):
    import torch
    lib = _lib()
    rng = np.random.default_rng([13, QTYPES.index(type_name), n_in, n_out])
    raw = loader.random_blocks(type_name, n_out, n_in, rng)
    x = rng.standard_normal(n_in, dtype=np.float32)
    want = loader.oracle_matvec(loader.load_oracle(), type_name, raw, x, n_in, n_out)
    planar = _upload(lib, type_name, raw, n_in, n_out)
    out0 = rng.standard_normal(n_out, dtype=np.float32)
    out = torch.from_numpy(out0.copy()).cuda()
    xd = torch.from_numpy(x).cuda()
    assert lib.ingot_quant_gemv(out.data_ptr(), planar.data_ptr(), loader.GGML_TYPES[type_name], xd.data_ptr(), n_in, n_out, accumulate, None) == 0
    torch.cuda.synchronize()
    if accumulate:
        want = want + out0.astype(np.float64)
    err = np.abs(out.cpu().numpy().astype(np.float64) - want).max()
    scale = np.abs(want).max()
    assert err <= 2e-6 * scale * max(1.0, (n_in / 1024) ** 0.5), (err, scale)  # f32 accumulation over n_in terms


def test_unsupported_types_and_shapes_are_rejected():
    lib = _lib()
    assert lib.ingot_quant_supported(loader.GGML_TYPES["Q8_0"], 3072) == 1
    assert lib.ingot_quant_supported(loader.GGML_TYPES["Q6_K"], 3072) == 1
    assert lib.ingot_quant_supported(loader.GGML_TYPES["Q6_K"], 96) == 0     # not a multiple of 256
    assert lib.ingot_quant_supported(loader.GGML_TYPES["F16"], 3072) == 0    # not a block format
    assert lib.ingot_quant_supported(6, 3072) == 0                           # Q5_0: the reference rejects it too
    assert lib.ingot_quant_gemv(None, None, loader.GGML_TYPES["Q8_0"], None, 16384, 8, 0, None) != 0  # row too long
