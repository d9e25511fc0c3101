"""The tensor-core form of CudaBackend's batched projections (backend/linear_sm100.cu) against float64 matmul.

out[t][r] (+)= sum_i W[r][i] x[t][i] with f16 weights and f32 activations split into f16 hi + lo parts: the
result has to be an f32-accurate product (the reference multiplies f32 activations with widened f16 weights,
src/ops.cpp:127-141), not an f16-activation one.
"""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENGINE = os.path.join(ROOT, "inference-agent_b200", "backend", "_build", "libingot_engine_cuda.so")


def _lib():
    if not os.path.exists(ENGINE):
        pytest.skip("libingot_engine_cuda.so not built (needs a reference checkout at build time)")
    lib = C.CDLL(ENGINE)
    lib.ingot_linear_ws_create.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int]
    lib.ingot_linear_ws_destroy.argtypes = [C.c_void_p]
    lib.ingot_linear_tc_supported.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]
    lib.ingot_linear_tc_prepare.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    lib.ingot_linear_tc_run.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.ingot_linear_ws_status.argtypes = [C.c_void_p]
    return lib


@pytest.mark.parametrize("x_scale", [1.0, 3e-4])
@pytest.mark.parametrize("n_tok,n_in,n_out,accumulate", [
    (128, 3072, 3072, 1),    # wo at the Llama-3.2-3B shape, one token tile, split-k
    (128, 3072, 1024, 0),    # wk / wv: few output tiles, deep split-k
    (130, 3072, 8192, 0),    # gate / up, a second, nearly empty token tile
    (512, 8192, 3072, 1),    # down projection of a full 512-token chunk
    (16, 64, 4, 0),          # smallest supported shape: one k-step, four outputs
    (77, 256, 132, 1),       # output count that is not a multiple of the tile
])
def test_linear_tc_matches_float64(n_tok, n_in, n_out, accumulate, x_scale):
    import torch
    lib = _lib()
    ws = C.c_void_p()
    assert lib.ingot_linear_ws_create(C.byref(ws), 512, 8192) == 0
    try:
        g = torch.Generator(device="cuda").manual_seed(n_tok * 31 + n_out)
        # x_scale 3e-4: activations of magnitude 1e-4..1e-3 (a SwiGLU product on random-init weights), where the lo
        # half of the split is an f16 subnormal and the split only bounds the ABSOLUTE error (2^-25 per element)
        x = torch.randn(n_tok, n_in, device="cuda", generator=g) * x_scale
        w = (torch.randn(n_out, n_in, device="cuda", generator=g) * 0.02).half()
        out0 = torch.randn(n_tok, n_out, device="cuda", generator=g) * x_scale
        out = out0.clone()
        assert lib.ingot_linear_tc_supported(ws, 1, n_in, n_out, n_tok) == 1
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert lib.ingot_linear_tc_prepare(ws, x.data_ptr(), n_in, n_tok, stream) == 0
        assert lib.ingot_linear_tc_run(ws, out.data_ptr(), w.data_ptr(), n_in, n_out, accumulate, stream) == 0
        torch.cuda.synchronize()
        want = x.double() @ w.double().t()
        if accumulate:
            want += out0.double()
        err = (out.double() - want).abs().max().item()
        scale = want.abs().max().item()
        # f32 accumulation over n_in terms plus the 2^-22 truncation of x; an f16-activation product would be ~1e-3
        tol = (1e-5 if x_scale == 1.0 else 2e-4) * scale * max(1.0, (n_in / 1024) ** 0.5)
        assert err <= tol, (err, scale)
        # a second run on the same workspace gives the same bits (fixed summation order over the k slices)
        out2 = out0.clone()
        assert lib.ingot_linear_tc_run(ws, out2.data_ptr(), w.data_ptr(), n_in, n_out, accumulate, stream) == 0
        torch.cuda.synchronize()
        assert torch.equal(out, out2)
        assert lib.ingot_linear_ws_status(ws) == 0
    finally:
        lib.ingot_linear_ws_destroy(ws)


def _quant_planes(lib, type_name, raw, n_in, n_out):
    """Raw GGUF rows -> repacked device planes and the address of their scale plane."""
    import torch
    from oracle import loader
    P, I = C.c_void_p, C.c_int
    lib.ingot_quant_planar_bytes.argtypes = [I, I, I]
    lib.ingot_quant_planar_bytes.restype = C.c_size_t
    lib.ingot_quant_scale_offset.argtypes = [I, I, I]
    lib.ingot_quant_scale_offset.restype = C.c_size_t
    lib.ingot_quant_repack.argtypes = [P, P, I, I, I, P]
    t = loader.GGML_TYPES[type_name]
    raw_d = torch.from_numpy(np.ascontiguousarray(raw)).cuda()
    planar = torch.empty(lib.ingot_quant_planar_bytes(t, n_in, n_out), dtype=torch.uint8, device="cuda")
    assert lib.ingot_quant_repack(planar.data_ptr(), raw_d.data_ptr(), t, n_in, n_out, None) == 0
    torch.cuda.synchronize()
    return planar, planar.data_ptr() + lib.ingot_quant_scale_offset(t, n_in, n_out)


@pytest.mark.parametrize("wtype", ["F16", "Q8_0", "Q4_0"])
@pytest.mark.parametrize("mode", ["qkv_norm", "swiglu", "plain_accumulate", "many_rows"])
def test_gemv_group_matches_float64(mode, wtype):
    """The single-token weight-streaming launch: RMS norm folded into up to three matrix-vector products,
    SwiGLU as the epilogue of gate/up, plain accumulate (wo / down), and a row count far above one wave (logits):
    against rmsnorm (src/ops.cpp:227-232) and float64 products - for f16 rows and for Q8_0 / Q4_0 rows read from
    their repacked planes (values decoded by the CPU checker)."""
    import torch
    from oracle import loader
    lib = _lib()
    lib.ingot_support_gemv_group.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int,
                                             C.POINTER(C.c_int), C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_float, C.c_int,
                                             C.c_int, C.c_void_p]
    swiglu = int(mode == "swiglu")
    norm = mode != "plain_accumulate"
    accumulate = int(mode == "plain_accumulate")
    n_in = 8192 if mode == "plain_accumulate" else 3072
    rows = {"qkv_norm": [3072, 1024, 1016], "swiglu": [8192, 8192], "plain_accumulate": [3072], "many_rows": [50001]}[mode]
    g = torch.Generator(device="cuda").manual_seed(len(mode))
    x = torch.randn(n_in, device="cuda", generator=g) * 3
    nw = 1 + 0.1 * torch.randn(n_in, device="cuda", generator=g)
    keep = []
    if wtype == "F16":
        ws = [(torch.randn(r, n_in, device="cuda", generator=g) * 0.02).half() for r in rows]
        w_ptrs, s_ptrs, fmt = [w.data_ptr() for w in ws], [None] * len(rows), 0
        w64 = [w.double() for w in ws]
    else:
        rng = np.random.default_rng([len(mode), len(wtype)])
        orc = loader.load_oracle()
        w_ptrs, s_ptrs, w64, fmt = [], [], [], {"Q8_0": 1, "Q4_0": 2}[wtype]
        for r in rows:
            raw = loader.random_blocks(wtype, r, n_in, rng)
            planar, scale_ptr = _quant_planes(lib, wtype, raw, n_in, r)
            keep.append(planar)
            w_ptrs.append(planar.data_ptr())
            s_ptrs.append(scale_ptr)
            vals = np.stack([loader.dequant(orc, "oracle_", wtype, raw[i], n_in) for i in range(r)])
            w64.append(torch.from_numpy(vals).cuda().double())
    outs0 = [torch.randn(r, device="cuda", generator=g) for r in rows]
    outs = [o.clone() for o in outs0]
    eps = 1e-5
    outs_p = (C.c_void_p * len(rows))(*[o.data_ptr() for o in outs])
    ws_p = (C.c_void_p * len(rows))(*w_ptrs)
    sc_p = (C.c_void_p * len(rows))(*s_ptrs)
    rows_p = (C.c_int * len(rows))(*rows)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for _ in range(2 if not accumulate else 1):  # a second launch right behind the first (dependent launch) gives the same result
        assert lib.ingot_support_gemv_group(outs_p, ws_p, sc_p, fmt, rows_p, len(rows), swiglu, x.data_ptr(),
                                            nw.data_ptr() if norm else None, eps, n_in, accumulate, stream) == 0
    torch.cuda.synchronize()
    xd = x.double()
    h = xd * torch.rsqrt((xd * xd).mean() + eps) * nw.double() if norm else xd
    want = [w @ h for w in w64]
    if swiglu:
        gate, up = want
        ref = gate / (1 + torch.exp(-gate)) * up
        err = (outs[0].double() - ref).abs().max().item()
        assert err <= 1e-5 * max(1.0, ref.abs().max().item()), err
        assert torch.equal(outs[1], outs0[1])  # the second output buffer is not touched
    else:
        for o, o0, r in zip(outs, outs0, want):
            ref = r + o0.double() if accumulate else r
            err = (o.double() - ref).abs().max().item()
            assert err <= 1e-5 * max(1.0, ref.abs().max().item()), err


def test_slice_consumers_match_float64():
    """Split-k products left as k slices and summed by their consumers: the grouped q/k/v sum, the residual add
    with the next RMS norm folded in, and the SwiGLU product, each checked through the projection that follows."""
    import torch
    lib = _lib()
    vp, ci, cf = C.c_void_p, C.c_int, C.c_float
    lib.ingot_linear_tc_run_partial.argtypes = [vp, vp, ci, ci, ci, vp]
    lib.ingot_linear_tc_finish_group.argtypes = [vp, C.POINTER(vp), ci, vp]
    lib.ingot_linear_tc_finish_residual_norm.argtypes = [vp, vp, vp, cf, ci, vp]
    lib.ingot_linear_tc_finish_swiglu.argtypes = [vp, ci, ci, vp]
    lib.ingot_linear_tc_prepare_norm.argtypes = [vp, vp, vp, cf, ci, ci, vp]
    ws = vp()
    assert lib.ingot_linear_ws_create(C.byref(ws), 256, 2048) == 0
    try:
        n_tok, d, ff, eps = 130, 512, 2048, 1e-5
        g = torch.Generator(device="cuda").manual_seed(11)
        rnd = lambda *shape: torch.randn(*shape, device="cuda", generator=g)
        x = rnd(n_tok, d)
        nw1, nw2 = 1 + 0.1 * rnd(d), 1 + 0.1 * rnd(d)
        wq, wk, wv = [(rnd(r, d) * 0.05).half() for r in (512, 128, 256)]
        wo = (rnd(d, 512) * 0.05).half()
        wg, wu = [(rnd(ff, d) * 0.05).half() for _ in range(2)]
        wd = (rnd(d, ff) * 0.05).half()
        st = vp(torch.cuda.current_stream().cuda_stream)
        rms = lambda t, w: t * torch.rsqrt((t * t).mean(dim=1, keepdim=True) + eps) * w.double()
        close = lambda got, want: (got.double() - want).abs().max().item() <= 2e-5 * max(1.0, want.abs().max().item())

        # norm -> q/k/v as slices -> one summing launch
        assert lib.ingot_linear_tc_prepare_norm(ws, x.data_ptr(), nw1.data_ptr(), eps, d, n_tok, st) == 0
        for slot, w in enumerate((wq, wk, wv)):
            assert lib.ingot_linear_tc_run_partial(ws, w.data_ptr(), d, w.shape[0], slot, st) == 0
        outs = [torch.zeros(n_tok, w.shape[0], device="cuda") for w in (wq, wk, wv)]
        assert lib.ingot_linear_tc_finish_group(ws, (vp * 3)(*[o.data_ptr() for o in outs]), 3, st) == 0
        torch.cuda.synchronize()
        h = rms(x.double(), nw1)
        for o, w in zip(outs, (wq, wk, wv)):
            assert close(o, h @ w.double().t())

        # wo product added to the residual, next norm folded in, checked through gate/up + SwiGLU + down
        a = rnd(n_tok, 512)
        lib.ingot_linear_tc_prepare.argtypes = [vp, vp, ci, ci, vp]
        assert lib.ingot_linear_tc_prepare(ws, a.data_ptr(), 512, n_tok, st) == 0
        assert lib.ingot_linear_tc_run_partial(ws, wo.data_ptr(), 512, d, 0, st) == 0
        xr = x.clone()
        assert lib.ingot_linear_tc_finish_residual_norm(ws, xr.data_ptr(), nw2.data_ptr(), eps, 0, st) == 0
        assert lib.ingot_linear_tc_run_partial(ws, wg.data_ptr(), d, ff, 0, st) == 0
        assert lib.ingot_linear_tc_run_partial(ws, wu.data_ptr(), d, ff, 1, st) == 0
        assert lib.ingot_linear_tc_finish_swiglu(ws, 0, 1, st) == 0
        assert lib.ingot_linear_tc_run_partial(ws, wd.data_ptr(), ff, d, 0, st) == 0
        xr2 = xr.clone()
        torch.cuda.synchronize()
        want_x = x.double() + a.double() @ wo.double().t()
        assert close(xr, want_x)
        assert lib.ingot_linear_tc_finish_residual_norm(ws, xr2.data_ptr(), None, eps, 0, st) == 0
        torch.cuda.synchronize()
        h2 = rms(want_x, nw2)
        gate, up = h2 @ wg.double().t(), h2 @ wu.double().t()
        want_x2 = want_x + (gate / (1 + torch.exp(-gate)) * up) @ wd.double().t()
        assert close(xr2, want_x2)
        assert lib.ingot_linear_ws_status(ws) == 0
    finally:
        lib.ingot_linear_ws_destroy(ws)


def test_grouped_projection_launch_matches_float64():
    """q/k/v (and gate/up) as ONE tensor-core launch over the output tiles of all matrices, k slices left in scratch
    slots 0..2 and summed by the consumer kernel: against float64, with widths that are not multiples of the tile."""
    import torch
    lib = _lib()
    vp, ci, cf = C.c_void_p, C.c_int, C.c_float
    lib.ingot_linear_tc_run_partial_group.argtypes = [vp, C.POINTER(vp), ci, C.POINTER(ci), ci, ci, ci, vp]
    lib.ingot_linear_tc_finish_group.argtypes = [vp, C.POINTER(vp), ci, vp]
    lib.ingot_linear_tc_prepare_norm.argtypes = [vp, vp, vp, cf, ci, ci, vp]
    ws = vp()
    assert lib.ingot_linear_ws_create(C.byref(ws), 256, 2048) == 0
    try:
        n_tok, d, eps = 130, 1024, 1e-5
        g = torch.Generator(device="cuda").manual_seed(21)
        rnd = lambda *shape: torch.randn(*shape, device="cuda", generator=g)
        x, nw = rnd(n_tok, d), 1 + 0.1 * rnd(d)
        mats = [(rnd(r, d) * 0.05).half() for r in (640, 132, 256)]
        st = vp(torch.cuda.current_stream().cuda_stream)
        assert lib.ingot_linear_tc_prepare_norm(ws, x.data_ptr(), nw.data_ptr(), eps, d, n_tok, st) == 0
        for count in (3, 2, 1):
            wp = (vp * count)(*[m.data_ptr() for m in mats[:count]])
            rows = (ci * count)(*[m.shape[0] for m in mats[:count]])
            assert lib.ingot_linear_tc_run_partial_group(ws, wp, d, rows, count, 0, 0, st) == 0
            if count == 2:  # a second product appended to the same slots: W + 0.5 W, as hi and lo planes of a quantised matrix would be
                halves = [(m * 0.5).contiguous() for m in mats[:count]]
                hp = (vp * count)(*[m.data_ptr() for m in halves])
                assert lib.ingot_linear_tc_run_partial_group(ws, hp, d, rows, count, 0, 1, st) == 0
            outs = [torch.zeros(n_tok, m.shape[0], device="cuda") for m in mats[:count]]
            assert lib.ingot_linear_tc_finish_group(ws, (vp * count)(*[o.data_ptr() for o in outs]), count, st) == 0
            torch.cuda.synchronize()
            xd = x.double()
            h = xd * torch.rsqrt((xd * xd).mean(dim=1, keepdim=True) + eps) * nw.double()
            for o, m in zip(outs, mats):
                want = h @ m.double().t() * (1.5 if count == 2 else 1.0)
                assert (o.double() - want).abs().max().item() <= 2e-5 * max(1.0, want.abs().max().item())
        assert lib.ingot_linear_ws_status(ws) == 0
    finally:
        lib.ingot_linear_ws_destroy(ws)
