"""K2 (causal GQA flash-attention prefill / chunked prefill) against the CPU reference."""
import numpy as np
import pytest

import helpers
from helpers import D, H, HKV
from ingot_b200 import workloads as W

pytestmark = pytest.mark.gpu

IMPLS = [1, 2]  # 1 = warp-MMA kernel, 2 = tcgen05/TMEM/TMA kernel


@pytest.mark.parametrize("impl", IMPLS)
def test_c1_prefill_128(impl):
    wl = W.c1_prefill128()
    want, q_rot, _ = helpers.oracle_prefill(wl)
    out, _, _ = helpers.gpu_prefill(wl, impl=impl)
    helpers.assert_parity(out.cpu().numpy(), want, f"C1 prefill 128 impl={impl}")


@pytest.mark.parametrize("impl", IMPLS)
def test_c3_chunked_prefill(impl):
    wl = W.c3_chunked()
    want, _, _ = helpers.oracle_prefill(wl)
    out, _, _ = helpers.gpu_prefill(wl, impl=impl)
    helpers.assert_parity(out.cpu().numpy(), want, f"C3 chunked prefill impl={impl}")


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("n_tok,pos0", [(1, 0), (2, 0), (7, 0), (43, 0), (85, 0), (86, 0), (100, 3), (129, 0), (300, 77), (64, 1000),
                                        (600, 0), (16, 5000), (200, 2000)])  # the last three split the keys over CTAs
def test_prefill_ragged_shapes(impl, n_tok, pos0):
    rng = np.random.default_rng(n_tok * 31 + pos0)
    q = rng.standard_normal((n_tok, H, D), dtype=np.float32)
    k = rng.standard_normal((n_tok, HKV, D), dtype=np.float32)
    v = rng.standard_normal((n_tok, HKV, D), dtype=np.float32)
    ck = cv = None
    if pos0:
        ck = rng.standard_normal((pos0, HKV, D), dtype=np.float32).astype(np.float16)
        cv = rng.standard_normal((pos0, HKV, D), dtype=np.float32).astype(np.float16)
    wl = W.Prefill(q, k, v, pos0, True, ck, cv)
    want, _, _ = helpers.oracle_prefill(wl)
    out, _, _ = helpers.gpu_prefill(wl, impl=impl)
    helpers.assert_parity(out.cpu().numpy(), want, f"prefill n_tok={n_tok} pos0={pos0} impl={impl}")


@pytest.mark.parametrize("impl", IMPLS)
def test_prefill_first_row_is_v0(impl):
    """Token 0 sees only key 0, so its output is v[0] rounded to f16, for every head of the group."""
    wl = W.c1_prefill128(seed=9, n_tok=40)
    out, _, _ = helpers.gpu_prefill(wl, impl=impl)
    got = out.cpu().numpy()[0].reshape(HKV, H // HKV, D)
    want = wl.v[0].astype(np.float16).astype(np.float32)
    for g in range(H // HKV):
        assert np.array_equal(got[:, g, :], want)


@pytest.mark.parametrize("n_head,n_head_kv", [(8, 8), (16, 8), (32, 8), (4, 1)])
def test_prefill_group_sizes(n_head, n_head_kv):
    rng = np.random.default_rng(n_head)
    n_tok = 150
    wl = W.Prefill(rng.standard_normal((n_tok, n_head, D), dtype=np.float32),
                   rng.standard_normal((n_tok, n_head_kv, D), dtype=np.float32),
                   rng.standard_normal((n_tok, n_head_kv, D), dtype=np.float32), 0, True)
    want, _, _ = helpers.oracle_prefill(wl)
    out, _, _ = helpers.gpu_prefill(wl, impl=1)
    helpers.assert_parity(out.cpu().numpy(), want, f"prefill H={n_head} Hkv={n_head_kv}")


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("n_tok,pos0", [(200, 0), (64, 1000), (700, 300)])
def test_prefill_paged_equals_contiguous(impl, n_tok, pos0):
    """A paged cache with a random block permutation gives the same bits as the contiguous cache: the
    kernels read the same values in the same order, only the addresses differ."""
    import torch
    rng = np.random.default_rng(n_tok + pos0)
    ck = cv = None
    if pos0:
        ck = rng.standard_normal((pos0, HKV, D), dtype=np.float32).astype(np.float16)
        cv = rng.standard_normal((pos0, HKV, D), dtype=np.float32).astype(np.float16)
    wl = W.Prefill(rng.standard_normal((n_tok, H, D), dtype=np.float32), rng.standard_normal((n_tok, HKV, D), dtype=np.float32),
                   rng.standard_normal((n_tok, HKV, D), dtype=np.float32), pos0, True, ck, cv)
    out_c, _, _ = helpers.gpu_prefill(wl, impl=impl)
    out_p, _, _ = helpers.gpu_prefill(wl, impl=impl, paged=True)
    assert torch.equal(out_c, out_p)


@pytest.mark.parametrize("impl", IMPLS)
def test_chunked_equals_one_shot(impl):
    """Prefilling 384 tokens in chunks of 128 matches one 384-token prefill row for row."""
    import torch
    import ingot_b200 as ib
    wl = W.c1_prefill128(seed=22, n_tok=384)
    out_full, _, _ = helpers.gpu_prefill(wl, impl=impl)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, HKV, 384)
    inv = helpers.to_dev(helpers.inv_freq())
    outs = []
    for c in range(3):
        sl = slice(c * 128, (c + 1) * 128)
        qr = ib.rope_kv_append(kv, 0, helpers.to_dev(wl.q[sl]), helpers.to_dev(wl.k[sl]), helpers.to_dev(wl.v[sl]), inv, c * 128)
        outs.append(ib.attn_prefill(kv, 0, qr, c * 128, impl=impl))
    torch.cuda.synchronize()
    got = torch.cat(outs).cpu().numpy()
    max_abs, rel = helpers.errors(got, out_full.cpu().numpy())
    assert max_abs <= 1e-5 and rel <= 1e-6, (max_abs, rel)


@pytest.mark.parametrize("impl", IMPLS)
def test_c5_long_prefill_sampled_rows(impl):
    """32768-token causal prefill (bf16 q, f16 k/v). The reference is evaluated on a stratified row
    sample (first rows, last rows, random rows); every sampled row must meet the tolerance."""
    import torch
    wl = W.c5_prefill32k()
    rng = np.random.default_rng(44)
    rows = np.unique(np.concatenate([np.arange(16), np.arange(32768 - 16, 32768), rng.integers(0, 32768, 32)]))
    want, _, _ = helpers.oracle_prefill(wl, rows=rows)
    out, _, _ = helpers.gpu_prefill(wl, impl=impl, out_f16=True)
    got = out[torch.from_numpy(rows).cuda()].float().cpu().numpy()
    assert np.isfinite(got).all()
    max_abs, rel = helpers.errors(got, want)
    # f16 output adds half an f16 ulp of the value (|out| < 8 -> 2e-3 at most, typically 1e-4).
    assert max_abs <= 2e-3 + 2e-3 and rel <= 1e-3, (max_abs, rel)
    # size-independent property: no row of the full output is non-finite, row 0 equals v[0]
    assert torch.isfinite(out).all().item()
    assert np.array_equal(out[0].float().cpu().numpy().reshape(HKV, 3, D)[:, 0], wl.v[0].astype(np.float32))


def test_prefill_rejects_bad_arguments():
    import ingot_b200 as ib
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, HKV, 64)
    q = helpers.to_dev(np.zeros((8, H, D), dtype=np.float16))
    with pytest.raises(ib.IngotError, match="context window exceeded"):
        ib.attn_prefill(kv, 0, q, 60)
    with pytest.raises(ib.IngotError, match="multiple of n_head_kv"):
        ib.attn_prefill(kv, 0, helpers.to_dev(np.zeros((8, 7, D), dtype=np.float16)), 0)


@pytest.mark.parametrize("n_shards,out_f16", [(2, True), (4, False), (8, True)])
def test_kv_head_shards_with_fused_gather_reproduce_unsharded_output(n_shards, out_f16):
    """KV-head sharding: every shard runs the same kernel on its own heads and stores its rows into every
    destination buffer (here: two buffers on one GPU standing in for this GPU's and a peer's). The
    gathered token-major result must equal the unsharded prefill bit for bit."""
    import torch
    import ingot_b200 as ib
    wl = W.c1_prefill128(seed=31, n_tok=300)
    dt = torch.float16 if out_f16 else torch.float32
    full, _, _ = helpers.gpu_prefill(wl, impl=2, out_f16=out_f16)
    inv = helpers.to_dev(helpers.inv_freq())
    dst = [torch.zeros(300, H, D, device="cuda", dtype=dt) for _ in range(2)]
    hkv_l, h_l = HKV // n_shards, H // n_shards
    for r in range(n_shards):
        kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, hkv_l, 300)
        q = helpers.to_dev(wl.q[:, r * h_l:(r + 1) * h_l])
        k = helpers.to_dev(wl.k[:, r * hkv_l:(r + 1) * hkv_l])
        v = helpers.to_dev(wl.v[:, r * hkv_l:(r + 1) * hkv_l])
        qr = ib.rope_kv_append(kv, 0, q, k, v, inv, 0)
        ib.attn_prefill_gather(kv, 0, qr, 0, [d.data_ptr() for d in dst], ib.F16 if out_f16 else ib.F32, H, r * h_l)
        torch.cuda.synchronize()
        assert kv.status() == 0
    assert torch.equal(dst[0], full) and torch.equal(dst[1], full)


def test_bounded_waits_expire_cleanly(monkeypatch):
    """Failure detection without a fault: with the TMA producer stalled by the test hook, every mbarrier wait
    of the tcgen05 kernel runs into its (shortened) limit, the kernel returns normally with the timeout bit in
    the status word, tensor memory is released, and the next launch on the same handle is correct again."""
    import torch
    import ingot_b200 as ib
    wl = W.c1_prefill128(seed=41, n_tok=40)
    want, _, _ = helpers.oracle_prefill(wl)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, HKV, 40)
    inv = helpers.to_dev(helpers.inv_freq())
    qr = ib.rope_kv_append(kv, 0, helpers.to_dev(wl.q), helpers.to_dev(wl.k), helpers.to_dev(wl.v), inv, 0)
    assert ib.lib().ingot_kv_test_stall_prefill(kv.handle, 50) == 0  # milliseconds; this handle only
    ib.attn_prefill(kv, 0, qr, 0, impl=2)
    torch.cuda.synchronize()
    assert kv.status() == 4  # kDevErrBarrierTimeout
    assert ib.lib().ingot_kv_test_stall_prefill(kv.handle, 0) == 0
    out = ib.attn_prefill(kv, 0, qr, 0, impl=2)
    torch.cuda.synchronize()
    assert kv.status() == 0
    helpers.assert_parity(out.cpu().numpy(), want, "prefill after an expired wait")


def test_gather_signal_and_bounded_wait():
    """The signalling form of the fused gather on one GPU. The call writes this GPU's own buffer and signals slot 0
    of a two-slot counter array. A wait for ONE source completes, takes the signal back (counter 0 again) and leaves
    the status word clear. A wait for TWO sources meets a peer that never signals - the host-made stand-in for a
    rank that dropped out: it gives up after its limit, raises the timeout bit without hanging or trapping, and the
    next call on the same handle is correct again."""
    import torch
    import ingot_b200 as ib
    wl = W.c5_prefill32k(seed=9, n_tok=2048)
    rows = np.array([0, 1, 700, 2047])
    want, _, _ = helpers.oracle_prefill(wl, rows=rows)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, HKV, 2048)
    kv.import_f16(0, helpers.to_dev(wl.k), helpers.to_dev(wl.v), 0)
    q = helpers.to_dev(wl.q, torch.bfloat16)
    out = torch.zeros(2048, H, D, device="cuda", dtype=torch.float16)
    sig = torch.zeros(2, device="cuda", dtype=torch.int32)
    ib.attn_prefill_gather_signal(kv, 0, q, 0, [out.data_ptr()], [sig.data_ptr()], 0, ib.F16, H, 0)
    ib.gather_wait(kv, sig, 1, timeout_ms=2000)
    torch.cuda.synchronize()
    assert kv.status() == 0 and sig.tolist() == [0, 0]
    helpers.assert_parity(out[torch.from_numpy(rows).cuda()].float().cpu().numpy(), want, "gather_signal output")
    # the second source never signals
    out.zero_()
    ib.attn_prefill_gather_signal(kv, 0, q, 0, [out.data_ptr()], [sig.data_ptr()], 0, ib.F16, H, 0)
    ib.gather_wait(kv, sig, 2, timeout_ms=50)
    torch.cuda.synchronize()
    assert kv.status() == 4 and sig.tolist() == [0, 0]  # slot 0 was consumed, slot 1 never arrived
    # and the handle is fine afterwards
    out.zero_()
    ib.attn_prefill_gather_signal(kv, 0, q, 0, [out.data_ptr()], [sig.data_ptr()], 0, ib.F16, H, 0)
    ib.gather_wait(kv, sig, 1)
    torch.cuda.synchronize()
    assert kv.status() == 0
    helpers.assert_parity(out[torch.from_numpy(rows).cuda()].float().cpu().numpy(), want, "gather_signal after an expired wait")


@pytest.mark.parametrize("n_tok,pos0,chunk,q_dtype,out_dtype", [(700, 0, 256, "float32", "float32"), (1300, 260, 512, "bfloat16", "float16"),
                                                             (100, 0, 0, "float16", "float32"), (513, 3584, 128, "float32", "float32")])
def test_prefill_host_pipelined_chunks(n_tok, pos0, chunk, q_dtype, out_dtype):
    """ingot_attn_prefill_host: queries and output in pinned host memory, the rows cut into chunks whose copies in,
    attention and copies out overlap on three streams. Against the CPU reference, against the device-buffer call on the
    same cache, and twice in a row (the staging buffers and events of the first call are reused by the second)."""
    import torch
    import ingot_b200 as ib
    rng = np.random.default_rng(n_tok + pos0)
    n_keys = pos0 + n_tok
    q = rng.standard_normal((n_tok, H, D), dtype=np.float32)
    k = rng.standard_normal((n_keys, HKV, D), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((n_keys, HKV, D), dtype=np.float32).astype(np.float16)
    tq, to = getattr(torch, q_dtype), getattr(torch, out_dtype)
    q_t = torch.from_numpy(q).to(tq)
    q_used = q_t.float().numpy()  # what the kernel sees (bf16 / f16 rounding of q is part of the input)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, HKV, n_keys)
    kv.import_f16(0, helpers.to_dev(k), helpers.to_dev(v), 0)
    want, _, _ = helpers.oracle_prefill(W.Prefill(q_used, k, v, pos0, False))  # k, v: every cache row, already rotated
    dev = ib.attn_prefill(kv, 0, helpers.to_dev(q_used, tq), pos0, out_dtype=to, impl=2)
    q_host = q_t.contiguous().pin_memory()
    outs = []
    for rep in range(2):
        out_host = torch.full((n_tok, H, D), 7.0, dtype=to).pin_memory()
        ib.attn_prefill_host(kv, 0, q_host, pos0, out_host, chunk_tokens=chunk)
        outs.append(out_host)
    torch.cuda.synchronize()
    assert kv.status() == 0
    for out_host in outs:
        got = out_host.float().numpy()
        helpers.assert_parity(got, want, "host-buffer prefill")
        # chunk boundaries move the key-tile boundaries, and with them the reference maxima P is rounded against
        assert np.abs(got - dev.float().cpu().numpy()).max() < 2e-3
    assert np.array_equal(outs[0].numpy(), outs[1].numpy())  # the second call reuses buffers and events: same bits


def test_prefill_host_paged_cache():
    """The host-buffer prefill on a paged cache (permuted 16-token blocks): same rows as on a contiguous cache."""
    import torch
    import ingot_b200 as ib
    rng = np.random.default_rng(77)
    n_tok, pos0 = 600, 200
    n_keys = pos0 + n_tok
    q = rng.standard_normal((n_tok, H, D), dtype=np.float32)
    k = rng.standard_normal((n_keys, HKV, D), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((n_keys, HKV, D), dtype=np.float32).astype(np.float16)
    nb = (n_keys + 15) // 16
    lens = np.array([n_keys], dtype=np.int32)
    bt = helpers.to_dev(W.block_tables(lens, rng.permutation(nb).astype(np.int32)))
    paged = ib.KVCache(ib.KV_PAGED, 1, HKV, nb, max_seqs=1)
    paged.import_f16(0, helpers.to_dev(k), helpers.to_dev(v), 0, bt[0])
    flat = ib.KVCache(ib.KV_CONTIGUOUS, 1, HKV, n_keys)
    flat.import_f16(0, helpers.to_dev(k), helpers.to_dev(v), 0)
    q_host = torch.from_numpy(q).pin_memory()
    out_p = torch.zeros(n_tok, H, D).pin_memory()
    out_f = torch.zeros(n_tok, H, D).pin_memory()
    ib.attn_prefill_host(paged, 0, q_host, pos0, out_p, block_table=bt[0], chunk_tokens=256)
    ib.attn_prefill_host(flat, 0, q_host, pos0, out_f, chunk_tokens=256)
    torch.cuda.synchronize()
    assert paged.status() == 0 and flat.status() == 0
    assert torch.equal(out_p, out_f)
    want, _, _ = helpers.oracle_prefill(W.Prefill(q, k, v, pos0, False))
    helpers.assert_parity(out_p.numpy(), want, "host-buffer prefill, paged cache")
