"""K3 (split-KV flash decoding) against the CPU reference's attention lambda."""
import numpy as np
import pytest

import helpers
from helpers import D, H, HKV
from ingot_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _decode_case(n_keys, n_head=H, n_head_kv=HKV, seed=0):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((1, n_head, D), dtype=np.float32)
    k = rng.standard_normal((n_keys, n_head_kv, D), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((n_keys, n_head_kv, D), dtype=np.float32).astype(np.float16)
    return W.Decode(q, [k], [v], np.array([n_keys], dtype=np.int32))


def test_c2_decode_4096():
    wl = W.c2_decode4096()
    want = helpers.oracle_decode(wl)
    out, _ = helpers.gpu_decode(wl)
    helpers.assert_parity(out.cpu().numpy(), want, "C2 decode @4096")


@pytest.mark.parametrize("n_keys", [1, 2, 7, 15, 16, 17, 31, 63, 64, 65, 255, 1000, 4095])
def test_decode_lengths(n_keys):
    wl = _decode_case(n_keys, seed=n_keys)
    want = helpers.oracle_decode(wl)
    out, _ = helpers.gpu_decode(wl)
    helpers.assert_parity(out.cpu().numpy(), want, f"decode n_keys={n_keys}")


def test_decode_single_key_returns_v0():
    """With one key the softmax weight is exactly 1, so the output is v[0] (stored as f16) exactly."""
    wl = _decode_case(1, seed=3)
    out, _ = helpers.gpu_decode(wl)
    got = out.cpu().numpy()[0].reshape(HKV, H // HKV, D)
    for g in range(H // HKV):
        assert np.array_equal(got[:, g, :], wl.v[0][0].astype(np.float32))


@pytest.mark.parametrize("n_head,n_head_kv", [(8, 8), (16, 8), (32, 8), (8, 1), (24, 4)])
def test_decode_group_sizes(n_head, n_head_kv):
    wl = _decode_case(777, n_head, n_head_kv, seed=n_head)
    want = helpers.oracle_decode(wl)
    out, _ = helpers.gpu_decode(wl)
    helpers.assert_parity(out.cpu().numpy(), want, f"decode H={n_head} Hkv={n_head_kv}")


@pytest.mark.parametrize("chunk", [16, 64, 112, 512, 4096])
def test_decode_split_sizes_agree(chunk):
    """Any split size gives the reference answer: the split merge is the attn_combine formula."""
    wl = _decode_case(2049, seed=11)
    want = helpers.oracle_decode(wl)
    out, _ = helpers.gpu_decode(wl, chunk_keys=chunk)
    helpers.assert_parity(out.cpu().numpy(), want, f"decode chunk={chunk}")


def test_decode_is_deterministic_and_reusable():
    """Two launches on the same handle give identical bits (the arrival counters reset themselves)."""
    import torch
    import ingot_b200 as ib
    wl = _decode_case(3000, seed=12)
    out1, kv = helpers.gpu_decode(wl)
    q = helpers.to_dev(wl.q)
    out2 = ib.attn_decode(kv, 0, q, max_seq_len=3000)
    out3 = ib.attn_decode(kv, 0, q, max_seq_len=3000)
    torch.cuda.synchronize()
    assert torch.equal(out1, out2) and torch.equal(out2, out3)


def test_decode_paged_equals_contiguous():
    """The paged layout (random block permutation) reads the same values in the same order."""
    import torch
    wl = _decode_case(1234, seed=13)
    out_c, _ = helpers.gpu_decode(wl, chunk_keys=128)
    out_p, _ = helpers.gpu_decode(wl, paged=True, chunk_keys=128)
    assert torch.equal(out_c, out_p)


def test_decode_bf16_query_f16_output():
    import torch
    wl = _decode_case(600, seed=14)
    wl.q = W.bf16_round(wl.q)
    wl.q_is_bf16 = True
    want = helpers.oracle_decode(wl)
    out, _ = helpers.gpu_decode(wl, out_f16=True)
    assert out.dtype == torch.float16
    got = out.float().cpu().numpy()
    max_abs, rel = helpers.errors(got, want)
    assert max_abs <= 2e-3 + 2e-3 and rel <= 1e-3  # plus the f16 rounding of the output itself


def test_c4_batched_paged_decode():
    """64 sequences, lengths U{256..8192}, paged cache with a random block permutation, bf16 queries."""
    wl = W.c4_batched_decode()
    assert len(wl.lens) == 64 and wl.lens.min() >= 256 and wl.lens.max() <= 8192
    want = helpers.oracle_decode(wl)
    out, _ = helpers.gpu_decode(wl, paged=True)
    helpers.assert_parity(out.cpu().numpy(), want, "C4 batched paged decode")


def test_decode_rejects_bad_arguments():
    import ingot_b200 as ib
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, HKV, 64)
    q = helpers.to_dev(np.zeros((1, H, D), dtype=np.float32))
    with pytest.raises(ib.IngotError, match="context window exceeded"):
        ib.attn_decode(kv, 0, q, max_seq_len=65)
    with pytest.raises(ib.IngotError, match="layer out of range"):
        ib.attn_decode(kv, 1, q, max_seq_len=10)
    with pytest.raises(ib.IngotError, match="multiple of 16"):
        ib.attn_decode(kv, 0, q, max_seq_len=10, chunk_keys=24)


def test_decode_very_long_context():
    """100 000 keys: the split size grows so that at most 64 partials per head exist; parity still holds."""
    wl = _decode_case(100_000, seed=21)
    want = helpers.oracle_decode(wl)
    out, _ = helpers.gpu_decode(wl)
    helpers.assert_parity(out.cpu().numpy(), want, "decode n_keys=100000")
    out16, _ = helpers.gpu_decode(wl, chunk_keys=16)  # a too-small request is raised to the same bound
    helpers.assert_parity(out16.cpu().numpy(), want, "decode n_keys=100000, chunk request 16")


def test_batched_append_then_decode_paged():
    """Three sequences in one paged pool: one K1 launch appends a token to each (device positions and
    sequence ids), one K3 launch decodes all three; each sequence must match its own reference."""
    import torch
    import ingot_b200 as ib
    rng = np.random.default_rng(55)
    lens = np.array([37, 260, 16], dtype=np.int32)  # lengths AFTER the append
    nb = int(((lens + 15) // 16).sum())
    perm = rng.permutation(nb + 4).astype(np.int32)[:nb]
    bt_np = W.block_tables(lens, perm)
    kv = ib.KVCache(ib.KV_PAGED, 1, HKV, nb + 4, max_seqs=3)
    bt = helpers.to_dev(bt_np)
    inv_np = helpers.inv_freq()
    ks, vs = [], []
    for s in range(3):
        k = rng.standard_normal((lens[s] - 1, HKV, D), dtype=np.float32).astype(np.float16)
        v = rng.standard_normal((lens[s] - 1, HKV, D), dtype=np.float32).astype(np.float16)
        if lens[s] > 1:
            kv.import_f16(0, helpers.to_dev(k), helpers.to_dev(v), 0, bt[s])
        ks.append(k)
        vs.append(v)
    q = rng.standard_normal((3, H, D), dtype=np.float32)
    k_new = rng.standard_normal((3, HKV, D), dtype=np.float32)
    v_new = rng.standard_normal((3, HKV, D), dtype=np.float32)
    q_rot = ib.rope_kv_append(kv, 0, helpers.to_dev(q), helpers.to_dev(k_new), helpers.to_dev(v_new), helpers.to_dev(inv_np),
                              positions=helpers.to_dev(lens - 1), seq_ids=helpers.to_dev(np.arange(3, dtype=np.int32)),
                              block_tables=bt)
    out = ib.attn_decode(kv, 0, q_rot, seq_lens=helpers.to_dev(lens), max_seq_len=int(lens.max()), block_tables=bt)
    torch.cuda.synchronize()
    assert kv.status() == 0
    for s in range(3):
        pos0 = int(lens[s]) - 1
        wl = W.Prefill(q[s:s + 1], k_new[s:s + 1], v_new[s:s + 1], pos0, True, ks[s] if pos0 else None, vs[s] if pos0 else None)
        want, _, _ = helpers.oracle_prefill(wl)
        helpers.assert_parity(out[s].cpu().numpy(), want[0], f"batched append+decode, sequence {s}")


@pytest.mark.parametrize("lens", [(2100, 300, 20), (1023, 1024, 1025, 257), (4096,), (300,)])
def test_decode_ragged_batches_library_plan_vs_explicit_split(lens):
    """Few sequences of very different lengths in one call: the library's own split plan and an explicit 256-key
    split (many empty split CTAs for the short sequences, single-split ranges written directly) against the CPU
    reference and against each other."""
    rng = np.random.default_rng(len(lens) * 1000 + lens[0])
    lens = np.array(lens, dtype=np.int32)
    q = rng.standard_normal((len(lens), H, D), dtype=np.float32)
    ks = [rng.standard_normal((n, HKV, D), dtype=np.float32).astype(np.float16) for n in lens]
    vs = [rng.standard_normal((n, HKV, D), dtype=np.float32).astype(np.float16) for n in lens]
    wl = W.Decode(q, ks, vs, lens)
    want = helpers.oracle_decode(wl)
    planned, _ = helpers.gpu_decode(wl, paged=True)
    launched, _ = helpers.gpu_decode(wl, paged=True, chunk_keys=256)
    helpers.assert_parity(planned.cpu().numpy(), want, "library plan")
    helpers.assert_parity(launched.cpu().numpy(), want, "256-key splits")
    assert np.abs(planned.cpu().numpy() - launched.cpu().numpy()).max() < 1e-4  # two summation orders of the same f16 products


@pytest.mark.parametrize("pos", [0, 1, 14, 15, 16, 17, 255, 256, 300, 1000, 4095])
def test_rope_append_decode_equals_k1_then_k3(pos):
    """ingot_rope_append_decode (RoPE, cache append and attention of one token in one launch) against
    ingot_rope_kv_append followed by ingot_attn_decode on a second, identically filled cache: the outputs and the
    appended K/V rows must be the same bits; and against the CPU reference. Once with the key count as an argument,
    once read from device memory with the capacity as the bound (the form a replayed CUDA graph uses)."""
    import torch
    import ingot_b200 as ib
    rng = np.random.default_rng(900 + pos)
    cap = max(pos + 1, 4096 if pos >= 256 else pos + 1)
    k_old = rng.standard_normal((pos, HKV, D), dtype=np.float32).astype(np.float16)
    v_old = rng.standard_normal((pos, HKV, D), dtype=np.float32).astype(np.float16)
    q = rng.standard_normal((1, H, D), dtype=np.float32)
    k_new = rng.standard_normal((1, HKV, D), dtype=np.float32)
    v_new = rng.standard_normal((1, HKV, D), dtype=np.float32)
    inv = helpers.to_dev(helpers.inv_freq())
    caches = []
    for _ in range(3):
        kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, HKV, cap)
        if pos:
            kv.import_f16(0, helpers.to_dev(k_old), helpers.to_dev(v_old), 0)
        caches.append(kv)
    qd, kd, vd = helpers.to_dev(q), helpers.to_dev(k_new), helpers.to_dev(v_new)
    q_rot = ib.rope_kv_append(caches[0], 0, qd, kd, vd, inv, pos)
    two = ib.attn_decode(caches[0], 0, q_rot, max_seq_len=pos + 1)
    one = ib.rope_append_decode(caches[1], 0, qd[0], kd[0], vd[0], inv, pos)
    count = helpers.to_dev(np.array([pos + 1], dtype=np.int32))
    one_dev = ib.rope_append_decode(caches[2], 0, qd[0], kd[0], vd[0], inv, 0, key_count=count, max_seq_len=cap)
    torch.cuda.synchronize()
    for kv in caches:
        assert kv.status() == 0
    for which in ("k", "v"):
        want_rows = caches[0].layer_view(0, which)
        assert torch.equal(caches[1].layer_view(0, which), want_rows) and torch.equal(caches[2].layer_view(0, which), want_rows)
    assert torch.equal(one, two[0])
    wl = W.Prefill(q, k_new, v_new, pos, True, k_old if pos else None, v_old if pos else None)
    want, _, _ = helpers.oracle_prefill(wl)
    helpers.assert_parity(one.cpu().numpy()[None], want, "fused rope + append + decode")
    helpers.assert_parity(one_dev.cpu().numpy()[None], want, "fused, key count from device memory")


def test_empty_calls_are_no_ops():
    import ingot_b200 as ib
    lib = ib.lib()
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, HKV, 16)
    z = helpers.to_dev(np.zeros((1, H, D), dtype=np.float16))
    import ctypes as C
    p = C.c_void_p(z.data_ptr())
    assert lib.ingot_attn_prefill(kv.handle, 0, p, ib.F16, p, ib.F16, H, 0, 0, None, 0, None) == 0      # n_tok == 0
    assert lib.ingot_rope_kv_append(kv.handle, 0, None, None, p, p, p, H, 0, 0, None, None, None, 0, None) == 0
    assert lib.ingot_kv_import_f16(kv.handle, 0, p, p, 0, 0, None, None) == 0
    assert lib.ingot_attn_decode_layers(kv.handle, 0, 0, p, ib.F16, p, ib.F16, H, 1, None, 1, None, 0, 0, None) == 0
    assert kv.status() == 0


def test_device_length_beyond_the_cache_is_clamped_and_flagged():
    """A sequence length read from device memory that exceeds the cache cannot be rejected on the host: the
    kernel clamps it to the capacity and raises the status word instead of reading past the cache."""
    import torch
    import ingot_b200 as ib
    wl = _decode_case(64, seed=31)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 2, HKV, 64)  # layer 1 follows layer 0 in memory
    kv.import_f16(0, helpers.to_dev(wl.k[0]), helpers.to_dev(wl.v[0]), 0)
    q = helpers.to_dev(wl.q)
    want = ib.attn_decode(kv, 0, q, max_seq_len=64)
    got = ib.attn_decode(kv, 0, q, seq_lens=helpers.to_dev(np.array([70], dtype=np.int32)), max_seq_len=64)
    torch.cuda.synchronize()
    assert kv.status() == 1
    assert torch.equal(got, want)
