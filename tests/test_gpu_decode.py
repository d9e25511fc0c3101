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
