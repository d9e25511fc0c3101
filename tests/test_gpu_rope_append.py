"""K1 (fused RoPE + KV append) against the CPU reference's ops::rope + cache append."""
import numpy as np
import pytest

import helpers
from helpers import D, H, HKV

pytestmark = pytest.mark.gpu


def _check_rounded(got_f16, want_f32, what):
    """got must be the f16 rounding of the reference's f32 value, up to the libm difference.

    CUDA's cosf/sinf and glibc's differ by at most a couple of f32 ulps of the rotated value (an
    absolute 1e-6 covers |x| <= 8), which can also move a value across an f16 rounding boundary. So:
    every element within half an f16 ulp (the rounding itself) plus 1e-6, and all but a small
    fraction bit-equal to the rounded reference."""
    want16 = want_f32.astype(np.float16)
    spacing = np.spacing(np.abs(want16)).astype(np.float64)  # f16 ulp at the reference value
    diff = np.abs(got_f16.astype(np.float64) - want_f32.astype(np.float64))
    assert (diff <= 0.5 * spacing + 1e-6).all(), f"{what}: max excess {(diff - 0.5 * spacing).max():.3e}"
    assert (got_f16 != want16).mean() < 5e-3, f"{what}: {(got_f16 != want16).mean():.2%} of elements differ"


@pytest.mark.parametrize("pos0,n_tok,paged", [(0, 128, False), (3584, 64, False), (32760, 8, False), (5, 37, True)])
def test_rope_append_matches_reference(pos0, n_tok, paged):
    import torch
    import ingot_b200 as ib
    rng = np.random.default_rng(100 + pos0)
    q = rng.standard_normal((n_tok, H, D), dtype=np.float32)
    k = rng.standard_normal((n_tok, HKV, D), dtype=np.float32)
    v = rng.standard_normal((n_tok, HKV, D), dtype=np.float32)
    inv = helpers.inv_freq()
    lib = helpers.oracle()
    q_ref, k_ref = q.copy(), k.copy()
    for i in range(n_tok):
        lib.oracle_rope(q_ref[i].reshape(-1), H, D, pos0 + i, inv)
        lib.oracle_rope(k_ref[i].reshape(-1), HKV, D, pos0 + i, inv)

    n_ctx = pos0 + n_tok
    if paged:
        nb = (n_ctx + 15) // 16
        perm = np.random.default_rng(1).permutation(nb + 2).astype(np.int32)[:nb]
        kv = ib.KVCache(ib.KV_PAGED, 2, HKV, nb + 2)
        bt = helpers.to_dev(perm).view(1, -1)
    else:
        kv = ib.KVCache(ib.KV_CONTIGUOUS, 2, HKV, n_ctx)
        bt = None
    q_out = ib.rope_kv_append(kv, 1, helpers.to_dev(q), helpers.to_dev(k), helpers.to_dev(v), helpers.to_dev(inv), pos0,
                              block_tables=bt)
    torch.cuda.synchronize()
    assert kv.status() == 0
    kc = kv.layer_view(1, "k").cpu().numpy()
    vc = kv.layer_view(1, "v").cpu().numpy()
    if paged:
        pos = pos0 + np.arange(n_tok)
        k_got = kc[perm[pos // 16], :, pos % 16, :]   # [n_tok, Hkv, d]
        v_got = vc[perm[pos // 16], :, pos % 16, :]
    else:
        k_got = kc[:, pos0:pos0 + n_tok, :].transpose(1, 0, 2)
        v_got = vc[:, pos0:pos0 + n_tok, :].transpose(1, 0, 2)
    _check_rounded(q_out.cpu().numpy(), q_ref, "rotated q")
    _check_rounded(k_got, k_ref, "rotated k in cache")
    assert np.array_equal(v_got, v.astype(np.float16)), "v must be the exact f16 rounding of the input"
    # layer 0 untouched
    assert not kv.layer_view(0, "k").any().item()


def test_append_rewind_overwrites():
    """The cache is a pure function of (layer, position): writing position p again replaces it."""
    import torch
    import ingot_b200 as ib
    rng = np.random.default_rng(5)
    inv = helpers.to_dev(helpers.inv_freq())
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, HKV, 32)
    k1 = rng.standard_normal((8, HKV, D), dtype=np.float32)
    k2 = rng.standard_normal((3, HKV, D), dtype=np.float32)
    ib.rope_kv_append(kv, 0, None, helpers.to_dev(k1), helpers.to_dev(k1), inv, 0)
    before = kv.layer_view(0, "v").cpu().numpy().copy()
    ib.rope_kv_append(kv, 0, None, helpers.to_dev(k2), helpers.to_dev(k2), inv, 2)
    torch.cuda.synchronize()
    after = kv.layer_view(0, "v").cpu().numpy()
    assert np.array_equal(after[:, 2:5], k2.astype(np.float16).transpose(1, 0, 2))
    assert np.array_equal(after[:, :2], before[:, :2]) and np.array_equal(after[:, 5:8], before[:, 5:8])


def test_append_out_of_range_is_rejected_on_host():
    import ingot_b200 as ib
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, HKV, 16)
    z = helpers.to_dev(np.zeros((4, HKV, D), dtype=np.float32))
    inv = helpers.to_dev(helpers.inv_freq())
    with pytest.raises(ib.IngotError, match="context window exceeded"):
        ib.rope_kv_append(kv, 0, None, z, z, inv, 14)


def test_append_device_positions_out_of_range_sets_status():
    """Positions supplied on the device cannot be validated on the host: the kernel skips the row
    and raises the status word instead of writing out of bounds."""
    import torch
    import ingot_b200 as ib
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 1, HKV, 16)
    z = helpers.to_dev(np.ones((2, HKV, D), dtype=np.float32))
    inv = helpers.to_dev(helpers.inv_freq())
    pos = helpers.to_dev(np.array([3, 99], dtype=np.int32))
    ib.rope_kv_append(kv, 0, None, z, z, inv, 0, positions=pos)
    torch.cuda.synchronize()
    assert kv.status() == 1
    assert kv.status() == 0  # cleared by the read
    v = kv.layer_view(0, "v").cpu().numpy()
    assert (v[:, 3] == 1).all() and not v[:, :3].any() and not v[:, 4:].any()
