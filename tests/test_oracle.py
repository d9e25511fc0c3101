"""The plain-C oracle against fixtures produced by the reference's own compiled code, and (when that
library was built on this machine) against the reference directly."""
import os

import numpy as np
import pytest

import helpers
from oracle import loader

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attn_golden.npz")


@pytest.fixture(scope="module")
def g():
    return np.load(GOLDEN)


@pytest.fixture(scope="module")
def lib():
    return loader.load_oracle()


def test_inv_freq_table(g, lib):
    assert np.array_equal(loader.inv_freq(lib, "oracle_"), g["inv_freq"])
    out = np.empty(64, dtype=np.float32)
    facs = np.ascontiguousarray(g["rope_factors"])
    lib.oracle_rope_inv_freq(out, 128, 500000.0, facs.ctypes.data)
    assert np.array_equal(out, g["inv_freq_factored"])


@pytest.mark.parametrize("pos", [0, 1, 127, 3584, 32767])
def test_rope(g, lib, pos):
    x = g["rope_in"].copy()
    lib.oracle_rope(x.reshape(-1), x.shape[0], x.shape[1], pos, np.ascontiguousarray(g["inv_freq"]))
    assert np.array_equal(x, g[f"rope_out_{pos}"])
    if pos == 0:
        assert np.array_equal(x, g["rope_in"])  # angle 0 is the identity


def test_softmax(g, lib):
    x = g["softmax_in"].copy()
    lib.oracle_softmax(x, x.size)
    assert np.array_equal(x, g["softmax_out"])
    assert abs(float(x.sum()) - 1.0) < 1e-6


def test_prefill_then_chunk_with_overwrite(g, lib):
    inv = np.ascontiguousarray(g["inv_freq"])
    o, _, _, kc, vc = loader.attn_forward(lib, "oracle_", g["p_q"], g["p_k"], g["p_v"], 0, 12, inv)
    assert np.array_equal(o, g["p_out"])
    o2, _, _, kc, vc = loader.attn_forward(lib, "oracle_", g["c_q"], g["c_k"], g["c_v"], 7, 12, inv, kc, vc)
    assert np.array_equal(o2, g["c_out"])
    assert np.array_equal(kc, g["c_kcache"]) and np.array_equal(vc, g["c_vcache"])


def test_attend_rows_equals_per_token_loop(g, lib):
    """The threaded row driver used for sampled long prefills is the same arithmetic as the token loop."""
    inv = np.ascontiguousarray(g["inv_freq"])
    o, q_rot, _, kc, vc = loader.attn_forward(lib, "oracle_", g["p_q"], g["p_k"], g["p_v"], 0, 12, inv)
    rows = np.array([0, 3, 8], dtype=np.int32)
    got = loader.attend_rows(lib, q_rot[rows], kc, vc, rows, 6, 2, 128, n_threads=2)
    assert np.array_equal(got, o[rows])
    assert loader.attend_rows(lib, q_rot[:0], kc, vc, rows[:0], 6, 2, 128).shape[0] == 0  # empty input


def test_first_token_returns_its_value_row(g, lib):
    """One visible key: the softmax weight is exactly 1 and the output is v[0] for every head of the group."""
    out = g["p_out"][0].reshape(2, 3, 128)
    for j in range(3):
        assert np.array_equal(out[:, j], g["p_v"][0])


def test_oracle_equals_compiled_reference_when_present(lib):
    ref = loader.load_ref()
    if ref is None:
        pytest.skip("oracle/_ref not built on this machine")
    rng = np.random.default_rng(3)
    q = rng.standard_normal((33, 24, 128), dtype=np.float32)
    k = rng.standard_normal((33, 8, 128), dtype=np.float32)
    v = rng.standard_normal((33, 8, 128), dtype=np.float32)
    inv_o, inv_r = loader.inv_freq(lib, "oracle_"), loader.inv_freq(ref, "ref_")
    assert np.array_equal(inv_o, inv_r)
    a = loader.attn_forward(lib, "oracle_", q, k, v, 100, 133, inv_o)
    b = loader.attn_forward(ref, "ref_", q, k, v, 100, 133, inv_r)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)


def test_parity_metric_helpers():
    a = np.ones((4, 4), dtype=np.float32)
    assert helpers.errors(a, a) == (0.0, 0.0)
    with pytest.raises(AssertionError):
        helpers.assert_parity(a + 1e-2, a)
    with pytest.raises(AssertionError):
        helpers.assert_parity(np.full((2, 2), np.nan), np.ones((2, 2)))
