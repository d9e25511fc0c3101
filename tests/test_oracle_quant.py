"""The CPU restatement of the reference's weight dequantisation (oracle/quant_oracle.c) against the committed
fixture generated from the reference's own compiled ops::dequant_row, and against that code directly when it was
built on this machine. Bit-exact: block decoding is integer/byte work plus one or two f32 multiplies."""
import os

import numpy as np
import pytest

from oracle import loader

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quant_golden.npz")
TYPES = ["F32", "F16", "BF16", "Q8_0", "Q4_0", "Q4_1", "Q6_K"]


@pytest.mark.parametrize("type_name", TYPES)
def test_dequant_matches_golden_fixture(type_name):
    lib = loader.load_oracle()
    g = np.load(GOLDEN)
    for kind in ("normal", "extreme"):
        raw, bits = g[f"{type_name}_{kind}_raw"], g[f"{type_name}_{kind}_bits"]
        for r in range(raw.shape[0]):
            got = loader.dequant(lib, "oracle_", type_name, raw[r], bits.shape[1])
            assert np.array_equal(got.view(np.uint32), bits[r]), f"{type_name} {kind} row {r}"


@pytest.mark.parametrize("type_name", TYPES)
def test_dequant_equals_compiled_reference_when_present(type_name):
    ref = loader.load_ref()
    if ref is None:
        pytest.skip("oracle/_ref not built on this machine")
    lib = loader.load_oracle()
    for extreme in (False, True):
        rng = np.random.default_rng([5, TYPES.index(type_name), int(extreme)])
        raw = loader.random_blocks(type_name, 16, 1024, rng, extreme=extreme)
        for r in range(raw.shape[0]):
            a = loader.dequant(lib, "oracle_", type_name, raw[r], 1024)
            b = loader.dequant(ref, "ref_", type_name, raw[r], 1024)
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), f"{type_name} extreme={extreme} row {r}"


def test_unsupported_type_is_rejected():
    lib = loader.load_oracle()
    with pytest.raises((ValueError, KeyError)):
        loader.dequant(lib, "oracle_", "Q5_0", np.zeros(64, dtype=np.uint8), 32)


def test_row_bytes():
    assert loader.row_bytes("Q8_0", 3072) == 3264 and loader.row_bytes("Q4_0", 3072) == 1728
    assert loader.row_bytes("Q4_1", 3072) == 1920 and loader.row_bytes("Q6_K", 3072) == 2520
