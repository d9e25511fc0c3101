"""Generates tests/golden/quant_golden.npz: weight rows in the reference's GGUF block layouts together with what
the reference's own ops::dequant_row (src/ops.cpp:22-104, 198-200) makes of them.

    python tests/golden/make_golden_quant.py          (needs oracle/_ref/libingot_ref.so, i.e. a reference checkout
                                                       at build time; the committed fixture was made this way)

Per type: 6 rows of 512 elements with weight-like scales and 6 rows whose f16 scale fields are arbitrary finite bit
patterns (zero, subnormals, 65504 included). Outputs are stored as uint32 bit patterns.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import loader  # noqa: E402

TYPES = ["F32", "F16", "BF16", "Q8_0", "Q4_0", "Q4_1", "Q6_K"]
N_IN, N_ROWS = 512, 6


def main():
    ref = loader.load_ref()
    if ref is None:
        raise SystemExit("oracle/_ref/libingot_ref.so is not built")
    out = {}
    for ti, t in enumerate(TYPES):
        for extreme in (False, True):
            rng = np.random.default_rng([77, ti, int(extreme)])
            raw = loader.random_blocks(t, N_ROWS, N_IN, rng, extreme=extreme)
            vals = np.stack([loader.dequant(ref, "ref_", t, raw[r], N_IN) for r in range(N_ROWS)])
            key = f"{t}_{'extreme' if extreme else 'normal'}"
            out[key + "_raw"] = raw
            out[key + "_bits"] = vals.view(np.uint32)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "quant_golden.npz"), **out)


if __name__ == "__main__":
    main()
