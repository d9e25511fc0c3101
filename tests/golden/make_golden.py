"""Generates tests/golden/attn_golden.npz from the reference's own compiled CPU code.

Run where oracle/_ref/libingot_ref.so exists (it is built from an Ingot checkout by oracle/Makefile):
    python tests/golden/make_golden.py
The fixture is small on purpose (2 KV heads, 6 query heads) and pins: the rotary inverse-frequency
table, ops::rope at small / chunk-offset / long-context positions, ops::softmax, and the attention
part of CpuBackend::forward for a fresh 9-token prefill and for a 5-token chunk appended at position 7.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import loader  # noqa: E402


def main():
    ref = loader.load_ref()
    if ref is None:
        raise SystemExit("oracle/_ref/libingot_ref.so not built")
    rng = np.random.default_rng(20250101)
    H, HKV, D = 6, 2, 128
    out = {}
    inv = loader.inv_freq(ref, "ref_")
    out["inv_freq"] = inv
    facs = (1.0 + np.arange(64, dtype=np.float32) / 16).astype(np.float32)
    inv_f = np.empty(64, dtype=np.float32)
    ref.ref_rope_inv_freq(inv_f, 128, 500000.0, facs.ctypes.data)
    out["rope_factors"], out["inv_freq_factored"] = facs, inv_f
    x = rng.standard_normal((H, D), dtype=np.float32)
    out["rope_in"] = x
    for pos in (0, 1, 127, 3584, 32767):
        y = x.copy()
        ref.ref_rope(y.reshape(-1), H, D, pos, inv)
        out[f"rope_out_{pos}"] = y
    sm = (rng.standard_normal(37, dtype=np.float32) * 3).astype(np.float32)
    out["softmax_in"] = sm
    y = sm.copy()
    ref.ref_softmax(y, y.size)
    out["softmax_out"] = y
    # fresh prefill of 9 tokens, then a 5-token chunk at position 7 (overwrites 7, 8 and extends to 11)
    q = rng.standard_normal((9, H, D), dtype=np.float32)
    k = rng.standard_normal((9, HKV, D), dtype=np.float32)
    v = rng.standard_normal((9, HKV, D), dtype=np.float32)
    o, _, _, kc, vc = loader.attn_forward(ref, "ref_", q, k, v, 0, 12, inv)
    out.update(p_q=q, p_k=k, p_v=v, p_out=o)
    q2 = rng.standard_normal((5, H, D), dtype=np.float32)
    k2 = rng.standard_normal((5, HKV, D), dtype=np.float32)
    v2 = rng.standard_normal((5, HKV, D), dtype=np.float32)
    o2, _, _, kc, vc = loader.attn_forward(ref, "ref_", q2, k2, v2, 7, 12, inv, kc, vc)
    out.update(c_q=q2, c_k=k2, c_v=v2, c_out=o2, c_kcache=kc, c_vcache=vc)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attn_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
