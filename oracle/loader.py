"""TEST INFRASTRUCTURE: ctypes loaders for the two CPU checkers.

`load_oracle()`  -> liboracle.so, the plain-C restatement (oracle/attn_oracle.c).
`load_ref()`     -> _ref/libingot_ref.so, the reference's own CPU sources compiled unmodified
                    (None when it was not built on this machine).

Only tests/, the smoke check and bench.py's CPU-baseline legs may import this module.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


def _declare_common(lib, prefix):
    getattr(lib, prefix + "rope_inv_freq").argtypes = [_f32p, C.c_int, C.c_float, C.c_void_p]
    getattr(lib, prefix + "rope_inv_freq").restype = None
    getattr(lib, prefix + "rope").argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _f32p]
    getattr(lib, prefix + "rope").restype = None
    getattr(lib, prefix + "softmax").argtypes = [_f32p, C.c_size_t]
    getattr(lib, prefix + "softmax").restype = None
    getattr(lib, prefix + "attend").argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int, _f32p, _f32p]
    getattr(lib, prefix + "attend").restype = None
    fwd = getattr(lib, prefix + "attn_forward")
    fwd.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _f32p, _f32p]


def load_oracle():
    path = os.path.join(_HERE, "liboracle.so")
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path} missing: run `make -C oracle` (or __graft_entry__.build())")
    lib = C.CDLL(path)
    _declare_common(lib, "oracle_")
    lib.oracle_attn_forward.restype = C.c_int
    lib.oracle_attend_rows.argtypes = [_f32p, _f32p, _f32p, _i32p, C.c_int, C.c_int, C.c_int, C.c_int, _f32p, C.c_int]
    lib.oracle_attend_rows.restype = C.c_int
    return lib


def load_ref():
    path = os.path.join(_HERE, "_ref", "libingot_ref.so")
    if not os.path.exists(path):
        return None
    lib = C.CDLL(path)
    _declare_common(lib, "ref_")
    lib.ref_attn_forward.restype = None
    lib.ref_thread_count.restype = C.c_int
    lib.ref_last_error.restype = C.c_char_p
    return lib


def inv_freq(lib, prefix, head_dim=128, theta=500000.0):
    out = np.empty(head_dim // 2, dtype=np.float32)
    getattr(lib, prefix + "rope_inv_freq")(out, head_dim, theta, None)
    return out


def attn_forward(lib, prefix, q, k, v, pos0, n_ctx, inv_f, kcache=None, vcache=None):
    """Runs rope + append + attend for n tokens starting at pos0 (the reference's per-token loop).

    q [n,H,d], k/v [n,Hkv,d] float32 (copied, not modified). kcache/vcache: optional existing
    f32 caches [n_ctx, Hkv*d] holding positions < pos0 (modified in place). Returns out [n,H,d].
    """
    n, H, d = q.shape
    Hkv = k.shape[1]
    q = np.ascontiguousarray(q, dtype=np.float32).copy()
    k = np.ascontiguousarray(k, dtype=np.float32).copy()
    v = np.ascontiguousarray(v, dtype=np.float32)
    if kcache is None:
        kcache = np.zeros((n_ctx, Hkv * d), dtype=np.float32)
        vcache = np.zeros((n_ctx, Hkv * d), dtype=np.float32)
    out = np.empty((n, H, d), dtype=np.float32)
    getattr(lib, prefix + "attn_forward")(q.reshape(-1), k.reshape(-1), v.reshape(-1), kcache.reshape(-1),
                                          vcache.reshape(-1), pos0, n, H, Hkv, d, inv_f, out.reshape(-1))
    return out, q, k, kcache, vcache


def attend_rows(lib, q_rows, kcache, vcache, positions, H, Hkv, d, n_threads=0):
    """oracle_attend_rows: q_rows [r,H,d] f32 (already rotated), caches [n_ctx,Hkv*d] f32."""
    q_rows = np.ascontiguousarray(q_rows, dtype=np.float32)
    positions = np.ascontiguousarray(positions, dtype=np.int32)
    out = np.empty_like(q_rows)
    rc = lib.oracle_attend_rows(q_rows.reshape(-1), kcache.reshape(-1), vcache.reshape(-1), positions,
                                len(positions), H, Hkv, d, out.reshape(-1), n_threads)
    if rc != 0:
        raise MemoryError("oracle_attend_rows")
    return out


# ---- weight formats (quant_oracle.c / ref_dequant) ----
GGML_TYPES = {"F32": 0, "F16": 1, "Q4_0": 2, "Q4_1": 3, "Q8_0": 8, "Q6_K": 14, "BF16": 30}
_u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")


def _declare_quant(lib, prefix):
    fn = getattr(lib, prefix + "dequant")
    fn.argtypes = [C.c_int, _u8p, _f32p, C.c_size_t]
    fn.restype = C.c_int
    return fn


def dequant(lib, prefix, type_name, raw, n):
    """Dequantises `n` elements of ggml type `type_name` from the uint8 array `raw` (reference block layout)."""
    out = np.empty(n, dtype=np.float32)
    rc = _declare_quant(lib, prefix)(GGML_TYPES[type_name], np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1), out, n)
    if rc != 0:
        raise ValueError(f"{prefix}dequant rejects {type_name}")
    return out


def row_bytes(type_name, n):
    block, nbytes = {"F32": (1, 4), "F16": (1, 2), "BF16": (1, 2), "Q4_0": (32, 18), "Q4_1": (32, 20), "Q8_0": (32, 34),
                     "Q6_K": (256, 210)}[type_name]
    return n // block * nbytes


def oracle_matvec(lib, type_name, raw, x, n_in, n_out):
    """float64 row products of the dequantised [n_out][n_in] matrix with x (tolerance reference)."""
    lib.oracle_matvec.argtypes = [C.c_int, _u8p, _f32p, C.c_size_t, C.c_size_t, _f64p, _f32p]
    lib.oracle_matvec.restype = C.c_int
    out = np.empty(n_out, dtype=np.float64)
    rc = lib.oracle_matvec(GGML_TYPES[type_name], np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1),
                           np.ascontiguousarray(x, dtype=np.float32), n_in, n_out, out, np.empty(n_in, dtype=np.float32))
    if rc != 0:
        raise ValueError(f"oracle_matvec rejects {type_name}")
    return out


def random_blocks(type_name, n_rows, n_in, rng, scale=0.02, extreme=False):
    """Random weight rows in the reference's block layout: uint8 [n_rows, row_bytes]. Quants are uniform random
    bits; scales are f16 values of magnitude about `scale` (extreme=True: any finite f16 bit pattern, including
    zero, subnormals and 65504)."""
    rb = row_bytes(type_name, n_in)
    raw = rng.integers(0, 256, size=(n_rows, rb), dtype=np.uint8)
    if type_name in ("F32", "F16", "BF16"):
        vals = rng.standard_normal((n_rows, n_in)).astype(np.float32) * scale
        if type_name == "F32":
            return vals.view(np.uint8).reshape(n_rows, rb)
        if type_name == "F16":
            return vals.astype(np.float16).view(np.uint8).reshape(n_rows, rb)
        return (vals.view(np.uint32) >> 16).astype(np.uint16).view(np.uint8).reshape(n_rows, rb)

    def f16_bits(shape):
        if extreme:
            b = rng.integers(0, 1 << 16, size=shape, dtype=np.uint32).astype(np.uint16)
            return np.where((b & 0x7C00) == 0x7C00, b & 0x83FF, b).astype(np.uint16)  # no inf / nan
        return (np.abs(rng.standard_normal(shape)) * scale + scale / 8).astype(np.float16).view(np.uint16)

    block, nbytes = {"Q4_0": (32, 18), "Q4_1": (32, 20), "Q8_0": (32, 34), "Q6_K": (256, 210)}[type_name]
    nb = n_in // block
    blocks = raw.reshape(n_rows, nb, nbytes)
    if type_name == "Q6_K":
        blocks[:, :, 208:210] = (f16_bits((n_rows, nb)) if extreme else
                                 (np.abs(rng.standard_normal((n_rows, nb))) * scale / 1000 + scale / 4000).astype(np.float16).view(np.uint16)
                                 ).view(np.uint8).reshape(n_rows, nb, 2)
    else:
        blocks[:, :, 0:2] = f16_bits((n_rows, nb)).view(np.uint8).reshape(n_rows, nb, 2)
        if type_name == "Q4_1":
            blocks[:, :, 2:4] = f16_bits((n_rows, nb)).view(np.uint8).reshape(n_rows, nb, 2)
    return blocks.reshape(n_rows, rb)
