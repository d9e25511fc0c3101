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
    lib.ref_e2e_greedy.argtypes = [C.c_char_p, _i32p, C.c_int, C.c_int, C.c_int, _i32p, C.c_void_p]
    lib.ref_e2e_greedy.restype = C.c_int
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
