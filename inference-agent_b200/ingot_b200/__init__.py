"""Python harness over libingot_cuda.so (the C ABI declared in include/ingot_cuda.h).

Used by the tests and bench.py. torch supplies device memory and streams only: every compute
call goes through the C ABI with raw device pointers. There is no fallback: importing this
module raises if the CUDA library has not been built.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# INGOT_CUDA_LIB points at another build of the same library (e.g. one compiled with different tuning macros).
LIB_PATH = os.environ.get("INGOT_CUDA_LIB") or os.path.join(os.path.dirname(_HERE), "libingot_cuda.so")

F32, F16, BF16 = 0, 1, 2
KV_CONTIGUOUS, KV_PAGED = 0, 1
BLOCK_TOKENS = 16
HEAD_DIM = 128

# name -> (restype, argtypes); every symbol include/ingot_cuda.h declares.
_P, _I, _SZ = C.c_void_p, C.c_int, C.c_size_t
ABI = {
    "ingot_status_string": (C.c_char_p, [_I]),
    "ingot_last_error": (C.c_char_p, []),
    "ingot_build_arch": (C.c_char_p, []),
    "ingot_build_flags": (C.c_char_p, []),
    "ingot_kv_create": (_I, [C.POINTER(_P), _I, _I, _I, _I, _I, _I]),
    "ingot_kv_destroy": (None, [_P]),
    "ingot_kv_k_dev": (_P, [_P, _I]),
    "ingot_kv_v_dev": (_P, [_P, _I]),
    "ingot_kv_layer_bytes": (_SZ, [_P]),
    "ingot_kv_status": (_I, [_P, _P, C.POINTER(_I)]),
    "ingot_kv_test_stall_prefill": (_I, [_P, _I]),
    "ingot_kv_test_shrink_extent": (_I, [_P, _SZ]),
    "ingot_rope_kv_append": (_I, [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P, _P, _I, _P]),
    "ingot_kv_import_f16": (_I, [_P, _I, _P, _P, _I, _I, _P, _P]),
    "ingot_attn_decode": (_I, [_P, _I, _P, _I, _P, _I, _I, _I, _P, _I, _P, _I, _I, _P]),
    "ingot_attn_decode_layers": (_I, [_P, _I, _I, _P, _I, _P, _I, _I, _I, _P, _I, _P, _I, _I, _P]),
    "ingot_attn_decode_noalloc": (_I, [_P, _P, _I, _I, _P, _I, _P, _I, _I, _I, _I, _P]),
    "ingot_attn_prefill": (_I, [_P, _I, _P, _I, _P, _I, _I, _I, _I, _P, _I, _P]),
    "ingot_attn_prefill_gather": (_I, [_P, _I, _P, _I, C.POINTER(_P), _I, _I, _I, _I, _I, _I, _I, _P]),
    "ingot_attn_prefill_gather_signal": (_I, [_P, _I, _P, _I, C.POINTER(_P), C.POINTER(_P), _I, _I, _I, _I, _I, _I, _I, _I, _P]),
    "ingot_gather_wait": (_I, [_P, _P, _I, _I, _P]),
    "ingot_mg_create": (_I, [C.POINTER(_P), _I, _I, _I, _I, _I, _I]),
    "ingot_mg_destroy": (None, [_P]),
    "ingot_mg_kv": (_P, [_P, _I]),
    "ingot_mg_out": (_P, [_P, _I]),
    "ingot_mg_stream": (_P, [_P, _I]),
    "ingot_mg_prefill": (_I, [_P, _I, C.POINTER(_P), _I, _I, _I, _I]),
    "ingot_lpt_assign": (_I, [C.POINTER(C.c_int32), _I, _I, C.POINTER(C.c_int32)]),
    "ingot_rope_append_decode": (_I, [_P, _I, _P, _P, _P, _P, _P, _I, _I, _P, _I, _I, _P]),
    "ingot_attn_prefill_host": (_I, [_P, _I, _P, _I, _P, _I, _I, _I, _I, _P, _I, _P]),
    "ingot_attn_layer_host": (_I, [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "ingot_attn_layers_host": (_I, [_P, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "ingot_stream_sync": (_I, [_P]),
    "ingot_hbm_read_probe": (_I, [_SZ, _I, C.POINTER(C.c_double), _P]),
}


# Canary-padded device allocations for the tests (INGOT_TEST_CANARY=1): every tensor this module allocates for a
# caller - and every input the test helpers upload - sits between two guard zones filled with a byte pattern;
# check_guards() verifies that no kernel wrote into them. A stand-in for a memory checker on the output side.
_CANARY = os.environ.get("INGOT_TEST_CANARY") == "1"
_GUARD_ELEMS = 256
_GUARD_BYTE = 0xA5
_guards = []


def guarded_empty(shape, dtype, device="cuda"):
    import torch
    if not _CANARY:
        return torch.empty(shape, dtype=dtype, device=device)
    n = 1
    for d in shape:
        n *= int(d)
    base = torch.empty(n + 2 * _GUARD_ELEMS, dtype=dtype, device=device)
    raw = base.view(torch.uint8)
    g = _GUARD_ELEMS * base.element_size()
    raw[:g] = _GUARD_BYTE
    raw[raw.numel() - g:] = _GUARD_BYTE
    _guards.append(base)
    return base[_GUARD_ELEMS:_GUARD_ELEMS + n].view(tuple(int(d) for d in shape))


def check_guards():
    """Number of guarded allocations whose guard zones were written to since the last call (0 = clean)."""
    import torch
    bad = 0
    for base in _guards:
        raw = base.view(torch.uint8)
        g = _GUARD_ELEMS * base.element_size()
        if not (bool((raw[:g] == _GUARD_BYTE).all()) and bool((raw[raw.numel() - g:] == _GUARD_BYTE).all())):
            bad += 1
    _guards.clear()
    return bad


class IngotError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"ingot status {status}: {message}")
        self.status = status


def load_library(path=LIB_PATH):
    if not os.path.exists(path):
        raise FileNotFoundError(
            f"{path} not found: build it with `make -C inference-agent_b200` or __graft_entry__.build(); "
            "there is no CPU fallback")
    lib = C.CDLL(path)
    for name, (res, args) in ABI.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = load_library()
    return _lib


def _check(status):
    if status != 0:
        raise IngotError(status, lib().ingot_last_error().decode() or lib().ingot_status_string(status).decode())


def _dtype_code(t):
    import torch
    return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[t.dtype]


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class KVCache:
    """Owns an ingot_kv handle on the current CUDA device."""

    def __init__(self, layout, n_layer, n_head_kv, capacity, max_seqs=1, head_dim=HEAD_DIM):
        self.layout, self.n_layer, self.n_head_kv, self.capacity, self.max_seqs = layout, n_layer, n_head_kv, capacity, max_seqs
        h = C.c_void_p()
        _check(lib().ingot_kv_create(C.byref(h), layout, n_layer, n_head_kv, head_dim, capacity, max_seqs))
        self.handle = h

    def close(self):
        if self.handle:
            lib().ingot_kv_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def layer_view(self, layer, which="k"):
        """torch view of one layer's K or V storage in its native layout (no copy)."""
        import torch
        fn = lib().ingot_kv_k_dev if which == "k" else lib().ingot_kv_v_dev
        ptr = fn(self.handle, layer)
        if self.layout == KV_CONTIGUOUS:
            shape = (self.n_head_kv, self.capacity, HEAD_DIM)
        else:
            shape = (self.capacity, self.n_head_kv, BLOCK_TOKENS, HEAD_DIM)

        class _DeviceArray:  # wraps the raw device pointer for torch through the CUDA array interface
            __cuda_array_interface__ = {"shape": shape, "typestr": "<f2", "data": (ptr, False), "version": 2}

        return torch.as_tensor(_DeviceArray(), device=torch.device("cuda", torch.cuda.current_device()))

    def status(self):
        out = C.c_int(0)
        _check(lib().ingot_kv_status(self.handle, _stream(), C.byref(out)))
        return out.value

    def import_f16(self, layer, k, v, pos0, block_table=None):
        """k, v: [n_tok, n_head_kv, 128] f16 cuda tensors."""
        assert k.is_contiguous() and v.is_contiguous() and _dtype_code(k) == F16 and _dtype_code(v) == F16
        _check(lib().ingot_kv_import_f16(self.handle, layer, _ptr(k), _ptr(v), pos0, k.shape[0], _ptr(block_table), _stream()))


def rope_kv_append(kv, layer, q, k, v, inv_freq, pos0=0, positions=None, seq_ids=None, block_tables=None):
    """q [n,H,128] f32 or None; k, v [n,Hkv,128] f32. Returns rotated q as f16 (or None)."""
    import torch
    n_tok = k.shape[0]
    q_out = None
    n_head = kv.n_head_kv
    if q is not None:
        assert q.is_contiguous() and q.dtype == torch.float32
        n_head = q.shape[1]
        q_out = guarded_empty(q.shape, torch.float16, q.device)
    assert k.is_contiguous() and v.is_contiguous() and k.dtype == torch.float32 and v.dtype == torch.float32
    mb = 0 if block_tables is None else block_tables.shape[-1]
    _check(lib().ingot_rope_kv_append(kv.handle, layer, _ptr(q), _ptr(q_out), _ptr(k), _ptr(v), _ptr(inv_freq), n_head,
                                      pos0, n_tok, _ptr(positions), _ptr(seq_ids), _ptr(block_tables), mb, _stream()))
    return q_out


def attn_decode(kv, layer, q, out=None, out_dtype=None, seq_lens=None, max_seq_len=None, block_tables=None,
                chunk_keys=0):
    """q [n_seq,H,128]; returns out [n_seq,H,128] (f32 unless out_dtype given)."""
    import torch
    assert q.is_contiguous()
    n_seq, n_head = q.shape[0], q.shape[1]
    if out is None:
        out = guarded_empty(q.shape, out_dtype or torch.float32, q.device)
    mb = 0 if block_tables is None else block_tables.shape[-1]
    _check(lib().ingot_attn_decode(kv.handle, layer, _ptr(q), _dtype_code(q), _ptr(out), _dtype_code(out), n_head, n_seq,
                                   _ptr(seq_lens), int(max_seq_len), _ptr(block_tables), mb, chunk_keys, _stream()))
    return out


def attn_decode_layers(kv, layer_begin, q, out, seq_lens=None, max_seq_len=None, block_tables=None, chunk_keys=0):
    """q, out [n_layers, n_seq, H, 128]: decode attention of consecutive layers in one call."""
    assert q.is_contiguous() and out.is_contiguous()
    n_layers, n_seq, n_head = q.shape[0], q.shape[1], q.shape[2]
    mb = 0 if block_tables is None else block_tables.shape[-1]
    _check(lib().ingot_attn_decode_layers(kv.handle, layer_begin, n_layers, _ptr(q), _dtype_code(q), _ptr(out),
                                          _dtype_code(out), n_head, n_seq, _ptr(seq_lens), int(max_seq_len),
                                          _ptr(block_tables), mb, chunk_keys, _stream()))
    return out


def attn_prefill(kv, layer, q, q_pos0, out=None, out_dtype=None, block_table=None, impl=0):
    """q [n_tok,H,128]; returns out [n_tok,H,128]."""
    import torch
    assert q.is_contiguous()
    n_tok, n_head = q.shape[0], q.shape[1]
    if out is None:
        out = guarded_empty(q.shape, out_dtype or torch.float32, q.device)
    _check(lib().ingot_attn_prefill(kv.handle, layer, _ptr(q), _dtype_code(q), _ptr(out), _dtype_code(out), n_head,
                                    q_pos0, n_tok, _ptr(block_table), impl, _stream()))
    return out


def attn_prefill_gather(kv, layer, q, q_pos0, out_ptrs, out_dtype_code, out_n_head, out_head0):
    """q [n_tok,H_local,128]; out_ptrs: device addresses (ints) of the destination buffers [n_tok,out_n_head,128]."""
    assert q.is_contiguous()
    arr = (C.c_void_p * len(out_ptrs))(*[C.c_void_p(int(x)) for x in out_ptrs])
    _check(lib().ingot_attn_prefill_gather(kv.handle, layer, _ptr(q), _dtype_code(q), arr, len(out_ptrs), out_dtype_code,
                                           q.shape[1], out_n_head, out_head0, q_pos0, q.shape[0], _stream()))


def attn_prefill_gather_signal(kv, layer, q, q_pos0, out_ptrs, signal_ptrs, src_index, out_dtype_code, out_n_head, out_head0):
    """attn_prefill_gather plus one completion signal per destination (counter src_index of each array in signal_ptrs)."""
    assert q.is_contiguous() and len(out_ptrs) == len(signal_ptrs)
    arr = (C.c_void_p * len(out_ptrs))(*[C.c_void_p(int(x)) for x in out_ptrs])
    sig = (C.c_void_p * len(signal_ptrs))(*[C.c_void_p(int(x)) for x in signal_ptrs])
    _check(lib().ingot_attn_prefill_gather_signal(kv.handle, layer, _ptr(q), _dtype_code(q), arr, sig, len(out_ptrs), src_index,
                                                  out_dtype_code, q.shape[1], out_n_head, out_head0, q_pos0, q.shape[0], _stream()))


def gather_wait(kv, counters, n_src, timeout_ms=2000):
    """Queues the bounded wait for n_src completion signals on this GPU's counter array (an int32 cuda tensor)."""
    _check(lib().ingot_gather_wait(kv.handle, _ptr(counters), n_src, timeout_ms, _stream()))


def rope_append_decode(kv, layer, q, k, v, inv_freq, pos, out=None, out_dtype=None, key_count=None, max_seq_len=0):
    """One token: q [H,128], k, v [Hkv,128] f32 projections (cuda). RoPE, append at `pos`, attention over keys 0..pos in one
    launch. key_count: optional int32 cuda tensor holding pos + 1 (then max_seq_len bounds it)."""
    import torch
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous() and q.dtype == torch.float32
    if out is None:
        out = guarded_empty(q.shape, out_dtype or torch.float32, q.device)
    _check(lib().ingot_rope_append_decode(kv.handle, layer, _ptr(q), _ptr(k), _ptr(v), _ptr(inv_freq), _ptr(out), _dtype_code(out),
                                          q.shape[0], _ptr(key_count), pos, max_seq_len, _stream()))
    return out


def attn_prefill_host(kv, layer, q_host, q_pos0, out_host, block_table=None, chunk_tokens=0):
    """q_host, out_host [n_tok,H,128]: (pinned) host tensors; the cache holds the keys already. Copies in, attention and
    copies out are pipelined chunk by chunk; asynchronous on the current stream."""
    assert q_host.is_contiguous() and out_host.is_contiguous() and not q_host.is_cuda and not out_host.is_cuda
    n_tok, n_head = q_host.shape[0], q_host.shape[1]
    _check(lib().ingot_attn_prefill_host(kv.handle, layer, _ptr(q_host), _dtype_code(q_host), _ptr(out_host), _dtype_code(out_host),
                                         n_head, q_pos0, n_tok, _ptr(block_table), chunk_tokens, _stream()))


def attn_layer_host(kv, layer, q_host, k_host, v_host, out_host, inv_freq_dev, pos0):
    """Pinned host tensors in/out; asynchronous on the current stream."""
    n_tok, n_head = q_host.shape[0], q_host.shape[1]
    _check(lib().ingot_attn_layer_host(kv.handle, layer, _ptr(q_host), _ptr(k_host), _ptr(v_host), _ptr(out_host),
                                       _ptr(inv_freq_dev), n_head, pos0, n_tok, _stream()))


def attn_layers_host(kv, layer_begin, q_host, k_host, v_host, out_host, inv_freq_dev, pos0):
    """q_host [L,n_tok,H,128], k/v_host [L,n_tok,Hkv,128], out_host like q_host: pinned host tensors."""
    n_layers, n_tok, n_head = q_host.shape[0], q_host.shape[1], q_host.shape[2]
    _check(lib().ingot_attn_layers_host(kv.handle, layer_begin, n_layers, _ptr(q_host), _ptr(k_host), _ptr(v_host),
                                        _ptr(out_host), _ptr(inv_freq_dev), n_head, pos0, n_tok, _stream()))


def hbm_read_probe(n_bytes, reps=5):
    """GB/s of a read-only sweep over n_bytes of device memory (best of reps)."""
    best = C.c_double(0.0)
    _check(lib().ingot_hbm_read_probe(n_bytes, reps, C.byref(best), _stream()))
    return n_bytes / best.value / 1e9
