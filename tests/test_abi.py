"""The C-ABI library loads without a GPU and exports every symbol include/ingot_cuda.h declares."""
import ctypes as C
import os
import re

import pytest

import ingot_b200 as ib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ingot_cuda.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ingot_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for must in ("ingot_kv_create", "ingot_rope_kv_append", "ingot_attn_decode", "ingot_attn_prefill",
                 "ingot_attn_decode_layers", "ingot_attn_layers_host", "ingot_attn_decode_noalloc"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(ib.LIB_PATH)
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, missing


def test_python_binding_table_matches_header():
    assert sorted(ib.ABI) == declared_functions()


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(FileNotFoundError, match="no CPU fallback"):
        ib.load_library(str(tmp_path / "libingot_cuda.so"))


def test_argument_errors_need_no_gpu():
    """Null handles and bad ranges are rejected on the host before any CUDA call."""
    lib = ib.lib()
    assert lib.ingot_build_arch() == b"sm_100a"
    assert lib.ingot_status_string(0) == b"ok"
    rc = lib.ingot_attn_decode(None, 0, None, 0, None, 0, 24, 1, None, 16, None, 0, 0, None)
    assert rc == 1 and b"kv is null" in lib.ingot_last_error()
    rc = lib.ingot_attn_prefill(None, 0, None, 0, None, 0, 24, 0, 16, None, 0, None)
    assert rc == 1
    rc = lib.ingot_rope_kv_append(None, 0, None, None, None, None, None, 24, 0, 1, None, None, None, 0, None)
    assert rc == 1
    h = C.c_void_p()
    assert lib.ingot_kv_create(C.byref(h), 7, 1, 8, 128, 16, 1) == 1          # bad layout
    assert lib.ingot_kv_create(C.byref(h), 0, 1, 8, 64, 16, 1) == 3           # head_dim != 128: unsupported
    assert lib.ingot_attn_decode_noalloc(None, None, 1, 1, None, 0, None, 0, 1, 1, 0, None) == 1
    lib.ingot_kv_destroy(None)  # no-op


def test_lpt_assign_in_the_library_matches_the_python_one():
    """ingot_lpt_assign is pure host code: the C assignment equals workloads.lpt_assign for the configs[3] lengths."""
    import ctypes as C
    import numpy as np
    import ingot_b200 as ib
    from ingot_b200 import workloads as W
    lens = W.c4_lengths()
    for n in (1, 2, 4, 8):
        got = np.zeros(len(lens), dtype=np.int32)
        rc = ib.lib().ingot_lpt_assign(lens.ctypes.data_as(C.POINTER(C.c_int32)), len(lens), n, got.ctypes.data_as(C.POINTER(C.c_int32)))
        assert rc == 0
        want = np.zeros(len(lens), dtype=np.int32)
        for r, idx in enumerate(W.lpt_assign(lens, n)):
            want[idx] = r
        assert np.array_equal(got, want)
