"""End to end: the CUDA backend behind the reference's own engine glue against the reference CpuBackend.

A seeded random-init Llama-3.2-3B-shaped F16 GGUF is generated on the machine, 128 uniformly drawn
token ids are prefilled and 32 tokens are decoded greedily through make_backend / prefill / Sampler
(src/engine.cpp, src/sampler.cpp) on both backends; the token lists must be identical.
The one-batch case runs the full 28-layer, 128256-token model (a 6.4 GB file written under /tmp or
INGOT_E2E_DIR; about 100 s on a B200 host; INGOT_E2E_SMALL=1 swaps in the small model). The chunked-prefill
case (n_batch 48) and the error checks use 2 layers and a 32064-token vocabulary (seconds).
"""
import ctypes as C
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENGINE = os.path.join(ROOT, "inference-agent_b200", "backend", "_build", "libingot_engine_cuda.so")


def _engine():
    if not os.path.exists(ENGINE):
        pytest.skip("libingot_engine_cuda.so not built (needs a reference checkout at build time)")
    lib = C.CDLL(ENGINE)
    i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
    f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
    lib.ingot_e2e_greedy.argtypes = [C.c_char_p, C.c_char_p, i32p, C.c_int, C.c_int, C.c_int, i32p, f32p]
    lib.ingot_e2e_greedy.restype = C.c_int
    lib.ingot_e2e_last_error.restype = C.c_char_p
    return lib


def _model(tmp_dir, full=False, wtype="F16", output_type=None):
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_random_gguf
    full = full and os.environ.get("INGOT_E2E_SMALL") != "1"
    n_layer, n_vocab = (28, 128256) if full else (2, 32064)
    tag = "" if wtype == "F16" else f"_{wtype}_{output_type or wtype}"
    path = os.path.join(tmp_dir, f"ingot_random_l{n_layer}_v{n_vocab}_s0{tag}.gguf")
    if not os.path.exists(path):
        make_random_gguf.write(path + ".tmp", n_layer, n_vocab, seed=0, wtype=wtype, output_type=output_type)
        os.replace(path + ".tmp", path)
    return path, n_vocab


def _greedy(lib, path, backend, prompt, n_gen, n_batch):
    ids = np.zeros(n_gen, dtype=np.int32)
    margin = np.zeros(n_gen, dtype=np.float32)
    rc = lib.ingot_e2e_greedy(path.encode(), backend, prompt, len(prompt), n_gen, n_batch, ids, margin)
    assert rc == 0, lib.ingot_e2e_last_error().decode()
    return ids, margin


@pytest.mark.parametrize("full,n_batch", [(True, 512), (False, 48)])
def test_greedy_tokens_match_cpu_reference(full, n_batch):
    lib = _engine()
    path, n_vocab = _model(os.environ.get("INGOT_E2E_DIR", "/tmp"), full)
    prompt = np.random.default_rng(0).integers(0, n_vocab, size=128).astype(np.int32)
    want, want_margin = _greedy(lib, path, b"cpu", prompt, 32, n_batch)
    got, got_margin = _greedy(lib, path, b"metal", prompt, 32, n_batch)  # "metal" = the GPU backend of this build
    first_bad = next((i for i in range(32) if want[i] != got[i]), None)
    detail = "" if first_bad is None else (f"first mismatch at step {first_bad}: cpu {want[first_bad]} (top-2 margin "
                                           f"{want_margin[first_bad]:.3e}) vs cuda {got[first_bad]} (margin {got_margin[first_bad]:.3e})")
    assert first_bad is None, detail
    print(f"\n32 greedy tokens identical (n_batch={n_batch}); smallest reference top-2 margin {want_margin.min():.3e}")


@pytest.mark.parametrize("wtype,output_type,n_batch,resident_planes", [
    ("Q8_0", None, 512, True),     # one 128-token batch: resident hi/lo planes through the tensor-core GEMM
    ("Q4_0", "Q6_K", 512, True),   # what llama.cpp's Q4_0 files look like: Q6_K embedding / output matrix
    ("Q4_1", None, 512, True),     # no streaming kernel for this format: the unfused single-token path
    ("Q8_0", None, 48, False),     # chunked prefill, hi/lo planes rebuilt in scratch per use
    ("Q4_0", "Q6_K", 5, True),     # chunks below the tensor-core minimum: the f32 fallback
])
def test_greedy_tokens_match_cpu_reference_quantised(wtype, output_type, n_batch, resident_planes, monkeypatch):
    """The same check on block-quantised GGUFs (2 layers, 32064 tokens): weights stay quantised on the device,
    single tokens go through the weight-streaming (Q8_0, Q4_0) or dequantise-in-GEMV kernels, batches through the
    hi/lo tensor-core path."""
    if not resident_planes:
        monkeypatch.setenv("INGOT_QUANT_PLANES", "0")
    lib = _engine()
    path, n_vocab = _model(os.environ.get("INGOT_E2E_DIR", "/tmp"), False, wtype, output_type)
    prompt = np.random.default_rng(0).integers(0, n_vocab, size=128).astype(np.int32)
    want, want_margin = _greedy(lib, path, b"cpu", prompt, 32, n_batch)
    got, got_margin = _greedy(lib, path, b"metal", prompt, 32, n_batch)
    first_bad = next((i for i in range(32) if want[i] != got[i]), None)
    detail = "" if first_bad is None else (f"first mismatch at step {first_bad}: cpu {want[first_bad]} (top-2 margin "
                                           f"{want_margin[first_bad]:.3e}) vs cuda {got[first_bad]} (margin {got_margin[first_bad]:.3e})")
    assert first_bad is None, detail
    assert len(set(want.tolist())) > 8  # the random model does not collapse onto one token
    print(f"\n{wtype}: 32 greedy tokens identical (n_batch={n_batch}); smallest reference top-2 margin {want_margin.min():.3e}")


@pytest.mark.parametrize("n_seq,wtype", [(5, "F16"), (24, "F16"), (5, "Q8_0")])
def test_batched_forward_multi_matches_single_sequence_reference(n_seq, wtype):
    """The batched extension (BatchedBackend::forward_multi on the paged cache): n_seq sequences with prompts of
    different lengths are prefilled and decoded together, each contributing one token per step, and every
    sequence must produce exactly the tokens the reference CpuBackend produces when it runs that sequence alone.
    24 sequences take the batched projections through the tensor-core kernels, 5 through the f32 ones."""
    lib = _engine()
    i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
    lib.ingot_e2e_multi_greedy.argtypes = [C.c_char_p, i32p, i32p, C.c_int, C.c_int, C.c_int, i32p]
    lib.ingot_e2e_multi_greedy.restype = C.c_int
    path, n_vocab = _model(os.environ.get("INGOT_E2E_DIR", "/tmp"), False, wtype)
    rng = np.random.default_rng(100 + n_seq)
    lens = rng.integers(3, 40, size=n_seq).astype(np.int32)
    prompts = [rng.integers(0, n_vocab, size=int(n)).astype(np.int32) for n in lens]
    n_gen = 12
    got = np.zeros((n_seq, n_gen), dtype=np.int32)
    rc = lib.ingot_e2e_multi_greedy(path.encode(), np.concatenate(prompts), lens, n_seq, n_gen, 64, got)
    assert rc == 0, lib.ingot_e2e_last_error().decode()
    for s in range(min(n_seq, 8)):  # the CPU reference is slow: the first eight sequences
        want, margin = _greedy(lib, path, b"cpu", prompts[s], n_gen, 512)
        assert np.array_equal(got[s], want), f"sequence {s} (prompt {lens[s]} tokens): batched {got[s]} vs reference {want}; margins {margin}"


def test_abench_and_bwtest_verbs():
    """The reference's diagnostics verbs through the link seam: `abench` (seconds per token of decode attention over
    all layers, bytes by the formula of src/main.cpp:446) and `bwtest` (read-bandwidth table)."""
    lib = _engine()
    path, _ = _model(os.environ.get("INGOT_E2E_DIR", "/tmp"))
    lib.ingot_e2e_abench.argtypes = [C.c_char_p, C.c_int, C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double)]
    secs, nbytes = C.c_double(0), C.c_double(0)
    assert lib.ingot_e2e_abench(path.encode(), 4095, 10, C.byref(secs), C.byref(nbytes)) == 0, lib.ingot_e2e_last_error()
    assert nbytes.value == 2.0 * 2 * 4096 * 8 * 128 * 2  # the 2-layer test model
    gbs = nbytes.value / secs.value / 1e9
    assert 100.0 < gbs < 20000.0, gbs  # a GPU-speed figure, not a CPU one and not a nonsense one
    lib.ingot_e2e_bwtest.argtypes = [C.c_char_p, C.c_double]
    assert lib.ingot_e2e_bwtest(path.encode(), 300.0) == 0, lib.ingot_e2e_last_error()


def test_backend_errors_match_reference():
    lib = _engine()
    path, n_vocab = _model(os.environ.get("INGOT_E2E_DIR", "/tmp"))
    ids = np.zeros(1, dtype=np.int32)
    m = np.zeros(1, dtype=np.float32)
    bad = np.array([n_vocab + 5], dtype=np.int32)
    for backend in (b"cpu", b"metal"):
        assert lib.ingot_e2e_greedy(path.encode(), backend, bad, 1, 1, 512, ids, m) == -1
        assert lib.ingot_e2e_last_error() == b"token id out of range"
    assert lib.ingot_e2e_greedy(path.encode(), b"nope", bad, 1, 1, 512, ids, m) == -1
    assert b"unknown backend" in lib.ingot_e2e_last_error()
