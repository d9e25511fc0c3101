"""BatchScheduler (backend/batch_scheduler.h) on the CPU: continuous batching over BatchedBackend must give every
request exactly the reply the reference's single-sequence loop gives it when it runs alone.

The scheduler is host code, so it is checked here without a GPU: make_batched_backend("cpu") puts one reference
CpuBackend behind each sequence slot, and the expected replies come from the reference's own glue (make_backend,
prefill, Sampler) through ingot_e2e_greedy on the same backend. The model is a seeded random-init GGUF small enough
for seconds of CPU time. The last test runs the same entry point on the CUDA backend.
"""
import ctypes as C
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENGINE = os.path.join(ROOT, "inference-agent_b200", "backend", "_build", "libingot_engine_cuda.so")
i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
N_VOCAB = 1000


def engine():
    if not os.path.exists(ENGINE):
        pytest.skip("libingot_engine_cuda.so not built (needs a reference checkout at build time)")
    lib = C.CDLL(ENGINE)
    lib.ingot_e2e_greedy.argtypes = [C.c_char_p, C.c_char_p, i32p, C.c_int, C.c_int, C.c_int, i32p, f32p]
    lib.ingot_e2e_sched_greedy.argtypes = [C.c_char_p, C.c_char_p, i32p, i32p, i32p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                           C.c_int, i32p, C.c_int, i32p, i32p, C.c_void_p, C.c_void_p]
    lib.ingot_e2e_generate.argtypes = [C.c_char_p, C.c_char_p, i32p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, i32p]
    lib.ingot_e2e_last_error.restype = C.c_char_p
    return lib


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_random_gguf
    path = str(tmp_path_factory.mktemp("sched") / "tiny.gguf")
    make_random_gguf.write(path, n_layer=2, n_vocab=N_VOCAB, seed=3, n_embd=256, n_head=2, n_head_kv=1, n_ff=512, n_ctx=256)
    return path


def alone(lib, path, prompt, n_gen):
    """The reply of one request run by itself through the reference's loop (greedy, no stop token)."""
    ids, margin = np.zeros(n_gen, dtype=np.int32), np.zeros(n_gen, dtype=np.float32)
    assert lib.ingot_e2e_greedy(path.encode(), b"cpu", prompt, len(prompt), n_gen, 512, ids, margin) == 0, lib.ingot_e2e_last_error()
    return ids


def _sampling(params):
    """{temperature, top_k, top_p, repeat_penalty, repeat_last_n, seed} as the C entries take it (None: greedy)."""
    return None if params is None else np.asarray(params, dtype=np.float64)


def served_alone(lib, path, prompt, max_tokens, sampling, stop_token):
    """The reply of one request through the reference server's loop (prefill, Sampler over prompt + reply, stop token)."""
    ids = np.zeros(max_tokens, dtype=np.int32)
    sp = _sampling(sampling)
    n = lib.ingot_e2e_generate(path.encode(), b"cpu", prompt, len(prompt), max_tokens, 512, None if sp is None else sp.ctypes.data,
                               stop_token, ids)
    assert n >= 0, lib.ingot_e2e_last_error()
    return ids[:n]


def scheduled(lib, path, prompts, max_tokens, arrivals, max_seqs, n_ctx, stop_token, backend=b"cpu", sampling=None):
    """max_tokens[r] = -(k + 1): request r has no limit of its own and is cancelled before step k."""
    sp = _sampling(sampling)
    n = len(prompts)
    lens = np.array([len(p) for p in prompts], dtype=np.int32)
    max_out = n_ctx if min(max_tokens) < 0 else int(max(max_tokens))
    out = np.full((n, max_out), -1, dtype=np.int32)
    counts, finish = np.zeros(n, dtype=np.int32), np.zeros(n, dtype=np.int32)
    stats = (C.c_longlong * 2)()
    arr = None if arrivals is None else np.ascontiguousarray(arrivals, dtype=np.int32)
    rc = lib.ingot_e2e_sched_greedy(path.encode(), backend, np.concatenate(prompts).astype(np.int32), lens,
                                    np.asarray(max_tokens, dtype=np.int32), None if arr is None else arr.ctypes.data, n, max_seqs, n_ctx,
                                    stop_token, out, max_out, counts, finish, C.cast(stats, C.c_void_p),
                                    None if sp is None else sp.ctypes.data)
    return rc, out, counts, finish, (stats[0], stats[1])


def test_replies_equal_the_single_sequence_loop_with_arrivals_stops_and_slot_reuse(model):
    lib = engine()
    rng = np.random.default_rng(11)
    n_req, max_seqs = 7, 3
    prompts = [rng.integers(0, N_VOCAB, size=int(n)).astype(np.int32) for n in rng.integers(1, 24, size=n_req)]
    prompts[2] = prompts[2][:1]  # a one-token prompt: its first step is sampled at once
    max_tokens = np.array([9, 4, 12, 1, 7, 10, 6], dtype=np.int32)
    arrivals = np.array([0, 0, 0, 0, 5, 9, 40], dtype=np.int32)  # four at the start for three slots, the rest later
    want = [alone(lib, model, p, int(m)) for p, m in zip(prompts, max_tokens)]
    # a stop token that cuts request 0 short (its 6th token); other requests stop wherever that token turns up in their own reply
    stop = int(want[0][5])
    expect, reason = [], []
    for w in want:
        hit = np.flatnonzero(w == stop)
        expect.append(w[:hit[0]] if len(hit) else w)
        reason.append(1 if len(hit) else 0)
    assert reason[0] == 1 and len(expect[0]) <= 5

    rc, out, counts, finish, (steps, rows) = scheduled(lib, model, prompts, max_tokens, arrivals, max_seqs, 64, stop)
    assert rc == 0, lib.ingot_e2e_last_error()
    for r in range(n_req):
        assert counts[r] == len(expect[r]) and np.array_equal(out[r, :counts[r]], expect[r]), (r, out[r], expect[r])
        assert finish[r] == reason[r], (r, finish[r], reason[r])
    # every request costs its prompt plus the reply tokens that were fed back: a reply that ends on its limit never feeds its
    # last token, one that ends on the stop token fed all of its tokens
    fed = sum(len(p) + len(e) - (0 if s else 1) for p, e, s in zip(prompts, expect, reason))
    assert rows == fed
    assert steps < rows  # steps were shared (three slots busy for most of the run)
    assert steps >= -(-rows // max_seqs)

    # the same requests all at once on a backend with a slot for each: same replies
    rc, out2, counts2, finish2, _ = scheduled(lib, model, prompts, max_tokens, None, n_req, 64, stop)
    assert rc == 0 and np.array_equal(counts2, counts) and np.array_equal(finish2, finish)
    assert all(np.array_equal(out2[r, :counts[r]], out[r, :counts[r]]) for r in range(n_req))


def test_limits_follow_the_reference_server(model):
    lib = engine()
    rng = np.random.default_rng(12)
    # context of 16 positions: a 10-token prompt may generate at most 16 - 10 - 1 = 5 tokens (src/server.cpp:140)
    p = rng.integers(0, N_VOCAB, size=10).astype(np.int32)
    rc, out, counts, finish, _ = scheduled(lib, model, [p], [50], None, 2, 16, -1)
    assert rc == 0 and counts[0] == 5 and finish[0] == 0
    assert np.array_equal(out[0, :5], alone(lib, model, p, 5))
    # a prompt that leaves no room is refused with the server's message (src/server.cpp:139)
    rc, *_ = scheduled(lib, model, [rng.integers(0, N_VOCAB, size=15).astype(np.int32)], [4], None, 2, 16, -1)
    assert rc == -1 and lib.ingot_e2e_last_error() == b"prompt is 15 tokens, context is 16"
    # a bad token id is refused when the request is submitted, before it can spoil a shared step
    rc, *_ = scheduled(lib, model, [np.array([5, N_VOCAB + 7], dtype=np.int32)], [4], None, 2, 16, -1)
    assert rc == -1 and lib.ingot_e2e_last_error() == b"token id out of range"
    # max_tokens 0: finished at once with an empty reply
    rc, out, counts, finish, (steps, rows) = scheduled(lib, model, [p, p], [0, 3], None, 2, 64, -1)
    assert rc == 0 and counts[0] == 0 and finish[0] == 0 and counts[1] == 3
    assert rows == len(p) + 2 and steps == rows  # only the second request ever reached the backend


@pytest.mark.parametrize("sampling", [
    (0.0, 40, 0.95, 1.5, 8, 7),     # greedy with a repetition penalty over the last 8 tokens of prompt + reply
    (0.9, 20, 0.9, 1.2, 64, 1234),  # temperature, top-k, top-p, penalty: every request seeds its own generator
])
def test_sampling_and_repetition_penalty_follow_the_reference_server_loop(model, sampling):
    """The sampler sees what the server's sees: this request's prompt + reply as history, its own seeded generator."""
    lib = engine()
    rng = np.random.default_rng(14)
    prompts = [rng.integers(0, 40, size=int(n)).astype(np.int32) for n in (5, 17, 2, 9)]  # a small alphabet: repeats happen
    max_tokens = [10, 6, 12, 8]
    stop = 3
    want = [served_alone(lib, model, p, m, sampling, stop) for p, m in zip(prompts, max_tokens)]
    rc, out, counts, finish, _ = scheduled(lib, model, prompts, max_tokens, [0, 0, 2, 6], 2, 64, stop, sampling=sampling)
    assert rc == 0, lib.ingot_e2e_last_error()
    for r in range(4):
        assert np.array_equal(out[r, :counts[r]], want[r]), (r, out[r, :counts[r]], want[r])
        assert finish[r] == (1 if len(want[r]) < max_tokens[r] else 0)
    # the penalty changes the replies (otherwise this test would not see a wrong history)
    plain = [served_alone(lib, model, p, m, None, stop) for p, m in zip(prompts, max_tokens)]
    assert any(not np.array_equal(a, b) for a, b in zip(plain, want))


def test_cancelled_requests_free_their_slot_and_keep_what_they_had(model):
    lib = engine()
    rng = np.random.default_rng(13)
    a, b, c = (rng.integers(0, N_VOCAB, size=n).astype(np.int32) for n in (4, 6, 3))
    # one slot: a runs first and its client goes away before step 9 (steps 0..8 done: 4 prompt tokens fed in steps 0..3, the
    # first reply token sampled in step 3, so 6 tokens by then); b is cancelled while still queued; c then gets the slot
    rc, out, counts, finish, (steps, rows) = scheduled(lib, model, [a, b, c], [-(9 + 1), -(2 + 1), 5], None, 1, 64, -1)
    assert rc == 0, lib.ingot_e2e_last_error()
    assert list(finish) == [2, 2, 0] and list(counts) == [6, 0, 5]
    assert np.array_equal(out[0, :6], alone(lib, model, a, 6)) and np.array_equal(out[2, :5], alone(lib, model, c, 5))
    assert steps == rows == 9 + (3 + 5 - 1)  # b never reached the backend


@pytest.mark.gpu
def test_scheduler_on_the_cuda_backend_matches_single_sequence_reference():
    """The same scheduler on the paged CUDA backend ("metal" is the name the reference's engine knows its GPU backend
    by) with two sequence slots for five requests - arrivals over time, a stop token, slots taken over by queued
    requests: every reply equals what the reference CpuBackend generates for that request alone, cut where the stop
    token would have appeared. The model is the 2-layer, 32064-token one of the end-to-end tests (head_dim 128)."""
    lib = engine()
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_random_gguf
    n_vocab = 32064
    path = os.path.join(os.environ.get("INGOT_E2E_DIR", "/tmp"), f"ingot_random_l2_v{n_vocab}_s0.gguf")
    if not os.path.exists(path):
        make_random_gguf.write(path + ".tmp", 2, n_vocab, seed=0)
        os.replace(path + ".tmp", path)
    rng = np.random.default_rng(100 + 5)
    prompts = [rng.integers(0, n_vocab, size=int(n)).astype(np.int32) for n in rng.integers(3, 40, size=5)]
    max_tokens = np.array([12, 5, 12, 8, 12], dtype=np.int32)
    arrivals = np.array([0, 0, 0, 3, 20], dtype=np.int32)
    want = [alone(lib, path, p, int(m)) for p, m in zip(prompts, max_tokens)]
    stop = int(want[0][7])
    expect = [w[:np.flatnonzero(w == stop)[0]] if (w == stop).any() else w for w in want]
    rc, out, counts, finish, (steps, rows) = scheduled(lib, path, prompts, max_tokens, arrivals, 2, 64, stop, backend=b"metal")
    assert rc == 0, lib.ingot_e2e_last_error().decode()
    for r in range(5):
        assert np.array_equal(out[r, :counts[r]], expect[r]), f"request {r}: scheduled {out[r, :counts[r]]} vs reference {expect[r]}"
        assert finish[r] == int((want[r] == stop).any())
    assert len(expect[0]) == 7 and steps < rows <= 2 * steps
