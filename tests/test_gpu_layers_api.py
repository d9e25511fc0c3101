"""The multi-layer and host-buffer entry points (the calls bench.py times) against the CPU reference."""
import numpy as np
import pytest

import helpers
from helpers import D, H, HKV
from ingot_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _fill_layers(kv, n_layers, n_keys, rng):
    ks, vs = [], []
    for l in range(n_layers):
        k = rng.standard_normal((n_keys, HKV, D), dtype=np.float32).astype(np.float16)
        v = rng.standard_normal((n_keys, HKV, D), dtype=np.float32).astype(np.float16)
        kv.import_f16(l, helpers.to_dev(k), helpers.to_dev(v), 0)
        ks.append(k)
        vs.append(v)
    return ks, vs


@pytest.mark.parametrize("n_layers,n_keys", [(1, 300), (3, 1000), (6, 4096), (9, 77)])
def test_decode_layers_matches_reference_per_layer(n_layers, n_keys):
    """ingot_attn_decode_layers runs all layers in one grid plus a merge launch; every layer's output must be
    the reference's, and a second call on the same handle must give identical bits."""
    import torch
    import ingot_b200 as ib
    rng = np.random.default_rng(n_layers * 1000 + n_keys)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, n_layers, HKV, n_keys)
    ks, vs = _fill_layers(kv, n_layers, n_keys, rng)
    q = rng.standard_normal((n_layers, 1, H, D), dtype=np.float32)
    qd = helpers.to_dev(q)
    out = torch.empty(n_layers, 1, H, D, device="cuda")
    ib.attn_decode_layers(kv, 0, qd, out, max_seq_len=n_keys)
    torch.cuda.synchronize()
    first = out.clone()
    for l in range(n_layers):
        wl = W.Decode(q[l], [ks[l]], [vs[l]], np.array([n_keys], dtype=np.int32))
        helpers.assert_parity(out[l].cpu().numpy(), helpers.oracle_decode(wl), f"layers decode, layer {l}")
    out.zero_()
    ib.attn_decode_layers(kv, 0, qd, out, max_seq_len=n_keys)
    torch.cuda.synchronize()
    assert torch.equal(out, first) and kv.status() == 0


def test_decode_layers_in_a_cuda_graph():
    """The call is capturable: replaying the graph reproduces the eager result."""
    import torch
    import ingot_b200 as ib
    rng = np.random.default_rng(5)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 5, HKV, 2048)
    _fill_layers(kv, 5, 2048, rng)
    q = helpers.to_dev(rng.standard_normal((5, 1, H, D), dtype=np.float32))
    out = torch.empty(5, 1, H, D, device="cuda")
    ib.attn_decode_layers(kv, 0, q, out, max_seq_len=2048)
    torch.cuda.synchronize()
    eager = out.clone()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ib.attn_decode_layers(kv, 0, q, out, max_seq_len=2048)
    for _ in range(3):
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager)


@pytest.mark.parametrize("n_tok,pos0", [(1, 511), (1, 0), (40, 100)])
def test_layers_host_matches_reference(n_tok, pos0):
    """Host buffers in and out (q/k/v projections -> attention rows), all layers in one call: RoPE + append
    + attention must equal the reference's per-token loop on every layer."""
    import torch
    import ingot_b200 as ib
    n_layers = 3
    rng = np.random.default_rng(n_tok * 7 + pos0)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, n_layers, HKV, pos0 + n_tok)
    ck = [rng.standard_normal((pos0, HKV, D), dtype=np.float32).astype(np.float16) for _ in range(n_layers)]
    cv = [rng.standard_normal((pos0, HKV, D), dtype=np.float32).astype(np.float16) for _ in range(n_layers)]
    if pos0:
        for l in range(n_layers):
            kv.import_f16(l, helpers.to_dev(ck[l]), helpers.to_dev(cv[l]), 0)
    q = rng.standard_normal((n_layers, n_tok, H, D), dtype=np.float32)
    k = rng.standard_normal((n_layers, n_tok, HKV, D), dtype=np.float32)
    v = rng.standard_normal((n_layers, n_tok, HKV, D), dtype=np.float32)
    qh, kh, vh = (torch.from_numpy(x).pin_memory() for x in (q, k, v))
    oh = torch.empty(n_layers, n_tok, H, D).pin_memory()
    inv = helpers.to_dev(helpers.inv_freq())
    ib.attn_layers_host(kv, 0, qh, kh, vh, oh, inv, pos0)
    torch.cuda.synchronize()
    assert kv.status() == 0
    for l in range(n_layers):
        wl = W.Prefill(q[l], k[l], v[l], pos0, True, ck[l] if pos0 else None, cv[l] if pos0 else None)
        want, _, _ = helpers.oracle_prefill(wl)
        helpers.assert_parity(oh[l].numpy(), want, f"layers_host n_tok={n_tok} pos0={pos0} layer {l}")
    # single-layer form writes the same rows
    oh1 = torch.empty(n_tok, H, D).pin_memory()
    ib.attn_layer_host(kv, 1, qh[1], kh[1], vh[1], oh1, inv, pos0)
    torch.cuda.synchronize()
    want1, _, _ = helpers.oracle_prefill(W.Prefill(q[1], k[1], v[1], pos0, True, ck[1] if pos0 else None, cv[1] if pos0 else None))
    helpers.assert_parity(oh1.numpy(), want1, "layer_host")


def test_layers_host_single_token_calls_in_a_row():
    """Five single-token calls at consecutive positions on one handle: the first runs eagerly, the second is
    captured into a graph, the others replay it with a new position read from device memory. Token i must
    see keys 0..pos0+i, exactly like row i of a five-token chunk in the reference."""
    import torch
    import ingot_b200 as ib
    n_layers, pos0, n_calls = 3, 200, 5
    rng = np.random.default_rng(321)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, n_layers, HKV, 512)
    ck = [rng.standard_normal((pos0, HKV, D), dtype=np.float32).astype(np.float16) for _ in range(n_layers)]
    cv = [rng.standard_normal((pos0, HKV, D), dtype=np.float32).astype(np.float16) for _ in range(n_layers)]
    for l in range(n_layers):
        kv.import_f16(l, helpers.to_dev(ck[l]), helpers.to_dev(cv[l]), 0)
    q = rng.standard_normal((n_layers, n_calls, H, D), dtype=np.float32)
    k = rng.standard_normal((n_layers, n_calls, HKV, D), dtype=np.float32)
    v = rng.standard_normal((n_layers, n_calls, HKV, D), dtype=np.float32)
    inv = helpers.to_dev(helpers.inv_freq())
    got = np.empty((n_layers, n_calls, H, D), dtype=np.float32)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(n_calls):
            qh, kh, vh = (torch.from_numpy(np.ascontiguousarray(x[:, i:i + 1])).pin_memory() for x in (q, k, v))
            oh = torch.empty(n_layers, 1, H, D).pin_memory()
            ib.attn_layers_host(kv, 0, qh, kh, vh, oh, inv, pos0 + i)
            stream.synchronize()
            got[:, i] = oh.numpy()[:, 0]
    assert kv.status() == 0
    for l in range(n_layers):
        want, _, _ = helpers.oracle_prefill(W.Prefill(q[l], k[l], v[l], pos0, True, ck[l], cv[l]))
        helpers.assert_parity(got[l], want, f"single-token host calls, layer {l}")
    # going back to an earlier position overwrites that row and attends over fewer keys (positions may go backwards)
    qh, kh, vh = (torch.from_numpy(np.ascontiguousarray(x[:, 1:2])).pin_memory() for x in (q, k, v))
    oh = torch.empty(n_layers, 1, H, D).pin_memory()
    ib.attn_layers_host(kv, 0, qh, kh, vh, oh, inv, pos0 + 1)
    torch.cuda.synchronize()
    for l in range(n_layers):
        want, _, _ = helpers.oracle_prefill(W.Prefill(q[l], k[l], v[l], pos0, True, ck[l], cv[l]))
        helpers.assert_parity(oh.numpy()[l, 0], want[1], f"single-token host call moved back, layer {l}")


def test_layers_host_rejects_overflow():
    import torch
    import ingot_b200 as ib
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 2, HKV, 8)
    z = torch.zeros(2, 1, H, D).pin_memory()
    zk = torch.zeros(2, 1, HKV, D).pin_memory()
    inv = helpers.to_dev(helpers.inv_freq())
    with pytest.raises(ib.IngotError, match="context window exceeded"):
        ib.attn_layers_host(kv, 0, z, zk, zk, z.clone().pin_memory(), inv, 8)


def test_decode_layers_paged_batch_of_uneven_lengths():
    """Several layers of a paged cache, sequences from one key to many splits long, in one call: every
    (layer, sequence) must match the reference; a second call gives the same bits and leaves the status
    word clear."""
    import torch
    import ingot_b200 as ib
    n_layers = 3
    lens = np.array([1, 17, 255, 256, 1000, 2049], dtype=np.int32)
    n_seq = len(lens)
    rng = np.random.default_rng(99)
    nb = int(((lens + 15) // 16).sum())
    perm = rng.permutation(nb).astype(np.int32)
    bt_np = W.block_tables(lens, perm)
    kv = ib.KVCache(ib.KV_PAGED, n_layers, HKV, nb, max_seqs=n_seq)
    bt = helpers.to_dev(bt_np)
    ks = [[rng.standard_normal((int(n), HKV, D), dtype=np.float32).astype(np.float16) for n in lens] for _ in range(n_layers)]
    vs = [[rng.standard_normal((int(n), HKV, D), dtype=np.float32).astype(np.float16) for n in lens] for _ in range(n_layers)]
    for l in range(n_layers):
        for s in range(n_seq):
            kv.import_f16(l, helpers.to_dev(ks[l][s]), helpers.to_dev(vs[l][s]), 0, bt[s])
    q = rng.standard_normal((n_layers, n_seq, H, D), dtype=np.float32)
    qd = helpers.to_dev(q)
    lens_d = helpers.to_dev(lens)
    out = torch.zeros(n_layers, n_seq, H, D, device="cuda")
    ib.attn_decode_layers(kv, 0, qd, out, seq_lens=lens_d, max_seq_len=int(lens.max()), block_tables=bt)
    torch.cuda.synchronize()
    first = out.clone()
    for l in range(n_layers):
        wl = W.Decode(q[l], ks[l], vs[l], lens)
        helpers.assert_parity(out[l].cpu().numpy(), helpers.oracle_decode(wl), f"paged layers decode, layer {l}")
    out.zero_()
    ib.attn_decode_layers(kv, 0, qd, out, seq_lens=lens_d, max_seq_len=int(lens.max()), block_tables=bt)
    torch.cuda.synchronize()
    assert torch.equal(out, first) and kv.status() == 0


@pytest.mark.parametrize("scratch_mb", [None, "1"])
def test_decode_28_layers_4096_keys_replayed_from_a_graph(scratch_mb, monkeypatch):
    """The call the benchmark times: 28 layers x 4096 keys through ingot_attn_decode_layers, captured once into a
    CUDA graph and replayed. Every layer of the replay must match the reference, a second replay must give the
    same bits, and the same holds when a small scratch forces the layers into several groups of launches."""
    import torch
    import ingot_b200 as ib
    if scratch_mb is not None:
        monkeypatch.setenv("INGOT_DECODE_SCRATCH_MB", scratch_mb)
    n_layers, n_keys = W.N_LAYER, 4096
    rng = np.random.default_rng(2024)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, n_layers, HKV, n_keys)
    ks, vs = _fill_layers(kv, n_layers, n_keys, rng)
    q = rng.standard_normal((n_layers, 1, H, D), dtype=np.float32)
    qd = helpers.to_dev(q)
    out = torch.zeros(n_layers, 1, H, D, device="cuda")
    ib.attn_decode_layers(kv, 0, qd, out, max_seq_len=n_keys)  # eager first: sizes the split scratch
    torch.cuda.synchronize()
    eager = out.clone()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ib.attn_decode_layers(kv, 0, qd, out, max_seq_len=n_keys)
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    first = out.clone()
    for l in range(n_layers):
        wl = W.Decode(q[l], [ks[l]], [vs[l]], np.array([n_keys], dtype=np.int32))
        helpers.assert_parity(first[l].cpu().numpy(), helpers.oracle_decode(wl), f"graph-replayed decode, layer {l}")
    assert torch.equal(first, eager)
    for _ in range(20):  # back-to-back replays overlap their tails: the scratch hand-over must hold
        g.replay()
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, first) and kv.status() == 0


def test_decode_scratch_follows_the_split_count():
    """A handle grows its split scratch to what the calls need (a graph captured before a growth keeps
    working, because outgrown buffers stay alive until the handle is destroyed)."""
    import torch
    import ingot_b200 as ib
    rng = np.random.default_rng(8)
    kv = ib.KVCache(ib.KV_CONTIGUOUS, 2, HKV, 4096)
    ks, vs = _fill_layers(kv, 2, 4096, rng)
    q = rng.standard_normal((2, 1, H, D), dtype=np.float32)
    qd = helpers.to_dev(q)
    small = torch.zeros(1, H, D, device="cuda")
    ib.attn_decode(kv, 0, qd[0], out=small, max_seq_len=300, chunk_keys=64)  # few splits
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ib.attn_decode(kv, 0, qd[0], out=small, max_seq_len=300, chunk_keys=64)
    big = torch.zeros(2, 1, H, D, device="cuda")
    ib.attn_decode_layers(kv, 0, qd, big, max_seq_len=4096, chunk_keys=64)  # 64 splits, two layers: the scratch grows
    torch.cuda.synchronize()
    for l in range(2):
        wl = W.Decode(q[l], [ks[l]], [vs[l]], np.array([4096], dtype=np.int32))
        helpers.assert_parity(big[l].cpu().numpy(), helpers.oracle_decode(wl), f"after growth, layer {l}")
    small.zero_()
    g.replay()
    torch.cuda.synchronize()
    wl = W.Decode(q[0], [ks[0][:300]], [vs[0][:300]], np.array([300], dtype=np.int32))
    helpers.assert_parity(small.cpu().numpy(), helpers.oracle_decode(wl), "graph captured before the growth")
    assert kv.status() == 0
