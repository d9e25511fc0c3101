"""Host-side sharding logic: KV-head split for prefill, length-balanced sequence split for decode, and
the rank-major layout of the gathered head outputs (2 gloo ranks on CPU)."""
import os
import socket
import sys

import numpy as np
import pytest

from ingot_b200 import workloads as W


def test_kv_head_shard_partitions_heads():
    for n in (1, 2, 4, 8):
        spans = [W.kv_head_shard(8, n, r) for r in range(n)]
        assert spans[0][0] == 0 and spans[-1][1] == 8
        assert all(spans[i][1] == spans[i + 1][0] for i in range(n - 1))
        assert all(e - b == 8 // n for b, e in spans)


def test_lpt_assign_is_a_balanced_partition():
    lens = W.c4_lengths()
    assert len(lens) == 64 and lens.min() >= 256 and lens.max() <= 8192
    for n in (1, 2, 4, 8):
        parts = W.lpt_assign(lens, n)
        flat = np.sort(np.concatenate(parts))
        assert np.array_equal(flat, np.arange(64))  # every sequence exactly once
        loads = np.array([lens[p].sum() for p in parts], dtype=np.int64)
        assert loads.max() - loads.min() <= lens.max()  # LPT bound
        assert loads.max() / loads.mean() < 1.05
    assert [len(p) for p in W.lpt_assign(np.array([5, 1, 1]), 4)] == [1, 1, 1, 0]  # more ranks than sequences


def test_block_tables_cover_the_permutation():
    lens = np.array([1, 16, 17, 300], dtype=np.int32)
    nb = int(((lens + 15) // 16).sum())
    perm = np.random.default_rng(0).permutation(nb).astype(np.int32)
    bt = W.block_tables(lens, perm)
    used = bt[bt >= 0]
    assert np.array_equal(np.sort(used), np.arange(nb))
    assert [(r >= 0).sum() for r in bt] == [1, 1, 2, 19]


def test_workloads_are_seeded_and_shaped():
    a, b = W.c2_decode4096(), W.c2_decode4096()
    assert np.array_equal(a.q, b.q) and np.array_equal(a.k[0], b.k[0])
    assert a.kv_bytes == 16777216 and a.k[0].dtype == np.float16
    c1 = W.c1_prefill128()
    assert c1.flops == 100663296 and c1.q.shape == (128, 24, 128)
    q = W.bf16_round(np.array([1.0 + 2 ** -9, 3.14159], dtype=np.float32))
    assert q[0] == 1.0 and (q.view(np.uint32) & 0xFFFF == 0).all()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _gather_worker(rank, world, port, ret):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        S, H, D = 5, 24, 4
        full = torch.arange(S * H * D, dtype=torch.float32).reshape(S, H, D)  # "attention output" of all heads
        b, e = W.kv_head_shard(8, world, rank)
        mine = full[:, b * 3:e * 3].contiguous()                               # this rank's 3 query heads per kv head
        gathered = torch.empty(world * S, (e - b) * 3, D)  # concatenated along dim 0: rank-major
        dist.all_gather_into_tensor(gathered, mine)
        gathered = gathered.view(world, S, (e - b) * 3, D)
        # rank-major [rank][tok][heads_local][d] -> token-major [tok][head][d], as the wo projection reads it
        rebuilt = gathered.permute(1, 0, 2, 3).reshape(S, H, D)
        ok = torch.equal(rebuilt, full)
        # sequence sharding: every rank gets a disjoint, balanced subset and the union is everything
        parts = W.lpt_assign(W.c4_lengths(), world)
        counts = torch.tensor([len(parts[rank])])
        dist.all_reduce(counts)
        ret[rank] = bool(ok) and int(counts.item()) == 64
    finally:
        dist.destroy_process_group()


def test_head_output_gather_layout_two_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    ret = mgr.dict()
    port = _free_port()
    procs = [ctx.Process(target=_gather_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret.get(0) is True and ret.get(1) is True


def _monitor_worker(rank, world, port, steps_alive, ret):
    """Rank `rank` runs `steps_alive[rank]` steps, then leaves between steps (no work in flight)."""
    from datetime import timedelta
    import torch.distributed as dist
    from ingot_b200.sharding import PeerLost, PeerMonitor
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=30), wait_for_workers=False)
    mon = PeerMonitor(store, rank, world)
    done = 0
    try:
        for step in range(steps_alive[rank]):
            mon.begin_step(step, timeout_s=1.0)
            done += 1  # the sharded kernels of this step would be launched here
        ret[rank] = ("left", done)
    except PeerLost as e:
        ret[rank] = ("peer lost", done, e.step, e.missing)
    if rank == 0:  # the store's host stays up until the other rank has stopped using it
        import time
        time.sleep(1.5)


def test_a_rank_that_leaves_is_noticed_on_the_host_before_the_next_launch():
    """Two CPU ranks share a store. Rank 1 leaves after three steps; rank 0 must complete exactly those three steps
    and then get PeerLost for step 3 within its time limit - on the host, with nothing launched for that step."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_monitor_worker, args=(r, 2, port, {0: 10, 1: 3}, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert ret.get(1) == ("left", 3)
    assert ret.get(0) == ("peer lost", 3, 3, [1])


def test_peer_monitor_with_a_fake_store_that_drops_a_message():
    """The same logic against a fake store: a peer's announcement that is dropped looks like a peer that left."""
    from ingot_b200.sharding import PeerLost, PeerMonitor

    class FakeStore:
        def __init__(self, drop):
            self.keys, self.drop = set(), drop

        def set(self, k, v):
            if k not in self.drop:
                self.keys.add(k)

        def check(self, ks):
            return all(k in self.keys for k in ks)

    shared = FakeStore(drop={"ingot/step/1/2"})  # rank 2's announcement of step 1 never arrives
    mons = [PeerMonitor(shared, r, 3) for r in range(3)]
    for m in mons:
        m.announce(0)
    for m in mons:
        m.begin_step(0, timeout_s=0.2)  # everybody present
    for m in mons:
        m.announce(1)
    with pytest.raises(PeerLost) as e:
        mons[0].begin_step(1, timeout_s=0.1)
    assert e.value.missing == [2] and e.value.step == 1
