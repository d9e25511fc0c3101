"""Seeded synthetic inputs for the five attention workloads the project is measured on.

All shapes are the Llama-3.2-3B attention shape: 24 query heads, 8 KV heads, head_dim 128,
scale 1/sqrt(128), RoPE theta 500000. No dataset is involved: every tensor is N(0,1) from
numpy.random.default_rng(seed), drawn as float32 in the order Q, K, V and then cast to the stated
storage type, so that the CUDA path and the CPU checker see identical bits. Lengths and block
permutations (batched decode) come from independent child streams default_rng([seed, 1]) and
default_rng([seed, 2]) so that they do not depend on tensor sizes.
"""
from dataclasses import dataclass

import numpy as np

N_HEAD, N_HEAD_KV, HEAD_DIM = 24, 8, 128
ROPE_THETA = 500000.0
N_LAYER = 28
BLOCK_TOKENS = 16


def _normal(rng, shape):
    return rng.standard_normal(shape, dtype=np.float32)


def bf16_round(x):
    """float32 -> nearest-even bfloat16, returned as float32 (numpy has no bf16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(x.shape)


def bf16_bits(x):
    """float32 (already bf16-representable) -> uint16 bit patterns."""
    return (np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16).reshape(x.shape)


@dataclass
class Prefill:
    """Causal prefill of n_tok tokens starting at position pos0 (pos0 > 0: chunked prefill)."""
    q: np.ndarray          # [n_tok, H, d] f32 (bf16-representable when q_is_bf16)
    k: np.ndarray          # [n_tok, Hkv, d] f32 projections (rope=True) or f16 cache rows (rope=False)
    v: np.ndarray
    pos0: int
    rope: bool             # True: q/k are raw projections and RoPE is part of the path
    cache_k: np.ndarray = None  # [pos0, Hkv, d] f16: existing cache rows, already rotated
    cache_v: np.ndarray = None
    q_is_bf16: bool = False

    @property
    def n_tok(self):
        return self.q.shape[0]

    @property
    def flops(self):
        """4*H*d*(n_tok*pos0 + n_tok^2/2): causal FLOPs of QK^T and PV."""
        n = self.n_tok
        return 4 * N_HEAD * HEAD_DIM * (n * self.pos0 + n * n // 2)


def c1_prefill128(seed=0, n_tok=128):
    rng = np.random.default_rng(seed)
    q = _normal(rng, (n_tok, N_HEAD, HEAD_DIM))
    k = _normal(rng, (n_tok, N_HEAD_KV, HEAD_DIM))
    v = _normal(rng, (n_tok, N_HEAD_KV, HEAD_DIM))
    return Prefill(q, k, v, 0, True)


@dataclass
class Decode:
    """One query token per sequence over an f16 cache; all len keys visible."""
    q: np.ndarray            # [n_seq, H, d] f32 (bf16-representable when q_is_bf16)
    k: list                  # per sequence [len, Hkv, d] f16
    v: list
    lens: np.ndarray         # [n_seq] int32
    q_is_bf16: bool = False
    block_perm: np.ndarray = None  # paged: physical block of each logical block, all sequences concatenated

    @property
    def kv_bytes(self):
        """K+V bytes one layer reads: 2 * len * Hkv * d * 2 per sequence (the reference's abench formula)."""
        return int(self.lens.astype(np.int64).sum()) * N_HEAD_KV * HEAD_DIM * 2 * 2


def c2_decode4096(seed=1, n_keys=4096):
    rng = np.random.default_rng(seed)
    q = _normal(rng, (1, N_HEAD, HEAD_DIM))
    k = _normal(rng, (n_keys, N_HEAD_KV, HEAD_DIM)).astype(np.float16)
    v = _normal(rng, (n_keys, N_HEAD_KV, HEAD_DIM)).astype(np.float16)
    return Decode(q, [k], [v], np.array([n_keys], dtype=np.int32))


def c3_chunked(seed=2, n_tok=512, pos0=3584):
    rng = np.random.default_rng(seed)
    q = _normal(rng, (n_tok, N_HEAD, HEAD_DIM))
    k = _normal(rng, (n_tok, N_HEAD_KV, HEAD_DIM))
    v = _normal(rng, (n_tok, N_HEAD_KV, HEAD_DIM))
    ck = _normal(rng, (pos0, N_HEAD_KV, HEAD_DIM)).astype(np.float16)
    cv = _normal(rng, (pos0, N_HEAD_KV, HEAD_DIM)).astype(np.float16)
    return Prefill(q, k, v, pos0, True, ck, cv)


def c4_lengths(seed=3, n_seq=64, lo=256, hi=8192):
    return np.random.default_rng([seed, 1]).integers(lo, hi + 1, size=n_seq).astype(np.int32)


def c4_batched_decode(seed=3, n_seq=64, lo=256, hi=8192):
    lens = c4_lengths(seed, n_seq, lo, hi)
    rng = np.random.default_rng(seed)
    q = bf16_round(_normal(rng, (n_seq, N_HEAD, HEAD_DIM)))
    total = int(lens.sum())
    k_all = _normal(rng, (total, N_HEAD_KV, HEAD_DIM)).astype(np.float16)
    v_all = _normal(rng, (total, N_HEAD_KV, HEAD_DIM)).astype(np.float16)
    offs = np.concatenate([[0], np.cumsum(lens)])
    k = [k_all[offs[i]:offs[i + 1]] for i in range(n_seq)]
    v = [v_all[offs[i]:offs[i + 1]] for i in range(n_seq)]
    n_blocks = int(((lens + BLOCK_TOKENS - 1) // BLOCK_TOKENS).sum())
    perm = np.random.default_rng([seed, 2]).permutation(n_blocks).astype(np.int32)
    return Decode(q, k, v, lens, True, perm)


def block_tables(lens, perm, max_blocks=None):
    """Per-sequence block tables [n_seq, max_blocks] from the concatenated permutation (-1 padded)."""
    nb = (np.asarray(lens) + BLOCK_TOKENS - 1) // BLOCK_TOKENS
    max_blocks = int(max_blocks or nb.max())
    bt = np.full((len(lens), max_blocks), -1, dtype=np.int32)
    o = 0
    for i, n in enumerate(nb):
        bt[i, :n] = perm[o:o + n]
        o += n
    return bt


def c5_prefill32k(seed=4, n_tok=32768):
    rng = np.random.default_rng(seed)
    q = bf16_round(_normal(rng, (n_tok, N_HEAD, HEAD_DIM)))
    k = _normal(rng, (n_tok, N_HEAD_KV, HEAD_DIM)).astype(np.float16)
    v = _normal(rng, (n_tok, N_HEAD_KV, HEAD_DIM)).astype(np.float16)
    return Prefill(q, k, v, 0, False, q_is_bf16=True)


def lpt_assign(lens, n_ranks):
    """Length-balanced assignment of sequences to ranks (longest processing time first).

    Returns a list of index arrays, one per rank. Deterministic: ties go to the lower rank."""
    order = np.argsort(-np.asarray(lens, dtype=np.int64), kind="stable")
    loads = np.zeros(n_ranks, dtype=np.int64)
    out = [[] for _ in range(n_ranks)]
    for i in order:
        r = int(np.argmin(loads))
        out[r].append(int(i))
        loads[r] += int(lens[i])
    return [np.array(sorted(x), dtype=np.int64) for x in out]


def kv_head_shard(n_head_kv, n_ranks, rank):
    """KV heads [begin, end) owned by `rank` when the heads are split evenly over n_ranks."""
    assert n_head_kv % n_ranks == 0
    per = n_head_kv // n_ranks
    return rank * per, (rank + 1) * per
