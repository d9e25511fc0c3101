// K3 — split-KV flash decoding for one-token queries over the f16 KV cache (contiguous or paged).
//
// Replaces the attention lambda of the CPU reference for a single query token
// (src/cpu_backend.cpp:51-69) and Metal's attn_decode_g3 + attn_combine pair
// (shaders/kernels.metal:428-516, dispatch src/metal_backend.mm:340-360).
//
// Work decomposition. grid = (splits, kv heads, layers x sequences). A CTA owns one KV head of one sequence
// of one layer over one split of `chunk_keys` keys and serves ALL query heads that share that KV head (GQA), so
// every K/V byte is fetched from HBM exactly once. Inside the CTA each warp walks its own 16-key
// units with a private online-softmax state (m, l, o); the warp states are merged through shared
// memory and the split's partial (o[128], m, l per head) goes to a global scratch. A small combine
// kernel chained behind it with programmatic dependent launch merges the partials:
// out = sum_s o_s 2^(m_s-M) / sum_s l_s 2^(m_s-M), the attn_combine formula. Split CTAs therefore
// retire as soon as their partial is written (no fence, ticket or polling), and the combine of one
// launch overlaps the K/V loads of the next.
//
// Data path. HBM-bound: 2 * len * 128 * 2 B per (sequence, kv head). Every lane issues 16-byte
// loads straight from global memory into registers, 16 of them (one whole 16-key unit, 8 KB per
// warp) before the first use and the next unit's 16 while the current one is consumed, so a warp
// keeps 8-16 KB in flight with no shared-memory staging and no barrier in the key loop.
// The math rides on warp-level m16n8k16 f16 MMAs with f32 accumulation: the (up to 8) query heads
// of the group are the M rows of QK^T and of PV. Registers loaded as 16-byte chunks are used as MMA
// fragments directly; the k-index permutation this implies is applied identically to the query
// fragments (QK^T) and undone when the output is written (PV), so no shuffles or shared-memory
// transposes are needed. Scores are scaled in f32 after the MMA (the Metal kernel pre-scales q in
// f16; scaling late keeps the error inside the f32-reference tolerance).
#include "attn_common.cuh"
#include "ingot_internal.cuh"
#include "attn_decode_params.cuh"

// This file is compiled twice. attn_decode_append.cu defines INGOT_DECODE_APPEND and includes it: the kernel then is
// the single-token form that also does K1's work (RoPE on q and on the new k, the K/V row written to the cache by the
// CTA that owns the last key, that row fed to the MMAs from the projections instead of from the cache) - one launch
// for what is otherwise rope_kv_append + decode. Everything outside the kernel is compiled in the plain build only,
// so this build's kernel is the same code as before.
#ifdef INGOT_DECODE_APPEND
#include "rope_unit.cuh"
#define DECODE_KERNEL attn_decode_append_kernel
#define DECODE_PARAMS DecodeAppendParams
struct DecodeAppendParams : DecodeParams {
    const float* q_f32;     // [n_head][128] projections of the token
    const float* k_new;     // [n_head_kv][128]
    const float* v_new;
    const float* inv_freq;  // [64]
    __half* kc_w;           // writable aliases of kc / vc
    __half* vc_w;
};
#else
#define DECODE_KERNEL attn_decode_kernel
#define DECODE_PARAMS DecodeParams
#endif

#include <algorithm>
#include <cstring>
#include <mutex>

namespace {

constexpr int kMaxDecodeWarps = 8;
constexpr int kMaxParts = 64;

// Merges the splits of one (sequence, kv head): out = sum_s o_s 2^(m_s-M) / sum_s l_s 2^(m_s-M)
// (the attn_combine formula, shaders/kernels.metal:502-516). Runs in one extra CTA per (kv head,
// sequence) of the launch that FOLLOWS the one that wrote the partials (or of a merge-only launch):
// programmatic dependent launch orders it behind that launch, so no fences, tickets or polling are
// involved, and the merge overlaps the K/V loads of the split CTAs it shares the grid with.
__device__ __forceinline__ void combine_splits(const DecodeParams& p, float* smem, int kvh, int layer, int seq) {
    const int n_keys = load_seq_len(p, seq);
    if (n_keys < 1) return;
    const int n_chunks = (n_keys + p.chunk_keys - 1) / p.chunk_keys;
    if (n_chunks == 1) return;  // the split CTA wrote the final output itself
    const int G = p.group;

    // Parallel merge. A thread owns one (head, 4-dim column) pair for a strided subset of the splits
    // ("slot"); all of its partial loads are independent and issued before anything waits on them, so
    // the merge costs about one L2 round trip instead of one per split.
    const int T = blockDim.x;
    const int pairs = G * 32;                     // (head, float4 column) pairs
    const int slots = max(1, T / pairs);          // threads per pair
    const int pair = threadIdx.x % pairs, slot = threadIdx.x / pairs;
    const bool active = slot < slots;
    const int gi_t = pair >> 5, col = pair & 31;
    const size_t step = (size_t)p.n_head * kPartStride;
    const size_t part0 = (size_t)layer * p.part_layer_stride, out0 = (size_t)layer * p.qo_layer_stride;
    // bounds-check build: the last partial row this merge reads, and the output rows it writes
    if (!INGOT_CHECK(part0 + (((size_t)seq * p.n_parts_max + (n_chunks - 1)) * p.n_head + (size_t)kvh * G) * kPartStride, (size_t)G * kPartStride,
                     p.part_extent, p.status) ||
        !INGOT_CHECK(out0 + ((size_t)seq * p.n_head + (size_t)kvh * G) * kHeadDim, (size_t)G * kHeadDim, p.out_extent, p.status))
        return;
    const float* base = p.c_part + part0 + (((size_t)seq * p.n_parts_max) * p.n_head + (size_t)kvh * G) * kPartStride;
    const float* my_rows = base + (size_t)gi_t * kPartStride + col * 4;

    float* mg_m = smem;                       // [G][kMaxParts] split maxima, then weights
    float* mg_l = mg_m + G * kMaxParts;       // [G][kMaxParts] split sums
    float* mg_acc = mg_l + G * kMaxParts;     // [slots][pairs] float4 partial outputs

    constexpr int kBatch = 16;
    float4 v[kBatch];
    if (active) {
#pragma unroll
        for (int u = 0; u < kBatch; u++) {
            const int c = slot + u * slots;
            if (c < n_chunks) v[u] = __ldcg(reinterpret_cast<const float4*>(my_rows + c * step));
        }
    }
    for (int idx = threadIdx.x; idx < G * n_chunks; idx += T) {
        const int gi = idx / n_chunks, c = idx - gi * n_chunks;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(base + (size_t)gi * kPartStride + c * step + 128));
        mg_m[gi * kMaxParts + c] = ml.x;
        mg_l[gi * kMaxParts + c] = ml.y;
    }
    __syncthreads();
    float w_mine[4];
    {
        // weight of split c for head gi: 2^(m_c - M), M = max over the head's splits
        int k = 0;
        for (int idx = threadIdx.x; idx < G * n_chunks; idx += T, k++) {
            const int gi = idx / n_chunks;
            float M = -INFINITY;
            for (int c = 0; c < n_chunks; c++) M = fmaxf(M, mg_m[gi * kMaxParts + c]);
            if (k < 4) w_mine[k] = exp2f(mg_m[gi * kMaxParts + (idx - gi * n_chunks)] - M);
        }
    }
    __syncthreads();
    {
        int k = 0;
        for (int idx = threadIdx.x; idx < G * n_chunks && k < 4; idx += T, k++) {
            const int gi = idx / n_chunks;
            mg_m[gi * kMaxParts + (idx - gi * n_chunks)] = w_mine[k];
        }
    }
    __syncthreads();
    if (active) {
        const float* wrow = mg_m + gi_t * kMaxParts;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < kBatch; u++) {
            const int c = slot + u * slots;
            if (c < n_chunks) {
                const float w = wrow[c];
                acc.x += v[u].x * w; acc.y += v[u].y * w; acc.z += v[u].z * w; acc.w += v[u].w * w;
            }
        }
        for (int c = slot + kBatch * slots; c < n_chunks; c += slots) {  // only when n_chunks > 16 * slots
            const float4 x = __ldcg(reinterpret_cast<const float4*>(my_rows + c * step));
            const float w = wrow[c];
            acc.x += x.x * w; acc.y += x.y * w; acc.z += x.z * w; acc.w += x.w * w;
        }
        reinterpret_cast<float4*>(mg_acc)[slot * pairs + pair] = acc;
    }
    // More (head, column) pairs than threads (large groups on a small CTA): remaining pairs, one slot.
    for (int pr = T + threadIdx.x; pr < pairs; pr += T) {
        const float* rows = base + (size_t)(pr >> 5) * kPartStride + (pr & 31) * 4;
        const float* wrow = mg_m + (pr >> 5) * kMaxParts;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int c0 = 0; c0 < n_chunks; c0 += kBatch) {
#pragma unroll
            for (int u = 0; u < kBatch; u++)
                if (c0 + u < n_chunks) v[u] = __ldcg(reinterpret_cast<const float4*>(rows + (c0 + u) * step));
#pragma unroll
            for (int u = 0; u < kBatch; u++)
                if (c0 + u < n_chunks) {
                    const float w = wrow[c0 + u];
                    acc.x += v[u].x * w; acc.y += v[u].y * w; acc.z += v[u].z * w; acc.w += v[u].w * w;
                }
        }
        reinterpret_cast<float4*>(mg_acc)[pr] = acc;  // slots == 1 here
    }
    __syncthreads();
    for (int pr = threadIdx.x; pr < pairs; pr += T) {
        const int gi = pr >> 5, cl = pr & 31;
        float L = 0.f;
        for (int c = 0; c < n_chunks; c++) L += mg_l[gi * kMaxParts + c] * mg_m[gi * kMaxParts + c];
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sl_i = 0; sl_i < slots; sl_i++) {
            const float4 x = reinterpret_cast<const float4*>(mg_acc)[sl_i * pairs + pr];
            acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
        }
        const float inv = L > 0.f ? 1.0f / L : 0.f;
        const size_t e = out0 + ((size_t)seq * p.n_head + (size_t)kvh * G + gi) * kHeadDim + cl * 4;
        store_out(p.c_out, p.out_dtype, e + 0, acc.x * inv);
        store_out(p.c_out, p.out_dtype, e + 1, acc.y * inv);
        store_out(p.c_out, p.out_dtype, e + 2, acc.z * inv);
        store_out(p.c_out, p.out_dtype, e + 3, acc.w * inv);
    }
}

struct KRegs { uint4 k[8]; };  // [n-tile 0/1][i=0..3]: key (nt*8 + g), 16-byte chunk (4i + j)
struct VRegs { uint4 v[8]; };  // [slot 0..3 -> keys 2j, 2j+1, 2j+8, 2j+9][chunk g / g+8]

__global__ void __launch_bounds__(kMaxDecodeWarps * 32, 1) DECODE_KERNEL(const DECODE_PARAMS p) {
    extern __shared__ float smem[];
    // Programmatic dependent launch: let the next kernel in the stream start as soon as SM resources allow, and
    // wait for the kernel before this one according to p.pdl_mode (see DecodeParams).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if ((int)blockIdx.x >= p.split_parts) {  // merge role: partials of the preceding launch
        asm volatile("griddepcontrol.wait;" ::: "memory");
        combine_splits(p, smem, blockIdx.y, blockIdx.z / p.n_seq, blockIdx.z % p.n_seq);
        return;
    }
    if (p.pdl_mode == kPdlWaitFirst) asm volatile("griddepcontrol.wait;" ::: "memory");

    const int chunk = blockIdx.x, kvh = blockIdx.y, layer = blockIdx.z / p.n_seq, seq = blockIdx.z % p.n_seq;
    const __half* const kc = p.kc + (size_t)layer * p.cache_layer_stride;
    const __half* const vc = p.vc + (size_t)layer * p.cache_layer_stride;
    const int n_keys = load_seq_len(p, seq);
    if (n_keys < 1) return;
    const int n_chunks = (n_keys + p.chunk_keys - 1) / p.chunk_keys;
    if (chunk >= n_chunks) return;
    const int k_begin = chunk * p.chunk_keys;
    const int k_end = min(n_keys, k_begin + p.chunk_keys);
    const int n_units = (k_end - k_begin + 15) >> 4;

    const int n_warps = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, j = lane & 3;
    const int G = p.group;

    const int32_t* bt = p.paged ? p.block_tables + (size_t)seq * p.max_blocks_per_seq : nullptr;

#ifdef INGOT_DECODE_APPEND
    // The token's projections, rotated for position n_keys - 1 and rounded to f16 once per CTA: the G query heads of this
    // KV head (the MMA A operand), the new K row and the new V row (what K1 writes to the cache). One 8-element unit
    // per thread.
    __shared__ __align__(16) __half new_q[8 * kHeadDim];
    __shared__ __align__(16) __half new_kv[2 * kHeadDim];
    {
        const float fpos = float(n_keys - 1);
        for (int u = threadIdx.x; u < (G + 2) * 16; u += blockDim.x) {
            const int h = u >> 4, c = u & 15;
            if (h < G)
                *reinterpret_cast<uint4*>(new_q + h * kHeadDim + c * 8) =
                    rope_pack8(p.q_f32 + ((size_t)kvh * G + h) * kHeadDim + c * 8, c * 4, fpos, p.inv_freq, true);
            else
                *reinterpret_cast<uint4*>(new_kv + (h - G) * kHeadDim + c * 8) =
                    rope_pack8((h == G ? p.k_new : p.v_new) + (size_t)kvh * kHeadDim + c * 8, c * 4, fpos, p.inv_freq, h == G);
        }
        __syncthreads();
    }
#endif

    // Base element offset (within the layer) of the 16 rows of unit u; keys of a unit are contiguous
    // rows in both layouts (a unit is exactly one block of a paged cache).
    auto unit_base = [&](int u) -> size_t {
        const int key0 = k_begin + (u << 4);
        if (!p.paged) return kv_row_offset_contig(p.capacity, kvh, key0);
        int blk = bt[key0 >> 4];
        if (blk < 0 || blk >= p.capacity) {
            if (lane == 0) atomicOr(p.status, kDevErrBlockRange);
            blk = 0;
        }
        return kv_row_offset_paged(p.n_head_kv, blk, kvh, 0);
    };
    auto load_k = [&](KRegs& r, int u) {
        const int last = n_keys - 1 - (k_begin + (u << 4));  // last valid row of this unit (>= 0)
        const size_t ub = unit_base(u);
        if (!INGOT_CHECK(ub, (size_t)(last + 1 < 16 ? last + 1 : 16) * kHeadDim, p.cache_extent, p.status)) return;
        const __half* kb = kc + ub;
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            const int row = min(nt * 8 + g, last);
#ifdef INGOT_DECODE_APPEND
            if (row == last && last < 16) {
                // The newest key (position n_keys - 1): taken from the CTA's rotated copy of the projection, and written to
                // the cache by the lanes whose own row it is (rows past the last key are clamped onto it and only read it).
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int c = 4 * i + j;
                    const uint4 val = *reinterpret_cast<const uint4*>(new_kv + c * 8);
                    r.k[nt * 4 + i] = val;
                    if (nt * 8 + g == last) *reinterpret_cast<uint4*>(p.kc_w + (size_t)layer * p.cache_layer_stride + ub + (size_t)row * kHeadDim + c * 8) = val;
                }
                continue;
            }
#endif
#pragma unroll
            for (int i = 0; i < 4; i++) r.k[nt * 4 + i] = ld_stream16(kb + (size_t)row * kHeadDim + (4 * i + j) * 8);
        }
    };
    auto load_v = [&](VRegs& r, int u) {
        const int last = n_keys - 1 - (k_begin + (u << 4));
        const size_t ub = unit_base(u);
        if (!INGOT_CHECK(ub, (size_t)(last + 1 < 16 ? last + 1 : 16) * kHeadDim, p.cache_extent, p.status)) return;
        const __half* vb = vc + ub;
#pragma unroll
        for (int s = 0; s < 4; s++) {
            const int row_own = 2 * j + (s & 1) + (s >> 1) * 8;
            const int row = min(row_own, last);
#ifdef INGOT_DECODE_APPEND
            if (row == last && last < 16) {  // the newest V row: from the CTA's f16 copy of the projection, stored by its owner lanes
#pragma unroll
                for (int hgh = 0; hgh < 2; hgh++) {
                    const int c = g + 8 * hgh;
                    const uint4 val = *reinterpret_cast<const uint4*>(new_kv + kHeadDim + c * 8);
                    r.v[s * 2 + hgh] = val;
                    if (row_own == last) *reinterpret_cast<uint4*>(p.vc_w + (size_t)layer * p.cache_layer_stride + ub + (size_t)row * kHeadDim + c * 8) = val;
                }
                continue;
            }
#endif
            r.v[s * 2 + 0] = ld_stream16(vb + (size_t)row * kHeadDim + g * 8);
            r.v[s * 2 + 1] = ld_stream16(vb + (size_t)row * kHeadDim + (g + 8) * 8);
        }
    };

    uint4 qa[4];
#pragma unroll
    for (int i = 0; i < 4; i++) qa[i] = make_uint4(0, 0, 0, 0);
    float m = -INFINITY, l = 0.f;
    // O^T accumulators: o[t] = {O[2j][8g+t], O[2j+1][8g+t], O[2j][64+8g+t], O[2j+1][64+8g+t]} (head, dim).
    float o[8][4];
#pragma unroll
    for (int t = 0; t < 8; t++) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;

    uint32_t pa0 = 0, pa2 = 0;
    auto compute_qk = [&](const KRegs& r, int u) {
        // S[head g][key] for two 8-key n-tiles; rows 8-15 of the M dimension are unused (zero A rows).
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int i = 0; i < 4; i++) {
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                const uint4 kk = r.k[nt * 4 + i];
                mma_16816(s[nt], qa[i].x, 0u, qa[i].y, 0u, kk.x, kk.y);
                mma_16816(s[nt], qa[i].z, 0u, qa[i].w, 0u, kk.z, kk.w);
            }
        }
        const int key0 = k_begin + (u << 4) + 2 * j;
        float x[2][2];
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const bool valid = key0 + nt * 8 + e < k_end;
                x[nt][e] = valid ? s[nt][e] * p.scale_log2 : -INFINITY;
                mx = fmaxf(mx, x[nt][e]);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m, mx);  // finite: every unit holds at least one valid key
        const float alpha = exp2f(m - m_new);
        float pr[2][2];
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) pr[nt][e] = exp2f(x[nt][e] - m_new);
        l = l * alpha + ((pr[0][0] + pr[0][1]) + (pr[1][0] + pr[1][1]));
        m = m_new;
        pa0 = pack_half2_rn(pr[0][0], pr[0][1]);
        pa2 = pack_half2_rn(pr[1][0], pr[1][1]);
        // The output accumulators are transposed (dims x heads): thread (g, j) holds heads 2j and
        // 2j+1, whose rescale factors live in the lanes with g == 2j and g == 2j+1.
        const float alpha_a = __shfl_sync(0xffffffffu, alpha, 8 * j);
        const float alpha_b = __shfl_sync(0xffffffffu, alpha, 8 * j + 4);
#pragma unroll
        for (int t = 0; t < 8; t++) { o[t][0] *= alpha_a; o[t][1] *= alpha_b; o[t][2] *= alpha_a; o[t][3] *= alpha_b; }
    };
    // O^T[dims][heads] += V^T[dims][keys] * P^T[keys][heads]: the packed P pairs are the B fragment
    // as they come out of the score tile; V pairs (two keys, one dim) are formed with byte permutes.
    auto compute_pv = [&](const VRegs& r) {
        const uint32_t va0[4] = {r.v[0].x, r.v[0].y, r.v[0].z, r.v[0].w};  // key 2j,   chunk g
        const uint32_t va1[4] = {r.v[1].x, r.v[1].y, r.v[1].z, r.v[1].w};  // key 2j,   chunk g+8
        const uint32_t vb0[4] = {r.v[2].x, r.v[2].y, r.v[2].z, r.v[2].w};  // key 2j+1, chunk g
        const uint32_t vb1[4] = {r.v[3].x, r.v[3].y, r.v[3].z, r.v[3].w};  // key 2j+1, chunk g+8
        const uint32_t vc0[4] = {r.v[4].x, r.v[4].y, r.v[4].z, r.v[4].w};  // key 2j+8, chunk g
        const uint32_t vc1[4] = {r.v[5].x, r.v[5].y, r.v[5].z, r.v[5].w};  // key 2j+8, chunk g+8
        const uint32_t vd0[4] = {r.v[6].x, r.v[6].y, r.v[6].z, r.v[6].w};  // key 2j+9, chunk g
        const uint32_t vd1[4] = {r.v[7].x, r.v[7].y, r.v[7].z, r.v[7].w};  // key 2j+9, chunk g+8
#pragma unroll
        for (int t = 0; t < 8; t++) {
            const int w = t >> 1;
            const uint32_t sel = (t & 1) ? 0x7632u : 0x5410u;
            mma_16816(o[t], prmt(va0[w], vb0[w], sel), prmt(va1[w], vb1[w], sel), prmt(vc0[w], vd0[w], sel),
                      prmt(vc1[w], vd1[w], sel), pa0, pa2);
        }
    };

    // Key loop, software-pipelined two units deep: both the K and the V rows of the warp's next two
    // 16-key units (16 KB) are requested before anything is consumed, and a unit's registers are
    // refilled as soon as it has been used. For a 4096-key decode every warp owns at most two units, so
    // all of its loads are in flight at once and the kernel pays the DRAM latency once.
    {
        KRegs k0, k1;
        VRegs v0, v1;
        int u0 = warp, u1 = warp + n_warps;
        if (u0 < n_units) { load_k(k0, u0); load_v(v0, u0); }
        if (u1 < n_units) { load_k(k1, u1); load_v(v1, u1); }
        // Query fragments (head row g, chunks 4i + j), requested after the K/V units so that the wait
        // for them overlaps the K/V latency instead of preceding it.
        if (g < G) {
#ifdef INGOT_DECODE_APPEND
#pragma unroll
            for (int i = 0; i < 4; i++) qa[i] = *reinterpret_cast<const uint4*>(new_q + g * kHeadDim + (4 * i + j) * 8);
#else
            const size_t qbase = (size_t)layer * p.qo_layer_stride + ((size_t)seq * p.n_head + (size_t)kvh * G + g) * kHeadDim;
#pragma unroll
            for (int i = 0; i < 4; i++) qa[i] = load_q8(p.q, p.q_dtype, qbase + (size_t)(4 * i + j) * 8);
#endif
        }
        while (u0 < n_units) {
            compute_qk(k0, u0);
            compute_pv(v0);
            const int u2 = u1 + n_warps;
            if (u2 < n_units) { load_k(k0, u2); load_v(v0, u2); }
            if (u1 >= n_units) break;
            compute_qk(k1, u1);
            compute_pv(v1);
            const int u3 = u2 + n_warps;
            if (u3 < n_units) { load_k(k1, u3); load_v(v1, u3); }
            u0 = u2;
            u1 = u3;
        }
    }
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);

    // ---- merge the warps' states through shared memory ----
    // layout: so[warp][G][128], sm[warp][G], sl[warp][G]
    float* so = smem;
    float* sm = so + (size_t)n_warps * G * kHeadDim;
    float* sl = sm + n_warps * G;
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const int head = 2 * j + e;
        if (head < G) {
            float* dst = so + ((size_t)warp * G + head) * kHeadDim + 8 * g;
            *reinterpret_cast<float4*>(dst) = make_float4(o[0][e], o[1][e], o[2][e], o[3][e]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(o[4][e], o[5][e], o[6][e], o[7][e]);
            *reinterpret_cast<float4*>(dst + 64) = make_float4(o[0][2 + e], o[1][2 + e], o[2][2 + e], o[3][2 + e]);
            *reinterpret_cast<float4*>(dst + 68) = make_float4(o[4][2 + e], o[5][2 + e], o[6][2 + e], o[7][2 + e]);
        }
    }
    if (g < G && j == 0) { sm[warp * G + g] = m; sl[warp * G + g] = l; }
    __syncthreads();
    if (p.pdl_mode == kPdlEarlyLoads) asm volatile("griddepcontrol.wait;" ::: "memory");

    const bool single = n_chunks == 1;
    const size_t part_row0 = ((size_t)seq * p.n_parts_max + chunk) * p.n_head + (size_t)kvh * G;
    const size_t part0 = (size_t)layer * p.part_layer_stride, out0 = (size_t)layer * p.qo_layer_stride;
    for (int idx = threadIdx.x; idx < G * kHeadDim; idx += blockDim.x) {
        const int gi = idx >> 7, dim = idx & 127;
        float M = -INFINITY;
        for (int w = 0; w < n_warps; w++) M = fmaxf(M, sm[w * G + gi]);
        float L = 0.f, O = 0.f;
        for (int w = 0; w < n_warps; w++) {
            const float wgt = exp2f(sm[w * G + gi] - M);
            L += sl[w * G + gi] * wgt;
            O += so[((size_t)w * G + gi) * kHeadDim + dim] * wgt;
        }
        if (single) {
            const size_t e = out0 + ((size_t)seq * p.n_head + (size_t)kvh * G + gi) * kHeadDim + dim;
            if (INGOT_CHECK(e, 1, p.out_extent, p.status)) store_out(p.out, p.out_dtype, e, O / L);
        } else if (INGOT_CHECK(part0 + (part_row0 + gi) * kPartStride, kPartStride, p.part_extent, p.status)) {
            float* row = p.part + part0 + (part_row0 + gi) * kPartStride;
            row[dim] = O;
            if (dim == 0) { row[128] = M; row[129] = L; }
        }
    }
}

}  // namespace

#ifndef INGOT_DECODE_APPEND
// Tuning knob, process-wide and read once (like the reference's LLM_ATTN_SPLITS): warps per CTA, 4 (two CTAs
// per SM) or 8.
int decode_warps_cfg() {
    static const int v = [] { const char* e = getenv("INGOT_DECODE_WARPS"); return (e && atoi(e) == 8) ? 8 : 4; }();
    return v;
}

// Split size and split count of one decode launch over `ranges` = layers x sequences x kv heads independent key
// ranges of up to max_seq_len keys (chunk_keys == 0: chosen here).
// A split CTA costs about 1.5 us of start-up and drain whatever its size - at a slot's share of the HBM bandwidth
// that is the time of ~64 keys - so long splits are the efficient ones, but the last wave of long splits leaves
// SMs idle. Measured on a B200, 28 layers x 4096 keys in one grid: 3.2 / 4.4 / 5.2 / 5.4 / 5.1 / 5.3 TB/s with
// 128 / 256 / 512 / 768 / 1024 / 2048 keys per split; a 64-sequence paged batch (lengths 256..8192, 4 layers):
// 5.4 / 5.7 / 5.9 / 6.1 TB/s with 512 / 768 / 1024 / 2048.
//   * Up to 256 keys: one split (the CTA writes the output itself; a merge launch would cost more than it saves).
//   * Jobs that do not fill the CTA slots of the GPU even with 512-key splits (a single layer of one sequence):
//     fill every slot once with whole 16-key units per warp.
//   * Batches (lengths differ, many items): 2048 keys per split.
//   * Otherwise the split size c, in multiples of 64 keys, that maximises keys streamed per slot and unit of time
//     when the CTAs run in rounds of (c + 64): ranges x keys / (slots x ceil(items / slots) x (c + 64)). (Counting the
//     short last split of a range as a full one, as an earlier form of this rule did, picked 960 for 28 x 4096 keys:
//     four rounds of 1024; 832 - five equal splits, four rounds of 896 - streams the same keys in 12 % less.)
DecodePlan decode_plan(const ingot_kv* kv, int n_layers, int n_seq, int max_seq_len, int chunk_keys) {
    const int n_warps = decode_warps_cfg();
    const int min_chunk = ((max_seq_len + kMaxParts - 1) / kMaxParts + 15) / 16 * 16;
    if (chunk_keys == 0) {
        const int slots = kv->num_sms * (8 / n_warps);
        const long long ranges = (long long)n_layers * n_seq * kv->n_head_kv;
        if (max_seq_len <= 256) {
            chunk_keys = 256;  // one split per range: its CTA writes the output itself and no merge launch is needed
        } else if (ranges * ((max_seq_len + 511) / 512) <= slots) {
            const int per_range = (int)std::max<long long>(1, slots / ranges);
            const int quantum = n_warps * 16;
            chunk_keys = ((max_seq_len + per_range - 1) / per_range + quantum - 1) / quantum * quantum;
            chunk_keys = std::min(std::max(chunk_keys, quantum), 512);
        } else if (n_seq > 1) {
            chunk_keys = 2048;
        } else {
            double best = -1.0;
            for (int c = 256; c <= 4096 && c < max_seq_len + 64; c += 64) {
                const long long items = ranges * ((max_seq_len + c - 1) / c);
                const long long rounds = (items + slots - 1) / slots;
                // keys streamed / (slots x time), a round costing a full split plus its start-up
                const double score = (double)ranges * max_seq_len / ((double)slots * rounds * (c + 64));
                if (score > best) { best = score; chunk_keys = c; }
            }
        }
    }
    chunk_keys = std::max(chunk_keys, min_chunk);
    DecodePlan plan;
    plan.chunk_keys = chunk_keys;
    plan.n_parts = (max_seq_len + chunk_keys - 1) / chunk_keys;
    return plan;
}
int decode_slots(const ingot_kv* kv) { return kv->num_sms * (8 / decode_warps_cfg()); }

size_t decode_part_floats(int n_seq, int n_parts, int n_head) {
    return (size_t)n_seq * n_parts * n_head * kPartStride;
}

// One launch of the decode kernel over `n_layers` consecutive layers starting at `layer`: either the split CTAs
// (merge_only == 0; partials of split ranges into `part`, outputs of single-split ranges straight into `out`) or
// one merge CTA per (kv head, layer, sequence) that turns the partials in `part` into `out` (merge_only != 0; a
// no-op when the plan has a single split). q and out are [n_layers][n_seq][n_head][128], `part` holds n_layers
// blocks of decode_part_floats(). pdl_mode: kPdlWaitFirst or kPdlEarlyLoads (see DecodeParams).
int launch_attn_decode(ingot_kv* kv, int layer, int n_layers, const void* q, int q_dtype, void* out, int out_dtype, int n_head,
                       int n_seq, const int32_t* seq_lens, int max_seq_len, const int32_t* block_tables,
                       int max_blocks_per_seq, DecodePlan plan, float* part, int merge_only, int pdl_mode, cudaStream_t stream) {
    if (merge_only && plan.n_parts <= 1) return INGOT_OK;
    const int n_warps = decode_warps_cfg();
    DecodeParams p;
    p.kc = kv->k + size_t(layer) * kv->layer_elems;
    p.vc = kv->v + size_t(layer) * kv->layer_elems;
    p.q = q; p.out = out; p.seq_lens = seq_lens; p.block_tables = block_tables;
    p.part = part; p.c_part = part; p.c_out = out; p.status = kv->status_dev;
    p.n_seq = n_seq;
    p.cache_layer_stride = kv->layer_elems;
    p.qo_layer_stride = (size_t)n_seq * n_head * kHeadDim;
    p.part_layer_stride = decode_part_floats(n_seq, plan.n_parts, n_head);
    p.cache_extent = kv->checked_cache_elems();
    p.part_extent = p.part_layer_stride * n_layers;
    p.out_extent = p.qo_layer_stride * n_layers;
    p.q_dtype = q_dtype; p.out_dtype = out_dtype;
    p.n_head = n_head; p.n_head_kv = kv->n_head_kv; p.group = n_head / kv->n_head_kv;
    p.capacity = kv->capacity; p.paged = kv->layout == INGOT_KV_PAGED; p.max_blocks_per_seq = max_blocks_per_seq;
    p.len0 = max_seq_len; p.chunk_keys = plan.chunk_keys; p.n_parts_max = plan.n_parts;
    p.pdl_mode = pdl_mode;
    p.split_parts = merge_only ? 0 : plan.n_parts;
    p.scale_log2 = 1.4426950408889634f / sqrtf(float(kHeadDim));
    const int threads = n_warps * 32;
    const size_t smem_split = (size_t)n_warps * p.group * (kHeadDim + 2);
    const size_t smem_merge = (size_t)2 * p.group * kMaxParts + (size_t)4 * std::max(threads, p.group * 32);
    const size_t smem = std::max(smem_split, smem_merge) * sizeof(float);
    const dim3 grid(merge_only ? 1 : plan.n_parts, kv->n_head_kv, (unsigned)(n_layers * n_seq));
    INGOT_CUDA_TRY(ingot_launch_pdl(attn_decode_kernel, grid, dim3(threads), smem, stream, p));
    return INGOT_OK;
}

// ---- decode without any allocation ----------------------------------------------------------------
// Some callers must not allocate device memory at all: code that runs inside a memory pool it does
// not own, a plugin that is only handed pre-allocated buffers by its host application, or a
// latency-critical serving loop where cudaMalloc/cudaFree (which synchronise the device) are
// forbidden. For them the split partials live in a fixed array inside the library image instead of
// the cache handle's heap scratch. Every GPU that loads the library holds these 2.06 MiB until exit.
namespace {
constexpr int kStaticMaxHeads = 64;  // most query heads one call may carry
constexpr int kStaticMaxDevices = 64;
static __device__ __align__(256) float g_static_part[(size_t)kMaxParts * kStaticMaxHeads * kPartStride];
float* g_static_part_addr[kStaticMaxDevices] = {};
int g_static_sms[kStaticMaxDevices] = {};
std::mutex g_static_mu;
}  // namespace

extern "C" int ingot_attn_decode_noalloc(const void* k_dev, const void* v_dev, int n_ctx, int n_head_kv, const void* q_dev,
                                         int q_dtype, void* out_dev, int out_dtype, int n_head, int n_keys, int chunk_keys,
                                         void* stream) {
    INGOT_REQUIRE(k_dev && v_dev && q_dev && out_dev, "ingot_attn_decode_noalloc: null pointer");
    INGOT_REQUIRE(n_head_kv >= 1 && n_head >= n_head_kv && n_head % n_head_kv == 0,
                  "ingot_attn_decode_noalloc: n_head must be a multiple of n_head_kv");
    INGOT_REQUIRE(n_keys >= 1 && n_keys <= n_ctx, "context window exceeded");
    INGOT_REQUIRE(chunk_keys >= 0 && chunk_keys % 16 == 0, "ingot_attn_decode_noalloc: chunk_keys must be a multiple of 16");
    if (n_head > kStaticMaxHeads) {
        ingot_set_error("ingot_attn_decode_noalloc: n_head exceeds the 64 heads the built-in scratch is sized for; "
                        "use ingot_attn_decode");
        return INGOT_ERR_INVALID;
    }
    if (n_head / n_head_kv > 8 || (q_dtype != INGOT_F32 && q_dtype != INGOT_F16 && q_dtype != INGOT_BF16) ||
        (out_dtype != INGOT_F32 && out_dtype != INGOT_F16)) {
        ingot_set_error("ingot_attn_decode_noalloc: group size > 8 or unsupported dtype");
        return INGOT_ERR_UNSUPPORTED;
    }
    int dev = 0;
    INGOT_CUDA_TRY(cudaGetDevice(&dev));
    INGOT_REQUIRE(dev >= 0 && dev < kStaticMaxDevices, "ingot_attn_decode_noalloc: device index too large");
    float* scratch = nullptr;
    int sms = 0;
    {
        // First call on this device: resolve the device address of the array. The array's name is only
        // a host-side handle; the kernel must be given the address cudaGetSymbolAddress reports, taken
        // with this device current.
        std::lock_guard<std::mutex> lk(g_static_mu);
        if (!g_static_part_addr[dev]) {
            void* addr = nullptr;
            INGOT_CUDA_TRY(cudaGetSymbolAddress(&addr, g_static_part));
            INGOT_CUDA_TRY(cudaDeviceGetAttribute(&g_static_sms[dev], cudaDevAttrMultiProcessorCount, dev));
            g_static_part_addr[dev] = static_cast<float*>(addr);
        }
        scratch = g_static_part_addr[dev];
        sms = g_static_sms[dev];
    }
    const int n_warps = 4;
    if (chunk_keys == 0) {
        const int per_head = max(1, sms * 2 / n_head_kv);
        chunk_keys = ((n_keys + per_head - 1) / per_head + 63) / 64 * 64;
        chunk_keys = min(max(chunk_keys, 64), 512);
    }
    chunk_keys = max(chunk_keys, ((n_keys + kMaxParts - 1) / kMaxParts + 15) / 16 * 16);
    const int n_parts = (n_keys + chunk_keys - 1) / chunk_keys;  // <= kMaxParts, so the partials fit the array

    DecodeParams p;
    p.kc = static_cast<const __half*>(k_dev);
    p.vc = static_cast<const __half*>(v_dev);
    p.q = q_dev; p.out = out_dev; p.seq_lens = nullptr; p.block_tables = nullptr;
    p.part = scratch; p.c_part = scratch; p.c_out = out_dev; p.status = nullptr;
    p.n_seq = 1; p.cache_layer_stride = 0; p.qo_layer_stride = 0; p.part_layer_stride = 0;
    p.cache_extent = (size_t)n_head_kv * n_ctx * kHeadDim;
    p.part_extent = (size_t)kMaxParts * kStaticMaxHeads * kPartStride;
    p.out_extent = (size_t)n_head * kHeadDim;
    p.q_dtype = q_dtype; p.out_dtype = out_dtype;
    p.n_head = n_head; p.n_head_kv = n_head_kv; p.group = n_head / n_head_kv;
    p.capacity = n_ctx; p.paged = 0; p.max_blocks_per_seq = 0;
    p.len0 = n_keys; p.chunk_keys = chunk_keys; p.n_parts_max = n_parts;
    p.pdl_mode = 0;
    p.scale_log2 = 1.4426950408889634f / sqrtf(float(kHeadDim));
    const int threads = n_warps * 32;
    const size_t smem_split = (size_t)n_warps * p.group * (kHeadDim + 2);
    const size_t smem_merge = (size_t)2 * p.group * kMaxParts + (size_t)4 * max(threads, p.group * 32);
    const size_t smem = max(smem_split, smem_merge) * sizeof(float);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    p.split_parts = n_parts;
    attn_decode_kernel<<<dim3(n_parts, n_head_kv, 1), threads, smem, s>>>(p);
    INGOT_CUDA_TRY(cudaGetLastError());
    if (n_parts > 1) {  // merge-only launch; stream order makes the partials visible
        p.split_parts = 0;
        attn_decode_kernel<<<dim3(1, n_head_kv, 1), threads, smem, s>>>(p);
        INGOT_CUDA_TRY(cudaGetLastError());
    }
    return INGOT_OK;
}
#endif  // !INGOT_DECODE_APPEND

#ifdef INGOT_DECODE_APPEND
// One launch of the fused form for one token of one sequence on a contiguous cache: q/k/v are the f32 projections, the
// key count (position + 1) comes from seq_lens (device) or max_seq_len. Splits and partials as in launch_attn_decode;
// with more than one split the caller follows up with the plain kernel's merge-only launch.
int launch_attn_decode_append(ingot_kv* kv, int layer, const float* q, const float* k, const float* v, const float* inv_freq, void* out,
                              int out_dtype, int n_head, const int32_t* seq_lens, int max_seq_len, DecodePlan plan, float* part,
                              cudaStream_t stream) {
    const int n_warps = decode_warps_cfg();
    DecodeAppendParams p;
    p.kc = kv->k + size_t(layer) * kv->layer_elems;
    p.vc = kv->v + size_t(layer) * kv->layer_elems;
    p.kc_w = kv->k + size_t(layer) * kv->layer_elems;
    p.vc_w = kv->v + size_t(layer) * kv->layer_elems;
    p.q = nullptr; p.out = out; p.seq_lens = seq_lens; p.block_tables = nullptr;
    p.part = part; p.c_part = part; p.c_out = out; p.status = kv->status_dev;
    p.q_f32 = q; p.k_new = k; p.v_new = v; p.inv_freq = inv_freq;
    p.n_seq = 1;
    p.cache_layer_stride = kv->layer_elems;
    p.qo_layer_stride = (size_t)n_head * kHeadDim;
    p.part_layer_stride = decode_part_floats(1, plan.n_parts, n_head);
    p.cache_extent = kv->checked_cache_elems();
    p.part_extent = p.part_layer_stride;
    p.out_extent = p.qo_layer_stride;
    p.q_dtype = INGOT_F32; p.out_dtype = out_dtype;
    p.n_head = n_head; p.n_head_kv = kv->n_head_kv; p.group = n_head / kv->n_head_kv;
    p.capacity = kv->capacity; p.paged = 0; p.max_blocks_per_seq = 0;
    p.len0 = max_seq_len; p.chunk_keys = plan.chunk_keys; p.n_parts_max = plan.n_parts;
    p.pdl_mode = kPdlWaitFirst;
    p.split_parts = plan.n_parts;
    p.scale_log2 = 1.4426950408889634f / sqrtf(float(kHeadDim));
    const int threads = n_warps * 32;
    const size_t smem_split = (size_t)n_warps * p.group * (kHeadDim + 2);
    const size_t smem_merge = (size_t)2 * p.group * kMaxParts + (size_t)4 * std::max(threads, p.group * 32);
    const size_t smem = std::max(smem_split, smem_merge) * sizeof(float);
    const dim3 grid(plan.n_parts, kv->n_head_kv, 1);
    INGOT_CUDA_TRY(ingot_launch_pdl(attn_decode_append_kernel, grid, dim3(threads), smem, stream, p));
    return INGOT_OK;
}
#endif
