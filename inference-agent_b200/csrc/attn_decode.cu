// K3 — split-KV flash decoding for one-token queries over the f16 KV cache (contiguous or paged).
//
// Replaces the attention lambda of the CPU reference for a single query token
// (src/cpu_backend.cpp:51-69) and Metal's attn_decode_g3 + attn_combine pair
// (shaders/kernels.metal:428-516, dispatch src/metal_backend.mm:340-360) with ONE launch.
//
// Work decomposition. grid = (splits, kv heads, sequences). A CTA owns one KV head of one sequence
// over one split of `chunk_keys` keys and serves ALL query heads that share that KV head (GQA), so
// every K/V byte is fetched from HBM exactly once. Inside the CTA each warp walks its own 16-key
// units with a private online-softmax state (m, l, o); the warp states are merged through shared
// memory, the split's partial (o[128], m, l per head) goes to a global scratch, and the last CTA
// of a (sequence, kv head) to arrive — found with an atomic ticket, nobody waits — merges the
// partials: out = sum_s o_s 2^(m_s-M) / sum_s l_s 2^(m_s-M), the attn_combine formula.
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

namespace {

constexpr int kMaxDecodeWarps = 8;
constexpr int kMaxParts = 64;

struct DecodeParams {
    const __half* kc;   // layer base
    const __half* vc;
    const void* q;
    void* out;
    const int32_t* seq_lens;
    const int32_t* block_tables;
    float* part;
    unsigned int* counters;
    int* status;
    int q_dtype, out_dtype;
    int n_head, n_head_kv, group;
    int capacity, paged, max_blocks_per_seq;
    int len0, chunk_keys, n_parts_max;
    float scale_log2;
};

struct KRegs { uint4 k[8]; };  // [n-tile 0/1][i=0..3]: key (nt*8 + g), 16-byte chunk (4i + j)
struct VRegs { uint4 v[8]; };  // [slot 0..3 -> keys 2j, 2j+1, 2j+8, 2j+9][chunk g / g+8]

__global__ void __launch_bounds__(kMaxDecodeWarps * 32, 1) attn_decode_kernel(const DecodeParams p) {
    extern __shared__ float smem[];
    const int chunk = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    const int n_keys = p.seq_lens ? p.seq_lens[seq] : p.len0;
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

    // Query fragments: head row g, chunks 4i + j.
    uint4 qa[4];
    if (g < G) {
        const size_t qbase = ((size_t)seq * p.n_head + (size_t)kvh * G + g) * kHeadDim;
#pragma unroll
        for (int i = 0; i < 4; i++) qa[i] = load_q8(p.q, p.q_dtype, qbase + (size_t)(4 * i + j) * 8);
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) qa[i] = make_uint4(0, 0, 0, 0);
    }

    const int32_t* bt = p.paged ? p.block_tables + (size_t)seq * p.max_blocks_per_seq : nullptr;

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
        const __half* kb = p.kc + unit_base(u);
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            const int row = min(nt * 8 + g, last);
#pragma unroll
            for (int i = 0; i < 4; i++) r.k[nt * 4 + i] = ld_stream16(kb + (size_t)row * kHeadDim + (4 * i + j) * 8);
        }
    };
    auto load_v = [&](VRegs& r, int u) {
        const int last = n_keys - 1 - (k_begin + (u << 4));
        const __half* vb = p.vc + unit_base(u);
#pragma unroll
        for (int s = 0; s < 4; s++) {
            const int row = min(2 * j + (s & 1) + (s >> 1) * 8, last);
            r.v[s * 2 + 0] = ld_stream16(vb + (size_t)row * kHeadDim + g * 8);
            r.v[s * 2 + 1] = ld_stream16(vb + (size_t)row * kHeadDim + (g + 8) * 8);
        }
    };

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

    // Key loop, software-pipelined: while unit u is consumed the loads of the warp's next unit are
    // in flight (K of the next unit is requested before QK^T of this one, V before PV), so a warp
    // keeps 8-12 KB outstanding and at most three 4 KB register sets are live at a time.
    {
        KRegs ka, kb;
        VRegs va, vb;
        int u = warp;
        if (u < n_units) { load_k(ka, u); load_v(va, u); }
        while (u < n_units) {
            const int u1 = u + n_warps;
            if (u1 < n_units) load_k(kb, u1);
            compute_qk(ka, u);
            if (u1 < n_units) load_v(vb, u1);
            compute_pv(va);
            if (u1 >= n_units) break;
            const int u2 = u1 + n_warps;
            if (u2 < n_units) load_k(ka, u2);
            compute_qk(kb, u1);
            if (u2 < n_units) load_v(va, u2);
            compute_pv(vb);
            u = u2;
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

    const bool single = n_chunks == 1;
    const size_t part_row0 = ((size_t)seq * p.n_parts_max + chunk) * p.n_head + (size_t)kvh * G;
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
            store_out(p.out, p.out_dtype, ((size_t)seq * p.n_head + (size_t)kvh * G + gi) * kHeadDim + dim, O / L);
        } else {
            float* row = p.part + (part_row0 + gi) * kPartStride;
            row[dim] = O;
            if (dim == 0) { row[128] = M; row[129] = L; }
        }
    }
    if (single) return;

    // ---- last CTA of this (sequence, kv head) merges the splits ----
    __shared__ int s_is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int* ctr = p.counters + (size_t)seq * p.n_head_kv + kvh;
        const unsigned int prev = atomicAdd(ctr, 1u);
        s_is_last = prev == (unsigned int)(n_chunks - 1);
        if (s_is_last) *ctr = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!s_is_last) return;
    __threadfence();
    for (int idx = threadIdx.x; idx < G * kHeadDim; idx += blockDim.x) {
        const int gi = idx >> 7, dim = idx & 127;
        const float* rows = p.part + (((size_t)seq * p.n_parts_max) * p.n_head + (size_t)kvh * G + gi) * kPartStride;
        const size_t step = (size_t)p.n_head * kPartStride;
        float M = -INFINITY;
        for (int c = 0; c < n_chunks; c++) M = fmaxf(M, __ldcg(rows + c * step + 128));
        float L = 0.f, O = 0.f;
        for (int c = 0; c < n_chunks; c++) {
            const float wgt = exp2f(__ldcg(rows + c * step + 128) - M);
            L += __ldcg(rows + c * step + 129) * wgt;
            O += __ldcg(rows + c * step + dim) * wgt;
        }
        store_out(p.out, p.out_dtype, ((size_t)seq * p.n_head + (size_t)kvh * G + gi) * kHeadDim + dim, L > 0.f ? O / L : 0.f);
    }
}

int g_num_sms = 0;

}  // namespace

size_t decode_part_floats(int n_seq, int /*max_seq_len*/, int n_head) {
    return (size_t)n_seq * kMaxParts * n_head * kPartStride;
}

int launch_attn_decode(ingot_kv* kv, int layer, const void* q, int q_dtype, void* out, int out_dtype, int n_head,
                       int n_seq, const int32_t* seq_lens, int max_seq_len, const int32_t* block_tables,
                       int max_blocks_per_seq, int chunk_keys, float* part, unsigned int* counters,
                       cudaStream_t stream) {
    if (g_num_sms == 0) {
        int dev = 0;
        INGOT_CUDA_TRY(cudaGetDevice(&dev));
        INGOT_CUDA_TRY(cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev));
    }
    const int n_warps = 4;
    if (chunk_keys == 0) {
        // Aim for two resident CTAs per SM; never fewer than 64 keys per split on small jobs and
        // never more than 512 on large ones (keeps variable-length batches balanced).
        const int target = 2 * g_num_sms;
        const int per_head = max(1, target / (n_seq * kv->n_head_kv));
        chunk_keys = ((max_seq_len + per_head - 1) / per_head + 15) / 16 * 16;
        chunk_keys = min(max(chunk_keys, 64), 512);
    }
    const int min_chunk = ((max_seq_len + kMaxParts - 1) / kMaxParts + 15) / 16 * 16;
    chunk_keys = max(chunk_keys, min_chunk);
    const int n_parts = (max_seq_len + chunk_keys - 1) / chunk_keys;

    DecodeParams p;
    p.kc = kv->k + size_t(layer) * kv->layer_elems;
    p.vc = kv->v + size_t(layer) * kv->layer_elems;
    p.q = q; p.out = out; p.seq_lens = seq_lens; p.block_tables = block_tables;
    p.part = part; p.counters = counters; p.status = kv->status_dev;
    p.q_dtype = q_dtype; p.out_dtype = out_dtype;
    p.n_head = n_head; p.n_head_kv = kv->n_head_kv; p.group = n_head / kv->n_head_kv;
    p.capacity = kv->capacity; p.paged = kv->layout == INGOT_KV_PAGED; p.max_blocks_per_seq = max_blocks_per_seq;
    p.len0 = max_seq_len; p.chunk_keys = chunk_keys; p.n_parts_max = n_parts;
    p.scale_log2 = 1.4426950408889634f / sqrtf(float(kHeadDim));
    const size_t smem = (size_t)n_warps * p.group * (kHeadDim + 2) * sizeof(float);
    dim3 grid(n_parts, kv->n_head_kv, n_seq);
    attn_decode_kernel<<<grid, n_warps * 32, smem, stream>>>(p);
    INGOT_CUDA_TRY(cudaGetLastError());
    return INGOT_OK;
}
