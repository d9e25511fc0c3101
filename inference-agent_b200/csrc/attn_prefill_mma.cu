// K2 (warp-MMA form) — causal GQA flash-attention prefill / chunked prefill on warp-level
// m16n8k16 f16 MMAs, for short chunks and paged caches. The tcgen05/TMEM/TMA kernel in
// attn_prefill_sm100.cu takes over for long contiguous prefills.
//
// Replaces n_tok iterations of the CPU reference's attention lambda (src/backend.h:16-20 looping
// src/cpu_backend.cpp:51-69) and Metal's attn_prefill (shaders/kernels.metal:518-633): query token
// i sits at position q_pos0 + i and attends to keys 0..q_pos0+i (mask `key <= qpos`,
// kernels.metal:578; chunk offset `pos`, :555).
//
// Work decomposition. One CTA = one KV head x 64 query ROWS, where a row is a (token, query head of
// the group) pair: row R -> token R / G, head R % G. Packing the G query heads that share a KV head
// into the M dimension means a K/V tile staged in shared memory is used by all of them (the Metal
// kernel re-reads K/V once per head and per 8 queries). Four warps, 16 rows each. K/V tiles of 64
// keys are staged with 16-byte cp.async copies, double buffered. Fragments are read from shared
// memory as 16-byte chunks and fed to the MMAs through the same k-permutation trick as the decode
// kernel (see attn_decode.cu); row strides of 320 B (K) and 272 B (V) make those reads conflict-free.
// Online softmax in the exp2 domain with f32 state; P is rounded to f16 for the PV MMA (bf16 would
// break the 2e-3 tolerance at early positions); scores are scaled in f32 after the MMA.
#include "attn_common.cuh"
#include "ingot_internal.cuh"

namespace {

constexpr int kBM = 64;       // query rows per CTA
constexpr int kBN = 64;       // keys per tile
constexpr int kKStride = 160; // halves per K row in shared memory (320 B)
constexpr int kVStride = 136; // halves per V row in shared memory (272 B)
constexpr int kPrefillThreads = 128;

struct PrefillParams {
    const __half* kc;
    const __half* vc;
    const void* q;
    void* out;
    const int32_t* block_table;
    int* status;
    int q_dtype, out_dtype;
    int n_head, n_head_kv, group;
    int capacity, paged;
    int q_pos0, n_tok;
    float scale_log2;
    size_t cache_extent;  // bounds-check build: elements of one cache layer
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ uint4 lds16(const __half* p) { return *reinterpret_cast<const uint4*>(p); }

__global__ void __launch_bounds__(kPrefillThreads) attn_prefill_mma_kernel(const PrefillParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* sK = reinterpret_cast<__half*>(smem_raw);                 // [2][kBN][kKStride]
    __half* sV = sK + 2 * kBN * kKStride;                            // [2][kBN][kVStride]

    INGOT_PDL_TRIGGER();
    INGOT_PDL_WAIT();  // q and the newest cache rows come from the kernel before
    const int G = p.group;
    const int kvh = blockIdx.y;
    const int n_rows = p.n_tok * G;
    // Heavier (later) tiles first: causal work grows with the row index.
    const int tile = gridDim.x - 1 - blockIdx.x;
    const int row0 = tile * kBM;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, j = lane & 3;

    const int r_lo = row0 + warp * 16 + g, r_hi = r_lo + 8;
    const bool ok_lo = r_lo < n_rows, ok_hi = r_hi < n_rows;
    const int tok_lo = r_lo / G, tok_hi = r_hi / G;
    const int n_keys_total = p.q_pos0 + p.n_tok;
    // Rows past the end behave like the last token so that they never see a fully masked tile.
    const int qpos_lo = p.q_pos0 + (ok_lo ? tok_lo : p.n_tok - 1);
    const int qpos_hi = p.q_pos0 + (ok_hi ? tok_hi : p.n_tok - 1);

    uint4 qlo[4], qhi[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        qlo[i] = ok_lo ? load_q8(p.q, p.q_dtype, ((size_t)tok_lo * p.n_head + (size_t)kvh * G + r_lo % G) * kHeadDim + (4 * i + j) * 8)
                       : make_uint4(0, 0, 0, 0);
        qhi[i] = ok_hi ? load_q8(p.q, p.q_dtype, ((size_t)tok_hi * p.n_head + (size_t)kvh * G + r_hi % G) * kHeadDim + (4 * i + j) * 8)
                       : make_uint4(0, 0, 0, 0);
    }

    // Keys this CTA needs: up to the position of its last valid row.
    const int last_row = min(row0 + kBM, n_rows) - 1;
    const int cta_keys = p.q_pos0 + last_row / G + 1;
    const int n_tiles = (cta_keys + kBN - 1) / kBN;
    // First tile that may need masking: the one holding the earliest row's position.
    const int first_masked_tile = (p.q_pos0 + row0 / G) / kBN;

    auto stage_tile = [&](int t, int buf) {
        __half* dK = sK + buf * kBN * kKStride;
        __half* dV = sV + buf * kBN * kVStride;
        // 64 rows x 16 chunks per matrix; 128 threads -> 8 K chunks + 8 V chunks each.
#pragma unroll
        for (int it = 0; it < 8; it++) {
            const int idx = it * kPrefillThreads + threadIdx.x;
            const int row = idx >> 4, c = idx & 15;
            const int key = min(t * kBN + row, n_keys_total - 1);  // clamped rows are masked below
            size_t off;
            if (!p.paged) {
                off = kv_row_offset_contig(p.capacity, kvh, key);
            } else {
                int blk = p.block_table[key >> 4];
                if (blk < 0 || blk >= p.capacity) {
                    if (c == 0) atomicOr(p.status, kDevErrBlockRange);
                    blk = 0;
                }
                off = kv_row_offset_paged(p.n_head_kv, blk, kvh, key);
            }
            if (!INGOT_CHECK(off + c * 8, 8, p.cache_extent, p.status)) off = 0;  // flagged; a harmless row instead
            cp_async16(smem_u32(dK + row * kKStride + c * 8), p.kc + off + c * 8);
            cp_async16(smem_u32(dV + row * kVStride + c * 8), p.vc + off + c * 8);
        }
        cp_async_commit();
    };

    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    float o[16][4];
#pragma unroll
    for (int t = 0; t < 16; t++) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;

    stage_tile(0, 0);
    for (int t = 0; t < n_tiles; t++) {
        const int buf = t & 1;
        if (t + 1 < n_tiles) {
            stage_tile(t + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const __half* tK = sK + buf * kBN * kKStride;
        const __half* tV = sV + buf * kBN * kVStride;

        // ---- S = Q K^T : 8 n-tiles of 8 keys ----
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint4 kk = lds16(tK + (nt * 8 + g) * kKStride + (4 * i + j) * 8);
                mma_16816(s[nt], qlo[i].x, qhi[i].x, qlo[i].y, qhi[i].y, kk.x, kk.y);
                mma_16816(s[nt], qlo[i].z, qhi[i].z, qlo[i].w, qhi[i].w, kk.z, kk.w);
            }
        }

        // ---- online softmax (exp2 domain) ----
        const bool need_mask = t >= first_masked_tile;
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int key = t * kBN + nt * 8 + 2 * j + e;
                float x_lo = s[nt][e] * p.scale_log2, x_hi = s[nt][2 + e] * p.scale_log2;
                if (need_mask) {
                    if (key > qpos_lo) x_lo = -INFINITY;
                    if (key > qpos_hi) x_hi = -INFINITY;
                }
                s[nt][e] = x_lo;
                s[nt][2 + e] = x_hi;
                mx_lo = fmaxf(mx_lo, x_lo);
                mx_hi = fmaxf(mx_hi, x_hi);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        // Key 0 is visible to every row, so after tile 0 the running max is finite.
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        const float a_lo = exp2f(m_lo - mn_lo), a_hi = exp2f(m_hi - mn_hi);
        m_lo = mn_lo;
        m_hi = mn_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
        uint32_t pa[8][2];  // [n-tile][row half] packed f16 pairs
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            const float p0 = exp2f(s[nt][0] - mn_lo), p1 = exp2f(s[nt][1] - mn_lo);
            const float p2 = exp2f(s[nt][2] - mn_hi), p3 = exp2f(s[nt][3] - mn_hi);
            sum_lo += p0 + p1;
            sum_hi += p2 + p3;
            pa[nt][0] = pack_half2_rn(p0, p1);
            pa[nt][1] = pack_half2_rn(p2, p3);
        }
        l_lo = l_lo * a_lo + sum_lo;
        l_hi = l_hi * a_hi + sum_hi;
#pragma unroll
        for (int tt = 0; tt < 16; tt++) {
            o[tt][0] *= a_lo; o[tt][1] *= a_lo;
            o[tt][2] *= a_hi; o[tt][3] *= a_hi;
        }

        // ---- O += P V : 4 k-steps of 16 keys x 16 n-tiles of dims ----
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            const __half* v0 = tV + (ks * 16 + 2 * j) * kVStride;
#pragma unroll
            for (int c = 0; c < 2; c++) {
                const int col = (g + 8 * c) * 8;
                const uint4 ra = lds16(v0 + col);                  // key 2j
                const uint4 rb = lds16(v0 + kVStride + col);       // key 2j+1
                const uint4 rc = lds16(v0 + 8 * kVStride + col);   // key 2j+8
                const uint4 rd = lds16(v0 + 9 * kVStride + col);   // key 2j+9
                const uint32_t va[4] = {ra.x, ra.y, ra.z, ra.w}, vb[4] = {rb.x, rb.y, rb.z, rb.w};
                const uint32_t vc[4] = {rc.x, rc.y, rc.z, rc.w}, vd[4] = {rd.x, rd.y, rd.z, rd.w};
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const int tt = c * 8 + 2 * w;
                    mma_16816(o[tt], pa[2 * ks][0], pa[2 * ks][1], pa[2 * ks + 1][0], pa[2 * ks + 1][1],
                              prmt(va[w], vb[w], 0x5410), prmt(vc[w], vd[w], 0x5410));
                    mma_16816(o[tt + 1], pa[2 * ks][0], pa[2 * ks][1], pa[2 * ks + 1][0], pa[2 * ks + 1][1],
                              prmt(va[w], vb[w], 0x7632), prmt(vc[w], vd[w], 0x7632));
                }
            }
        }
        __syncthreads();  // everyone is done with this buffer before it is refilled
    }

    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

    // Thread (g, j) holds, for its two rows, dims [16j, 16j+16) and [64+16j, 64+16j+16):
    // o[t][0] / o[t][1] (row g) and o[t][2] / o[t][3] (row g+8) with dim = (t>>3)*64 + 16j + 8*e + (t&7).
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const bool ok = half ? ok_hi : ok_lo;
        if (!ok) continue;
        const int r = half ? r_hi : r_lo;
        const float inv = 1.0f / (half ? l_hi : l_lo);
        const size_t base = ((size_t)(r / G) * p.n_head + (size_t)kvh * G + r % G) * kHeadDim;
#pragma unroll
        for (int c = 0; c < 2; c++) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                float vals[8];
#pragma unroll
                for (int w = 0; w < 8; w++) vals[w] = o[c * 8 + w][half * 2 + e] * inv;
                const size_t off = base + c * 64 + 16 * j + 8 * e;
                if (p.out_dtype == INGOT_F32) {
                    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.out) + off);
                    dst[0] = make_float4(vals[0], vals[1], vals[2], vals[3]);
                    dst[1] = make_float4(vals[4], vals[5], vals[6], vals[7]);
                } else {
                    uint4 pk = make_uint4(pack_half2_rn(vals[0], vals[1]), pack_half2_rn(vals[2], vals[3]),
                                          pack_half2_rn(vals[4], vals[5]), pack_half2_rn(vals[6], vals[7]));
                    *reinterpret_cast<uint4*>(static_cast<__half*>(p.out) + off) = pk;
                }
            }
        }
    }
}

}  // namespace

int launch_attn_prefill_mma(ingot_kv* kv, int layer, const void* q, int q_dtype, void* out, int out_dtype,
                            int n_head, int q_pos0, int n_tok, const int32_t* block_table, cudaStream_t stream) {
    PrefillParams p;
    p.kc = kv->k + size_t(layer) * kv->layer_elems;
    p.vc = kv->v + size_t(layer) * kv->layer_elems;
    p.q = q; p.out = out; p.block_table = block_table; p.status = kv->status_dev;
    p.q_dtype = q_dtype; p.out_dtype = out_dtype;
    p.n_head = n_head; p.n_head_kv = kv->n_head_kv; p.group = n_head / kv->n_head_kv;
    p.capacity = kv->capacity; p.paged = kv->layout == INGOT_KV_PAGED;
    p.q_pos0 = q_pos0; p.n_tok = n_tok;
    p.cache_extent = kv->checked_cache_elems();
    p.scale_log2 = 1.4426950408889634f / sqrtf(float(kHeadDim));
    const size_t smem = size_t(2) * kBN * (kKStride + kVStride) * sizeof(__half);
    if (!kv->prefill_mma_attr_set) {  // function attributes belong to a device context: once per handle, not per process
        INGOT_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        kv->prefill_mma_attr_set = true;
    }
    const long long n_rows = (long long)n_tok * p.group;
    dim3 grid(unsigned((n_rows + kBM - 1) / kBM), kv->n_head_kv);
    INGOT_CUDA_TRY(ingot_launch_pdl(attn_prefill_mma_kernel, grid, dim3(kPrefillThreads), smem, stream, p));
    return INGOT_OK;
}
