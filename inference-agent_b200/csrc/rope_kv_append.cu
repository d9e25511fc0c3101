// K1 — fused rotary embedding + KV-cache append (+ rotated-query f16 cast), one launch per layer.
//
// Replaces, per token: ops::rope on q and k and the two cache memcpys of the CPU reference
// (src/ops.cpp:243-255, src/cpu_backend.cpp:43-49), i.e. the three Metal dispatches rope,
// rope_k_to_cache and to_half (shaders/kernels.metal:256-282, 779-782).
//
// Arithmetic follows src/ops.cpp:248-253 exactly in f32: angle = float(pos) * inv_freq[i], then
// (x0, x1) <- (x0*c - x1*s, x0*s + x1*c) on ADJACENT elements (2i, 2i+1). cosf/sinf are the
// full-range library versions (angles reach ~3e4 rad at position 32767), never the fast
// intrinsics. Results are rounded once to f16 for the cache / the tensor-core query operand.
//
// HBM-bound elementwise work: each thread moves 8 consecutive elements (two 16-byte f32 loads,
// one 16-byte f16 store), fully coalesced on both sides. Algorithmic bytes per token:
// (n_head + 2*n_head_kv) * 128 * (4 in + 2 out).
#include "ingot_internal.cuh"
#include "rope_unit.cuh"

namespace {

struct AppendParams {
    const float* q;       // [n_tok][n_head][128] or null
    __half* q_out;        // [n_tok][n_head][128]
    const float* k;       // [n_tok][n_head_kv][128]
    const float* v;
    const float* inv_freq;  // [64]
    __half* kc;           // layer base of the K cache
    __half* vc;
    const int32_t* positions;
    const int32_t* seq_ids;
    const int32_t* block_tables;
    int* status;
    int n_head, n_head_kv, n_tok, pos0;
    int capacity;            // positions (contiguous) or blocks (paged)
    int max_blocks_per_seq;
    int paged;
    size_t layer_elems;      // cache elements between consecutive layers (blockIdx.y = layer offset)
    size_t cache_extent;     // elements of one layer the kernel may touch (bounds-check build)
};

// Destination element offset of (kv head h, position pos) for token `tok`, or -1 if out of range.
__device__ __forceinline__ long long cache_row(const AppendParams& p, int tok, int h, int pos) {
    if (pos < 0) return -1;
    if (!p.paged) {
        if (pos >= p.capacity) return -1;
        return (long long)kv_row_offset_contig(p.capacity, h, pos);
    }
    const int lb = pos / kBlockTokens;
    if (lb >= p.max_blocks_per_seq) return -1;
    const int seq = p.seq_ids ? p.seq_ids[tok] : 0;
    const int blk = p.block_tables[(size_t)seq * p.max_blocks_per_seq + lb];
    if (blk < 0 || blk >= p.capacity) return -2;
    return (long long)kv_row_offset_paged(p.n_head_kv, blk, h, pos);
}

__global__ void __launch_bounds__(256) rope_kv_append_kernel(const AppendParams p) {
    INGOT_PDL_TRIGGER();
    INGOT_PDL_WAIT();  // q/k/v come from the kernel before; the cache rows written here may still be read by it
    const int q_units = p.q ? p.n_head * 16 : 0;  // 16 units of 8 elements per head
    const int kv_units = p.n_head_kv * 16;
    const int units_per_tok = q_units + 2 * kv_units;
    const long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= (long long)units_per_tok * p.n_tok) return;
    const int tok = int(u / units_per_tok);
    int r = int(u % units_per_tok);
    const int pos = p.positions ? p.positions[tok] : p.pos0 + tok;
    // blockIdx.y selects one of several consecutive layers whose inputs are stacked [layer][token][...].
    const size_t lq = (size_t)blockIdx.y * p.n_tok * p.n_head * kHeadDim;
    const size_t lkv = (size_t)blockIdx.y * p.n_tok * p.n_head_kv * kHeadDim;
    const size_t lc = (size_t)blockIdx.y * p.layer_elems;

    const float* src;
    __half* dst;
    bool rotate = true;
    if (r < q_units) {
        src = p.q + lq + ((size_t)tok * p.n_head) * kHeadDim + (size_t)r * 8;
        dst = p.q_out + lq + ((size_t)tok * p.n_head) * kHeadDim + (size_t)r * 8;
    } else {
        r -= q_units;
        const bool is_v = r >= kv_units;
        if (is_v) r -= kv_units;
        const int h = r / 16;
        const long long row = cache_row(p, tok, h, pos);
        if (row < 0) {
            if ((r & 15) == 0) atomicOr(p.status, row == -1 ? kDevErrPosRange : kDevErrBlockRange);
            return;
        }
        if (!INGOT_CHECK(row + (size_t)(r & 15) * 8, 8, p.cache_extent, p.status)) return;
        src = (is_v ? p.v : p.k) + lkv + ((size_t)tok * p.n_head_kv) * kHeadDim + (size_t)r * 8;
        dst = (is_v ? p.vc : p.kc) + lc + row + (size_t)(r & 15) * 8;
        rotate = !is_v;
    }
    *reinterpret_cast<uint4*>(dst) = rope_pack8(src, (r & 15) * 4, float(pos), p.inv_freq, rotate);
}

struct ImportParams {
    const __half* k;
    const __half* v;
    __half* kc;
    __half* vc;
    const int32_t* block_table;
    int* status;
    int n_head_kv, n_tok, pos0, capacity, paged;
    size_t cache_extent;
};

// Token-major [n_tok][n_head_kv][128] f16 rows -> cache layout. One 16-byte chunk per thread.
__global__ void __launch_bounds__(256) kv_import_f16_kernel(const ImportParams p) {
    const int units_per_tok = p.n_head_kv * 16;
    const long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= (long long)units_per_tok * p.n_tok * 2) return;
    const bool is_v = u >= (long long)units_per_tok * p.n_tok;
    const long long uu = is_v ? u - (long long)units_per_tok * p.n_tok : u;
    const int tok = int(uu / units_per_tok);
    const int r = int(uu % units_per_tok);
    const int h = r / 16, c = r & 15;
    const int pos = p.pos0 + tok;
    size_t row;
    if (!p.paged) {
        row = kv_row_offset_contig(p.capacity, h, pos);
    } else {
        const int blk = p.block_table[pos / kBlockTokens];
        if (blk < 0 || blk >= p.capacity) {
            if (c == 0) atomicOr(p.status, kDevErrBlockRange);
            return;
        }
        row = kv_row_offset_paged(p.n_head_kv, blk, h, pos);
    }
    if (!INGOT_CHECK(row + (size_t)c * 8, 8, p.cache_extent, p.status)) return;
    const uint4 val = __ldg(reinterpret_cast<const uint4*>((is_v ? p.v : p.k) + (size_t)tok * units_per_tok * 8) + r);
    *reinterpret_cast<uint4*>((is_v ? p.vc : p.kc) + row + (size_t)c * 8) = val;
}

}  // namespace

int launch_rope_kv_append(ingot_kv* kv, int layer, const float* q, __half* q_out, const float* k, const float* v,
                          const float* inv_freq, int n_head, int pos0, int n_tok, const int32_t* positions,
                          const int32_t* seq_ids, const int32_t* block_tables, int max_blocks_per_seq,
                          int layer_count, cudaStream_t stream) {
    AppendParams p;
    p.q = q; p.q_out = q_out; p.k = k; p.v = v; p.inv_freq = inv_freq;
    p.kc = kv->k + size_t(layer) * kv->layer_elems;
    p.vc = kv->v + size_t(layer) * kv->layer_elems;
    p.positions = positions; p.seq_ids = seq_ids; p.block_tables = block_tables;
    p.status = kv->status_dev;
    p.n_head = n_head; p.n_head_kv = kv->n_head_kv; p.n_tok = n_tok; p.pos0 = pos0;
    p.capacity = kv->capacity; p.max_blocks_per_seq = max_blocks_per_seq;
    p.paged = kv->layout == INGOT_KV_PAGED;
    p.layer_elems = kv->layer_elems;
    p.cache_extent = kv->checked_cache_elems();
    const long long units = (long long)((q ? n_head : 0) + 2 * kv->n_head_kv) * 16 * n_tok;
    const unsigned blocks = unsigned((units + 255) / 256);
    INGOT_CUDA_TRY(ingot_launch_pdl(rope_kv_append_kernel, dim3(blocks, layer_count), dim3(256), 0, stream, p));
    return INGOT_OK;
}

int launch_kv_import_f16(ingot_kv* kv, int layer, const __half* k, const __half* v, int pos0, int n_tok,
                         const int32_t* block_table, cudaStream_t stream) {
    ImportParams p;
    p.k = k; p.v = v;
    p.kc = kv->k + size_t(layer) * kv->layer_elems;
    p.vc = kv->v + size_t(layer) * kv->layer_elems;
    p.block_table = block_table; p.status = kv->status_dev;
    p.n_head_kv = kv->n_head_kv; p.n_tok = n_tok; p.pos0 = pos0; p.capacity = kv->capacity;
    p.paged = kv->layout == INGOT_KV_PAGED;
    p.cache_extent = kv->checked_cache_elems();
    const long long units = (long long)kv->n_head_kv * 16 * n_tok * 2;
    const unsigned blocks = unsigned((units + 255) / 256);
    kv_import_f16_kernel<<<blocks, 256, 0, stream>>>(p);
    INGOT_CUDA_TRY(cudaGetLastError());
    return INGOT_OK;
}
