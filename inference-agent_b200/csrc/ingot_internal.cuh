// Internal declarations shared by the .cu files of libingot_cuda.so. Not installed.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "ingot_cuda.h"

constexpr int kHeadDim = INGOT_HEAD_DIM;
constexpr int kBlockTokens = INGOT_BLOCK_TOKENS;
// Floats per (split, head) partial of the split-KV decode: o[128], running max m, running sum l,
// padded to a 16-byte multiple. The Metal reference keeps the same triple with stride 130
// (shaders/kernels.metal:291).
constexpr int kPartStride = 132;
// Most independent launch chains the multi-layer decode call spreads its layers over
// (INGOT_DECODE_STREAMS picks how many are used; the default is this bound).
constexpr int kDecodeStreams = 8;
constexpr int kHostPosSlots = 256;  // host-buffer calls that may be queued before the caller synchronises

// Bits of the device status word (ingot_kv::status_dev).
enum : int {
    kDevErrPosRange = 1,      // K1: a position fell outside the cache; the row was skipped
    kDevErrBlockRange = 2,    // a block-table entry fell outside the pool; the access was skipped
    kDevErrBarrierTimeout = 4 // prefill: a bounded mbarrier wait expired; the CTA gave up cleanly
};

struct ingot_kv {
    int device = 0;
    int num_sms = 0;  // of `device`
    int layout = INGOT_KV_CONTIGUOUS;
    int n_layer = 0, n_head_kv = 0, head_dim = kHeadDim;
    int capacity = 0;   // positions (contiguous) or blocks (paged)
    int max_seqs = 1;
    size_t layer_elems = 0;  // f16 elements per layer in each of K and V
    __half* k = nullptr;
    __half* v = nullptr;
    int* status_dev = nullptr;  // [0] the status word, [1] the ticket of the signalling prefill form
    // split-KV decode scratch: part_bufs buffers of partials [n_seq][splits][n_head][kPartStride], each with its
    // arrival counters part_sync [max_seqs][n_head_kv][2] (zero when idle). A single decode call uses buffer 0;
    // the multi-layer call gives every launch chain two buffers that its consecutive launches alternate between.
    // Sized on first use from the split count actually needed and only ever grown; a buffer that is outgrown is
    // parked in `retired` until the handle is destroyed, because a CUDA graph captured earlier may still point
    // into it.
    float* part = nullptr;
    int* part_sync = nullptr;
    size_t part_floats = 0;  // floats per buffer
    int part_bufs = 0;
    std::vector<void*> retired;
    size_t decode_smem_opt_in = 0;      // largest dynamic shared memory the decode kernel was opted in for on `device`
    bool prefill_mma_attr_set = false;
    int test_stall_ms = 0;              // test hook, see ingot_kv_test_stall_prefill  // the warp-MMA prefill kernel's shared-memory opt-in was made on `device`
    // staging for the host-buffer entry points (grown on demand)
    void* stage = nullptr;
    size_t stage_bytes = 0;
    // single-token form of the host-buffer multi-layer call: its kernels captured once into a graph that reads the
    // position and key count from device memory (fed from a ring of pinned slots), replayed by later calls
    cudaGraph_t host_graph = nullptr;
    cudaGraphExec_t host_exec = nullptr;
    cudaStream_t capture_stream = nullptr;
    int host_key[3] = {-1, -1, -1};      // layer_begin, layer_count, n_head the graph was captured for
    const float* host_inv_freq = nullptr;
    int host_calls = 0;                  // calls seen with this key (the first runs eagerly and sizes the scratch)
    int32_t* host_pos_dev = nullptr;     // {position, key count}
    int32_t* host_pos_pinned = nullptr;  // kHostPosSlots pairs
    unsigned host_pos_next = 0;
    // side streams of the multi-layer decode call (created on first use) and their fork/join events
    cudaStream_t side_stream[kDecodeStreams] = {};
    cudaEvent_t side_done[kDecodeStreams] = {};
    cudaEvent_t fork_event = nullptr;
    // tensor maps for the TMA prefill kernel, one per layer and per tile height, built on first use
    void* tmaps = nullptr;  // host array, see attn_prefill_sm100.cu
};

void ingot_set_error(const std::string& msg);
int ingot_cuda_fail(cudaError_t e, const char* what);

#define INGOT_CUDA_TRY(expr)                                          \
    do {                                                              \
        cudaError_t e__ = (expr);                                     \
        if (e__ != cudaSuccess) return ingot_cuda_fail(e__, #expr);   \
    } while (0)

// Entry points that take a cache handle must run with the handle's device current: kernels, streams and
// function attributes all belong to that device's context.
#define INGOT_REQUIRE_DEVICE(kv)                                                          \
    do {                                                                                  \
        int dev__ = -1;                                                                   \
        INGOT_CUDA_TRY(cudaGetDevice(&dev__));                                            \
        if (dev__ != (kv)->device) {                                                      \
            ingot_set_error("the cache was created on device " + std::to_string((kv)->device) + \
                            " but device " + std::to_string(dev__) + " is current");     \
            return INGOT_ERR_INVALID;                                                     \
        }                                                                                 \
    } while (0)

#define INGOT_REQUIRE(cond, msg)                                      \
    do {                                                              \
        if (!(cond)) {                                                \
            ingot_set_error(msg);                                     \
            return INGOT_ERR_INVALID;                                 \
        }                                                             \
    } while (0)

// Element offset of (layer-local) row `pos` of kv head `h` — contiguous layout.
__host__ __device__ inline size_t kv_row_offset_contig(int n_ctx, int h, int pos) {
    return (size_t(h) * n_ctx + pos) * kHeadDim;
}
// Element offset of token slot `pos % 16` of kv head `h` in physical block `blk` — paged layout.
__host__ __device__ inline size_t kv_row_offset_paged(int n_head_kv, int blk, int h, int pos) {
    return ((size_t(blk) * n_head_kv + h) * kBlockTokens + (pos % kBlockTokens)) * kHeadDim;
}

// Launchers implemented in the kernel files.
int launch_rope_kv_append(ingot_kv* kv, int layer, const float* q, __half* q_out, const float* k, const float* v,
                          const float* inv_freq, int n_head, int pos0, int n_tok, const int32_t* positions,
                          const int32_t* seq_ids, const int32_t* block_tables, int max_blocks_per_seq,
                          int layer_count, cudaStream_t stream);
int launch_kv_import_f16(ingot_kv* kv, int layer, const __half* k, const __half* v, int pos0, int n_tok,
                         const int32_t* block_table, cudaStream_t stream);
struct DecodePlan { int chunk_keys, n_parts; };
DecodePlan decode_plan(const ingot_kv* kv, int n_seq, int max_seq_len, int chunk_keys, int concurrency, int n_head);
size_t decode_part_floats(int n_seq, int n_parts, int n_head);
int launch_attn_decode(ingot_kv* kv, int layer, const void* q, int q_dtype, void* out, int out_dtype, int n_head,
                       int n_seq, const int32_t* seq_lens, int max_seq_len, const int32_t* block_tables,
                       int max_blocks_per_seq, DecodePlan plan, float* part, int* sync, int tag, int early_loads,
                       cudaStream_t stream);
int launch_attn_prefill_mma(ingot_kv* kv, int layer, const void* q, int q_dtype, void* out, int out_dtype,
                            int n_head, int q_pos0, int n_tok, const int32_t* block_table, cudaStream_t stream);
int launch_attn_prefill_sm100(ingot_kv* kv, int layer, const void* q, int q_dtype, void* const* outs, int n_outs,
                              int out_dtype, int n_head, int out_n_head, int out_head0, int q_pos0, int n_tok,
                              const int32_t* block_table, void* const* signals, int src_index, cudaStream_t stream);
int launch_gather_wait(ingot_kv* kv, void* counters, int n_src, int timeout_ms, cudaStream_t stream);
void free_prefill_sm100_state(ingot_kv* kv);
