// Internal declarations shared by the .cu files of libingot_cuda.so. Not installed.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <utility>
#include <vector>

#include "ingot_cuda.h"

constexpr int kHeadDim = INGOT_HEAD_DIM;
constexpr int kBlockTokens = INGOT_BLOCK_TOKENS;
// Floats per (split, head) partial of the split-KV decode: o[128], running max m, running sum l,
// padded to a 16-byte multiple. The Metal reference keeps the same triple with stride 130
// (shaders/kernels.metal:291).
constexpr int kPartStride = 132;
constexpr int kHostPosSlots = 256;  // host-buffer calls that may be queued before the caller synchronises

// Bits of the device status word (ingot_kv::status_dev).
enum : int {
    kDevErrPosRange = 1,      // K1: a position fell outside the cache; the row was skipped
    kDevErrBlockRange = 2,    // a block-table entry fell outside the pool; the access was skipped
    kDevErrBarrierTimeout = 4,// a bounded wait expired; the kernel gave up cleanly
    kDevErrBounds = 8         // bounds-check build only: an offset fell outside its buffer; the access was skipped
};

// Bounds-check build (-DINGOT_BOUNDS_CHECK, `make check` -> libingot_cuda_check.so). Every offset the kernels
// compute into the KV cache, the split scratch, the query and the output is compared with the extent of its
// buffer before the access; a violation raises kDevErrBounds in the status word and the access is skipped - no
// trap, no assert, the context stays usable. It stands in for a memory checker on machines where none can run,
// and is compiled out of the production library.
#ifdef INGOT_BOUNDS_CHECK
__device__ __forceinline__ bool ingot_in_bounds(size_t first, size_t count, size_t extent, int* status) {
    if (first + count <= extent && first + count >= first) return true;
    if (status) atomicOr(status, kDevErrBounds);
    return false;
}
#define INGOT_CHECK(first, count, extent, status) ingot_in_bounds((size_t)(first), (size_t)(count), (size_t)(extent), (status))
#else
#define INGOT_CHECK(first, count, extent, status) true
#endif

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
    // split-KV decode scratch: partials [layer][n_seq][splits][n_head][kPartStride] of the layers one launch covers.
    // Sized on first use from the split count actually needed and only ever grown; a buffer that is outgrown is
    // parked in `retired` until the handle is destroyed, because a CUDA graph captured earlier may still point
    // into it.
    float* part = nullptr;
    size_t part_floats = 0;
    std::vector<void*> retired;
    bool prefill_mma_attr_set = false;
    int test_stall_ms = 0;              // test hook, see ingot_kv_test_stall_prefill
    size_t test_cache_extent = 0;       // test hook of the bounds-check build, see ingot_kv_test_shrink_extent (0: real extent)
    size_t checked_cache_elems() const { return test_cache_extent ? test_cache_extent : layer_elems; }  // the warp-MMA prefill kernel's shared-memory opt-in was made on `device`
    // staging for the host-buffer entry points (grown on demand)
    void* stage = nullptr;
    size_t stage_bytes = 0;
    // single-token form of the host-buffer multi-layer call: its kernels captured once into a graph that reads the
    // position and key count from device memory (fed from a ring of pinned slots), replayed by later calls
    cudaGraph_t host_graph = nullptr;
    cudaGraphExec_t host_exec = nullptr;
    cudaStream_t capture_stream = nullptr;
    // ingot_attn_prefill_host: copy streams and the events that hand its two staging buffers round
    cudaStream_t copy_in_stream = nullptr, copy_out_stream = nullptr;
    cudaEvent_t ev_entry = nullptr, ev_in[2] = {nullptr, nullptr}, ev_done[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
    int host_key[3] = {-1, -1, -1};      // layer_begin, layer_count, n_head the graph was captured for
    const float* host_inv_freq = nullptr;
    int host_calls = 0;                  // calls seen with this key (the first runs eagerly and sizes the scratch)
    int32_t* host_pos_dev = nullptr;     // {position, key count}
    int32_t* host_pos_pinned = nullptr;  // kHostPosSlots pairs
    unsigned host_pos_next = 0;
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

// Launch with programmatic dependent launch allowed: the kernel may start while the kernel before it in the stream
// is still running. Every kernel launched this way executes griddepcontrol.launch_dependents early and
// griddepcontrol.wait before it touches anything the preceding kernel may have written (or may still be reading),
// so only its set-up - barrier initialisation, tensor-memory allocation, index arithmetic - overlaps the
// predecessor's tail. INGOT_NO_PDL=1 turns the attribute off (plain stream order; diagnostics).
bool ingot_use_pdl();
template <typename... KArgs, typename... Args>
inline cudaError_t ingot_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ingot_use_pdl() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#define INGOT_PDL_TRIGGER() asm volatile("griddepcontrol.launch_dependents;" ::: "memory")
#define INGOT_PDL_WAIT() asm volatile("griddepcontrol.wait;" ::: "memory")

// Launchers implemented in the kernel files.
int launch_rope_kv_append(ingot_kv* kv, int layer, const float* q, __half* q_out, const float* k, const float* v,
                          const float* inv_freq, int n_head, int pos0, int n_tok, const int32_t* positions,
                          const int32_t* seq_ids, const int32_t* block_tables, int max_blocks_per_seq,
                          int layer_count, cudaStream_t stream);
int launch_kv_import_f16(ingot_kv* kv, int layer, const __half* k, const __half* v, int pos0, int n_tok,
                         const int32_t* block_table, cudaStream_t stream);
struct DecodePlan { int chunk_keys, n_parts; };
DecodePlan decode_plan(const ingot_kv* kv, int n_layers, int n_seq, int max_seq_len, int chunk_keys);
int decode_slots(const ingot_kv* kv);
int decode_warps_cfg();
int launch_attn_decode_append(ingot_kv* kv, int layer, const float* q, const float* k, const float* v, const float* inv_freq, void* out,
                              int out_dtype, int n_head, const int32_t* seq_lens, int max_seq_len, DecodePlan plan, float* part,
                              cudaStream_t stream);
size_t decode_part_floats(int n_seq, int n_parts, int n_head);
int launch_attn_decode(ingot_kv* kv, int layer, int n_layers, const void* q, int q_dtype, void* out, int out_dtype, int n_head,
                       int n_seq, const int32_t* seq_lens, int max_seq_len, const int32_t* block_tables,
                       int max_blocks_per_seq, DecodePlan plan, float* part, int merge_only, int pdl_mode, cudaStream_t stream);
int launch_attn_prefill_mma(ingot_kv* kv, int layer, const void* q, int q_dtype, void* out, int out_dtype,
                            int n_head, int q_pos0, int n_tok, const int32_t* block_table, cudaStream_t stream);
int launch_attn_prefill_sm100(ingot_kv* kv, int layer, const void* q, int q_dtype, void* const* outs, int n_outs,
                              int out_dtype, int n_head, int out_n_head, int out_head0, int q_pos0, int n_tok,
                              const int32_t* block_table, void* const* signals, int src_index, cudaStream_t stream);
int launch_gather_wait(ingot_kv* kv, void* counters, int n_src, int timeout_ms, cudaStream_t stream);
void free_prefill_sm100_state(ingot_kv* kv);
