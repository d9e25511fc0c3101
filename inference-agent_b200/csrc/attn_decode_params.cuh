// Parameters of the split-KV decode kernel (attn_decode.cu) and its sequence-length helper.
#pragma once

#include "ingot_internal.cuh"

constexpr int kMaxDecodeParts = 64;  // most splits of one (sequence, kv head) range

struct DecodeParams {
    const __half* kc;   // layer base
    const __half* vc;
    const void* q;
    void* out;
    const int32_t* seq_lens;
    const int32_t* block_tables;
    float* part;          // split role: partials written here
    const float* c_part;  // combine role: partials of the launch being merged
    void* c_out;          // combine role: its output
    int* status;
    // Several layers in one launch (blockIdx.z = layer * n_seq + sequence): strides between consecutive layers of
    // the cache (elements), of q and out ([layer][sequence][head][128], elements) and of the partials (floats).
    int n_seq;
    size_t cache_layer_stride, qo_layer_stride, part_layer_stride;
    size_t cache_extent, part_extent, out_extent;  // bounds-check build: elements of one cache layer, floats of the scratch, elements of out
    int q_dtype, out_dtype;
    int n_head, n_head_kv, group;
    int capacity, paged, max_blocks_per_seq;
    int len0, chunk_keys, n_parts_max;
    // How the launch relates to the kernel before it in the stream (programmatic dependent launch):
    //   kPdlWaitFirst   wait for the predecessor before the first global read (the default)
    //   kPdlEarlyLoads  nothing read here was written by the predecessor: load at once, wait before the first write
    int pdl_mode;
    int split_parts;  // grid.x values below this are split CTAs; the one CTA above it (if any) merges
    float scale_log2;
};
enum : int { kPdlWaitFirst = 0, kPdlEarlyLoads = 1 };

// Number of keys of sequence `seq`. Lengths that come from device memory cannot be checked on the host:
// one that exceeds what the cache (or the block table) can hold is clamped and raises the status word.
__device__ __forceinline__ int load_seq_len(const DecodeParams& p, int seq) {
    int n = p.seq_lens ? p.seq_lens[seq] : p.len0;
    const int bound = p.paged ? p.max_blocks_per_seq * kBlockTokens : p.capacity;
    if (n > bound) {
        if (threadIdx.x == 0 && p.status) atomicOr(p.status, kDevErrPosRange);
        n = bound;
    }
    return n;
}

