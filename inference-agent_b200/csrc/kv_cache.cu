// KV-cache handle, error reporting and the host-buffer convenience entry point of libingot_cuda.so.
//
// The cache replaces the one each reference backend owns (src/backend.h:1): f32
// [n_layer][n_ctx][n_head_kv*head_dim] on the CPU (src/cpu_backend.h:23) and f16 with the same
// order on Metal (src/metal_backend.mm:197-198). Here it is f16 in HBM and head-major, so that one
// KV head's keys are a dense [positions][128] matrix: a decode split reads one contiguous byte
// range, a prefill tile is one 2-D TMA box, and a KV-head shard of the cache is one slab.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <new>

#include "ingot_internal.cuh"
#include "attn_decode_params.cuh"

static thread_local std::string g_last_error;

void ingot_set_error(const std::string& msg) { g_last_error = msg; }

int ingot_cuda_fail(cudaError_t e, const char* what) {
    g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
    return e == cudaErrorMemoryAllocation ? INGOT_ERR_NOMEM : INGOT_ERR_CUDA;
}

bool ingot_use_pdl() {
    static const bool v = getenv("INGOT_NO_PDL") == nullptr;
    return v;
}

extern "C" {

const char* ingot_status_string(int status) {
    switch (status) {
        case INGOT_OK: return "ok";
        case INGOT_ERR_INVALID: return "invalid argument";
        case INGOT_ERR_CUDA: return "CUDA call failed";
        case INGOT_ERR_UNSUPPORTED: return "unsupported shape or dtype";
        case INGOT_ERR_NOMEM: return "out of device memory";
        case INGOT_ERR_DEVICE: return "a kernel reported an error";
        default: return "unknown status";
    }
}

const char* ingot_last_error(void) { return g_last_error.c_str(); }

const char* ingot_build_arch(void) { return "sm_100a"; }

const char* ingot_build_flags(void) {
#ifdef INGOT_BOUNDS_CHECK
    return "bounds-check";
#else
    return "";
#endif
}

int ingot_kv_create(ingot_kv** out, int layout, int n_layer, int n_head_kv, int head_dim, int capacity,
                    int max_seqs) {
    INGOT_REQUIRE(out != nullptr, "ingot_kv_create: out is null");
    *out = nullptr;
    INGOT_REQUIRE(layout == INGOT_KV_CONTIGUOUS || layout == INGOT_KV_PAGED, "ingot_kv_create: bad layout");
    INGOT_REQUIRE(n_layer >= 1 && n_head_kv >= 1 && capacity >= 1 && max_seqs >= 1, "ingot_kv_create: bad sizes");
    if (head_dim != kHeadDim) {
        ingot_set_error("ingot_kv_create: head_dim must be 128");
        return INGOT_ERR_UNSUPPORTED;
    }
    ingot_kv* kv = new (std::nothrow) ingot_kv();
    if (!kv) return INGOT_ERR_NOMEM;
    cudaError_t e = cudaGetDevice(&kv->device);
    if (e != cudaSuccess) { delete kv; return ingot_cuda_fail(e, "cudaGetDevice"); }
    e = cudaDeviceGetAttribute(&kv->num_sms, cudaDevAttrMultiProcessorCount, kv->device);
    if (e != cudaSuccess) { delete kv; return ingot_cuda_fail(e, "cudaDeviceGetAttribute"); }
    kv->layout = layout;
    kv->n_layer = n_layer;
    kv->n_head_kv = n_head_kv;
    kv->capacity = capacity;
    kv->max_seqs = max_seqs;
    const size_t rows = layout == INGOT_KV_CONTIGUOUS ? size_t(capacity) : size_t(capacity) * kBlockTokens;
    kv->layer_elems = rows * n_head_kv * kHeadDim;
    const size_t bytes = kv->layer_elems * n_layer * sizeof(__half);
    auto fail = [&](cudaError_t err, const char* what) {
        int rc = ingot_cuda_fail(err, what);
        ingot_kv_destroy(kv);
        return rc;
    };
    if ((e = cudaMalloc(&kv->k, bytes)) != cudaSuccess) return fail(e, "cudaMalloc(K cache)");
    if ((e = cudaMalloc(&kv->v, bytes)) != cudaSuccess) return fail(e, "cudaMalloc(V cache)");
    if ((e = cudaMalloc(&kv->status_dev, 2 * sizeof(int))) != cudaSuccess) return fail(e, "cudaMalloc(status)");
    // Zero-filled cache: rows that were never appended hold finite values, so a masked key can never
    // inject NaN through 0 * garbage.
    if ((e = cudaMemset(kv->k, 0, bytes)) != cudaSuccess) return fail(e, "cudaMemset(K)");
    if ((e = cudaMemset(kv->v, 0, bytes)) != cudaSuccess) return fail(e, "cudaMemset(V)");
    if ((e = cudaMemset(kv->status_dev, 0, 2 * sizeof(int))) != cudaSuccess) return fail(e, "cudaMemset(status)");
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) return fail(e, "cudaDeviceSynchronize");
    *out = kv;
    return INGOT_OK;
}

void ingot_kv_destroy(ingot_kv* kv) {
    if (!kv) return;
    free_prefill_sm100_state(kv);
    cudaFree(kv->k);
    cudaFree(kv->v);
    cudaFree(kv->status_dev);
    cudaFree(kv->part);
    for (void* p : kv->retired) cudaFree(p);
    cudaFree(kv->stage);
    if (kv->host_exec) cudaGraphExecDestroy(kv->host_exec);
    if (kv->host_graph) cudaGraphDestroy(kv->host_graph);
    cudaFree(kv->host_pos_dev);
    cudaFreeHost(kv->host_pos_pinned);
    if (kv->capture_stream) cudaStreamDestroy(kv->capture_stream);
    if (kv->copy_in_stream) cudaStreamDestroy(kv->copy_in_stream);
    if (kv->copy_out_stream) cudaStreamDestroy(kv->copy_out_stream);
    if (kv->ev_entry) cudaEventDestroy(kv->ev_entry);
    for (int b = 0; b < 2; b++) {
        if (kv->ev_in[b]) cudaEventDestroy(kv->ev_in[b]);
        if (kv->ev_done[b]) cudaEventDestroy(kv->ev_done[b]);
        if (kv->ev_out[b]) cudaEventDestroy(kv->ev_out[b]);
    }
    delete kv;
}

void* ingot_kv_k_dev(ingot_kv* kv, int layer) {
    if (!kv || layer < 0 || layer >= kv->n_layer) return nullptr;
    return kv->k + size_t(layer) * kv->layer_elems;
}

void* ingot_kv_v_dev(ingot_kv* kv, int layer) {
    if (!kv || layer < 0 || layer >= kv->n_layer) return nullptr;
    return kv->v + size_t(layer) * kv->layer_elems;
}

size_t ingot_kv_layer_bytes(const ingot_kv* kv) { return kv ? kv->layer_elems * sizeof(__half) : 0; }

int ingot_kv_test_shrink_extent(ingot_kv* kv, size_t elems) {
    INGOT_REQUIRE(kv != nullptr && elems <= kv->layer_elems, "ingot_kv_test_shrink_extent: bad argument");
    kv->test_cache_extent = elems;
    return INGOT_OK;
}

int ingot_kv_test_stall_prefill(ingot_kv* kv, int stall_ms) {
    INGOT_REQUIRE(kv != nullptr && stall_ms >= 0, "ingot_kv_test_stall_prefill: bad argument");
    kv->test_stall_ms = stall_ms;
    return INGOT_OK;
}

int ingot_kv_status(ingot_kv* kv, void* stream, int* status_out) {
    INGOT_REQUIRE(kv && status_out, "ingot_kv_status: null argument");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int host = 0;
    INGOT_CUDA_TRY(cudaMemcpyAsync(&host, kv->status_dev, sizeof(int), cudaMemcpyDeviceToHost, s));
    INGOT_CUDA_TRY(cudaMemsetAsync(kv->status_dev, 0, sizeof(int), s));
    INGOT_CUDA_TRY(cudaStreamSynchronize(s));
    *status_out = host;
    return INGOT_OK;
}

int ingot_rope_kv_append(ingot_kv* kv, int layer, const float* q_dev, void* q_out_dev, const float* k_dev,
                         const float* v_dev, const float* inv_freq_dev, int n_head, int pos0, int n_tok,
                         const int32_t* positions_dev, const int32_t* seq_ids_dev,
                         const int32_t* block_tables_dev, int max_blocks_per_seq, void* stream) {
    INGOT_REQUIRE(kv != nullptr, "ingot_rope_kv_append: kv is null");
    INGOT_REQUIRE_DEVICE(kv);
    INGOT_REQUIRE(layer >= 0 && layer < kv->n_layer, "ingot_rope_kv_append: layer out of range");
    INGOT_REQUIRE(n_tok >= 0, "ingot_rope_kv_append: n_tok < 0");
    if (n_tok == 0) return INGOT_OK;
    INGOT_REQUIRE(k_dev && v_dev && inv_freq_dev, "ingot_rope_kv_append: null k/v/inv_freq");
    INGOT_REQUIRE((q_dev == nullptr) == (q_out_dev == nullptr), "ingot_rope_kv_append: q and q_out must both be given or both be null");
    INGOT_REQUIRE(q_dev == nullptr || (n_head >= kv->n_head_kv && n_head % kv->n_head_kv == 0),
                  "ingot_rope_kv_append: n_head must be a multiple of n_head_kv");
    if (kv->layout == INGOT_KV_CONTIGUOUS) {
        INGOT_REQUIRE(positions_dev != nullptr || (pos0 >= 0 && size_t(pos0) + n_tok <= size_t(kv->capacity)),
                      "context window exceeded");
    } else {
        INGOT_REQUIRE(block_tables_dev != nullptr && max_blocks_per_seq >= 1,
                      "ingot_rope_kv_append: paged cache needs a block table");
        INGOT_REQUIRE(positions_dev != nullptr ||
                          (pos0 >= 0 && (size_t(pos0) + n_tok + kBlockTokens - 1) / kBlockTokens <= size_t(max_blocks_per_seq)),
                      "context window exceeded");
    }
    return launch_rope_kv_append(kv, layer, q_dev, static_cast<__half*>(q_out_dev), k_dev, v_dev, inv_freq_dev, n_head,
                                 pos0, n_tok, positions_dev, seq_ids_dev, block_tables_dev, max_blocks_per_seq, 1,
                                 static_cast<cudaStream_t>(stream));
}

int ingot_kv_import_f16(ingot_kv* kv, int layer, const void* k_f16_dev, const void* v_f16_dev, int pos0,
                        int n_tok, const int32_t* block_table_dev, void* stream) {
    INGOT_REQUIRE(kv != nullptr, "ingot_kv_import_f16: kv is null");
    INGOT_REQUIRE_DEVICE(kv);
    INGOT_REQUIRE(layer >= 0 && layer < kv->n_layer, "ingot_kv_import_f16: layer out of range");
    INGOT_REQUIRE(n_tok >= 0 && pos0 >= 0, "ingot_kv_import_f16: negative range");
    if (n_tok == 0) return INGOT_OK;
    INGOT_REQUIRE(k_f16_dev && v_f16_dev, "ingot_kv_import_f16: null k/v");
    if (kv->layout == INGOT_KV_CONTIGUOUS)
        INGOT_REQUIRE(size_t(pos0) + n_tok <= size_t(kv->capacity), "context window exceeded");
    else
        INGOT_REQUIRE(block_table_dev != nullptr, "ingot_kv_import_f16: paged cache needs a block table");
    return launch_kv_import_f16(kv, layer, static_cast<const __half*>(k_f16_dev), static_cast<const __half*>(v_f16_dev),
                                pos0, n_tok, block_table_dev, static_cast<cudaStream_t>(stream));
}

// Makes sure the handle's split scratch holds `floats` floats. Growing allocates, so the first call with a larger
// shape must not happen under stream capture; a buffer that is outgrown stays allocated until the handle is
// destroyed (a graph captured earlier may point into it).
static int ensure_decode_scratch(ingot_kv* kv, size_t floats) {
    if (floats <= kv->part_floats) return INGOT_OK;
    float* part = nullptr;
    INGOT_CUDA_TRY(cudaMalloc(&part, floats * sizeof(float)));
    if (kv->part) kv->retired.push_back(kv->part);
    kv->part = part;
    kv->part_floats = floats;
    kv->host_key[0] = -1;  // the host-buffer call's captured graph points into the old scratch
    return INGOT_OK;
}

// Argument checks shared by the decode entry points.
static int decode_checked(ingot_kv* kv, int layer, const void* q_dev, int q_dtype, void* out_dev, int out_dtype,
                          int n_head, int n_seq, const int32_t* seq_lens_dev, int max_seq_len,
                          const int32_t* block_tables_dev, int max_blocks_per_seq, int chunk_keys) {
    INGOT_REQUIRE(kv != nullptr, "ingot_attn_decode: kv is null");
    INGOT_REQUIRE_DEVICE(kv);
    INGOT_REQUIRE(layer >= 0 && layer < kv->n_layer, "ingot_attn_decode: layer out of range");
    INGOT_REQUIRE(q_dev && out_dev, "ingot_attn_decode: null q/out");
    INGOT_REQUIRE(n_seq >= 1 && n_seq <= kv->max_seqs, "ingot_attn_decode: n_seq exceeds max_seqs of the cache");
    INGOT_REQUIRE(seq_lens_dev != nullptr || n_seq == 1, "ingot_attn_decode: seq_lens_dev required for n_seq > 1");
    INGOT_REQUIRE(max_seq_len >= 1, "ingot_attn_decode: max_seq_len < 1");
    INGOT_REQUIRE(n_head >= kv->n_head_kv && n_head % kv->n_head_kv == 0, "ingot_attn_decode: n_head must be a multiple of n_head_kv");
    INGOT_REQUIRE(chunk_keys >= 0 && chunk_keys % 16 == 0, "ingot_attn_decode: chunk_keys must be a multiple of 16");
    if (n_head / kv->n_head_kv > 8 || (q_dtype != INGOT_F32 && q_dtype != INGOT_F16 && q_dtype != INGOT_BF16) ||
        (out_dtype != INGOT_F32 && out_dtype != INGOT_F16)) {
        ingot_set_error("ingot_attn_decode: group size > 8 or unsupported dtype");
        return INGOT_ERR_UNSUPPORTED;
    }
    if (kv->layout == INGOT_KV_CONTIGUOUS) {
        INGOT_REQUIRE(n_seq == 1, "ingot_attn_decode: a contiguous cache holds one sequence");
        INGOT_REQUIRE(max_seq_len <= kv->capacity, "context window exceeded");
    } else {
        INGOT_REQUIRE(block_tables_dev != nullptr && max_blocks_per_seq >= 1, "ingot_attn_decode: paged cache needs block tables");
        INGOT_REQUIRE((max_seq_len + kBlockTokens - 1) / kBlockTokens <= max_blocks_per_seq, "ingot_attn_decode: max_seq_len exceeds the block table");
    }
    return INGOT_OK;
}

int ingot_attn_decode(ingot_kv* kv, int layer, const void* q_dev, int q_dtype, void* out_dev, int out_dtype,
                      int n_head, int n_seq, const int32_t* seq_lens_dev, int max_seq_len,
                      const int32_t* block_tables_dev, int max_blocks_per_seq, int chunk_keys, void* stream) {
    INGOT_REQUIRE(kv != nullptr, "ingot_attn_decode: kv is null");
    INGOT_REQUIRE(layer >= 0 && layer < kv->n_layer, "ingot_attn_decode: layer out of range");
    return ingot_attn_decode_layers(kv, layer, 1, q_dev, q_dtype, out_dev, out_dtype, n_head, n_seq, seq_lens_dev, max_seq_len,
                                    block_tables_dev, max_blocks_per_seq, chunk_keys, stream);
}

int ingot_attn_decode_layers(ingot_kv* kv, int layer_begin, int layer_count, const void* q_dev, int q_dtype,
                             void* out_dev, int out_dtype, int n_head, int n_seq, const int32_t* seq_lens_dev,
                             int max_seq_len, const int32_t* block_tables_dev, int max_blocks_per_seq,
                             int chunk_keys, void* stream) {
    INGOT_REQUIRE(kv != nullptr, "ingot_attn_decode_layers: kv is null");
    INGOT_REQUIRE(layer_begin >= 0 && layer_count >= 0 && layer_begin + layer_count <= kv->n_layer,
                  "ingot_attn_decode_layers: layer range out of bounds");
    if (layer_count == 0) return INGOT_OK;
    int rc = decode_checked(kv, layer_begin, q_dev, q_dtype, out_dev, out_dtype, n_head, n_seq, seq_lens_dev, max_seq_len,
                            block_tables_dev, max_blocks_per_seq, chunk_keys);
    if (rc != INGOT_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t q_bytes = size_t(n_seq) * n_head * kHeadDim * (q_dtype == INGOT_F32 ? 4 : 2);
    const size_t o_bytes = size_t(n_seq) * n_head * kHeadDim * (out_dtype == INGOT_F32 ? 4 : 2);
    // The layers are independent of one another, so their split CTAs share a grid: blockIdx.z runs over (layer,
    // sequence), there is no launch boundary between layers and the block scheduler refills an SM the moment a CTA
    // retires. A merge-only launch (chained with programmatic dependent launch, so its CTAs are resident and
    // waiting when the split grid drains) then turns the split partials into the outputs. A single layer is the
    // same two launches. Only the size of the split scratch bounds how many layers share a launch:
    // INGOT_DECODE_SCRATCH_MB (default 256) caps it, and more layers than fit are done in groups.
    const DecodePlan plan = decode_plan(kv, layer_count, n_seq, max_seq_len, chunk_keys);
    const size_t per_layer = decode_part_floats(n_seq, plan.n_parts, n_head);
    size_t cap_mb = 256;
    if (const char* e = getenv("INGOT_DECODE_SCRATCH_MB")) cap_mb = size_t(std::max(1, atoi(e)));
    int group = plan.n_parts > 1 ? int(std::max<size_t>(1, std::min<size_t>(size_t(layer_count), (cap_mb << 20) / (per_layer * sizeof(float)))))
                                 : layer_count;
    group = std::min(group, std::max(1, 65535 / n_seq));  // gridDim.z
    if (plan.n_parts > 1) {
        rc = ensure_decode_scratch(kv, per_layer * size_t(group));
        if (rc != INGOT_OK) return rc;
    }
    for (int l0 = 0; l0 < layer_count; l0 += group) {
        const int n = std::min(group, layer_count - l0);
        const void* q_l = static_cast<const char*>(q_dev) + size_t(l0) * q_bytes;
        void* out_l = static_cast<char*>(out_dev) + size_t(l0) * o_bytes;
        // From the second group on nothing a split CTA READS was written by the launch before it (the previous
        // group's merge): it starts loading at once and waits for that launch only before it overwrites the scratch.
        rc = launch_attn_decode(kv, layer_begin + l0, n, q_l, q_dtype, out_l, out_dtype, n_head, n_seq, seq_lens_dev, max_seq_len,
                                block_tables_dev, max_blocks_per_seq, plan, kv->part, 0, l0 > 0 ? kPdlEarlyLoads : kPdlWaitFirst, s);
        if (rc != INGOT_OK) return rc;
        rc = launch_attn_decode(kv, layer_begin + l0, n, q_l, q_dtype, out_l, out_dtype, n_head, n_seq, seq_lens_dev, max_seq_len,
                                block_tables_dev, max_blocks_per_seq, plan, kv->part, 1, kPdlWaitFirst, s);
        if (rc != INGOT_OK) return rc;
    }
    return INGOT_OK;
}

// K1 + K3 for one token of the one sequence of a contiguous cache, in one launch (plus the merge launch when the keys
// are split): see attn_decode_append.cu.
int ingot_rope_append_decode(ingot_kv* kv, int layer, const float* q_dev, const float* k_dev, const float* v_dev,
                             const float* inv_freq_dev, void* out_dev, int out_dtype, int n_head, const int32_t* key_count_dev,
                             int pos, int max_seq_len, void* stream) {
    INGOT_REQUIRE(kv != nullptr, "ingot_rope_append_decode: kv is null");
    INGOT_REQUIRE_DEVICE(kv);
    INGOT_REQUIRE(kv->layout == INGOT_KV_CONTIGUOUS, "ingot_rope_append_decode: contiguous cache only");
    INGOT_REQUIRE(layer >= 0 && layer < kv->n_layer, "ingot_rope_append_decode: layer out of range");
    INGOT_REQUIRE(q_dev && k_dev && v_dev && inv_freq_dev && out_dev, "ingot_rope_append_decode: null argument");
    INGOT_REQUIRE(n_head >= kv->n_head_kv && n_head % kv->n_head_kv == 0, "ingot_rope_append_decode: n_head must be a multiple of n_head_kv");
    if (n_head / kv->n_head_kv > 8 || (out_dtype != INGOT_F32 && out_dtype != INGOT_F16)) {
        ingot_set_error("ingot_rope_append_decode: group size > 8 or unsupported dtype");
        return INGOT_ERR_UNSUPPORTED;
    }
    if (key_count_dev == nullptr) {
        INGOT_REQUIRE(pos >= 0 && size_t(pos) + 1 <= size_t(kv->capacity), "context window exceeded");
        max_seq_len = pos + 1;
    }
    INGOT_REQUIRE(max_seq_len >= 1 && max_seq_len <= kv->capacity, "ingot_rope_append_decode: max_seq_len out of range");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const DecodePlan plan = decode_plan(kv, 1, 1, max_seq_len, 0);
    if (plan.n_parts > 1) {
        const int rc = ensure_decode_scratch(kv, decode_part_floats(1, plan.n_parts, n_head));
        if (rc != INGOT_OK) return rc;
    }
    int rc = launch_attn_decode_append(kv, layer, q_dev, k_dev, v_dev, inv_freq_dev, out_dev, out_dtype, n_head, key_count_dev, max_seq_len,
                                       plan, kv->part, s);
    if (rc != INGOT_OK) return rc;
    return launch_attn_decode(kv, layer, 1, nullptr, INGOT_F16, out_dev, out_dtype, n_head, 1, key_count_dev, max_seq_len, nullptr, 0, plan,
                              kv->part, 1, kPdlWaitFirst, s);  // a no-op with a single split
}

int ingot_attn_prefill(ingot_kv* kv, int layer, const void* q_dev, int q_dtype, void* out_dev, int out_dtype,
                       int n_head, int q_pos0, int n_tok, const int32_t* block_table_dev, int impl, void* stream) {
    INGOT_REQUIRE(kv != nullptr, "ingot_attn_prefill: kv is null");
    INGOT_REQUIRE_DEVICE(kv);
    INGOT_REQUIRE(layer >= 0 && layer < kv->n_layer, "ingot_attn_prefill: layer out of range");
    INGOT_REQUIRE(n_tok >= 0 && q_pos0 >= 0, "ingot_attn_prefill: negative range");
    if (n_tok == 0) return INGOT_OK;
    INGOT_REQUIRE(q_dev && out_dev, "ingot_attn_prefill: null q/out");
    INGOT_REQUIRE(n_head >= kv->n_head_kv && n_head % kv->n_head_kv == 0, "ingot_attn_prefill: n_head must be a multiple of n_head_kv");
    INGOT_REQUIRE(impl >= 0 && impl <= 2, "ingot_attn_prefill: impl must be 0, 1 or 2");
    if ((q_dtype != INGOT_F32 && q_dtype != INGOT_F16 && q_dtype != INGOT_BF16) ||
        (out_dtype != INGOT_F32 && out_dtype != INGOT_F16)) {
        ingot_set_error("ingot_attn_prefill: unsupported dtype");
        return INGOT_ERR_UNSUPPORTED;
    }
    if (kv->layout == INGOT_KV_CONTIGUOUS)
        INGOT_REQUIRE(size_t(q_pos0) + n_tok <= size_t(kv->capacity), "context window exceeded");
    else
        INGOT_REQUIRE(block_table_dev != nullptr, "ingot_attn_prefill: paged cache needs a block table");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The tcgen05 kernel works on 256-row tiles of one KV head (and splits the keys over CTAs when there
    // are few row tiles). Measured on a B200, K1 + K2 per layer: a 512-token chunk onto 3584 cached positions takes
    // 42 us against 162 us for the warp-MMA kernel, 128 tokens at position 0 take 11.9 us against 13.4 us.
    // The tcgen05 kernel has a floor of about 10 us per launch; the warp-MMA kernel undercuts it only for a short chunk
    // at the very start of a sequence (measured at 24/8 heads: 64 tokens at position 0 are a tie, 16 tokens onto 1024
    // keys already take twice as long on the warp-MMA kernel).
    const bool use_sm100 = impl == 2 || (impl == 0 && q_pos0 + n_tok > 64);
    if (use_sm100)
        return launch_attn_prefill_sm100(kv, layer, q_dev, q_dtype, &out_dev, 1, out_dtype, n_head, n_head, 0, q_pos0, n_tok,
                                         block_table_dev, nullptr, 0, s);
    return launch_attn_prefill_mma(kv, layer, q_dev, q_dtype, out_dev, out_dtype, n_head, q_pos0, n_tok, block_table_dev, s);
}

static int prefill_gather_checked(ingot_kv* kv, int layer, const void* q_dev, int q_dtype, void* const* out_ptrs, int n_out,
                                  int out_dtype, int n_head, int out_n_head, int out_head0, int q_pos0, int n_tok) {
    INGOT_REQUIRE(kv != nullptr, "ingot_attn_prefill_gather: kv is null");
    INGOT_REQUIRE_DEVICE(kv);
    INGOT_REQUIRE(layer >= 0 && layer < kv->n_layer, "ingot_attn_prefill_gather: layer out of range");
    INGOT_REQUIRE(n_tok >= 1 && q_pos0 >= 0, "ingot_attn_prefill_gather: bad range");
    INGOT_REQUIRE(q_dev && out_ptrs && n_out >= 1 && n_out <= 8, "ingot_attn_prefill_gather: 1 to 8 output buffers");
    for (int i = 0; i < n_out; i++) INGOT_REQUIRE(out_ptrs[i] != nullptr, "ingot_attn_prefill_gather: null output buffer");
    INGOT_REQUIRE(n_head >= kv->n_head_kv && n_head % kv->n_head_kv == 0, "ingot_attn_prefill_gather: n_head must be a multiple of n_head_kv");
    INGOT_REQUIRE(out_head0 >= 0 && out_head0 + n_head <= out_n_head, "ingot_attn_prefill_gather: head range exceeds the destination layout");
    if (kv->layout != INGOT_KV_CONTIGUOUS || (q_dtype != INGOT_F32 && q_dtype != INGOT_F16 && q_dtype != INGOT_BF16) ||
        (out_dtype != INGOT_F32 && out_dtype != INGOT_F16)) {
        ingot_set_error("ingot_attn_prefill_gather: needs a contiguous cache and f32/f16/bf16 q, f32/f16 out");
        return INGOT_ERR_UNSUPPORTED;
    }
    INGOT_REQUIRE(size_t(q_pos0) + n_tok <= size_t(kv->capacity), "context window exceeded");
    return INGOT_OK;
}

int ingot_attn_prefill_gather(ingot_kv* kv, int layer, const void* q_dev, int q_dtype, void* const* out_ptrs, int n_out,
                              int out_dtype, int n_head, int out_n_head, int out_head0, int q_pos0, int n_tok,
                              void* stream) {
    if (kv && n_tok == 0) return INGOT_OK;
    int rc = prefill_gather_checked(kv, layer, q_dev, q_dtype, out_ptrs, n_out, out_dtype, n_head, out_n_head, out_head0, q_pos0, n_tok);
    if (rc != INGOT_OK) return rc;
    return launch_attn_prefill_sm100(kv, layer, q_dev, q_dtype, out_ptrs, n_out, out_dtype, n_head, out_n_head, out_head0,
                                     q_pos0, n_tok, nullptr, nullptr, 0, static_cast<cudaStream_t>(stream));
}

int ingot_attn_prefill_gather_signal(ingot_kv* kv, int layer, const void* q_dev, int q_dtype, void* const* out_ptrs,
                                     void* const* signal_ptrs, int n_out, int src_index, int out_dtype, int n_head,
                                     int out_n_head, int out_head0, int q_pos0, int n_tok, void* stream) {
    int rc = prefill_gather_checked(kv, layer, q_dev, q_dtype, out_ptrs, n_out, out_dtype, n_head, out_n_head, out_head0, q_pos0, n_tok);
    if (rc != INGOT_OK) return rc;
    INGOT_REQUIRE(signal_ptrs != nullptr && src_index >= 0 && src_index < 64, "ingot_attn_prefill_gather_signal: bad signal arguments");
    for (int i = 0; i < n_out; i++) INGOT_REQUIRE(signal_ptrs[i] != nullptr, "ingot_attn_prefill_gather_signal: null counter array");
    return launch_attn_prefill_sm100(kv, layer, q_dev, q_dtype, out_ptrs, n_out, out_dtype, n_head, out_n_head, out_head0,
                                     q_pos0, n_tok, nullptr, signal_ptrs, src_index, static_cast<cudaStream_t>(stream));
}

int ingot_gather_wait(ingot_kv* kv, void* counters_dev, int n_src, int timeout_ms, void* stream) {
    INGOT_REQUIRE(kv != nullptr && counters_dev != nullptr, "ingot_gather_wait: null argument");
    INGOT_REQUIRE_DEVICE(kv);
    INGOT_REQUIRE(n_src >= 1 && n_src <= 32 && timeout_ms >= 1, "ingot_gather_wait: 1 to 32 sources, timeout of at least 1 ms");
    return launch_gather_wait(kv, counters_dev, n_src, timeout_ms, static_cast<cudaStream_t>(stream));
}

int ingot_attn_layers_host(ingot_kv* kv, int layer_begin, int layer_count, const float* q_host, const float* k_host,
                           const float* v_host, float* out_host, const float* inv_freq_dev, int n_head, int pos0,
                           int n_tok, void* stream) {
    INGOT_REQUIRE(kv != nullptr, "ingot_attn_layers_host: kv is null");
    INGOT_REQUIRE_DEVICE(kv);
    INGOT_REQUIRE(kv->layout == INGOT_KV_CONTIGUOUS, "ingot_attn_layers_host: contiguous cache only");
    INGOT_REQUIRE(layer_begin >= 0 && layer_count >= 0 && layer_begin + layer_count <= kv->n_layer,
                  "ingot_attn_layers_host: layer range out of bounds");
    if (layer_count == 0) return INGOT_OK;
    INGOT_REQUIRE(q_host && k_host && v_host && out_host && inv_freq_dev, "ingot_attn_layers_host: null argument");
    INGOT_REQUIRE(n_tok >= 1 && pos0 >= 0, "ingot_attn_layers_host: bad range");
    INGOT_REQUIRE(n_head >= kv->n_head_kv && n_head % kv->n_head_kv == 0, "ingot_attn_layers_host: n_head must be a multiple of n_head_kv");
    INGOT_REQUIRE(size_t(pos0) + n_tok <= size_t(kv->capacity), "context window exceeded");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t L = size_t(layer_count);
    const size_t q_elems = size_t(n_tok) * n_head * kHeadDim, kv_elems = size_t(n_tok) * kv->n_head_kv * kHeadDim;
    // Device staging: q, k, v (f32), out (f32), rotated q (f16), each stacked over the layers so that the
    // whole call needs three host->device copies and one device->host copy.
    const size_t need = L * (q_elems * 4 + kv_elems * 8 + q_elems * 4 + q_elems * 2);
    if (need > kv->stage_bytes) {
        void* bigger = nullptr;
        INGOT_CUDA_TRY(cudaMalloc(&bigger, need));
        if (kv->stage) kv->retired.push_back(kv->stage);  // kernels in flight (or a captured graph) may still use it
        kv->stage = bigger;
        kv->stage_bytes = need;
        kv->host_key[0] = -1;  // the captured graph of the single-token form points into the old staging area
    }
    float* q_d = static_cast<float*>(kv->stage);
    float* k_d = q_d + L * q_elems;
    float* v_d = k_d + L * kv_elems;
    float* o_d = v_d + L * kv_elems;
    __half* qh_d = reinterpret_cast<__half*>(o_d + L * q_elems);
    if (k_host == q_host + L * q_elems && v_host == k_host + L * kv_elems) {
        // the caller keeps q, k and v in one block, in the order of the device staging area: one copy instead of three
        INGOT_CUDA_TRY(cudaMemcpyAsync(q_d, q_host, L * (q_elems + 2 * kv_elems) * 4, cudaMemcpyHostToDevice, s));
    } else {
        INGOT_CUDA_TRY(cudaMemcpyAsync(q_d, q_host, L * q_elems * 4, cudaMemcpyHostToDevice, s));
        INGOT_CUDA_TRY(cudaMemcpyAsync(k_d, k_host, L * kv_elems * 4, cudaMemcpyHostToDevice, s));
        INGOT_CUDA_TRY(cudaMemcpyAsync(v_d, v_host, L * kv_elems * 4, cudaMemcpyHostToDevice, s));
    }
    int rc = INGOT_OK;
    if (n_tok == 1) {
        // Single token: about 35 launches over several side streams. They are captured once per (layer range, head
        // count) into a graph whose kernels read the position and the key count from device memory; later
        // calls copy the new pair in and replay it, which takes the launch cost off the host.
        if (!kv->host_pos_dev) {
            INGOT_CUDA_TRY(cudaMalloc(&kv->host_pos_dev, 2 * sizeof(int32_t)));
            INGOT_CUDA_TRY(cudaMallocHost(&kv->host_pos_pinned, kHostPosSlots * 2 * sizeof(int32_t)));
        }
        const bool same = kv->host_key[0] == layer_begin && kv->host_key[1] == layer_count && kv->host_key[2] == n_head &&
                          kv->host_inv_freq == inv_freq_dev;
        if (!same) {
            if (kv->host_exec) { cudaGraphExecDestroy(kv->host_exec); kv->host_exec = nullptr; }
            if (kv->host_graph) { cudaGraphDestroy(kv->host_graph); kv->host_graph = nullptr; }
            kv->host_key[0] = layer_begin; kv->host_key[1] = layer_count; kv->host_key[2] = n_head;
            kv->host_inv_freq = inv_freq_dev;
            kv->host_calls = 0;
        }
        static const bool use_graph = getenv("INGOT_HOST_GRAPH") == nullptr || atoi(getenv("INGOT_HOST_GRAPH")) != 0;
        if (!use_graph) {
            // Plain launches: position and key count travel as kernel arguments, so there is no position copy either.
            rc = launch_rope_kv_append(kv, layer_begin, q_d, qh_d, k_d, v_d, inv_freq_dev, n_head, pos0, 1, nullptr, nullptr, nullptr, 0,
                                       layer_count, s);
            if (rc != INGOT_OK) return rc;
            rc = ingot_attn_decode_layers(kv, layer_begin, layer_count, qh_d, INGOT_F16, o_d, INGOT_F32, n_head, 1, nullptr, pos0 + 1,
                                          nullptr, 0, 0, s);
            if (rc != INGOT_OK) return rc;
            INGOT_CUDA_TRY(cudaMemcpyAsync(out_host, o_d, L * q_elems * 4, cudaMemcpyDeviceToHost, s));
            return INGOT_OK;
        }
        int32_t* slot = kv->host_pos_pinned + 2 * (kv->host_pos_next++ % kHostPosSlots);
        slot[0] = pos0;
        slot[1] = pos0 + 1;
        INGOT_CUDA_TRY(cudaMemcpyAsync(kv->host_pos_dev, slot, 2 * sizeof(int32_t), cudaMemcpyHostToDevice, s));
        auto encode = [&](cudaStream_t on) -> int {
            int r = launch_rope_kv_append(kv, layer_begin, q_d, qh_d, k_d, v_d, inv_freq_dev, n_head, pos0, 1, kv->host_pos_dev,
                                          nullptr, nullptr, 0, layer_count, on);
            if (r != INGOT_OK) return r;
            return ingot_attn_decode_layers(kv, layer_begin, layer_count, qh_d, INGOT_F16, o_d, INGOT_F32, n_head, 1,
                                            kv->host_pos_dev + 1, kv->capacity, nullptr, 0, 0, on);
        };
        if (kv->host_exec) {
            INGOT_CUDA_TRY(cudaGraphLaunch(kv->host_exec, s));
        } else if (kv->host_calls++ == 0) {
            rc = encode(s);  // first call with this shape: eager (it sizes the decode scratch, which cannot happen under capture)
            if (rc != INGOT_OK) return rc;
        } else {
            // Captured on a stream of the handle's own (the caller's may be the legacy default stream, which cannot
            // be captured); the graph is then launched into the caller's stream like any other work.
            if (!kv->capture_stream) INGOT_CUDA_TRY(cudaStreamCreateWithFlags(&kv->capture_stream, cudaStreamNonBlocking));
            INGOT_CUDA_TRY(cudaStreamBeginCapture(kv->capture_stream, cudaStreamCaptureModeThreadLocal));
            rc = encode(kv->capture_stream);
            cudaGraph_t g = nullptr;
            const cudaError_t ce = cudaStreamEndCapture(kv->capture_stream, &g);
            if (rc != INGOT_OK || ce != cudaSuccess) {
                if (g) cudaGraphDestroy(g);
                kv->host_key[0] = -1;
                return rc != INGOT_OK ? rc : ingot_cuda_fail(ce, "cudaStreamEndCapture");
            }
            kv->host_graph = g;
            INGOT_CUDA_TRY(cudaGraphInstantiate(&kv->host_exec, g, 0));
            INGOT_CUDA_TRY(cudaGraphLaunch(kv->host_exec, s));
        }
        INGOT_CUDA_TRY(cudaMemcpyAsync(out_host, o_d, L * q_elems * 4, cudaMemcpyDeviceToHost, s));
        return INGOT_OK;
    }
    rc = launch_rope_kv_append(kv, layer_begin, q_d, qh_d, k_d, v_d, inv_freq_dev, n_head, pos0, n_tok, nullptr, nullptr,
                               nullptr, 0, layer_count, s);
    if (rc != INGOT_OK) return rc;
    for (int i = 0; i < layer_count; i++) {
        rc = ingot_attn_prefill(kv, layer_begin + i, qh_d + i * q_elems, INGOT_F16, o_d + i * q_elems, INGOT_F32, n_head, pos0,
                                n_tok, nullptr, 0, stream);
        if (rc != INGOT_OK) return rc;
    }
    INGOT_CUDA_TRY(cudaMemcpyAsync(out_host, o_d, L * q_elems * 4, cudaMemcpyDeviceToHost, s));
    return INGOT_OK;
}

// Prefill with the queries and the output in host memory, the cache resident: the rows are cut into chunks and the
// copy of chunk c+1 in, the attention of chunk c and the copy of chunk c-1 out run at the same time (two copy streams
// of the handle's own beside the caller's stream, two staging buffers in each direction handed round with events).
int ingot_attn_prefill_host(ingot_kv* kv, int layer, const void* q_host, int q_dtype, void* out_host, int out_dtype, int n_head,
                            int q_pos0, int n_tok, const int32_t* block_table_dev, int chunk_tokens, void* stream) {
    INGOT_REQUIRE(kv != nullptr, "ingot_attn_prefill_host: kv is null");
    INGOT_REQUIRE_DEVICE(kv);
    INGOT_REQUIRE(layer >= 0 && layer < kv->n_layer, "ingot_attn_prefill_host: layer out of range");
    INGOT_REQUIRE(n_tok >= 0 && q_pos0 >= 0 && chunk_tokens >= 0, "ingot_attn_prefill_host: negative range");
    if (n_tok == 0) return INGOT_OK;
    INGOT_REQUIRE(q_host && out_host, "ingot_attn_prefill_host: null q/out");
    INGOT_REQUIRE(n_head >= kv->n_head_kv && n_head % kv->n_head_kv == 0, "ingot_attn_prefill_host: n_head must be a multiple of n_head_kv");
    if ((q_dtype != INGOT_F32 && q_dtype != INGOT_F16 && q_dtype != INGOT_BF16) || (out_dtype != INGOT_F32 && out_dtype != INGOT_F16)) {
        ingot_set_error("ingot_attn_prefill_host: unsupported dtype");
        return INGOT_ERR_UNSUPPORTED;
    }
    if (kv->layout == INGOT_KV_CONTIGUOUS)
        INGOT_REQUIRE(size_t(q_pos0) + n_tok <= size_t(kv->capacity), "context window exceeded");
    else
        INGOT_REQUIRE(block_table_dev != nullptr, "ingot_attn_prefill_host: paged cache needs a block table");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    INGOT_CUDA_TRY(cudaStreamIsCapturing(s, &cap));
    INGOT_REQUIRE(cap == cudaStreamCaptureStatusNone, "ingot_attn_prefill_host: not capturable (it uses streams of its own)");
    // Default chunk: as many tokens as give three full waves of the tcgen05 kernel's CTAs (one CTA per SM, 256 (token,
    // head) rows of one KV head each) - 4693 tokens at 24/8 heads on 148 SMs; a 4096-token chunk is 2.6 waves.
    const int group = n_head / kv->n_head_kv;
    const int auto_chunk = std::max(512, (3 * kv->num_sms / kv->n_head_kv) * 256 / group);
    const int chunk = std::min(n_tok, chunk_tokens > 0 ? chunk_tokens : auto_chunk);
    // (Smaller first and last chunks, whose copies overlap nothing, were measured and are not faster: 901 against 918 TFLOP/s.)
    const int n_chunks = (n_tok + chunk - 1) / chunk;
    const size_t q_row = size_t(n_head) * kHeadDim * (q_dtype == INGOT_F32 ? 4 : 2);
    const size_t o_row = size_t(n_head) * kHeadDim * (out_dtype == INGOT_F32 ? 4 : 2);
    const size_t q_buf = (size_t(chunk) * q_row + 255) / 256 * 256, o_buf = (size_t(chunk) * o_row + 255) / 256 * 256;
    const size_t need = 2 * (q_buf + o_buf);
    if (need > kv->stage_bytes) {
        void* bigger = nullptr;
        INGOT_CUDA_TRY(cudaMalloc(&bigger, need));
        if (kv->stage) kv->retired.push_back(kv->stage);  // kernels in flight (or a captured graph) may still use it
        kv->stage = bigger;
        kv->stage_bytes = need;
        kv->host_key[0] = -1;  // the captured graph of the single-token host form points into the old staging area
    }
    if (!kv->copy_in_stream) {
        INGOT_CUDA_TRY(cudaStreamCreateWithFlags(&kv->copy_in_stream, cudaStreamNonBlocking));
        INGOT_CUDA_TRY(cudaStreamCreateWithFlags(&kv->copy_out_stream, cudaStreamNonBlocking));
        INGOT_CUDA_TRY(cudaEventCreateWithFlags(&kv->ev_entry, cudaEventDisableTiming));
        for (int b = 0; b < 2; b++) {
            INGOT_CUDA_TRY(cudaEventCreateWithFlags(&kv->ev_in[b], cudaEventDisableTiming));
            INGOT_CUDA_TRY(cudaEventCreateWithFlags(&kv->ev_done[b], cudaEventDisableTiming));
            INGOT_CUDA_TRY(cudaEventCreateWithFlags(&kv->ev_out[b], cudaEventDisableTiming));
        }
    }
    char* base = static_cast<char*>(kv->stage);
    char* q_stage[2] = {base, base + q_buf};
    char* o_stage[2] = {base + 2 * q_buf, base + 2 * q_buf + o_buf};
    // Whatever the caller's stream still has to do with the staging buffers (an earlier call of this function ends with
    // the stream waiting for its last copy out) comes before the first copy in.
    INGOT_CUDA_TRY(cudaEventRecord(kv->ev_entry, s));
    INGOT_CUDA_TRY(cudaStreamWaitEvent(kv->copy_in_stream, kv->ev_entry, 0));
    for (int c = 0; c < n_chunks; c++) {
        const int b = c & 1;
        const int t0 = c * chunk, n = std::min(chunk, n_tok - t0);
        // in: buffer b is free once the attention of chunk c-2 has read it
        if (c >= 2) INGOT_CUDA_TRY(cudaStreamWaitEvent(kv->copy_in_stream, kv->ev_done[b], 0));
        INGOT_CUDA_TRY(cudaMemcpyAsync(q_stage[b], static_cast<const char*>(q_host) + size_t(t0) * q_row, size_t(n) * q_row,
                                       cudaMemcpyHostToDevice, kv->copy_in_stream));
        INGOT_CUDA_TRY(cudaEventRecord(kv->ev_in[b], kv->copy_in_stream));
        // attention on the caller's stream: needs the chunk's rows, and the output buffer back from the copy of chunk c-2
        INGOT_CUDA_TRY(cudaStreamWaitEvent(s, kv->ev_in[b], 0));
        if (c >= 2) INGOT_CUDA_TRY(cudaStreamWaitEvent(s, kv->ev_out[b], 0));
        const int rc = ingot_attn_prefill(kv, layer, q_stage[b], q_dtype, o_stage[b], out_dtype, n_head, q_pos0 + t0, n, block_table_dev,
                                          0, s);
        if (rc != INGOT_OK) return rc;
        INGOT_CUDA_TRY(cudaEventRecord(kv->ev_done[b], s));
        // out
        INGOT_CUDA_TRY(cudaStreamWaitEvent(kv->copy_out_stream, kv->ev_done[b], 0));
        INGOT_CUDA_TRY(cudaMemcpyAsync(static_cast<char*>(out_host) + size_t(t0) * o_row, o_stage[b], size_t(n) * o_row,
                                       cudaMemcpyDeviceToHost, kv->copy_out_stream));
        INGOT_CUDA_TRY(cudaEventRecord(kv->ev_out[b], kv->copy_out_stream));
    }
    // the caller's stream is done when the last copies out are
    INGOT_CUDA_TRY(cudaStreamWaitEvent(s, kv->ev_out[(n_chunks - 1) & 1], 0));
    if (n_chunks >= 2) INGOT_CUDA_TRY(cudaStreamWaitEvent(s, kv->ev_out[(n_chunks - 2) & 1], 0));
    return INGOT_OK;
}

int ingot_attn_layer_host(ingot_kv* kv, int layer, const float* q_host, const float* k_host, const float* v_host,
                          float* out_host, const float* inv_freq_dev, int n_head, int pos0, int n_tok, void* stream) {
    return ingot_attn_layers_host(kv, layer, 1, q_host, k_host, v_host, out_host, inv_freq_dev, n_head, pos0, n_tok, stream);
}

int ingot_stream_sync(void* stream) {
    INGOT_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    return INGOT_OK;
}

}  // extern "C"
