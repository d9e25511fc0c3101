// Library-level orchestration of the two sharded paths over the GPUs of one NVLink/NVSwitch box, for a single
// process that drives several devices (a C or C++ caller that does not bring torch.distributed):
//   * long prefill sharded by KV head: ingot_mg_* creates one cache shard per GPU, one token-major destination
//     buffer and one counter array per GPU, maps them into every peer (peer access), runs the signalling form of
//     the fused gather on every GPU and queues the bounded wait behind it - no collective library involved;
//   * batched decode sharded by sequence: ingot_lpt_assign is the length-balanced (longest processing time first)
//     assignment of sequences to GPUs; each GPU then decodes its own sequences with ingot_attn_decode.
// The reference is single-device (src/backend.h:9-23 runs one sequence on one device); there is no counterpart.
// Everything that waits is bounded: see ingot_gather_wait.
#include "ingot_internal.cuh"

#include <algorithm>
#include <new>
#include <numeric>
#include <vector>

struct ingot_mg {
    int n_dev = 0, n_head = 0, n_head_kv = 0, n_ctx = 0, out_dtype = INGOT_F16;
    std::vector<ingot_kv*> kv;
    std::vector<void*> out;            // [n_ctx][n_head][128] per GPU
    std::vector<void*> counters;       // 64 x u32 per GPU
    std::vector<cudaStream_t> stream;
};

namespace {
struct DeviceGuard {
    int saved = 0;
    DeviceGuard() { cudaGetDevice(&saved); }
    ~DeviceGuard() { cudaSetDevice(saved); }
};
}  // namespace

extern "C" {

int ingot_lpt_assign(const int32_t* lens, int n_seq, int n_ranks, int32_t* rank_of_seq) {
    INGOT_REQUIRE(lens != nullptr && rank_of_seq != nullptr && n_seq >= 0 && n_ranks >= 1, "ingot_lpt_assign: bad argument");
    std::vector<int> order(static_cast<size_t>(n_seq));
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return lens[a] > lens[b]; });
    std::vector<long long> load(static_cast<size_t>(n_ranks), 0);
    for (int i : order) {  // longest first, each to the least loaded rank; ties go to the lower rank
        const int r = int(std::min_element(load.begin(), load.end()) - load.begin());
        rank_of_seq[i] = r;
        load[r] += lens[i];
    }
    return INGOT_OK;
}

void ingot_mg_destroy(ingot_mg* mg) {
    if (!mg) return;
    DeviceGuard guard;
    for (int d = 0; d < mg->n_dev; d++) {
        cudaSetDevice(d);
        if (d < (int)mg->stream.size() && mg->stream[d]) { cudaStreamSynchronize(mg->stream[d]); cudaStreamDestroy(mg->stream[d]); }
        if (d < (int)mg->kv.size()) ingot_kv_destroy(mg->kv[d]);
        if (d < (int)mg->out.size()) cudaFree(mg->out[d]);
        if (d < (int)mg->counters.size()) cudaFree(mg->counters[d]);
    }
    delete mg;
}

int ingot_mg_create(ingot_mg** out, int n_dev, int n_layer, int n_head, int n_head_kv, int n_ctx, int out_dtype) {
    INGOT_REQUIRE(out != nullptr, "ingot_mg_create: out is null");
    *out = nullptr;
    INGOT_REQUIRE(n_dev >= 1 && n_dev <= 8 && n_head_kv % n_dev == 0 && n_head % n_head_kv == 0 && n_ctx >= 1,
                  "ingot_mg_create: 1 to 8 GPUs, and the KV heads must divide evenly over them");
    INGOT_REQUIRE(out_dtype == INGOT_F16 || out_dtype == INGOT_F32, "ingot_mg_create: out_dtype must be f16 or f32");
    int have = 0;
    INGOT_CUDA_TRY(cudaGetDeviceCount(&have));
    INGOT_REQUIRE(have >= n_dev, "ingot_mg_create: fewer GPUs visible than asked for");
    DeviceGuard guard;
    ingot_mg* mg = new (std::nothrow) ingot_mg();
    if (!mg) return INGOT_ERR_NOMEM;
    mg->n_dev = n_dev; mg->n_head = n_head; mg->n_head_kv = n_head_kv; mg->n_ctx = n_ctx; mg->out_dtype = out_dtype;
    mg->kv.assign(n_dev, nullptr); mg->out.assign(n_dev, nullptr); mg->counters.assign(n_dev, nullptr); mg->stream.assign(n_dev, nullptr);
    const size_t out_bytes = size_t(n_ctx) * n_head * kHeadDim * (out_dtype == INGOT_F32 ? 4 : 2);
    int rc = INGOT_OK;
    for (int d = 0; d < n_dev && rc == INGOT_OK; d++) {
        cudaError_t e = cudaSetDevice(d);
        for (int p = 0; p < n_dev && e == cudaSuccess; p++) {
            if (p == d) continue;
            int can = 0;
            e = cudaDeviceCanAccessPeer(&can, d, p);
            if (e == cudaSuccess && !can) { ingot_set_error("ingot_mg_create: GPUs without peer access"); rc = INGOT_ERR_UNSUPPORTED; break; }
            if (e == cudaSuccess) {
                e = cudaDeviceEnablePeerAccess(p, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) { e = cudaSuccess; cudaGetLastError(); }
            }
        }
        if (rc != INGOT_OK) break;
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&mg->stream[d], cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaMalloc(&mg->out[d], out_bytes);
        if (e == cudaSuccess) e = cudaMalloc(&mg->counters[d], 64 * sizeof(unsigned int));
        if (e == cudaSuccess) e = cudaMemset(mg->counters[d], 0, 64 * sizeof(unsigned int));
        if (e != cudaSuccess) { rc = ingot_cuda_fail(e, "ingot_mg_create"); break; }
        rc = ingot_kv_create(&mg->kv[d], INGOT_KV_CONTIGUOUS, n_layer, n_head_kv / n_dev, kHeadDim, n_ctx, 1);
    }
    if (rc == INGOT_OK) {
        for (int d = 0; d < n_dev; d++) { cudaSetDevice(d); cudaDeviceSynchronize(); }  // counters are zero before anyone signals
        *out = mg;
    } else {
        ingot_mg_destroy(mg);
    }
    return rc;
}

ingot_kv* ingot_mg_kv(ingot_mg* mg, int dev) { return (mg && dev >= 0 && dev < mg->n_dev) ? mg->kv[dev] : nullptr; }
void* ingot_mg_out(ingot_mg* mg, int dev) { return (mg && dev >= 0 && dev < mg->n_dev) ? mg->out[dev] : nullptr; }
void* ingot_mg_stream(ingot_mg* mg, int dev) { return (mg && dev >= 0 && dev < mg->n_dev) ? mg->stream[dev] : nullptr; }

int ingot_mg_prefill(ingot_mg* mg, int layer, const void* const* q_dev, int q_dtype, int q_pos0, int n_tok, int timeout_ms) {
    INGOT_REQUIRE(mg != nullptr && q_dev != nullptr, "ingot_mg_prefill: null argument");
    INGOT_REQUIRE(q_pos0 >= 0 && n_tok >= 1 && size_t(q_pos0) + n_tok <= size_t(mg->n_ctx), "context window exceeded");
    DeviceGuard guard;
    const int h_l = mg->n_head / mg->n_dev;
    // every GPU: its KV heads' rows into every GPU's buffer, then one signal per destination
    for (int d = 0; d < mg->n_dev; d++) {
        INGOT_CUDA_TRY(cudaSetDevice(d));
        int rc = ingot_attn_prefill_gather_signal(mg->kv[d], layer, q_dev[d], q_dtype, mg->out.data(), mg->counters.data(), mg->n_dev, d,
                                                  mg->out_dtype, h_l, mg->n_head, d * h_l, q_pos0, n_tok, mg->stream[d]);
        if (rc != INGOT_OK) return rc;
    }
    // every GPU: bounded wait for all sources' signals, behind its own kernel on its stream
    for (int d = 0; d < mg->n_dev; d++) {
        INGOT_CUDA_TRY(cudaSetDevice(d));
        int rc = ingot_gather_wait(mg->kv[d], mg->counters[d], mg->n_dev, timeout_ms, mg->stream[d]);
        if (rc != INGOT_OK) return rc;
    }
    int bad = 0;
    for (int d = 0; d < mg->n_dev; d++) {
        INGOT_CUDA_TRY(cudaSetDevice(d));
        int status = 0;
        int rc = ingot_kv_status(mg->kv[d], mg->stream[d], &status);  // synchronises the stream
        if (rc != INGOT_OK) return rc;
        bad |= status;
    }
    if (bad) {
        ingot_set_error("ingot_mg_prefill: a kernel raised status " + std::to_string(bad) + " (4 = a wait for a peer ran out)");
        return INGOT_ERR_DEVICE;
    }
    return INGOT_OK;
}

}  // extern "C"
