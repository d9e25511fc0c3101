// HBM read-bandwidth probe: the CUDA counterpart of the reference's `bwtest` diagnostic
// (src/main.cpp:450-455 -> MetalBackend::bandwidth_test, src/metal_backend.mm:533-592, kernels bw_fill / bw_sum,
// shaders/kernels.metal:949-991). It times a kernel that only reads: every thread walks the buffer with 16-byte
// streaming loads, folds what it read into one word and stores it only if an impossible condition holds, so the
// loads cannot be optimised away and nothing is written. The figure is the read roofline the decode kernel
// (which is a pure reader too) is up against on the GPU at hand, next to the read+write copy bandwidth.
#include "attn_common.cuh"
#include "ingot_internal.cuh"

#include <algorithm>

namespace {

__global__ void hbm_fill_kernel(uint4* dst, size_t n16) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
        const uint32_t x = (uint32_t)i * 2654435761u;
        dst[i] = make_uint4(x, x ^ 0x9e3779b9u, x + 1, ~x);  // no untouched or all-zero pages
    }
}

constexpr int kProbeUnroll = 8;  // 16-byte loads each thread keeps in flight

__global__ void __launch_bounds__(256) hbm_read_kernel(const uint4* __restrict__ src, size_t n16, unsigned* sink) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t acc = 0;
    for (; i + (kProbeUnroll - 1) * stride < n16; i += kProbeUnroll * stride) {
        uint4 v[kProbeUnroll];
#pragma unroll
        for (int u = 0; u < kProbeUnroll; u++) v[u] = ld_stream16(src + i + u * stride);
#pragma unroll
        for (int u = 0; u < kProbeUnroll; u++) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
    }
    for (; i < n16; i += stride) {
        const uint4 v = ld_stream16(src + i);
        acc ^= v.x ^ v.y ^ v.z ^ v.w;
    }
    if (acc == 0x5bd1e995u && sink) atomicAdd(sink, 1u);  // practically never: keeps the loads alive
}

}  // namespace

extern "C" int ingot_hbm_read_probe(size_t bytes, int reps, double* best_seconds, void* stream) {
    INGOT_REQUIRE(bytes >= 4096 && reps >= 1 && best_seconds != nullptr, "ingot_hbm_read_probe: bad argument");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int dev = 0, sms = 0;
    INGOT_CUDA_TRY(cudaGetDevice(&dev));
    INGOT_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const size_t n16 = bytes / 16;
    uint4* buf = nullptr;
    unsigned* sink = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    INGOT_CUDA_TRY(cudaMalloc(&buf, n16 * 16));
    int rc = INGOT_OK;
    auto fail = [&](cudaError_t e, const char* what) { if (e != cudaSuccess && rc == INGOT_OK) rc = ingot_cuda_fail(e, what); return e != cudaSuccess; };
    if (!fail(cudaMalloc(&sink, sizeof(unsigned)), "cudaMalloc") && !fail(cudaMemsetAsync(sink, 0, sizeof(unsigned), s), "cudaMemset") &&
        !fail(cudaEventCreate(&e0), "cudaEventCreate") && !fail(cudaEventCreate(&e1), "cudaEventCreate")) {
        const int grid = sms * 8;  // eight 256-thread CTAs per SM: one resident wave
        hbm_fill_kernel<<<grid, 256, 0, s>>>(buf, n16);
        hbm_read_kernel<<<grid, 256, 0, s>>>(buf, n16, sink);  // warm-up
        double best = 1e30;
        for (int r = 0; r < reps && rc == INGOT_OK; r++) {
            cudaEventRecord(e0, s);
            hbm_read_kernel<<<grid, 256, 0, s>>>(buf, n16, sink);
            cudaEventRecord(e1, s);
            if (fail(cudaEventSynchronize(e1), "hbm read probe")) break;
            float ms = 0.f;
            cudaEventElapsedTime(&ms, e0, e1);
            best = std::min(best, (double)ms * 1e-3);
        }
        *best_seconds = best;
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(sink);
    cudaFree(buf);
    return rc;
}
