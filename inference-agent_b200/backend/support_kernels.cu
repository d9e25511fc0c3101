// Correctness-first support kernels for CudaBackend: the non-attention stages of the forward pass
// (src/cpu_backend.cpp:39-42, 71-85; Metal: rmsnorm / matvec_f16 / silu_mul,
// shaders/kernels.metal:129-252, 706-710). Activations stay f32 everywhere, weights are read in their
// stored type (f16 or f32) and widened, products accumulate in f32 — the arithmetic of ops::dot_row
// (src/ops.cpp:127-141) up to summation order — so that greedy decoding follows the CPU reference.
// These are not the tuned part of this library; the attention path is.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// out[row][i] = x[row][i] * rsqrt(mean(x[row]^2) + eps) * w[i]      (ops::rmsnorm, src/ops.cpp:227-232)
__global__ void rmsnorm_kernel(float* out, const float* x, const float* w, int n, float eps) {
    __shared__ float red[32];
    const float* xr = x + (size_t)blockIdx.x * n;
    float* orow = out + (size_t)blockIdx.x * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += xr[i] * xr[i];
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) red[0] = 1.0f / sqrtf(v / float(n) + eps);
    }
    __syncthreads();
    const float scale = red[0];
    for (int i = threadIdx.x; i < n; i += blockDim.x) orow[i] = xr[i] * scale * w[i];
}

// gate[i] = silu(gate[i]) * up[i]      (src/cpu_backend.cpp:79, ops::silu src/ops.h:35)
__global__ void silu_mul_kernel(float* gate, const float* up, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float g = gate[i];
        gate[i] = g / (1.0f + expf(-g)) * up[i];
    }
}

template <typename W>
__device__ __forceinline__ void load8(const W* p, float (&w)[8]);
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&w)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __half22float2(h[i]);
        w[2 * i] = f.x;
        w[2 * i + 1] = f.y;
    }
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&w)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
}

// out[t][r] (+)= dot(W[r][:], x[t][:]) for a tile of TT tokens; one warp per output row.
// W is [n_out][n_in] row-major (ggml ne = [n_in, n_out]); n_in is a multiple of 8.
template <typename W, int TT>
__global__ void linear_kernel(float* out, const W* w, const float* x, int n_in, int n_out, int n_tok, int accumulate) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int t0 = blockIdx.y * TT;
    if (row >= n_out) return;
    const W* wr = w + (size_t)row * n_in;
    float acc[TT];
#pragma unroll
    for (int t = 0; t < TT; t++) acc[t] = 0.f;
    for (int i = lane * 8; i < n_in; i += 256) {
        float wv[8];
        load8<W>(wr + i, wv);
#pragma unroll
        for (int t = 0; t < TT; t++) {
            if (t0 + t < n_tok) {
                const float* xr = x + (size_t)(t0 + t) * n_in + i;
                const float4 a = *reinterpret_cast<const float4*>(xr), b = *reinterpret_cast<const float4*>(xr + 4);
                acc[t] = fmaf(wv[0], a.x, acc[t]); acc[t] = fmaf(wv[1], a.y, acc[t]);
                acc[t] = fmaf(wv[2], a.z, acc[t]); acc[t] = fmaf(wv[3], a.w, acc[t]);
                acc[t] = fmaf(wv[4], b.x, acc[t]); acc[t] = fmaf(wv[5], b.y, acc[t]);
                acc[t] = fmaf(wv[6], b.z, acc[t]); acc[t] = fmaf(wv[7], b.w, acc[t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TT; t++) {
        const float v = warp_sum(acc[t]);
        if (lane == 0 && t0 + t < n_tok) {
            float* o = out + (size_t)(t0 + t) * n_out + row;
            *o = accumulate ? *o + v : v;
        }
    }
}

}  // namespace

extern "C" {

cudaError_t ingot_support_rmsnorm(float* out, const float* x, const float* w, int n_rows, int n, float eps, cudaStream_t s) {
    rmsnorm_kernel<<<n_rows, 256, 0, s>>>(out, x, w, n, eps);
    return cudaGetLastError();
}

cudaError_t ingot_support_silu_mul(float* gate, const float* up, size_t n, cudaStream_t s) {
    silu_mul_kernel<<<unsigned((n + 255) / 256), 256, 0, s>>>(gate, up, n);
    return cudaGetLastError();
}

// w_is_f16: 1 = __half weights, 0 = float weights.
cudaError_t ingot_support_linear(float* out, const void* w, int w_is_f16, const float* x, int n_in, int n_out, int n_tok,
                                 int accumulate, cudaStream_t s) {
    const int warps = 8;
    if (n_tok == 1) {
        dim3 grid((n_out + warps - 1) / warps, 1);
        if (w_is_f16) linear_kernel<__half, 1><<<grid, warps * 32, 0, s>>>(out, static_cast<const __half*>(w), x, n_in, n_out, n_tok, accumulate);
        else linear_kernel<float, 1><<<grid, warps * 32, 0, s>>>(out, static_cast<const float*>(w), x, n_in, n_out, n_tok, accumulate);
    } else {
        dim3 grid((n_out + warps - 1) / warps, (n_tok + 7) / 8);
        if (w_is_f16) linear_kernel<__half, 8><<<grid, warps * 32, 0, s>>>(out, static_cast<const __half*>(w), x, n_in, n_out, n_tok, accumulate);
        else linear_kernel<float, 8><<<grid, warps * 32, 0, s>>>(out, static_cast<const float*>(w), x, n_in, n_out, n_tok, accumulate);
    }
    return cudaGetLastError();
}

}  // extern "C"
