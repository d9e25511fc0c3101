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


// Single-token form (decode): HBM-bound streaming of the weight matrix. One warp per output row; each lane
// keeps four 16-byte weight loads in flight (2 KB per warp, up to 128 KB per SM) and reads x through L1.
// out[r] (+)= dot(W[r][:], x).
template <typename W>
__global__ void __launch_bounds__(256) gemv_kernel(float* out, const W* w, const float* x, int n_in, int n_out, int accumulate) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= n_out) return;
    const W* wr = w + (size_t)row * n_in;
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
    auto fma8 = [&](float& acc, const float (&wv)[8], const float* xs) {
        const float4 xa = __ldg(reinterpret_cast<const float4*>(xs)), xb = __ldg(reinterpret_cast<const float4*>(xs + 4));
        acc = fmaf(wv[0], xa.x, acc); acc = fmaf(wv[1], xa.y, acc); acc = fmaf(wv[2], xa.z, acc); acc = fmaf(wv[3], xa.w, acc);
        acc = fmaf(wv[4], xb.x, acc); acc = fmaf(wv[5], xb.y, acc); acc = fmaf(wv[6], xb.z, acc); acc = fmaf(wv[7], xb.w, acc);
    };
    int i = lane * 8;
    for (; i + 768 < n_in; i += 1024) {
        float p0[8], p1[8], p2[8], p3[8];
        load8<W>(wr + i, p0); load8<W>(wr + i + 256, p1); load8<W>(wr + i + 512, p2); load8<W>(wr + i + 768, p3);
        fma8(acc0, p0, x + i); fma8(acc1, p1, x + i + 256); fma8(acc2, p2, x + i + 512); fma8(acc3, p3, x + i + 768);
    }
    for (; i < n_in; i += 256) {
        float p0[8];
        load8<W>(wr + i, p0);
        fma8(acc0, p0, x + i);
    }
    const float v = warp_sum((acc0 + acc1) + (acc2 + acc3));
    if (lane == 0) out[row] = accumulate ? out[row] + v : v;
}

// Single-token form with the RMS norm folded in, for up to three f16 matrices that read the same vector
// (q/k/v; or gate/up with the SwiGLU product as the epilogue): out_m[r] = scale * dot(W_m[r][:], x .* norm_w),
// scale = rsqrt(mean(x^2) + eps). Every warp sees the whole of x while it walks its row, so it gets the sum of
// squares for free; the scale is applied to the finished dot product (ops::rmsnorm, src/ops.cpp:227-232, scales
// the vector first: the same product up to rounding order). One launch replaces the norm and two or three
// matrix-vector launches of a layer.
struct GemvGroup {
    const __half* w[3];
    float* out[3];
    int row_end[3];  // running totals of the matrices' row counts
    int n_mat;
};

template <bool kSwiGLU>
__global__ void __launch_bounds__(256) gemv_norm_group_kernel(const GemvGroup g, const float* x, const float* norm_w, float eps, int n_in) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int row = blockIdx.x * (blockDim.x >> 5) + warp;
    const int total = kSwiGLU ? g.row_end[0] : g.row_end[g.n_mat - 1];
    if (row >= total) return;
    int mat = 0;
    if (!kSwiGLU) {
        while (row >= g.row_end[mat]) mat++;
        if (mat > 0) row -= g.row_end[mat - 1];
    }
    const __half* wa = g.w[mat] + (size_t)row * n_in;
    const __half* wb = kSwiGLU ? g.w[1] + (size_t)row * n_in : nullptr;
    float acc_a = 0.f, acc_b = 0.f, ss = 0.f;
    // four 16-byte weight loads in flight per lane (4 chunks of one matrix, or 2 of each of gate and up), all
    // issued before the first use
    constexpr int kChunks = kSwiGLU ? 2 : 4;
    for (int i = lane * 8; i < n_in; i += 256 * kChunks) {
        float a[kChunks][8], b[kChunks][8];
#pragma unroll
        for (int h = 0; h < kChunks; h++) {
            if (i + h * 256 < n_in) {
                load8<__half>(wa + i + h * 256, a[h]);
                if (kSwiGLU) load8<__half>(wb + i + h * 256, b[h]);
            }
        }
#pragma unroll
        for (int h = 0; h < kChunks; h++) {
            const int o = i + h * 256;
            if (o < n_in) {
                const float4 xa = __ldg(reinterpret_cast<const float4*>(x + o)), xb = __ldg(reinterpret_cast<const float4*>(x + o + 4));
                const float4 na = __ldg(reinterpret_cast<const float4*>(norm_w + o)), nb = __ldg(reinterpret_cast<const float4*>(norm_w + o + 4));
                const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
                const float nv[8] = {na.x, na.y, na.z, na.w, nb.x, nb.y, nb.z, nb.w};
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    ss = fmaf(xv[e], xv[e], ss);
                    const float xn = xv[e] * nv[e];
                    acc_a = fmaf(a[h][e], xn, acc_a);
                    if (kSwiGLU) acc_b = fmaf(b[h][e], xn, acc_b);
                }
            }
        }
    }
    ss = warp_sum(ss);
    acc_a = warp_sum(acc_a);
    if (kSwiGLU) acc_b = warp_sum(acc_b);
    if (lane == 0) {
        const float scale = 1.0f / sqrtf(ss / float(n_in) + eps);
        if (kSwiGLU) {
            const float gt = acc_a * scale, up = acc_b * scale;
            g.out[0][row] = gt / (1.0f + expf(-gt)) * up;  // silu(gate) * up, src/cpu_backend.cpp:79
        } else {
            g.out[mat][row] = acc_a * scale;
        }
    }
}

// Batched form (prefill): out[t][r] (+)= dot(W[r][:], x[t][:]) as a shared-memory tiled f32 GEMM on the FMA
// pipes: 128 tokens x 64 outputs per CTA, k-steps of 16, 8x4 outputs per thread; weights are widened to
// f32 when they are staged. The whole token batch of a prefill chunk up to 128 sits in one tile, so the
// weight matrix is read once per 128 tokens.
constexpr int kGM = 128, kGN = 64, kGK = 16;
template <typename W>
__global__ void __launch_bounds__(256) gemm_kernel(float* out, const W* w, const float* x, int n_in, int n_out, int n_tok, int accumulate) {
    __shared__ __align__(16) float xs[kGK][kGM + 4];
    __shared__ __align__(16) float ws[kGK][kGN + 4];
    const int t0 = blockIdx.y * kGM, r0 = blockIdx.x * kGN;
    const int tid = threadIdx.x;
    const int tm = (tid >> 4) * 8, tn = (tid & 15) * 4;  // this thread's 8 tokens x 4 outputs
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    // staging assignments: x tile 128 x 16 floats = 512 float4 (2 per thread); w tile 64 x 16 = 128 chunks of 8 (threads 0..127)
    for (int k0 = 0; k0 < n_in; k0 += kGK) {
#pragma unroll
        for (int it = 0; it < 2; it++) {
            const int idx = it * 256 + tid;
            const int row = idx >> 2, c4 = (idx & 3) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t0 + row < n_tok) v = *reinterpret_cast<const float4*>(x + (size_t)(t0 + row) * n_in + k0 + c4);
            xs[c4 + 0][row] = v.x; xs[c4 + 1][row] = v.y; xs[c4 + 2][row] = v.z; xs[c4 + 3][row] = v.w;
        }
        if (tid < 128) {
            const int row = tid >> 1, c8 = (tid & 1) * 8;
            float wv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (r0 + row < n_out) load8<W>(w + (size_t)(r0 + row) * n_in + k0 + c8, wv);
#pragma unroll
            for (int i = 0; i < 8; i++) ws[c8 + i][row] = wv[i];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kGK; k++) {
            const float4 xa = *reinterpret_cast<const float4*>(&xs[k][tm]), xb = *reinterpret_cast<const float4*>(&xs[k][tm + 4]);
            const float4 wv = *reinterpret_cast<const float4*>(&ws[k][tn]);
            const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
            const float wq[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(xv[i], wq[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int t = t0 + tm + i;
        if (t >= n_tok) continue;
        float* o = out + (size_t)t * n_out + r0 + tn;
        if (r0 + tn + 3 < n_out) {
            float4 v = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
            if (accumulate) {
                const float4 old = *reinterpret_cast<const float4*>(o);
                v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
            }
            *reinterpret_cast<float4*>(o) = v;
        } else {
            for (int j = 0; j < 4; j++)
                if (r0 + tn + j < n_out) o[j] = accumulate ? o[j] + acc[i][j] : acc[i][j];
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

// One token: out_m = (W_m . rmsnorm(x; norm_w, eps)) for n_mat <= 3 f16 matrices [n_out[m]][n_in] that share x; with
// swiglu != 0 there are exactly two matrices of equal height (gate, up) and outs[0] receives silu(gate) * up.
cudaError_t ingot_support_gemv_norm_group(float* const* outs, const void* const* ws, const int* n_out, int n_mat, int swiglu,
                                          const float* x, const float* norm_w, float eps, int n_in, cudaStream_t s) {
    if (n_mat < 1 || n_mat > 3 || n_in % 8 != 0 || (swiglu && (n_mat != 2 || n_out[0] != n_out[1]))) return cudaErrorInvalidValue;
    GemvGroup g = {};
    int total = 0;
    for (int m = 0; m < n_mat; m++) {
        g.w[m] = static_cast<const __half*>(ws[m]);
        g.out[m] = outs[m];
        total += n_out[m];
        g.row_end[m] = swiglu ? n_out[0] : total;
    }
    g.n_mat = n_mat;
    const int warps = 8;
    const int rows = swiglu ? n_out[0] : total;
    const unsigned grid = (rows + warps - 1) / warps;
    if (swiglu) gemv_norm_group_kernel<true><<<grid, warps * 32, 0, s>>>(g, x, norm_w, eps, n_in);
    else gemv_norm_group_kernel<false><<<grid, warps * 32, 0, s>>>(g, x, norm_w, eps, n_in);
    return cudaGetLastError();
}

// w_is_f16: 1 = __half weights, 0 = float weights.
cudaError_t ingot_support_linear(float* out, const void* w, int w_is_f16, const float* x, int n_in, int n_out, int n_tok,
                                 int accumulate, cudaStream_t s) {
    const int warps = 8;
    if (n_tok == 1) {
        const unsigned grid = (n_out + warps - 1) / warps;
        if (w_is_f16) gemv_kernel<__half><<<grid, warps * 32, 0, s>>>(out, static_cast<const __half*>(w), x, n_in, n_out, accumulate);
        else gemv_kernel<float><<<grid, warps * 32, 0, s>>>(out, static_cast<const float*>(w), x, n_in, n_out, accumulate);
    } else if (n_tok >= 16 && n_in % kGK == 0 && n_out % 4 == 0) {
        dim3 grid((n_out + kGN - 1) / kGN, (n_tok + kGM - 1) / kGM);
        if (w_is_f16) gemm_kernel<__half><<<grid, 256, 0, s>>>(out, static_cast<const __half*>(w), x, n_in, n_out, n_tok, accumulate);
        else gemm_kernel<float><<<grid, 256, 0, s>>>(out, static_cast<const float*>(w), x, n_in, n_out, n_tok, accumulate);
    } else {
        dim3 grid((n_out + warps - 1) / warps, (n_tok + 7) / 8);
        if (w_is_f16) linear_kernel<__half, 8><<<grid, warps * 32, 0, s>>>(out, static_cast<const __half*>(w), x, n_in, n_out, n_tok, accumulate);
        else linear_kernel<float, 8><<<grid, warps * 32, 0, s>>>(out, static_cast<const float*>(w), x, n_in, n_out, n_tok, accumulate);
    }
    return cudaGetLastError();
}

}  // extern "C"
