// Support kernels for CudaBackend: the non-attention stages of the forward pass
// (src/cpu_backend.cpp:39-42, 71-85; Metal: rmsnorm / matvec_f16 / silu_mul,
// shaders/kernels.metal:129-252, 706-710). Activations stay f32 everywhere, weights are read in their
// stored type (f16 or f32) and widened, products accumulate in f32 — the arithmetic of ops::dot_row
// (src/ops.cpp:127-141) up to summation order — so that greedy decoding follows the CPU reference.
// Single-token steps with f16 weights use the weight-streaming kernel (gemv_stream_kernel); batches use the
// tensor-core kernel of linear_sm100.cu; the plain kernels here cover f32 weights and odd shapes.
#include <cuda_fp16.h>
#include <type_traits>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

// Longest input row the weight-streaming GEMV stages in shared memory: n_in floats plus a few words of static
// shared memory must stay inside the 48 KB a kernel gets without an opt-in.
constexpr int kGemvMaxIn = 12032;

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

// Single-token products with f16 weights: a weight-streaming kernel, HBM-bound by design.
//   out_m[r] (+)= dot(W_m[r][:], x')            x' = x, or x .* norm_w with the result scaled by
//   rsqrt(mean(x^2) + eps) (the RMS norm of ops::rmsnorm, src/ops.cpp:227-232, folded in; the same product up to
//   rounding order), for up to three matrices that read the same vector (q/k/v), or for the gate/up pair with
//   out[r] = silu(gate[r]) * up[r] as the epilogue (src/cpu_backend.cpp:79).
// One launch is one resident wave of CTAs; a warp owns whole rows (r, r + W, ...), W chosen so that all warps get
// the same number of rows. A lane keeps four (or six) 16-byte weight loads in flight and requests the next set before
// it consumes the current ones, across row boundaries too, so a warp streams without gaps. x' is staged in
// shared memory once per CTA. Under programmatic dependent launch the first weight loads are issued before
// the wait for the preceding kernel (weights never depend on it), which hides the ramp of every launch
// behind the tail of the previous one.
struct GemvGroup {
    const void* w[3];      // weight rows: f16 values, or the quant plane of a repacked Q8_0 / Q4_0 matrix
    const __half* d[3];    // block scales of a quantised matrix (one per 32 weights), else null
    float* out[3];
    int row_end[3];  // running totals of the matrices' row counts
    int n_mat;
};

__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// x' is staged in shared memory in the order the lanes consume it: the j-th float4 that lane l needs for a chunk
// sits at float4 index (chunk * J + j) * 32 + l (J = float4s per lane and chunk), so that the 32 lanes of a warp
// read 32 consecutive float4s - conflict-free - instead of 32 segments that are 32 to 128 bytes apart (a 2- to 8-way
// bank conflict on every read, which cost more shared-memory cycles than the weights cost HBM cycles).
__device__ __forceinline__ float dot8(const uint4& raw, const float4* x4) {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
    const float4 xa = x4[0], xb = x4[32];
    const float2 w0 = __half22float2(h[0]), w1 = __half22float2(h[1]), w2 = __half22float2(h[2]), w3 = __half22float2(h[3]);
    float acc = w0.x * xa.x;
    acc = fmaf(w0.y, xa.y, acc); acc = fmaf(w1.x, xa.z, acc); acc = fmaf(w1.y, xa.w, acc);
    acc = fmaf(w2.x, xb.x, acc); acc = fmaf(w2.y, xb.y, acc); acc = fmaf(w3.x, xb.z, acc); acc = fmaf(w3.y, xb.w, acc);
    return acc;
}

// Weight formats of the streaming kernel. A lane's 16-byte load covers kElems weights: 8 f16 values, 16 Q8_0
// quants (half a block) or the 32 nibbles of one Q4_0 block; the 32 lanes of a warp therefore cover 512 bytes =
// 256 / 512 / 1024 consecutive weights per load. Quantised rows come from the repacked planes of
// quant_kernels.cu: quants contiguous per row, one f16 scale per 32 weights in a plane of its own.
enum : int { kFmtF16 = 0, kFmtQ8_0 = 1, kFmtQ4_0 = 2 };
template <int kFmt> struct FmtTraits { static constexpr int kElems = kFmt == kFmtF16 ? 8 : kFmt == kFmtQ8_0 ? 16 : 32; };

__device__ __forceinline__ uint32_t prmt_b(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
// byte k of `word` as a float: the byte becomes the low mantissa bits of 2^23, then 2^23 + bias is subtracted
__device__ __forceinline__ float byte_f(uint32_t word, int k, float bias) {
    return __uint_as_float(prmt_b(word, 0x4B000000u, 0x7650u + (uint32_t)k)) - bias;
}
// d * sum_i q_i x_i over the weights of one 16-byte load (the grouping of dot_q8_0 / dot_q4_0, src/ops.cpp:143-180)
template <int kFmt>
__device__ __forceinline__ float dot_load(const uint4& raw, const float4* x4, unsigned short scale_bits) {
    if (kFmt == kFmtF16) return dot8(raw, x4);
    const float d = __half2float(__ushort_as_half(scale_bits));
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    if (kFmt == kFmtQ8_0) {
#pragma unroll
        for (int j = 0; j < 4; j++) {  // signed byte = (byte ^ 0x80) - 128
            const uint32_t u = w[j] ^ 0x80808080u;
            const float4 xv = x4[j * 32];
            s0 = fmaf(byte_f(u, 0, 8388608.f + 128.f), xv.x, s0);
            s1 = fmaf(byte_f(u, 1, 8388608.f + 128.f), xv.y, s1);
            s2 = fmaf(byte_f(u, 2, 8388608.f + 128.f), xv.z, s2);
            s3 = fmaf(byte_f(u, 3, 8388608.f + 128.f), xv.w, s3);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 4; j++) {  // bytes 4j..4j+3: low nibbles are weights 4j.., high nibbles weights 16+4j..
            const uint32_t lo = w[j] & 0x0F0F0F0Fu, hi = (w[j] >> 4) & 0x0F0F0F0Fu;
            const float4 xl = x4[j * 32];
            const float4 xh = x4[(4 + j) * 32];
            s0 = fmaf(byte_f(lo, 0, 8388608.f + 8.f), xl.x, s0);
            s1 = fmaf(byte_f(lo, 1, 8388608.f + 8.f), xl.y, s1);
            s2 = fmaf(byte_f(lo, 2, 8388608.f + 8.f), xl.z, s2);
            s3 = fmaf(byte_f(lo, 3, 8388608.f + 8.f), xl.w, s3);
            s0 = fmaf(byte_f(hi, 0, 8388608.f + 8.f), xh.x, s0);
            s1 = fmaf(byte_f(hi, 1, 8388608.f + 8.f), xh.y, s1);
            s2 = fmaf(byte_f(hi, 2, 8388608.f + 8.f), xh.z, s2);
            s3 = fmaf(byte_f(hi, 3, 8388608.f + 8.f), xh.w, s3);
        }
    }
    return ((s0 + s1) + (s2 + s3)) * d;
}

// kLoads: 16-byte weight loads per lane and step (split between gate and up under kSwiGLU). Current and next step
// are in flight together, so with kLoads = 6 a whole row of 3072 weights (12 chunks) is requested at once.
// Threads per CTA: every CTA stages x' (and reads the norm weights) for itself, so fewer, larger CTAs mean less of that
// L2 traffic per launch. f16 rows need 80 registers per thread and fit 768 threads (24 warps, one CTA per SM);
// the quantised formats need up to 122 and stay at 256 threads, two or three CTAs per SM (512-thread CTAs measured:
// Q8_0 tg32 561 -> 536 tok/s, Q4_0 539 -> 544).
template <int kFmt>
struct StreamThreads { static constexpr int value = kFmt == 0 ? 768 : 256; };

template <bool kNorm, bool kSwiGLU, int kLoads, int kFmt>
__global__ void __launch_bounds__(StreamThreads<kFmt>::value) gemv_stream_kernel(const GemvGroup g, const float* x, const float* norm_w, float eps, int n_in,
                                                          int total_rows, int accumulate, int use_pdl) {
    extern __shared__ float xs[];  // x', n_in floats
    __shared__ float red[25];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Rows go round-robin over all warps of the grid, warp-major (warp w of CTA b is number w * gridDim.x + b): when the
    // rows do not divide by the warp count, the warps with one row more are the low-numbered warps of EVERY CTA, so
    // every SM streams the same number of bytes.
    const int W = gridDim.x * (blockDim.x >> 5), gw = warp * gridDim.x + blockIdx.x;
    if (use_pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int kPer = kSwiGLU ? kLoads / 2 : kLoads;  // 512-byte chunks per matrix and step
    constexpr int kElems = FmtTraits<kFmt>::kElems;       // weights per lane and load
    const int n_chunks = n_in / (32 * kElems);
    const int steps = (n_chunks + kPer - 1) / kPer;
    const size_t row_bytes = (size_t)n_chunks * 512;
    const int row_scales = n_in >> 5;

    auto row_base = [&](int r, const char*& wa, const char*& wb, const __half*& da, const __half*& db) {
        if (kSwiGLU) {
            wa = static_cast<const char*>(g.w[0]) + (size_t)r * row_bytes;
            wb = static_cast<const char*>(g.w[1]) + (size_t)r * row_bytes;
            da = kFmt == kFmtF16 ? nullptr : g.d[0] + (size_t)r * row_scales;
            db = kFmt == kFmtF16 ? nullptr : g.d[1] + (size_t)r * row_scales;
        } else {
            const int m = (r >= g.row_end[0]) + (r >= g.row_end[1] && g.n_mat > 2);
            const int local = m == 0 ? r : r - (m == 1 ? g.row_end[0] : g.row_end[1]);
            wa = static_cast<const char*>(m == 0 ? g.w[0] : m == 1 ? g.w[1] : g.w[2]) + (size_t)local * row_bytes;
            da = kFmt == kFmtF16 ? nullptr : (m == 0 ? g.d[0] : m == 1 ? g.d[1] : g.d[2]) + (size_t)local * row_scales;
            wb = nullptr;
            db = nullptr;
        }
    };
    // SA / SB: the block scale that goes with each load (quantised formats)
    auto issue = [&](uint4 (&A)[kPer], uint4 (&B)[kPer], unsigned short (&SA)[kPer], unsigned short (&SB)[kPer], int r, int st) {
        const char *wa, *wb;
        const __half *da, *db;
        row_base(r, wa, wb, da, db);
#pragma unroll
        for (int h = 0; h < kPer; h++) {
            const int c = st * kPer + h;
            if (c < n_chunks) {
                A[h] = ld_stream_u4(wa + (size_t)c * 512 + lane * 16);
                if (kSwiGLU) B[h] = ld_stream_u4(wb + (size_t)c * 512 + lane * 16);
                if (kFmt != kFmtF16) {
                    const int blk = ((c * 32 + lane) * kElems) >> 5;
                    SA[h] = __ldg(reinterpret_cast<const unsigned short*>(da) + blk);
                    if (kSwiGLU) SB[h] = __ldg(reinterpret_cast<const unsigned short*>(db) + blk);
                }
            }
        }
    };

    uint4 cur_a[kPer], cur_b[kPer], nxt_a[kPer], nxt_b[kPer];
    unsigned short cs_a[kPer] = {}, cs_b[kPer] = {}, ns_a[kPer] = {}, ns_b[kPer] = {};
    int r = gw, st = 0;
    bool have = r < total_rows;
    if (have) issue(cur_a, cur_b, cs_a, cs_b, r, 0);  // before the wait below: weights do not depend on the preceding kernel

    if (use_pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < n_in; i += blockDim.x * 4) {
        float4 v = *reinterpret_cast<const float4*>(x + i);
        if (kNorm) {
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            const float4 n = *reinterpret_cast<const float4*>(norm_w + i);
            v.x *= n.x; v.y *= n.y; v.z *= n.z; v.w *= n.w;
        }
        // element i = chunk * 32 * kElems + lane * kElems + 4 j + t  ->  float4 index (chunk * J + j) * 32 + lane
        const int chunk_e = 32 * kElems, c = i / chunk_e, rem = i - c * chunk_e, l = rem / kElems, jj = (rem - l * kElems) >> 2;
        reinterpret_cast<float4*>(xs)[(c * (kElems / 4) + jj) * 32 + l] = v;
    }
    if (kNorm) {
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
    }
    __syncthreads();
    float scale = 1.0f;
    if (kNorm) {
        float t = 0.f;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) t += red[w];
        scale = 1.0f / sqrtf(t / float(n_in) + eps);
    }

    float acc_a = 0.f, acc_b = 0.f;
    while (have) {
        int r2 = r, st2 = st + 1;
        if (st2 == steps) { st2 = 0; r2 = r + W; }
        const bool have2 = r2 < total_rows;
        if (have2) issue(nxt_a, nxt_b, ns_a, ns_b, r2, st2);
#pragma unroll
        for (int h = 0; h < kPer; h++) {
            const int c = st * kPer + h;
            if (c < n_chunks) {
                const float4* xp = reinterpret_cast<const float4*>(xs) + c * (kElems / 4) * 32 + lane;
                acc_a += dot_load<kFmt>(cur_a[h], xp, cs_a[h]);
                if (kSwiGLU) acc_b += dot_load<kFmt>(cur_b[h], xp, cs_b[h]);
            }
        }
        if (st == steps - 1) {
            acc_a = warp_sum(acc_a);
            if (kSwiGLU) acc_b = warp_sum(acc_b);
            if (lane == 0) {
                if (kSwiGLU) {
                    const float gt = acc_a * scale, up = acc_b * scale;
                    g.out[0][r] = gt / (1.0f + expf(-gt)) * up;
                } else {
                    const int m = (r >= g.row_end[0]) + (r >= g.row_end[1] && g.n_mat > 2);
                    const int local = m == 0 ? r : r - (m == 1 ? g.row_end[0] : g.row_end[1]);
                    float* o = (m == 0 ? g.out[0] : m == 1 ? g.out[1] : g.out[2]) + local;
                    const float v = acc_a * scale;
                    *o = accumulate ? *o + v : v;
                }
            }
            acc_a = 0.f;
            acc_b = 0.f;
        }
#pragma unroll
        for (int h = 0; h < kPer; h++) { cur_a[h] = nxt_a[h]; cs_a[h] = ns_a[h]; if (kSwiGLU) { cur_b[h] = nxt_b[h]; cs_b[h] = ns_b[h]; } }
        r = r2; st = st2; have = have2;
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

__device__ __forceinline__ float embed_to_f32(float v) { return v; }
__device__ __forceinline__ float embed_to_f32(__half v) { return __half2float(v); }

// Embedding gather: out[r][:] = table[rows[r]][:] widened to f32 (src/cpu_backend.cpp:33 does this with
// ops::dequant_row on the host). A row index outside the table gives zeros and raises *status.
template <typename W>
__global__ void embed_rows_kernel(float* out, const W* __restrict__ table, int n_in, int n_rows_table, const int32_t* __restrict__ rows,
                                  int* status) {
    const int row = rows[blockIdx.x];
    float* o = out + (size_t)blockIdx.x * n_in;
    if (row < 0 || row >= n_rows_table) {
        if (threadIdx.x == 0 && status) atomicOr(status, 1);
        for (int i = threadIdx.x; i < n_in; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const W* src = table + (size_t)row * n_in;
    for (int i = threadIdx.x; i < n_in; i += blockDim.x) o[i] = embed_to_f32(src[i]);
}

}  // namespace

extern "C" {

cudaError_t ingot_support_embed_rows(float* out, const void* table, int is_f16, int n_in, int n_rows_table, const int32_t* rows_dev,
                                     int n_rows, int* status_dev, cudaStream_t s) {
    if (n_rows < 1 || n_in < 1) return cudaErrorInvalidValue;
    if (is_f16) embed_rows_kernel<__half><<<n_rows, 256, 0, s>>>(out, static_cast<const __half*>(table), n_in, n_rows_table, rows_dev, status_dev);
    else embed_rows_kernel<float><<<n_rows, 256, 0, s>>>(out, static_cast<const float*>(table), n_in, n_rows_table, rows_dev, status_dev);
    return cudaGetLastError();
}

cudaError_t ingot_support_rmsnorm(float* out, const float* x, const float* w, int n_rows, int n, float eps, cudaStream_t s) {
    rmsnorm_kernel<<<n_rows, 256, 0, s>>>(out, x, w, n, eps);
    return cudaGetLastError();
}

cudaError_t ingot_support_silu_mul(float* gate, const float* up, size_t n, cudaStream_t s) {
    silu_mul_kernel<<<unsigned((n + 255) / 256), 256, 0, s>>>(gate, up, n);
    return cudaGetLastError();
}

// One token: out_m (+)= W_m . x' for n_mat <= 3 matrices [n_out[m]][n_in] of one format that share x (see
// gemv_stream_kernel). fmt: 0 f16 rows, 1 Q8_0, 2 Q4_0 (ws[m] = the quant plane, scales[m] = the scale plane of a
// matrix repacked by ingot_quant_repack). norm_w != nullptr folds the RMS norm in; swiglu != 0 takes exactly two
// matrices of equal height (gate, up) and outs[0] receives silu(gate) * up. n_in must be a multiple of 256 (f16),
// 512 (Q8_0) or 1024 (Q4_0).
cudaError_t ingot_support_gemv_group(float* const* outs, const void* const* ws, const void* const* scales, int fmt, const int* n_out, int n_mat,
                                     int swiglu, const float* x, const float* norm_w, float eps, int n_in, int accumulate, cudaStream_t s) {
    const int chunk = fmt == kFmtF16 ? 256 : fmt == kFmtQ8_0 ? 512 : 1024;
    if (fmt < 0 || fmt > 2 || n_mat < 1 || n_mat > 3 || n_in % chunk != 0 || n_in > kGemvMaxIn ||
        (swiglu && (n_mat != 2 || n_out[0] != n_out[1] || !norm_w)) || (fmt != kFmtF16 && !scales))
        return cudaErrorInvalidValue;
    GemvGroup g = {};
    int total = 0;
    for (int m = 0; m < 3; m++) {
        const int mm = m < n_mat ? m : n_mat - 1;
        g.w[m] = ws[mm];
        g.d[m] = fmt == kFmtF16 ? nullptr : static_cast<const __half*>(scales[mm]);
        g.out[m] = outs[mm];
        if (m < n_mat) total += n_out[m];
        g.row_end[m] = swiglu ? n_out[0] : total;
    }
    g.n_mat = n_mat;
    const int rows = swiglu ? n_out[0] : total;
    const size_t smem = (size_t)n_in * sizeof(float);
    // kLoads = 6 for short rows: with the current and the next step in flight the whole row is requested at once
    const bool short_rows = n_in / chunk <= 12;  // current and next step together cover the row
    typedef void (*Kernel)(GemvGroup, const float*, const float*, float, int, int, int, int);
    auto pick = [&](auto fmt_tag) -> Kernel {
        constexpr int F = decltype(fmt_tag)::value;
        return short_rows ? (swiglu ? gemv_stream_kernel<true, true, 6, F> : norm_w ? gemv_stream_kernel<true, false, 6, F> : gemv_stream_kernel<false, false, 6, F>)
                          : (swiglu ? gemv_stream_kernel<true, true, 4, F> : norm_w ? gemv_stream_kernel<true, false, 4, F> : gemv_stream_kernel<false, false, 4, F>);
    };
    Kernel kernel = fmt == kFmtF16 ? pick(std::integral_constant<int, kFmtF16>()) : fmt == kFmtQ8_0 ? pick(std::integral_constant<int, kFmtQ8_0>())
                                                                                               : pick(std::integral_constant<int, kFmtQ4_0>());
    // Environment knobs are process-wide and read once; the SM count belongs to the current device and is looked up
    // on every call (a cached attribute read), so that one process may drive several GPUs.
    static const bool use_pdl = getenv("INGOT_NO_PDL") == nullptr;
    // CTAs of one launch per SM. Fewer than fit leaves room for the next launch's CTAs, which then request
    // their first weights while this launch is still streaming (programmatic dependent launch).
    static const int ctas_per_sm_cap = [] { const char* c = getenv("INGOT_GEMV_CTAS_PER_SM"); return c ? atoi(c) : 0; }();
    int dev = 0, num_sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    int occ = 0;
    const int threads = fmt == kFmtF16 ? StreamThreads<kFmtF16>::value : StreamThreads<kFmtQ8_0>::value, cta_warps = threads / 32;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, threads, smem);
    if (e != cudaSuccess) return e;
    if (occ < 1) occ = 1;
    if (ctas_per_sm_cap > 0) occ = occ < ctas_per_sm_cap ? occ : ctas_per_sm_cap;
    // One resident wave. Quantised rows: a CTA slot on every SM is used, the rows go round-robin over all warps (warps of
    // every CTA alike get the odd row more). f16 rows: as many warps as give every warp the same number of rows, which
    // leaves some SMs without a CTA but has no uneven tail - measured tg32 589 against 578 tok/s with the full grid,
    // while the quantised formats gain from it (Q8_0 561 -> 565, Q4_0 540 -> 554).
    int ctas;
    if (fmt == kFmtF16) {
        const int capacity = num_sms * occ * cta_warps;
        const int rows_per_warp = (rows + capacity - 1) / capacity;
        ctas = ((rows + rows_per_warp - 1) / rows_per_warp + cta_warps - 1) / cta_warps;
    } else {
        ctas = std::min(num_sms * occ, (rows + cta_warps - 1) / cta_warps);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, g, x, norm_w, eps, n_in, rows, accumulate, use_pdl ? 1 : 0);
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
