// GGUF block-quantised weights (Q8_0, Q4_0, Q4_1, Q6_K) on the GPU for CudaBackend.
//
// The reference keeps such weights in their file layout and decodes them inside its dot products
// (src/ops.cpp:22-104 dequant_*, :143-180 dot_q8_0 / dot_q4_0, :198-225 dequant_row / dot_row / matvec); its Metal
// backend does the same in matvec_q8_0 / q4_0 / q4_1 / q6_k (shaders/kernels.metal:73-226) and dequantises tiles to
// f16 for its batched matmuls (kernels.metal:725-771). Here:
//
//   * Layout in HBM. The file's blocks interleave a 2-byte scale with 16 or 32 bytes of quants, so nothing in them is
//     16-byte aligned. At load time each matrix is repacked ON THE GPU into planes - all quants of a row contiguous,
//     then the scales (and minimums / sub-block scales) - with exactly the same bits, so every lane can fetch 16
//     aligned bytes of quants per load. Bytes per weight do not change (Q8_0 1.0625, Q4_0 0.5625, Q4_1 0.625,
//     Q6_K 0.8203).
//   * Decoding follows the reference arithmetic to the bit: Q8_0 d*q; Q4_0 d*(nibble-8); Q4_1 fma(d, nibble, m);
//     Q6_K (d*scale)*(q6-32) - one or two f32 multiplies of exactly representable integers.
//   * Single tokens: dequantise-in-GEMV. One warp per output row, lanes stride over the row's blocks with 16-byte
//     loads, the input vector sits in shared memory in f32, accumulation in f32: sum_b d_b * (sum_i q_i x_i), the
//     grouping of dot_q8_0 / dot_q4_0. HBM-bound: the roofline is the quantised bytes over the copy bandwidth.
//   * Batches: a matrix is expanded into two f16 planes hi = f16(w), lo = f16(w - hi) (w = hi + lo exactly: a product
//     of an 11-bit scale and a 4-to-8-bit integer has at most 19 significant bits) which the tensor-core GEMM of
//     linear_sm100.cu consumes as two f16 weight matrices accumulating into the same output.
//   * Embedding rows are dequantised on the GPU from the uploaded table (the reference does this on the host,
//     src/cpu_backend.cpp:33, src/metal_backend.mm:426-428).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>

namespace {

enum : int { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q4_1 = 3, T_Q8_0 = 8, T_Q6_K = 14, T_BF16 = 30 };

__host__ __device__ inline size_t align256(size_t x) { return (x + 255) / 256 * 256; }

// Byte offsets of the planes of a repacked [n_out][n_in] matrix.
struct Planes {
    size_t q, d, m, qh, sc, total;
};
__host__ __device__ inline Planes planes_of(int type, size_t n_in, size_t n_out) {
    Planes p = {};
    const size_t n = n_in * n_out;
    switch (type) {
        case T_Q8_0: p.q = 0; p.d = align256(n); p.total = p.d + align256(n / 32 * 2); break;
        case T_Q4_0: p.q = 0; p.d = align256(n / 2); p.total = p.d + align256(n / 32 * 2); break;
        case T_Q4_1: p.q = 0; p.d = align256(n / 2); p.m = p.d + align256(n / 32 * 2); p.total = p.m + align256(n / 32 * 2); break;
        case T_Q6_K: p.q = 0; p.qh = align256(n / 2); p.sc = p.qh + align256(n / 4); p.d = p.sc + align256(n / 16);
                     p.total = p.d + align256(n / 256 * 2); break;
        default: break;
    }
    return p;
}
__host__ __device__ inline bool is_block_type(int type) { return type == T_Q8_0 || type == T_Q4_0 || type == T_Q4_1 || type == T_Q6_K; }
__host__ __device__ inline int block_elems(int type) { return type == T_Q6_K ? 256 : 32; }
__host__ __device__ inline int block_bytes(int type) { return type == T_Q8_0 ? 34 : type == T_Q4_0 ? 18 : type == T_Q4_1 ? 20 : 210; }

// ---- repack: file blocks -> planes (same bits) ----
__global__ void repack_kernel(unsigned char* dst, const unsigned char* __restrict__ raw, int type, size_t n_in, size_t n_out) {
    const Planes pl = planes_of(type, n_in, n_out);
    const size_t n_blocks = n_in * n_out / block_elems(type);
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x; b < n_blocks; b += stride) {
        const unsigned char* src = raw + b * block_bytes(type);
        if (type == T_Q8_0) {
            dst[pl.d + 2 * b] = src[0]; dst[pl.d + 2 * b + 1] = src[1];
            for (int i = 0; i < 32; i++) dst[pl.q + b * 32 + i] = src[2 + i];
        } else if (type == T_Q4_0) {
            dst[pl.d + 2 * b] = src[0]; dst[pl.d + 2 * b + 1] = src[1];
            for (int i = 0; i < 16; i++) dst[pl.q + b * 16 + i] = src[2 + i];
        } else if (type == T_Q4_1) {
            dst[pl.d + 2 * b] = src[0]; dst[pl.d + 2 * b + 1] = src[1];
            dst[pl.m + 2 * b] = src[2]; dst[pl.m + 2 * b + 1] = src[3];
            for (int i = 0; i < 16; i++) dst[pl.q + b * 16 + i] = src[4 + i];
        } else {  // Q6_K: ql[128] qh[64] scales[16] d
            for (int i = 0; i < 128; i++) dst[pl.q + b * 128 + i] = src[i];
            for (int i = 0; i < 64; i++) dst[pl.qh + b * 64 + i] = src[128 + i];
            for (int i = 0; i < 16; i++) dst[pl.sc + b * 16 + i] = src[192 + i];
            dst[pl.d + 2 * b] = src[208]; dst[pl.d + 2 * b + 1] = src[209];
        }
    }
}

// Value of element i of row `row`, exactly as the reference's dequant_* computes it (src/ops.cpp:33-91).
__device__ __forceinline__ float decode_elem(const unsigned char* __restrict__ w, const Planes& pl, int type, size_t n_in, size_t row, size_t i) {
    const size_t e = row * n_in + i;
    if (type == T_Q8_0) {
        const float d = __half2float(reinterpret_cast<const __half*>(w + pl.d)[e >> 5]);
        return __fmul_rn(d, (float)reinterpret_cast<const signed char*>(w + pl.q)[e]);
    }
    if (type == T_Q4_0 || type == T_Q4_1) {
        const size_t b = e >> 5;
        const int r = (int)(e & 31);
        const unsigned char byte = w[pl.q + b * 16 + (r & 15)];
        const int nib = r < 16 ? (byte & 0xF) : (byte >> 4);
        const float d = __half2float(reinterpret_cast<const __half*>(w + pl.d)[b]);
        if (type == T_Q4_0) return __fmul_rn(d, (float)(nib - 8));
        return __fmaf_rn(d, (float)nib, __half2float(reinterpret_cast<const __half*>(w + pl.m)[b]));
    }
    // Q6_K (src/ops.cpp:68-91)
    const size_t sb = e >> 8;
    const int r = (int)(e & 255), half = r >> 7, rr = r & 127, k = rr >> 5, l = rr & 31, is = l >> 4;
    const unsigned char qlb = w[pl.q + sb * 128 + half * 64 + (k & 1) * 32 + l];
    const int lo4 = k < 2 ? (qlb & 0xF) : (qlb >> 4);
    const int hi2 = (w[pl.qh + sb * 64 + half * 32 + l] >> (2 * k)) & 3;
    const int q = (lo4 | (hi2 << 4)) - 32;
    const float sc = (float)reinterpret_cast<const signed char*>(w + pl.sc)[sb * 16 + half * 8 + is + 2 * k];
    const float d = __half2float(reinterpret_cast<const __half*>(w + pl.d)[sb]);
    return __fmul_rn(__fmul_rn(d, sc), (float)q);
}

// out[r][:] = row rows[r] (or r when rows is null) of the matrix, in f32. Rows outside the matrix give zeros and
// raise *status (a token id out of range is rejected on the host before this is reached).
__global__ void dequant_rows_kernel(float* out, const unsigned char* __restrict__ w, int type, size_t n_in, size_t n_out,
                                    const int32_t* __restrict__ rows, int* status) {
    const Planes pl = planes_of(type, n_in, n_out);
    const long long row = rows ? rows[blockIdx.x] : blockIdx.x;
    float* o = out + (size_t)blockIdx.x * n_in;
    if (row < 0 || row >= (long long)n_out) {
        if (threadIdx.x == 0 && status) atomicOr(status, 1);
        for (size_t i = threadIdx.x; i < n_in; i += blockDim.x) o[i] = 0.f;
        return;
    }
    for (size_t i = threadIdx.x; i < n_in; i += blockDim.x) o[i] = decode_elem(w, pl, type, n_in, (size_t)row, i);
}

// hi = f16(w), lo = f16(w - hi) for the whole matrix; a thread writes 8 consecutive elements of each plane.
__global__ void dequant_hilo_kernel(__half* hi, __half* lo, const unsigned char* __restrict__ w, int type, size_t n_in, size_t n_out) {
    const Planes pl = planes_of(type, n_in, n_out);
    const size_t n8 = n_in * n_out / 8;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < n8; t += stride) {
        const size_t e0 = t * 8;
        const size_t row = e0 / n_in, i0 = e0 - row * n_in;
        __align__(16) __half h[8];
        __align__(16) __half l[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float v = decode_elem(w, pl, type, n_in, row, i0 + j);
            h[j] = __float2half_rn(v);
            l[j] = __float2half_rn(v - __half2float(h[j]));
        }
        *reinterpret_cast<uint4*>(hi + e0) = *reinterpret_cast<const uint4*>(h);
        *reinterpret_cast<uint4*>(lo + e0) = *reinterpret_cast<const uint4*>(l);
    }
}

__global__ void bf16_to_f32_kernel(float* out, const uint16_t* __restrict__ in, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = __uint_as_float((uint32_t)in[i] << 16);
}

// ---- single-token products ----
__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
// Byte k of `word` (0..255) as a float: the byte becomes the low mantissa bits of 2^23, then 2^23 (+bias) is
// subtracted - a byte permute and an add instead of an integer-to-float conversion.
__device__ __forceinline__ float byte_to_float(uint32_t word, int k, float bias) {
    return __uint_as_float(prmt(word, 0x4B000000u, 0x7650u + (uint32_t)k)) - bias;
}

constexpr int kGemvWarps = 8;
constexpr float kTwo23 = 8388608.f;

// One warp per output row (R rows per warp, strided by the CTA's warp count). x sits in shared memory; for Q4_1 the
// per-block sums of x follow it. acc = sum_b d_b * (sum_i q_i x_i) [+ m_b * sum_i x_i].
template <int TYPE>
__global__ void __launch_bounds__(kGemvWarps * 32) quant_gemv_kernel(float* out, const unsigned char* __restrict__ w, const float* __restrict__ x,
                                                                     int n_in, int n_out, int rows_per_cta, int accumulate) {
    extern __shared__ __align__(16) float xs[];
    const Planes pl = planes_of(TYPE, (size_t)n_in, (size_t)n_out);
    for (int i = threadIdx.x * 4; i < n_in; i += blockDim.x * 4) *reinterpret_cast<float4*>(xs + i) = __ldg(reinterpret_cast<const float4*>(x + i));
    __syncthreads();
    float* xsum = xs + n_in;  // Q4_1 only
    if (TYPE == T_Q4_1) {
        for (int b = threadIdx.x; b < n_in / 32; b += blockDim.x) {
            float s = 0.f;
            for (int i = 0; i < 32; i++) s += xs[b * 32 + i];
            xsum[b] = s;
        }
        __syncthreads();
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row_end = min(n_out, (int)(blockIdx.x + 1) * rows_per_cta);
    for (int row = blockIdx.x * rows_per_cta + warp; row < row_end; row += kGemvWarps) {
        float acc = 0.f;
        if (TYPE == T_Q8_0) {
            const int nb = n_in >> 5;
            const unsigned char* q = w + pl.q + (size_t)row * n_in;
            const __half* d = reinterpret_cast<const __half*>(w + pl.d) + (size_t)row * nb;
            for (int b = lane; b < nb; b += 32) {
                const uint4 a = ldg16(q + b * 32), c = ldg16(q + b * 32 + 16);
                const float dv = __half2float(__ldg(d + b));
                const uint32_t wd[8] = {a.x ^ 0x80808080u, a.y ^ 0x80808080u, a.z ^ 0x80808080u, a.w ^ 0x80808080u,
                                        c.x ^ 0x80808080u, c.y ^ 0x80808080u, c.z ^ 0x80808080u, c.w ^ 0x80808080u};
                float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
                for (int j = 0; j < 8; j++) {  // signed byte = (byte ^ 0x80) - 128
                    const float4 xv = *reinterpret_cast<const float4*>(xs + b * 32 + j * 4);
                    s0 = fmaf(byte_to_float(wd[j], 0, kTwo23 + 128.f), xv.x, s0);
                    s1 = fmaf(byte_to_float(wd[j], 1, kTwo23 + 128.f), xv.y, s1);
                    s2 = fmaf(byte_to_float(wd[j], 2, kTwo23 + 128.f), xv.z, s2);
                    s3 = fmaf(byte_to_float(wd[j], 3, kTwo23 + 128.f), xv.w, s3);
                }
                acc = fmaf((s0 + s1) + (s2 + s3), dv, acc);
            }
        } else if (TYPE == T_Q4_0 || TYPE == T_Q4_1) {
            const int nb = n_in >> 5;
            const unsigned char* q = w + pl.q + (size_t)row * (n_in / 2);
            const __half* d = reinterpret_cast<const __half*>(w + pl.d) + (size_t)row * nb;
            const __half* mm = reinterpret_cast<const __half*>(w + pl.m) + (size_t)row * nb;
            const float bias = TYPE == T_Q4_0 ? kTwo23 + 8.f : kTwo23;
            for (int b = lane; b < nb; b += 32) {
                const uint4 a = ldg16(q + b * 16);
                const float dv = __half2float(__ldg(d + b));
                const uint32_t wd[4] = {a.x, a.y, a.z, a.w};
                float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
                for (int j = 0; j < 4; j++) {  // bytes 4j..4j+3: low nibbles are elements 4j.., high nibbles 16+4j..
                    const uint32_t lo = wd[j] & 0x0F0F0F0Fu, hi = (wd[j] >> 4) & 0x0F0F0F0Fu;
                    const float4 xl = *reinterpret_cast<const float4*>(xs + b * 32 + j * 4);
                    const float4 xh = *reinterpret_cast<const float4*>(xs + b * 32 + 16 + j * 4);
                    s0 = fmaf(byte_to_float(lo, 0, bias), xl.x, s0);
                    s1 = fmaf(byte_to_float(lo, 1, bias), xl.y, s1);
                    s2 = fmaf(byte_to_float(lo, 2, bias), xl.z, s2);
                    s3 = fmaf(byte_to_float(lo, 3, bias), xl.w, s3);
                    s0 = fmaf(byte_to_float(hi, 0, bias), xh.x, s0);
                    s1 = fmaf(byte_to_float(hi, 1, bias), xh.y, s1);
                    s2 = fmaf(byte_to_float(hi, 2, bias), xh.z, s2);
                    s3 = fmaf(byte_to_float(hi, 3, bias), xh.w, s3);
                }
                acc = fmaf((s0 + s1) + (s2 + s3), dv, acc);
                if (TYPE == T_Q4_1) acc = fmaf(__half2float(__ldg(mm + b)), xsum[b], acc);
            }
        } else {  // Q6_K: a lane takes 16 consecutive elements (one sub-block scale) at a time
            const int n_sub = n_in >> 4;
            const unsigned char* ql = w + pl.q + (size_t)row * (n_in / 2);
            const unsigned char* qh = w + pl.qh + (size_t)row * (n_in / 4);
            const signed char* sc = reinterpret_cast<const signed char*>(w + pl.sc) + (size_t)row * n_sub;
            const __half* d = reinterpret_cast<const __half*>(w + pl.d) + (size_t)row * (n_in >> 8);
            for (int s = lane; s < n_sub; s += 32) {
                // sub-block s covers elements 16 s .. 16 s + 15: super-block sb, half, k (which 32-group), is (which 16)
                const int sb = s >> 4, r = s & 15, half = r >> 3, k = (r >> 1) & 3, is = r & 1;
                const uint4 lq = ldg16(ql + sb * 128 + half * 64 + (k & 1) * 32 + is * 16);
                const uint4 hq = ldg16(qh + sb * 64 + half * 32 + is * 16);
                const float scale = __half2float(__ldg(d + sb)) * (float)sc[sb * 16 + half * 8 + is + 2 * k];
                const uint32_t lw[4] = {lq.x, lq.y, lq.z, lq.w}, hw[4] = {hq.x, hq.y, hq.z, hq.w};
                float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint32_t lo4 = (k < 2 ? lw[j] : (lw[j] >> 4)) & 0x0F0F0F0Fu;
                    const uint32_t hi2 = ((hw[j] >> (2 * k)) & 0x03030303u) << 4;
                    const uint32_t q6 = lo4 | hi2;  // 0..63 per byte
                    const float4 xv = *reinterpret_cast<const float4*>(xs + s * 16 + j * 4);
                    s0 = fmaf(byte_to_float(q6, 0, kTwo23 + 32.f), xv.x, s0);
                    s1 = fmaf(byte_to_float(q6, 1, kTwo23 + 32.f), xv.y, s1);
                    s2 = fmaf(byte_to_float(q6, 2, kTwo23 + 32.f), xv.z, s2);
                    s3 = fmaf(byte_to_float(q6, 3, kTwo23 + 32.f), xv.w, s3);
                }
                acc = fmaf((s0 + s1) + (s2 + s3), scale, acc);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) out[row] = accumulate ? out[row] + acc : acc;
    }
}

}  // namespace

extern "C" {

// 1 if `type` (a ggml type code) is one of the block formats these kernels read and the row length fits them.
int ingot_quant_supported(int type, int n_in) { return is_block_type(type) && n_in > 0 && n_in % block_elems(type) == 0 && n_in % 32 == 0; }

size_t ingot_quant_planar_bytes(int type, int n_in, int n_out) { return planes_of(type, (size_t)n_in, (size_t)n_out).total; }
// Byte offset of the f16 block-scale plane inside a repacked matrix (the quant plane starts at offset 0).
size_t ingot_quant_scale_offset(int type, int n_in, int n_out) { return planes_of(type, (size_t)n_in, (size_t)n_out).d; }
size_t ingot_quant_raw_bytes(int type, int n_in, int n_out) { return (size_t)n_in * n_out / block_elems(type) * block_bytes(type); }

// raw_dev: the matrix as it lies in the GGUF file, already copied to the device. planar_dev: ingot_quant_planar_bytes.
cudaError_t ingot_quant_repack(void* planar_dev, const void* raw_dev, int type, int n_in, int n_out, cudaStream_t s) {
    if (!ingot_quant_supported(type, n_in) || n_out < 1) return cudaErrorInvalidValue;
    const size_t n_blocks = (size_t)n_in * n_out / block_elems(type);
    repack_kernel<<<(unsigned)std::min<size_t>((n_blocks + 255) / 256, 65535), 256, 0, s>>>(static_cast<unsigned char*>(planar_dev),
                                                                                           static_cast<const unsigned char*>(raw_dev), type, n_in, n_out);
    return cudaGetLastError();
}

// out [n_rows][n_in] f32 <- rows rows_dev[0..n_rows) of the matrix (rows_dev == null: rows 0..n_rows-1).
// status_dev (may be null): bit 0 is raised if a row index falls outside the matrix.
cudaError_t ingot_quant_dequant_rows(float* out, const void* planar_dev, int type, int n_in, int n_out, const int32_t* rows_dev, int n_rows,
                                     int* status_dev, cudaStream_t s) {
    if (!ingot_quant_supported(type, n_in) || n_rows < 1) return cudaErrorInvalidValue;
    dequant_rows_kernel<<<n_rows, 256, 0, s>>>(out, static_cast<const unsigned char*>(planar_dev), type, n_in, n_out, rows_dev, status_dev);
    return cudaGetLastError();
}

cudaError_t ingot_quant_dequant_hilo(void* hi_f16, void* lo_f16, const void* planar_dev, int type, int n_in, int n_out, cudaStream_t s) {
    if (!ingot_quant_supported(type, n_in) || n_out < 1) return cudaErrorInvalidValue;
    const size_t n8 = (size_t)n_in * n_out / 8;
    dequant_hilo_kernel<<<(unsigned)std::min<size_t>((n8 + 255) / 256, 148 * 32), 256, 0, s>>>(
        static_cast<__half*>(hi_f16), static_cast<__half*>(lo_f16), static_cast<const unsigned char*>(planar_dev), type, n_in, n_out);
    return cudaGetLastError();
}

cudaError_t ingot_quant_bf16_to_f32(float* out, const void* in_bf16, size_t n, cudaStream_t s) {
    bf16_to_f32_kernel<<<(unsigned)std::min<size_t>((n + 255) / 256, 148 * 32), 256, 0, s>>>(out, static_cast<const uint16_t*>(in_bf16), n);
    return cudaGetLastError();
}

// out[r] (+)= sum_i W[r][i] x[i] for one token. n_in a multiple of 32 (256 for Q6_K) and at most 11776.
cudaError_t ingot_quant_gemv(float* out, const void* planar_dev, int type, const float* x, int n_in, int n_out, int accumulate, cudaStream_t s) {
    if (!ingot_quant_supported(type, n_in) || n_in > 11776 || n_out < 1) return cudaErrorInvalidValue;
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    // about four CTAs per SM; a CTA's warps take its rows round-robin
    const int target_ctas = sms * 4;
    int rows_per_cta = (n_out + target_ctas - 1) / target_ctas;
    rows_per_cta = (rows_per_cta + kGemvWarps - 1) / kGemvWarps * kGemvWarps;
    const unsigned grid = (unsigned)((n_out + rows_per_cta - 1) / rows_per_cta);
    const size_t smem = ((size_t)n_in + (type == T_Q4_1 ? n_in / 32 : 0)) * sizeof(float);
    const unsigned char* w = static_cast<const unsigned char*>(planar_dev);
    switch (type) {
        case T_Q8_0: quant_gemv_kernel<T_Q8_0><<<grid, kGemvWarps * 32, smem, s>>>(out, w, x, n_in, n_out, rows_per_cta, accumulate); break;
        case T_Q4_0: quant_gemv_kernel<T_Q4_0><<<grid, kGemvWarps * 32, smem, s>>>(out, w, x, n_in, n_out, rows_per_cta, accumulate); break;
        case T_Q4_1: quant_gemv_kernel<T_Q4_1><<<grid, kGemvWarps * 32, smem, s>>>(out, w, x, n_in, n_out, rows_per_cta, accumulate); break;
        default: quant_gemv_kernel<T_Q6_K><<<grid, kGemvWarps * 32, smem, s>>>(out, w, x, n_in, n_out, rows_per_cta, accumulate); break;
    }
    return cudaGetLastError();
}

}  // extern "C"
