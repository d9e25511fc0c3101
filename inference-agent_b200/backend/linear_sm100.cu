// Batched projections of CudaBackend::forward_batch on the sm_100a tensor cores:
//   out[t][r] (+)= sum_i W[r][i] * x[t][i]      W f16 [n_out][n_in] (ggml ne = [n_in, n_out]), x and out f32
// — the job of the matmul loops of the CPU reference (src/cpu_backend.cpp:39-42, 71-85 over
// ops::dot_row, src/ops.cpp:127-141) and of Metal's matmul_f16 (src/metal_backend.mm:282-322) for a
// prefill chunk of up to n_batch tokens.
//
// Precision. The reference multiplies f32 activations with widened f16 weights and accumulates in f32, and
// greedy decoding on a random-init model has to reproduce its token choices, so activations are NOT
// rounded to f16: x is split as x = hi + lo with hi = f16(x), lo = f16(x - hi), and every k-step issues two MMAs
// into the same f32 accumulator, hi*W and lo*W. The pair carries 22 significant bits while lo is a normal f16,
// i.e. for |x| above about 2^-4; below that lo falls into the f16 subnormals (spacing 2^-24), so what the split
// guarantees for every x is an ABSOLUTE error of at most 2^-25 per element (relative 3e-5 for an activation
// near 1e-3). The weights are used as stored, the products are exact, the accumulation is f32: the result
// differs from the reference only by summation order and that truncation of x.
//
// Kernel. One CTA = 128 tokens x 128 outputs over a slice of k (split-k fills the GPU when there are few
// output tiles; slices go to a scratch and are summed in slice order, by a small kernel or by the kernel
// that consumes the product, so results are reproducible). 6 warps: warp 0 streams [128 rows][64 k] boxes of hi, lo and W (128-byte swizzle, 48 KB per
// stage, 4 stages) with TMA; warp 1 issues tcgen05.mma (kind::f16, M = N = 128, K = 16; all lanes walk the
// loop, one elected lane issues); warps 2-5 read the 128x128 f32 accumulator out of tensor memory, one
// thread per token row. Rows past n_tok and outputs past n_out are zero-filled by TMA and not stored.
// Every mbarrier wait is bounded; on expiry the CTA raises the workspace's status word and leaves.
#include "../csrc/sm100_ptx.cuh"

#include <cuda_fp16.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>

namespace {

using namespace ingot_sm100;

#ifndef INGOT_GEMM_BN
#define INGOT_GEMM_BN 128
#endif
constexpr int kBM = 128, kBN = INGOT_GEMM_BN, kBK = 64;  // outputs per CTA: 128, or 256 (a third less L2 traffic per output)
static_assert(kBN == 128 || kBN == 256, "128 or 256 outputs per CTA");
constexpr int kStages = kBN == 256 ? 3 : 4;
constexpr int kBoxBytes = 128 * kBK * 2;        // 16 KB: 128 rows x 64 f16
constexpr int kWBytes = kBN * kBK * 2;          // the W box: kBN rows
constexpr int kStageBytes = 2 * kBoxBytes + kWBytes;  // hi, lo, W
constexpr int kThreads = 192;
constexpr int kOffBar = kStages * kStageBytes;
constexpr int kSmemBytes = kOffBar + 128 + 1024;  // barriers + alignment slack
constexpr uint32_t kTmemCols = kBN;
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);  // f16 x f16 -> f32, both K-major
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Programmatic dependent launch, as in the attention kernels: every kernel of the batched path lets its successor
// start early (launch_dependents at its top) and waits for its predecessor before it touches anything the predecessor
// wrote; launch latency and per-CTA set-up then overlap the predecessor's tail. INGOT_NO_PDL=1: plain stream order.
#define LINEAR_PDL_TRIGGER() asm volatile("griddepcontrol.launch_dependents;" ::: "memory")
#define LINEAR_PDL_WAIT() asm volatile("griddepcontrol.wait;" ::: "memory")
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    static const bool use_pdl = getenv("INGOT_NO_PDL") == nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

struct Bars {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t done;
    uint32_t tmem_base;
    uint32_t abort_flag;
};

// One launch covers up to three weight matrices that read the same activations (q/k/v, gate/up): grid.x runs over
// the output tiles of all of them, tile_end[m] being the running total of tiles up to and including matrix m.
struct GemmParams {
    float* out;           // [n_tok][n_out] (single matrix only)
    float* partial[3];    // per matrix: [n_split][n_tok][n_out] when n_split > 1 or to_partial
    int* status;
    int n_tok, k_steps, n_split, accumulate;
    int n_out[3], tile_end[3];
    int to_partial;  // write the slice(s) to `partial` even when there is only one (a consumer kernel sums them)
};

__global__ void __launch_bounds__(kThreads, 1)
linear_sm100_kernel(const __grid_constant__ CUtensorMap map_hi, const __grid_constant__ CUtensorMap map_lo,
                    const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1,
                    const __grid_constant__ CUtensorMap map_w2, const GemmParams p) {
    extern __shared__ unsigned char smem_dyn[];
    LINEAR_PDL_TRIGGER();
    const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char* smem_al = smem_dyn + (smem_base - smem_u32(smem_dyn));
    Bars* bars = reinterpret_cast<Bars*>(smem_al + kOffBar);
    volatile uint32_t* abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warp_u = __shfl_sync(0xffffffffu, warp, 0);
    const int mat = ((int)blockIdx.x >= p.tile_end[0]) + ((int)blockIdx.x >= p.tile_end[1]);  // warp-uniform
    const CUtensorMap* const map_w_p = mat == 0 ? &map_w0 : mat == 1 ? &map_w1 : &map_w2;
    const int mat_n_out = mat == 0 ? p.n_out[0] : mat == 1 ? p.n_out[1] : p.n_out[2];
    float* const mat_partial = mat == 0 ? p.partial[0] : mat == 1 ? p.partial[1] : p.partial[2];
    const int n0 = ((int)blockIdx.x - (mat == 0 ? 0 : mat == 1 ? p.tile_end[0] : p.tile_end[1])) * kBN;
    const int m0 = blockIdx.y * kBM, split = blockIdx.z;
    const int ks_begin = (int)((long long)p.k_steps * split / p.n_split);
    const int ks_end = (int)((long long)p.k_steps * (split + 1) / p.n_split);
    const int n_it = ks_end - ks_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) { mbar_init(smem_u32(&bars->full[s]), 1); mbar_init(smem_u32(&bars->empty[s]), 1); }
        mbar_init(smem_u32(&bars->done), 1);
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    // Barriers and tensor memory are this CTA's own and the weights never depend on the kernel before: the W boxes of
    // the first ring stages are requested now, the activation boxes (and, under accumulate, the output) only after the
    // wait for the predecessor. A stage's barrier is armed once for all three boxes.
    const int n_pre = min(n_it, kStages);
    if (warp_u == 0 && lane == 0) {
        for (int it = 0; it < n_pre; it++) {
            const uint32_t full = smem_u32(&bars->full[it]);
            mbar_expect_tx(full, kStageBytes);
            tma_load_2d(smem_base + it * kStageBytes + 2 * kBoxBytes, map_w_p, (ks_begin + it) * kBK, n0, full);
        }
    }
    LINEAR_PDL_WAIT();

    if (warp_u == 0) {
        // ---------------- TMA producer ----------------
        int armed = 0;
        bool ok = true;
        for (int it = 0; it < n_it && ok; it++) {
            const int s = it % kStages;
            const uint32_t full = smem_u32(&bars->full[s]);
            if (lane == 0) {
                const uint32_t dst = smem_base + s * kStageBytes;
                const int k = (ks_begin + it) * kBK;
                if (it < n_pre) {  // first use of the slot: armed and its W box requested before the wait above
                    tma_load_2d(dst, &map_hi, k, m0, full);
                    tma_load_2d(dst + kBoxBytes, &map_lo, k, m0, full);
                } else {
                    ok = mbar_wait(smem_u32(&bars->empty[s]), (uint32_t)(((it / kStages) & 1) ^ 1), abort_flag, kWaitLimitNs);
                    if (ok) {
                        mbar_expect_tx(full, kStageBytes);
                        tma_load_2d(dst, &map_hi, k, m0, full);
                        tma_load_2d(dst + kBoxBytes, &map_lo, k, m0, full);
                        tma_load_2d(dst + 2 * kBoxBytes, map_w_p, k, n0, full);
                    }
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (ok) armed = it + 1;
        }
        if (!ok && lane == 0) {
            // copies already issued must land before the CTA's shared memory is released
            for (int it = max(0, armed - kStages); it < armed; it++) {
                const uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(smem_u32(&bars->full[it % kStages]), (uint32_t)((it / kStages) & 1)) &&
                       globaltimer_ns() - t0 < 100000000ull) {}
            }
        }
    } else if (warp_u == 1) {
        // ---------------- MMA issuer ----------------
        bool ok = true;
        for (int it = 0; it < n_it && ok; it++) {
            const int s = it % kStages;
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->full[s]), (uint32_t)((it / kStages) & 1), abort_flag, kWaitLimitNs)) != 0;
            if (!ok) break;
            tc_fence_after();
            if (elect_one()) {
                const uint32_t a_hi = smem_base + s * kStageBytes, a_lo = a_hi + kBoxBytes, b = a_hi + 2 * kBoxBytes;
#pragma unroll
                for (int ks = 0; ks < kBK / 16; ks++)
                    tc_mma_ss(tmem, make_desc(a_hi + ks * 32, 16, 1024), make_desc(b + ks * 32, 16, 1024), kIdesc, (it > 0 || ks > 0) ? 1u : 0u);
#pragma unroll
                for (int ks = 0; ks < kBK / 16; ks++)
                    tc_mma_ss(tmem, make_desc(a_lo + ks * 32, 16, 1024), make_desc(b + ks * 32, 16, 1024), kIdesc, 1u);
                tc_commit(smem_u32(&bars->empty[s]));
                if (it == n_it - 1) tc_commit(smem_u32(&bars->done));
            }
            __syncwarp();
        }
    } else {
        // ---------------- epilogue: accumulator -> global, one thread per token row ----------------
        const int lg = warp & 3;  // the tensor-memory lane group this warp may read
        const int row = m0 + lg * 32 + lane;
        bool ok = n_it > 0 && mbar_wait(smem_u32(&bars->done), 0, abort_flag, kWaitLimitNs);
        ok = __all_sync(0xffffffffu, ok) != 0;
        const bool split_k = p.n_split > 1 || p.to_partial;
        if (ok) {
            tc_fence_after();
            float* dst = (split_k ? mat_partial + (size_t)split * p.n_tok * mat_n_out : p.out) + (size_t)row * mat_n_out + n0;
            const bool add = !split_k && p.accumulate;
#pragma unroll
            for (int c = 0; c < kBN / 32; c++) {
                float v[32];
                tmem_ld32(tmem + ((uint32_t)(lg * 32) << 16) + c * 32, v);
                tmem_wait_ld();
                if (row < p.n_tok) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        const int col = n0 + c * 32 + i;
                        if (col + 3 < mat_n_out) {
                            float4* d4 = reinterpret_cast<float4*>(dst + c * 32 + i);
                            float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                            if (add) { const float4 old = *d4; o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; }
                            *d4 = o;
                        } else {
                            for (int e = 0; e < 4; e++)
                                if (col + e < mat_n_out) dst[c * 32 + i + e] = add ? dst[c * 32 + i + e] + v[i + e] : v[i + e];
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(p.status, 1);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// out (+)= sum over the k slices, in slice order
__global__ void splitk_reduce_kernel(float* out, const float* partial, int n_split, size_t n, int accumulate) {
    LINEAR_PDL_TRIGGER();
    LINEAR_PDL_WAIT();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    float4 acc = accumulate ? *reinterpret_cast<const float4*>(out + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < n_split; s++) {
        const float4 v = *reinterpret_cast<const float4*>(partial + (size_t)s * n + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4*>(out + i) = acc;
}

// hi = f16(x), lo = f16(x - hi)
__global__ void split_f16_kernel(__half* hi, __half* lo, const float* x, size_t n) {
    LINEAR_PDL_TRIGGER();
    LINEAR_PDL_WAIT();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    const float4 v = *reinterpret_cast<const float4*>(x + i);
    const float f[4] = {v.x, v.y, v.z, v.w};
    __half h[4], l[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        h[e] = __float2half_rn(f[e]);
        l[e] = __float2half_rn(f[e] - __half2float(h[e]));
    }
    *reinterpret_cast<uint2*>(hi + i) = *reinterpret_cast<const uint2*>(h);
    *reinterpret_cast<uint2*>(lo + i) = *reinterpret_cast<const uint2*>(l);
}

__device__ __forceinline__ void store_split4(__half* hi, __half* lo, size_t i, const float (&f)[4]) {
    __half h[4], l[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        h[e] = __float2half_rn(f[e]);
        l[e] = __float2half_rn(f[e] - __half2float(h[e]));
    }
    *reinterpret_cast<uint2*>(hi + i) = *reinterpret_cast<const uint2*>(h);
    *reinterpret_cast<uint2*>(lo + i) = *reinterpret_cast<const uint2*>(l);
}

// hi/lo of rmsnorm(x) = x * rsqrt(mean(x^2) + eps) * w, one CTA per token row (ops::rmsnorm, src/ops.cpp:227-232,
// with the same expression order as the standalone norm kernel, so the split sees the same f32 values).
__global__ void rmsnorm_split_kernel(__half* hi, __half* lo, const float* x, const float* w, int n, float eps) {
    LINEAR_PDL_TRIGGER();
    LINEAR_PDL_WAIT();
    __shared__ float red[32];
    const float* xr = x + (size_t)blockIdx.x * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += xr[i] * xr[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (threadIdx.x == 0) red[0] = 1.0f / sqrtf(v / float(n) + eps);
    }
    __syncthreads();
    const float scale = red[0];
    for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(xr + i), g = *reinterpret_cast<const float4*>(w + i);
        const float f[4] = {v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w};
        store_split4(hi, lo, (size_t)blockIdx.x * n + i, f);
    }
}

// Consumers of k-slice partials [n_split][n_tok][n_out]: the sum over slices (always in slice order) is folded into
// the kernel that needs the result, so a split-k GEMM costs no reduction launch of its own.
struct Slices {
    const float* base;
    int n_split;
};
__device__ __forceinline__ float4 sum_slices(const Slices& p, size_t idx, size_t slice_elems, float4 acc) {
    for (int sl = 0; sl < p.n_split; sl++) {
        const float4 v = *reinterpret_cast<const float4*>(p.base + sl * slice_elems + idx);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    return acc;
}

// Up to three plain outputs (q, k, v): out_m = sum of its slices. grid.y selects the output.
struct FinishGroup {
    Slices in[3];
    float* out[3];
    int n_out[3];
};
__global__ void finish_group_kernel(const FinishGroup g, int n_tok) {
    LINEAR_PDL_TRIGGER();
    LINEAR_PDL_WAIT();
    const int m = blockIdx.y;
    const Slices in = m == 0 ? g.in[0] : m == 1 ? g.in[1] : g.in[2];
    float* out = m == 0 ? g.out[0] : m == 1 ? g.out[1] : g.out[2];
    const size_t n = (size_t)n_tok * (m == 0 ? g.n_out[0] : m == 1 ? g.n_out[1] : g.n_out[2]);
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    *reinterpret_cast<float4*>(out + i) = sum_slices(in, i, n, make_float4(0.f, 0.f, 0.f, 0.f));
}

// x[t][:] += sum of slices (the residual add of wo / down), then, if norm_w is given, hi/lo of rmsnorm(x[t]) for the
// next projections. One CTA per token.
__global__ void finish_residual_norm_kernel(float* x, const Slices in, __half* hi, __half* lo, const float* norm_w, int n, int n_tok,
                                            float eps) {
    __shared__ float red[32];
    LINEAR_PDL_TRIGGER();
    LINEAR_PDL_WAIT();
    const size_t row = (size_t)blockIdx.x * n;
    const size_t slice = (size_t)n_tok * n;
    float ss = 0.f;
    for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
        const float4 v = sum_slices(in, row + i, slice, *reinterpret_cast<const float4*>(x + row + i));
        *reinterpret_cast<float4*>(x + row + i) = v;
        ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
    }
    if (norm_w == nullptr) return;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (threadIdx.x == 0) red[0] = 1.0f / sqrtf(v / float(n) + eps);
    }
    __syncthreads();
    const float scale = red[0];
    for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(x + row + i), g = *reinterpret_cast<const float4*>(norm_w + i);
        const float f[4] = {v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w};
        store_split4(hi, lo, row + i, f);
    }
}

// hi/lo of silu(sum of gate slices) * (sum of up slices)
__global__ void finish_swiglu_kernel(__half* hi, __half* lo, const Slices gate, const Slices up, size_t n) {
    LINEAR_PDL_TRIGGER();
    LINEAR_PDL_WAIT();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 g = sum_slices(gate, i, n, z), u = sum_slices(up, i, n, z);
    const float f[4] = {g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y, g.z / (1.0f + expf(-g.z)) * u.z,
                        g.w / (1.0f + expf(-g.w)) * u.w};
    store_split4(hi, lo, i, f);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

// f16 matrix [rows][cols] row-major, boxes of box_rows rows x 64 columns, 128-byte swizzle, zero fill outside
bool make_map(CUtensorMap* map, const void* base, int rows, int cols, int box_rows = 128) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

struct ingot_linear_ws {
    __half* hi = nullptr;
    __half* lo = nullptr;
    float* partial = nullptr;
    int* status = nullptr;
    size_t act_elems = 0, partial_floats = 0;  // partial_floats: per slot; kSlots slots
    int slot_split[3] = {0, 0, 0};             // slices the last GEMM into each slot produced
    int slot_out[3] = {0, 0, 0};               // and its output width
    int num_sms = 0;
    int prepared_tok = 0, prepared_in = 0;
    CUtensorMap map_hi, map_lo;
    std::map<std::tuple<const void*, int, int>, CUtensorMap> w_maps;  // one per weight matrix
};

// (Re)builds the activation tensor maps when the prepared shape changes.
static cudaError_t set_prepared(ingot_linear_ws* ws, int n_in, int n_tok) {
    if (ws->prepared_tok != n_tok || ws->prepared_in != n_in) {
        if (!make_map(&ws->map_hi, ws->hi, n_tok, n_in) || !make_map(&ws->map_lo, ws->lo, n_tok, n_in)) return cudaErrorUnknown;
        ws->prepared_tok = n_tok;
        ws->prepared_in = n_in;
    }
    return cudaGetLastError();
}

extern "C" {

// max_tok x max_in: the largest activation matrix that will be prepared; also the largest output (tokens x width).
cudaError_t ingot_linear_ws_create(ingot_linear_ws** out, int max_tok, int max_in) {
    *out = nullptr;
    ingot_linear_ws* ws = new ingot_linear_ws();
    ws->act_elems = (size_t)max_tok * max_in;
    // k-slice partials: three slots, each at least two full-width slices of the largest batch (the hi-plane and the
    // lo-plane product of a quantised matrix), 24 MB or more
    ws->partial_floats = std::max((size_t)6 << 20, 2 * ws->act_elems);
    int dev = 0;
    cudaError_t e;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&ws->num_sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess ||
        (e = cudaMalloc(&ws->hi, ws->act_elems * 2)) != cudaSuccess || (e = cudaMalloc(&ws->lo, ws->act_elems * 2)) != cudaSuccess ||
        (e = cudaMalloc(&ws->partial, 3 * ws->partial_floats * 4)) != cudaSuccess || (e = cudaMalloc(&ws->status, sizeof(int))) != cudaSuccess ||
        (e = cudaMemset(ws->status, 0, sizeof(int))) != cudaSuccess ||
        (e = cudaFuncSetAttribute(linear_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes)) != cudaSuccess) {
        cudaFree(ws->hi); cudaFree(ws->lo); cudaFree(ws->partial); cudaFree(ws->status);
        delete ws;
        return e;
    }
    *out = ws;
    return cudaSuccess;
}

void ingot_linear_ws_destroy(ingot_linear_ws* ws) {
    if (!ws) return;
    cudaFree(ws->hi); cudaFree(ws->lo); cudaFree(ws->partial); cudaFree(ws->status);
    delete ws;
}

// Whether a projection of this shape can take the tensor-core path.
int ingot_linear_tc_supported(const ingot_linear_ws* ws, int w_is_f16, int n_in, int n_out, int n_tok) {
    return ws && encode_fn() && w_is_f16 && n_tok >= 16 && n_in % kBK == 0 && n_out % 4 == 0 && (size_t)n_tok * n_in <= ws->act_elems;
}

// Splits x [n_tok][n_in] f32 into the workspace's hi/lo f16 matrices; the following ingot_linear_tc_run calls use them.
cudaError_t ingot_linear_tc_prepare(ingot_linear_ws* ws, const float* x, int n_in, int n_tok, cudaStream_t s) {
    const size_t n = (size_t)n_tok * n_in;
    if (n > ws->act_elems || n_in % kBK != 0) return cudaErrorInvalidValue;
    cudaError_t le = launch_pdl(split_f16_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, s, ws->hi, ws->lo, x, n);
    if (le != cudaSuccess) return le;
    return set_prepared(ws, n_in, n_tok);
}

// The same with the producer of the activations folded in: rmsnorm(x; norm_w, eps).
cudaError_t ingot_linear_tc_prepare_norm(ingot_linear_ws* ws, const float* x, const float* norm_w, float eps, int n_in, int n_tok,
                                         cudaStream_t s) {
    if ((size_t)n_tok * n_in > ws->act_elems || n_in % kBK != 0) return cudaErrorInvalidValue;
    cudaError_t le = launch_pdl(rmsnorm_split_kernel, dim3(n_tok), dim3(256), 0, s, ws->hi, ws->lo, x, norm_w, n_in, eps);
    if (le != cudaSuccess) return le;
    return set_prepared(ws, n_in, n_tok);
}

// count <= 3 matrices W_m [n_out_m][n_in] in one launch; matrix m goes to `out` (count == 1, !to_partial) or as k slices to
// scratch slot first_slot + m.
// append: the slices are written behind the ones the slots already hold (all slots of the group must hold the same
// number), so that a second product - the lo plane of a quantised matrix after its hi plane - simply adds k slices
// for the consumer kernel to sum.
static cudaError_t launch_gemm(ingot_linear_ws* ws, float* out, const void* const* w, int n_in, const int* n_out, int count,
                               int accumulate, int first_slot, bool to_partial, bool append, cudaStream_t s) {
    const int n_tok = ws->prepared_tok;
    if (n_in != ws->prepared_in || n_tok < 1 || count < 1 || first_slot < 0 || first_slot + count > 3 || (count > 1 && !to_partial) ||
        (append && !to_partial))
        return cudaErrorInvalidValue;
    const int held = append ? ws->slot_split[first_slot] : 0;
    for (int m = 0; m < count && append; m++)
        if (ws->slot_split[first_slot + m] != held || ws->slot_out[first_slot + m] != n_out[m]) return cudaErrorInvalidValue;
    const CUtensorMap* maps[3] = {nullptr, nullptr, nullptr};
    GemmParams p = {};
    int tiles_n = 0, fit = 1 << 30;
    for (int m = 0; m < count; m++) {
        const auto key = std::make_tuple(w[m], n_out[m], n_in);
        auto it = ws->w_maps.find(key);
        if (it == ws->w_maps.end()) {
            CUtensorMap tm;
            if (!make_map(&tm, w[m], n_out[m], n_in, kBN)) return cudaErrorUnknown;
            it = ws->w_maps.emplace(key, tm).first;
        }
        maps[m] = &it->second;
        tiles_n += (n_out[m] + kBN - 1) / kBN;
        p.tile_end[m] = tiles_n;
        p.n_out[m] = n_out[m];
        p.partial[m] = ws->partial + (size_t)(first_slot + m) * ws->partial_floats + (size_t)held * n_tok * n_out[m];
        fit = std::min(fit, (int)(ws->partial_floats / ((size_t)n_tok * n_out[m])) - held);
    }
    for (int m = count; m < 3; m++) { maps[m] = maps[count - 1]; p.tile_end[m] = tiles_n; p.n_out[m] = n_out[count - 1]; p.partial[m] = p.partial[count - 1]; }
    const int tiles = tiles_n * ((n_tok + kBM - 1) / kBM);
    const int k_steps = n_in / kBK;
    // enough k slices to give every SM a CTA, at least 4 k-steps each, and no more than the slots hold
    if (to_partial && fit < 1) return cudaErrorInvalidValue;
    const int n_split = std::max(1, std::min({ws->num_sms / tiles, k_steps / 4, fit}));
    p.out = out; p.status = ws->status;
    p.n_tok = n_tok; p.k_steps = k_steps; p.n_split = n_split; p.accumulate = accumulate;
    p.to_partial = to_partial ? 1 : 0;
    dim3 grid(tiles_n, (n_tok + kBM - 1) / kBM, n_split);
    cudaError_t le = launch_pdl(linear_sm100_kernel, grid, dim3(kThreads), (size_t)kSmemBytes, s, ws->map_hi, ws->map_lo, *maps[0], *maps[1],
                                *maps[2], p);
    if (le != cudaSuccess) return le;
    for (int m = 0; m < count; m++) {
        ws->slot_split[first_slot + m] = held + n_split;
        ws->slot_out[first_slot + m] = n_out[m];
    }
    if (!to_partial && n_split > 1) {
        const size_t n = (size_t)n_tok * n_out[0];
        le = launch_pdl(splitk_reduce_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, s, out, (const float*)p.partial[0], n_split, n,
                        accumulate);
        if (le != cudaSuccess) return le;
    }
    return cudaGetLastError();
}

// out [n_tok][n_out] (+)= prepared activations x W^T, W f16 [n_out][n_in] on the device.
cudaError_t ingot_linear_tc_run(ingot_linear_ws* ws, float* out, const void* w, int n_in, int n_out, int accumulate, cudaStream_t s) {
    return launch_gemm(ws, out, &w, n_in, &n_out, 1, accumulate, 0, false, false, s);
}

// The same product left as k slices in scratch slot 0..2 for one of the ingot_linear_tc_finish_* calls below.
cudaError_t ingot_linear_tc_run_partial(ingot_linear_ws* ws, const void* w, int n_in, int n_out, int slot, cudaStream_t s) {
    return launch_gemm(ws, nullptr, &w, n_in, &n_out, 1, 0, slot, true, false, s);
}

// The products of count <= 3 matrices that read the same prepared activations (q/k/v, gate/up), as one launch:
// matrix m is left as k slices in scratch slot m.
// append != 0: the slices are added behind those the slots hold from the call before (same widths).
cudaError_t ingot_linear_tc_run_partial_group(ingot_linear_ws* ws, const void* const* w, int n_in, const int* n_out, int count,
                                              int first_slot, int append, cudaStream_t s) {
    return launch_gemm(ws, nullptr, w, n_in, n_out, count, 0, first_slot, true, append != 0, s);
}

static Slices slices_of(const ingot_linear_ws* ws, int slot) {
    return Slices{ws->partial + (size_t)slot * ws->partial_floats, ws->slot_split[slot]};
}

// outs[m] = product left in slot m, for count <= 3 outputs (q, k, v) in one launch.
cudaError_t ingot_linear_tc_finish_group(ingot_linear_ws* ws, float* const* outs, int count, cudaStream_t s) {
    if (count < 1 || count > 3) return cudaErrorInvalidValue;
    FinishGroup g = {};
    int widest = 0;
    for (int m = 0; m < count; m++) {
        g.in[m] = slices_of(ws, m);
        g.out[m] = outs[m];
        g.n_out[m] = ws->slot_out[m];
        widest = std::max(widest, ws->slot_out[m]);
    }
    const size_t n = (size_t)ws->prepared_tok * widest;
    cudaError_t le = launch_pdl(finish_group_kernel, dim3((unsigned)((n / 4 + 255) / 256), count), dim3(256), 0, s, g, ws->prepared_tok);
    if (le != cudaSuccess) return le;
    return cudaGetLastError();
}

// x += product left in `slot` (the residual add), then, with norm_w, the hi/lo activations of rmsnorm(x; norm_w, eps)
// become the prepared input of the next projections (n_in = the product's width).
cudaError_t ingot_linear_tc_finish_residual_norm(ingot_linear_ws* ws, float* x, const float* norm_w, float eps, int slot, cudaStream_t s) {
    const int n = ws->slot_out[slot], n_tok = ws->prepared_tok;
    if (n % 4 != 0 || (norm_w && ((size_t)n_tok * n > ws->act_elems || n % kBK != 0))) return cudaErrorInvalidValue;
    cudaError_t le = launch_pdl(finish_residual_norm_kernel, dim3(n_tok), dim3(256), 0, s, x, slices_of(ws, slot), ws->hi, ws->lo, norm_w, n, n_tok, eps);
    if (le != cudaSuccess) return le;
    return norm_w ? set_prepared(ws, n, n_tok) : cudaGetLastError();
}

// hi/lo of silu(slot_gate) .* slot_up become the prepared input of the next projection.
cudaError_t ingot_linear_tc_finish_swiglu(ingot_linear_ws* ws, int slot_gate, int slot_up, cudaStream_t s) {
    const int n_in = ws->slot_out[slot_gate], n_tok = ws->prepared_tok;
    const size_t n = (size_t)n_tok * n_in;
    if (ws->slot_out[slot_up] != n_in || n > ws->act_elems || n_in % kBK != 0) return cudaErrorInvalidValue;
    cudaError_t le = launch_pdl(finish_swiglu_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, s, ws->hi, ws->lo, slices_of(ws, slot_gate), slices_of(ws, slot_up), n);
    if (le != cudaSuccess) return le;
    return set_prepared(ws, n_in, n_tok);
}

// The status word: non-zero after a bounded wait expired in some launch since the last call. Synchronises the device.
int ingot_linear_ws_status(ingot_linear_ws* ws) {
    int v = 0;
    if (cudaMemcpy(&v, ws->status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (v) cudaMemset(ws->status, 0, sizeof(int));
    return v;
}

}  // extern "C"
