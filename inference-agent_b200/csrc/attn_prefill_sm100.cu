// K2 (tcgen05 form) — causal GQA flash-attention prefill / chunked prefill for sm_100a:
// TMA-staged K/V tiles, tcgen05.mma with accumulators in tensor memory, online softmax.
//
// Replaces n_tok iterations of the CPU reference's attention lambda (src/backend.h:16-20 looping
// src/cpu_backend.cpp:51-69) and Metal's attn_prefill (shaders/kernels.metal:518-633) for long
// prefills on a contiguous cache. Query token i sits at position q_pos0 + i and sees keys
// 0..q_pos0+i (kernels.metal:555,578).
//
// Work decomposition. One CTA = one KV head x 256 query ROWS (two 128-row tiles). A row is a
// (token, query head of the GQA group) pair: row R -> token R / G, head R % G, so the G query heads
// that share the KV head sit in the M dimension of the MMAs and every staged K/V tile serves all of
// them. The CTA walks the keys in tiles of 128.
//
// Roles (12 warps, one CTA per SM):
//   warp 0       TMA producer: K_j and V_j tiles ([128 keys][128 dims] f16 = 32 KB, as two
//                128-byte-swizzled boxes of 64 dims) into a 4-slot shared-memory ring.
//   warp 1       MMA issuer (one elected thread): S_q = Q_q K_j^T (SS MMA, 128x128x128) and
//                O_q += P_q V_j (A operand = P from tensor memory, B = V tile, MN-major).
//   warps 4-7    softmax for Q tile 0; warps 8-11 for Q tile 1: one thread per row. tcgen05.ld the
//                128 scores of the row, running max / sum in the exp2 domain, P = exp2(..) rounded to
//                f16 and stored over the first 64 columns of the same S region (tcgen05.st).
//                The O accumulator is rescaled only when the running max grew by more than 2^8
//                (P <= 256 stays exact enough in f16; l and O carry the same reference max).
// Tensor memory (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_q aliases S_q.
// The tensor pipe executes one thread's MMAs in issue order, which is what makes the aliasing safe:
//   QK(0,0) QK(1,0) | PV(0,j) QK(0,j+1) PV(1,j) QK(1,j+1) | ...
// so while the softmax warps of one tile work, the tensor pipe runs the other tile's MMAs.
//
// Every mbarrier wait is bounded (wall-clock limit): on expiry the CTA raises a bit in the cache's
// status word, every role leaves its loop, outstanding TMA copies are drained with a bounded wait
// and tensor memory is released before the CTA exits.
#include "attn_common.cuh"
#include "ingot_internal.cuh"
#include "sm100_ptx.cuh"

#include <algorithm>
#include <mutex>
#include <vector>

namespace {

using namespace ingot_sm100;

constexpr int kTileRows = 128;        // rows per Q tile (= TMEM lanes)
constexpr int kTileKeys = 128;        // keys per K/V tile
constexpr int kStages = 4;            // K/V ring slots
constexpr int kStageBytes = kTileKeys * kHeadDim * 2;   // 32 KB
constexpr int kHalfBytes = kStageBytes / 2;             // one 64-dim box
constexpr int kQBytes = kTileRows * kHeadDim * 2;       // 32 KB per Q tile
constexpr int kThreads = 384;
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
#ifndef INGOT_POLY_EVERY
#define INGOT_POLY_EVERY 1000000
#endif
// One score pair in this many takes the FMA-pipe polynomial exp2 instead of MUFU ex2. Measured on a B200
// at 32768 tokens: never 1233, every 6th 1129, every 4th 1103, every 2nd 1088 TFLOP/s — the softmax warps
// are bound by instruction issue and latency, not by MUFU throughput, so the default is "never".
constexpr int kPolyEvery = INGOT_POLY_EVERY;

// shared memory map (dynamic, 1024-byte aligned base)
constexpr int kOffQ = 0;                                  // 2 Q tiles
constexpr int kOffKV = 2 * kQBytes;                       // ring
constexpr int kOffBar = kOffKV + kStages * kStageBytes;   // barriers
constexpr int kSmemBytes = kOffBar + 256 + 1024;          // + alignment slack

struct Bars {
    uint64_t kv_full[kStages];
    uint64_t kv_empty[kStages];
    uint64_t q_ready;
    uint64_t s_ready[2];
    uint64_t p_ready[2];
    uint64_t o_final[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

constexpr int kMaxOutputs = 8;

struct Sm100Params {
    const void* q;
    void* outs[kMaxOutputs];  // every output row is stored to each of these (this GPU's buffer and, for a
    int n_outs;               // KV-head-sharded prefill, the peers' buffers: plain peer stores over NVLink)
    int out_n_head;           // heads per token in the destination layout [token][out_n_head][128]
    int out_head0;            // destination index of this call's first query head
    // Completion signalling for the multi-destination form (null: none). The CTA that finishes last - found with a
    // ticket in this GPU's memory - adds 1 to counter `src_index` of every destination's counter array, released
    // at system scope behind all of the grid's stores.
    unsigned int* signals[kMaxOutputs];
    int src_index;
    int* ticket;
    int* status;
    int q_dtype, out_dtype;
    int n_head, group;
    int q_pos0, n_tok;
    const int32_t* block_table;  // paged cache: this sequence's block-table row (device), else null
    int capacity;             // paged: blocks in the pool
    int n_split;              // > 1: grid.z CTAs share a row tile, each walks a slice of the key tiles and writes an
    float* part;              //      unnormalised partial (o[128], m, l per row) here for prefill_merge_kernel
    unsigned long long wait_limit_ns;  // bound of every mbarrier wait
    int test_stall_producer;  // test hook: the TMA producer issues nothing, so that the bounded waits expire
    float scale_log2;
    size_t q_extent, out_extent, part_extent;  // bounds-check build: elements of q, of each output, floats of the partials
};

// Build with -DINGOT_PREFILL_TIMING to make CTA (0,0,0) print, per key tile, the cycles its MMA warp and
// its first softmax warps spend in each phase (diagnostics only; the printing build is not for production).
#ifdef INGOT_PREFILL_TIMING
#define TIMING(...) __VA_ARGS__
#else
#define TIMING(...)
#endif

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Packed f32x2 arithmetic (sm_100): one instruction works on two floats.
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
    asm("{\n.reg .b64 ra, rb, rc, rd;\n"
        "mov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\nmov.b64 rc, {%6, %7};\n"
        "fma.rn.f32x2 rd, ra, rb, rc;\nmov.b64 {%0, %1}, rd;\n}\n"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void fadd2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    asm("{\n.reg .b64 ra, rb, rd;\n"
        "mov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\n"
        "add.rn.f32x2 rd, ra, rb;\nmov.b64 {%0, %1}, rd;\n}\n"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}

// 2^x for a pair on the FMA pipe instead of the MUFU pipe: round x to an integer n with the
// 1.5*2^23 trick, evaluate a degree-4 minimax polynomial of 2^f on f = x - n in [-0.5, 0.5]
// (max relative error 2.7e-6, far below the f16 rounding of P) and add n to the exponent field.
// Inputs are clamped at -126 (masked scores are -inf; anything that small rounds to 0 in f16 anyway).
__device__ __forceinline__ void exp2_poly2(float& r0, float& r1, float x0, float x1) {
    constexpr float kMagic = 12582912.f;  // 1.5 * 2^23
    x0 = fmaxf(x0, -126.f);
    x1 = fmaxf(x1, -126.f);
    float t0, t1, n0, n1, f0, f1, p0, p1;
    fadd2(t0, t1, x0, x1, kMagic, kMagic);
    fadd2(n0, n1, t0, t1, -kMagic, -kMagic);
    ffma2(f0, f1, n0, n1, -1.f, -1.f, x0, x1);
    ffma2(p0, p1, f0, f1, 0.009570102207362652f, 0.009570102207362652f, 0.05591785907745361f, 0.05591785907745361f);
    ffma2(p0, p1, p0, p1, f0, f1, 0.240247443318367f, 0.240247443318367f);
    ffma2(p0, p1, p0, p1, f0, f1, 0.6931217908859253f, 0.6931217908859253f);
    ffma2(p0, p1, p0, p1, f0, f1, 0.9999992847442627f, 0.9999992847442627f);
    r0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
    r1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}

// Instruction descriptor, kind::f16: f16 A and B, f32 accumulate, M = 128, N = 128.
constexpr uint32_t kIdescBase = (1u << 4) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kIdescQK = kIdescBase;               // A K-major, B K-major
constexpr uint32_t kIdescPV = kIdescBase | (1u << 16);  // B (= V) MN-major

__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_sm100_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                          const Sm100Params p) {
    extern __shared__ unsigned char smem_dyn[];
    TIMING(const long long t_entry = clock64();)
    INGOT_PDL_TRIGGER();
    const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char* smem_al = smem_dyn + (smem_base - smem_u32(smem_dyn));
    Bars* bars = reinterpret_cast<Bars*>(smem_al + kOffBar);
    volatile uint32_t* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warp_u = __shfl_sync(0xffffffffu, warp, 0);  // the same number, known to the compiler as warp-uniform
    const int G = p.group;
    const int kvh = blockIdx.y;
    const int n_rows = p.n_tok * G;
    const int tile256 = gridDim.x - 1 - blockIdx.x;  // heavier (later) tiles first
    const int row_base = tile256 * 2 * kTileRows;
    const int last_row = min(row_base + 2 * kTileRows, n_rows) - 1;
    const int n_kv = (p.q_pos0 + last_row / G + 1 + kTileKeys - 1) / kTileKeys;  // K/V tiles these rows need
    // Split-KV prefill (few row tiles, e.g. a 512-token chunk onto a long cache): grid.z CTAs share the rows
    // and each walks key tiles [j0, j1). n_it may be 0 for early row tiles; such a CTA writes an empty partial.
    const int split = blockIdx.z;
    const int j0 = (int)((long long)n_kv * split / p.n_split), j1 = (int)((long long)n_kv * (split + 1) / p.n_split);
    const int n_it = j1 - j0;

    auto bar_addr = [&](const uint64_t* b) { return smem_u32(b); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) { mbar_init(bar_addr(&bars->kv_full[s]), 1); mbar_init(bar_addr(&bars->kv_empty[s]), 1); }
        mbar_init(bar_addr(&bars->q_ready), 8);      // one arrival per softmax warp
        for (int q = 0; q < 2; q++) {
            mbar_init(bar_addr(&bars->s_ready[q]), 1);
            mbar_init(bar_addr(&bars->p_ready[q]), 4);  // one arrival per warp of the tile
            mbar_init(bar_addr(&bars->o_final[q]), 1);
        }
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Everything above (barriers, tensor memory) is this CTA's own; from here on the kernel reads what the kernel
    // before it in the stream produced (q, the newest cache rows) and writes what that kernel may still be reading.
    INGOT_PDL_WAIT();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    TIMING(const long long t_setup = clock64();)

    if (warp_u < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        if (warp_u == 0) {
            // ---------------- TMA producer ----------------
            // Contiguous cache: lane 0 issues two boxes of [128 keys][64 dims] per tile. Paged cache: a tile
            // is eight 16-token blocks; lanes 0-7 look their block up in the block table and each issue the
            // two [16 keys][64 dims] boxes of it, 2 KB apart in the same swizzled tile. Blocks past the last
            // key (or invalid entries, which also raise the status word) are replaced by block 0: their
            // columns are masked, they only have to be finite.
            int armed = 0;  // ring slots handed to TMA so far
            bool ok = true;
            const int last_block = (p.q_pos0 + p.n_tok - 1) / kBlockTokens;
            for (int it = 0; it < (p.test_stall_producer ? 0 : 2 * n_it) && ok; it++) {
                const int s = it % kStages;
                const uint32_t par = (uint32_t)((it / kStages) & 1);
                const uint32_t full = bar_addr(&bars->kv_full[s]);
                if (lane == 0) {
                    ok = mbar_wait(bar_addr(&bars->kv_empty[s]), par ^ 1u, abort_flag, p.wait_limit_ns);
                    if (ok) mbar_expect_tx(full, kStageBytes);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                const uint32_t dst = smem_base + kOffKV + s * kStageBytes;
                const CUtensorMap* map = (it & 1) ? &map_v : &map_k;
                const int key0 = (j0 + (it >> 1)) * kTileKeys;
                if (p.block_table == nullptr) {
                    if (lane == 0) {
                        tma_load_3d(dst, map, 0, key0, kvh, full);
                        tma_load_3d(dst + kHalfBytes, map, 64, key0, kvh, full);
                    }
                } else if (lane < kTileKeys / kBlockTokens) {
                    const int lb = key0 / kBlockTokens + lane;
                    int blk = lb <= last_block ? p.block_table[lb] : 0;
                    if (blk < 0 || blk >= p.capacity) {
                        atomicOr(p.status, kDevErrBlockRange);
                        blk = 0;
                    }
                    const int z = blk * (int)gridDim.y + kvh;  // pool is [block][kv head][16][128]
                    tma_load_3d(dst + lane * (kBlockTokens * 128), map, 0, 0, z, full);
                    tma_load_3d(dst + kHalfBytes + lane * (kBlockTokens * 128), map, 64, 0, z, full);
                }
                armed = it + 1;
            }
            if (!ok && lane == 0) {
                // Drain: copies already issued must land before the CTA's shared memory is released.
                for (int it = max(0, armed - kStages); it < armed; it++) {
                    const uint64_t t0 = globaltimer_ns();
                    const uint32_t full = bar_addr(&bars->kv_full[it % kStages]);
                    while (!mbar_try_wait(full, (uint32_t)((it / kStages) & 1)) && globaltimer_ns() - t0 < 100000000ull) {}
                }
            }
        } else if (warp_u == 1) {
            // ---------------- MMA issuer ----------------
            // The whole warp walks this loop and only the tcgen05 instructions sit under an elected lane.
            // With warp-uniform control flow the compiler keeps descriptors and addresses in uniform
            // registers, which is what tcgen05.mma reads; a loop run by one lane of a diverged warp has to
            // move every descriptor from vector to uniform registers first and then issues an MMA every
            // ~88 cycles instead of the tensor pipe's 64.
            const uint32_t q_base = smem_base + kOffQ;
            auto stage_addr = [&](int it) { return smem_base + kOffKV + (it % kStages) * kStageBytes; };
            auto wait_full = [&](int it) {
                return __all_sync(0xffffffffu, mbar_wait(bar_addr(&bars->kv_full[it % kStages]), (uint32_t)((it / kStages) & 1),
                                                         abort_flag, p.wait_limit_ns));
            };
            // S_q = Q_q K^T : 8 k-steps of 16 dims; dims 0-63 in the first 16 KB box, 64-127 in the second.
            auto issue_qk = [&](int q, uint32_t k_addr) {
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    const uint32_t off = (ks >> 2) * kHalfBytes + (ks & 3) * 32;
                    tc_mma_ss(tmem + q * 128, make_desc(q_base + q * kQBytes + off, 16, 1024), make_desc(k_addr + off, 16, 1024),
                              kIdescQK, ks > 0);
                }
                tc_commit(bar_addr(&bars->s_ready[q]));
            };
            // O_q += P_q V : 8 k-steps of 16 keys; P packed f16 in TMEM (8 columns per step);
            // V rows are 128-byte swizzled, 16 keys = 2048 B further per step, dims 64-127 one box further.
            auto issue_pv = [&](int q, uint32_t v_addr, bool first) {
#pragma unroll
                for (int ks = 0; ks < 8; ks++)
                    tc_mma_ts(tmem + 256 + q * 128, tmem + q * 128 + ks * 8, make_desc(v_addr + ks * 2048, kHalfBytes, 1024),
                              kIdescPV, (!first || ks > 0) ? 1u : 0u);
            };
            bool ok = __all_sync(0xffffffffu, mbar_wait(bar_addr(&bars->q_ready), 0, abort_flag, p.wait_limit_ns));
            ok = ok && (n_it == 0 || wait_full(0));
            TIMING(const long long t_begin = clock64(); const uint64_t g_begin = globaltimer_ns(); long long w_full = 0, w_p = 0, t_iss = 0, c0, c1;)
            if (ok && n_it > 0) {
                tc_fence_after();
                if (elect_one()) {
                    issue_qk(0, stage_addr(0));
                    issue_qk(1, stage_addr(0));
                    tc_commit(bar_addr(&bars->kv_empty[0]));
                }
                __syncwarp();
            }
            for (int j = 0; j < n_it && ok; j++) {  // j counts this CTA's key tiles from j0
                const int it_v = 2 * j + 1, it_k = 2 * j + 2;
                const bool more = j + 1 < n_it;
                TIMING(c0 = clock64();)
                ok = wait_full(it_v) && (!more || wait_full(it_k));
                TIMING(w_full += clock64() - c0;)
                if (!ok) break;
                const uint32_t v_addr = stage_addr(it_v), k_addr = stage_addr(it_k);
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    TIMING(c0 = clock64();)
                    ok = __all_sync(0xffffffffu, mbar_wait(bar_addr(&bars->p_ready[q]), (uint32_t)(j & 1), abort_flag, p.wait_limit_ns));
                    if (!ok) break;
                    tc_fence_after();
                    TIMING(c1 = clock64(); w_p += c1 - c0;)
                    if (elect_one()) {
                        issue_pv(q, v_addr, j == 0);
                        if (q == 1) tc_commit(bar_addr(&bars->kv_empty[it_v % kStages]));
                        if (more) {
                            issue_qk(q, k_addr);
                            if (q == 1) tc_commit(bar_addr(&bars->kv_empty[it_k % kStages]));
                        } else {
                            tc_commit(bar_addr(&bars->o_final[q]));
                        }
                    }
                    __syncwarp();
                    TIMING(t_iss += clock64() - c1;)
                }
            }
            TIMING(if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0 && n_it > 0)
                       printf("MMA warp: %d key tiles, cycles/tile %lld: wait K/V %lld, wait P (2 tiles) %lld, issue 32 MMAs %lld; SM clock %.3f GHz\n", n_it,
                              (clock64() - t_begin) / n_it, w_full / n_it, w_p / n_it, t_iss / n_it,
                              (double)(clock64() - t_begin) / (double)(globaltimer_ns() - g_begin));)
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
        // ---------------- softmax warps: one thread per query row ----------------
        const int q = (warp - 4) >> 2;              // Q tile 0 or 1
        const int row_in_tile = ((warp & 3) << 5) | lane;
        const int R = row_base + q * kTileRows + row_in_tile;
        const bool valid = R < n_rows;
        const int tok = valid ? R / G : 0;
        const int head = kvh * G + (valid ? R % G : 0);
        const int qpos = valid ? p.q_pos0 + tok : 0x3fffffff;  // rows past the end are never masked
        const uint32_t lane_sel = (uint32_t)((warp & 3) << 5) << 16;
        const uint32_t s_tmem = tmem + q * 128 + lane_sel;
        const uint32_t o_tmem = tmem + 256 + q * 128 + lane_sel;

        // Q_q in shared memory is a [128 rows][128 dims] f16 K-major operand with 128-byte swizzle: 16-byte chunk c of
        // row r lands at r*128 + ((c & 7) ^ (r & 7))*16 in the box of dims (c>>3)*64.
        {
            // Stage the tile's Q rows. Each warp stages the 32 rows of its own lanes, two rows (2 x 256 bytes of f16) per
            // load instruction with lane = 16-byte piece, so that global reads are whole 128-byte lines; the owner
            // of a row hands its source row index to the copying lanes. All sixteen loads are issued before the
            // first store: one round trip to L2 instead of sixteen.
            const int my_src = valid ? tok * p.n_head + head : -1;  // row of q [n_tok * n_head][128]
            unsigned char* qtile = smem_al + kOffQ + q * kQBytes;
            const int piece = lane & 15, warp_row0 = (warp & 3) << 5;
            auto put = [&](int it, const uint4& v) {
                const int r = warp_row0 + it * 2 + (lane >> 4);
                *reinterpret_cast<uint4*>(qtile + (piece >> 3) * kHalfBytes + r * 128 + (((piece & 7) ^ (r & 7)) << 4)) = v;
            };
            // One loop per element type, so that the loads of a loop are straight-line code the compiler can issue together.
            if (p.q_dtype == INGOT_F32) {
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    float4 lo[8], hi[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int it = half * 8 + i;
                        const int src = __shfl_sync(0xffffffffu, my_src, it * 2 + (lane >> 4));
                        const size_t e = (size_t)max(src, 0) * kHeadDim + piece * 8;
                        const bool in = src >= 0 && INGOT_CHECK(e, 8, p.q_extent, p.status);
                        const float4* g = reinterpret_cast<const float4*>(static_cast<const float*>(p.q) + e);
                        lo[i] = in ? __ldg(g) : make_float4(0.f, 0.f, 0.f, 0.f);
                        hi[i] = in ? __ldg(g + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int i = 0; i < 8; i++)
                        put(half * 8 + i, make_uint4(pack_half2_rn(lo[i].x, lo[i].y), pack_half2_rn(lo[i].z, lo[i].w),
                                                     pack_half2_rn(hi[i].x, hi[i].y), pack_half2_rn(hi[i].z, hi[i].w)));
                }
            } else {
                const bool bf16 = p.q_dtype == INGOT_BF16;  // same size as f16: the raw loads are the same
                uint4 qv[16];
#pragma unroll
                for (int it = 0; it < 16; it++) {
                    const int src = __shfl_sync(0xffffffffu, my_src, it * 2 + (lane >> 4));
                    const size_t e = (size_t)max(src, 0) * kHeadDim + piece * 8;
                    qv[it] = src >= 0 && INGOT_CHECK(e, 8, p.q_extent, p.status)
                                 ? __ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned short*>(p.q) + e))
                                 : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int it = 0; it < 16; it++) {
                    uint4 v = qv[it];
                    if (bf16) {  // bf16 -> f32 is a 16-bit shift; f32 -> f16 rounds to nearest
                        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int i = 0; i < 4; i++) w[i] = pack_half2_rn(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
                        v = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                    put(it, v);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> async proxy (MMA)
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_addr(&bars->q_ready));
        }
        TIMING(const long long t_q = clock64(); long long t_s0 = 0;)

        float m_ref = 0.f, l = 0.f;
        bool ok = true;
        const int qpos_warp_min = __shfl_sync(0xffffffffu, qpos, 0);  // rows ascend with the lane
        TIMING(long long t_w = 0, t_ld = 0, t_mx = 0, t_ex = 0, t_st = 0, c0, c1, c2, c3, c4; const long long t_begin = clock64();)
        for (int jj = 0; jj < n_it; jj++) {
            const int j = j0 + jj;
            TIMING(c0 = clock64();)
            ok = mbar_wait(bar_addr(&bars->s_ready[q]), (uint32_t)(jj & 1), abort_flag, p.wait_limit_ns);
            TIMING(c1 = clock64(); if (jj == 0) t_s0 = c1;)
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            float s[128];
#pragma unroll
            for (int c = 0; c < 4; c++) tmem_ld32(s_tmem + c * 32, *reinterpret_cast<float(*)[32]>(&s[c * 32]));
            tmem_wait_ld();
            TIMING(c2 = clock64();)

            const int key0 = j * kTileKeys;
            if (key0 + kTileKeys - 1 > qpos_warp_min) {  // warp-uniform: some row of this warp needs the mask
                const int limit = qpos - key0;           // columns > limit are in the future
#pragma unroll
                for (int i = 0; i < 128; i++) s[i] = i <= limit ? s[i] : -INFINITY;
            }
            // Row maximum: four independent chains of nested max (maps onto 3-input max instructions).
            float mxa = fmaxf(s[0], s[1]), mxb = fmaxf(s[2], s[3]), mxc = fmaxf(s[4], s[5]), mxd = fmaxf(s[6], s[7]);
#pragma unroll
            for (int i = 8; i < 128; i += 8) {
                mxa = fmaxf(mxa, fmaxf(s[i], s[i + 1]));
                mxb = fmaxf(mxb, fmaxf(s[i + 2], s[i + 3]));
                mxc = fmaxf(mxc, fmaxf(s[i + 4], s[i + 5]));
                mxd = fmaxf(mxd, fmaxf(s[i + 6], s[i + 7]));
            }
            float mx = fmaxf(fmaxf(mxa, mxb), fmaxf(mxc, mxd));
            mx *= p.scale_log2;  // scale > 0: max commutes with the scaling

            // Lazy rescale: keep the old reference max unless the new one is more than 2^8 above it.
            // (With split keys a row may see nothing but masked columns at first: m_ref stays -inf, every P is
            // 0, and the first finite maximum later "grows" from -inf with a rescale factor of exactly 0.)
            bool grow = jj == 0 || mx > m_ref + kRescaleThreshold;
            if (jj == 0) {
                m_ref = mx;  // finite whenever key 0 is among this CTA's keys (it is visible to every row)
            } else if (__any_sync(0xffffffffu, grow)) {
                const float alpha = grow ? ex2(m_ref - mx) : 1.0f;
                if (grow) { m_ref = mx; l *= alpha; }
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    float o[32];
                    tmem_ld32(o_tmem + c * 32, o);
                    tmem_wait_ld();
                    uint32_t ob[32];
#pragma unroll
                    for (int i = 0; i < 32; i++) ob[i] = __float_as_uint(o[i] * alpha);
                    tmem_st32(o_tmem + c * 32, ob);
                }
            }
            // P = 2^(s*scale - m_ref). A 128x128 tile costs as many MUFU (ex2) cycles as it costs tensor-core
            // cycles, so one pair in kPolyEvery goes to the FMA pipe instead (exp2_poly2); scaling and the
            // row sum use packed f32x2 instructions.
            TIMING(c3 = clock64();)
            const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    float x0, x1, p0, p1;
                    ffma2(x0, x1, s[c * 64 + 2 * i], s[c * 64 + 2 * i + 1], p.scale_log2, p.scale_log2, neg_m, neg_m);
                    if (i % kPolyEvery == kPolyEvery - 1) {
                        exp2_poly2(p0, p1, x0, x1);
                    } else {
                        p0 = ex2(x0);
                        p1 = ex2(x1);
                    }
                    fadd2(sum0, sum1, sum0, sum1, p0, p1);
                    pk[i] = pack_half2_rn(p0, p1);
                }
                tmem_st32(s_tmem + c * 32, pk);
            }
            l += sum0 + sum1;
            TIMING(c4 = clock64();)
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_addr(&bars->p_ready[q]));
            TIMING(t_w += c1 - c0; t_ld += c2 - c1; t_mx += c3 - c2; t_ex += c4 - c3; t_st += clock64() - c4;)
        }
        TIMING(if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (warp & 3) == 0 && lane == 0 && n_it > 0)
                   printf("softmax warp of Q tile %d, cycles/tile %lld: wait S %lld, tcgen05.ld %lld, max+rescale %lld, exp+pack %lld, st+arrive %lld\n", q,
                          (clock64() - t_begin) / n_it, t_w / n_it, t_ld / n_it, t_mx / n_it, t_ex / n_it, t_st / n_it);)

        // ---------------- epilogue: O / l -> global ----------------
        TIMING(const long long t_loop = clock64();)
        if (ok && n_it > 0) {
            ok = mbar_wait(bar_addr(&bars->o_final[q]), 0, abort_flag, p.wait_limit_ns);
            ok = __all_sync(0xffffffffu, ok);
        }
        TIMING(const long long t_of = clock64();)
        const bool partial = p.n_split > 1;
        float* part_row = nullptr;
        if (partial && valid) {
            part_row = p.part + (((size_t)split * gridDim.y + kvh) * n_rows + R) * kPartStride;
            if (n_it == 0) { m_ref = -INFINITY; l = 0.f; }
            part_row[128] = m_ref;
            part_row[129] = l;
        }
        if (ok && n_it == 0 && partial && valid) {
            // No key tile fell to this CTA: an empty partial (weight 0 in the merge).
            for (int i = 0; i < 32; i++) reinterpret_cast<float4*>(part_row)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (ok && n_it > 0) {
            tc_fence_after();
            // O / l goes through shared memory (the tile's Q buffer, idle once its last MMA has retired) so
            // that the global stores are row-contiguous: a warp instruction writes two whole 256-byte row
            // slices instead of 32 scattered 16-byte pieces. That matters most when the rows also go to
            // peer GPUs. One pass moves 256 bytes per row: all 128 dims as f16, or 64 dims as f32.
            const float inv = partial ? 1.0f : 1.0f / l;  // partials stay unnormalised
            const bool f32_out = partial || p.out_dtype == INGOT_F32;
            unsigned char* stage = smem_al + kOffQ + q * kQBytes;  // [128 rows][256 B], 16-byte pieces XOR-swizzled by row
            const int n_pass = f32_out ? 2 : 1;
            const int warp_row0 = (warp & 3) << 5;
            // Destination row of this thread's query row, handed to the lanes that copy it out (no division there):
            // a row of the partials, or (token, head) of the output; -1 past the end.
            const int my_dst = !valid ? -1 : partial ? R : tok * p.out_n_head + p.out_head0 + head;
            const size_t dst_row_bytes = partial ? (size_t)kPartStride * 4 : (size_t)kHeadDim * (f32_out ? 4 : 2);
            unsigned char* dst0 = partial ? reinterpret_cast<unsigned char*>(p.part + ((size_t)split * gridDim.y + kvh) * n_rows * kPartStride)
                                          : static_cast<unsigned char*>(p.outs[0]);
            for (int ps = 0; ps < n_pass; ps++) {
                if (ps) __syncwarp();
                unsigned char* my = stage + row_in_tile * 256;
                if (f32_out) {
#pragma unroll
                    for (int c = 0; c < 2; c++) {
                        float o[32];
                        tmem_ld32(o_tmem + ps * 64 + c * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            const int piece = c * 8 + i;
                            *reinterpret_cast<float4*>(my + ((piece ^ (row_in_tile & 7)) << 4)) =
                                make_float4(o[4 * i] * inv, o[4 * i + 1] * inv, o[4 * i + 2] * inv, o[4 * i + 3] * inv);
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        float o[32];
                        tmem_ld32(o_tmem + c * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int piece = c * 4 + i;
                            *reinterpret_cast<uint4*>(my + ((piece ^ (row_in_tile & 7)) << 4)) =
                                make_uint4(pack_half2_rn(o[8 * i] * inv, o[8 * i + 1] * inv),
                                           pack_half2_rn(o[8 * i + 2] * inv, o[8 * i + 3] * inv),
                                           pack_half2_rn(o[8 * i + 4] * inv, o[8 * i + 5] * inv),
                                           pack_half2_rn(o[8 * i + 6] * inv, o[8 * i + 7] * inv));
                        }
                    }
                }
                __syncwarp();
                // Each warp copies out the 32 rows its own lanes staged: two rows per instruction.
                const int piece = lane & 15;
                const size_t col_bytes = (size_t)(f32_out ? ps * 256 : 0) + piece * 16;
#pragma unroll 4
                for (int it = 0; it < 16; it++) {
                    const int owner = it * 2 + (lane >> 4);
                    const int dr = __shfl_sync(0xffffffffu, my_dst, owner);
                    if (dr >= 0) {
                        const int r = warp_row0 + owner;
                        const uint4 val = *reinterpret_cast<const uint4*>(stage + r * 256 + ((piece ^ (r & 7)) << 4));
                        const size_t byte_off = (size_t)dr * dst_row_bytes + col_bytes;
                        if (partial) {
                            if (INGOT_CHECK((reinterpret_cast<unsigned char*>(dst0) - reinterpret_cast<unsigned char*>(p.part) + byte_off) / 4, 4,
                                            p.part_extent, p.status))
                                *reinterpret_cast<uint4*>(dst0 + byte_off) = val;
                        } else if (INGOT_CHECK(byte_off / (f32_out ? 4 : 2), f32_out ? 4 : 8, p.out_extent, p.status)) {
                            *reinterpret_cast<uint4*>(dst0 + byte_off) = val;
                            if (p.n_outs > 1) {
#pragma unroll
                                for (int d = 1; d < kMaxOutputs; d++)  // unrolled: keeps the pointer table in the parameter bank
                                    if (d < p.n_outs) *reinterpret_cast<uint4*>(static_cast<unsigned char*>(p.outs[d]) + byte_off) = val;
                            }
                        }
                    }
                }
            }
        }
        TIMING(if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && warp == 4 && lane == 0)
                   printf("CTA phases (cycles): set-up + wait for the kernel before %lld, Q staged %lld, first S ready %lld, %d key tiles %lld, "
                          "last PV retired %lld, O stored %lld\n", t_setup - t_entry, t_q - t_setup, t_s0 - t_q, n_it, t_loop - t_s0, t_of - t_loop,
                          clock64() - t_of);)
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(p.status, kDevErrBarrierTimeout);
    if (threadIdx.x == 0 && p.ticket != nullptr) {
        // Every thread's output stores precede the barrier above; the fence orders them, at system scope (they
        // may have gone to peer GPUs), before this CTA's ticket. Whoever draws the last ticket has therefore
        // every CTA's stores before its own fence, and releases one signal per destination.
        __threadfence_system();
        const int total = (int)(gridDim.x * gridDim.y * gridDim.z);
        if (atomicAdd(p.ticket, 1) == total - 1) {
            atomicExch(p.ticket, 0);
            __threadfence_system();
#pragma unroll
            for (int d = 0; d < kMaxOutputs; d++)
                if (d < p.n_outs && p.signals[d] != nullptr)
                    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.signals[d] + p.src_index) : "memory");
        }
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// Merges the key-split partials of a prefill: one warp per (kv head, row), lane = 4 dims.
// out = sum_s o_s 2^(m_s-M) / sum_s l_s 2^(m_s-M), the same formula the decode merge uses.
__global__ void __launch_bounds__(256) prefill_merge_kernel(const float* __restrict__ part, void* out, int out_dtype, int n_split,
                                                            int n_kvh, int n_rows, int G, int out_n_head, int out_head0) {
    INGOT_PDL_TRIGGER();
    INGOT_PDL_WAIT();  // the partials come from the kernel before
    const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= (long long)n_kvh * n_rows) return;
    const int kvh = int(w / n_rows), R = int(w % n_rows);
    const size_t split_stride = (size_t)n_kvh * n_rows * kPartStride;
    const float* row = part + ((size_t)kvh * n_rows + R) * kPartStride;
    float M = -INFINITY;
    for (int s = 0; s < n_split; s++) M = fmaxf(M, row[s * split_stride + 128]);
    float L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < n_split; s++) {
        const float wgt = ex2(row[s * split_stride + 128] - M);  // an empty partial has m = -inf: weight 0
        L += row[s * split_stride + 129] * wgt;
        const float4 o = *reinterpret_cast<const float4*>(row + s * split_stride + lane * 4);
        acc.x += o.x * wgt; acc.y += o.y * wgt; acc.z += o.z * wgt; acc.w += o.w * wgt;
    }
    const float inv = 1.0f / L;
    const size_t e = ((size_t)(R / G) * out_n_head + out_head0 + kvh * G + R % G) * kHeadDim + lane * 4;
    if (out_dtype == INGOT_F32) {
        *reinterpret_cast<float4*>(static_cast<float*>(out) + e) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
    } else {
        *reinterpret_cast<uint2*>(static_cast<__half*>(out) + e) =
            make_uint2(pack_half2_rn(acc.x * inv, acc.y * inv), pack_half2_rn(acc.z * inv, acc.w * inv));
    }
}

// Consumer side of the completion signalling: thread i waits until counter i is non-zero (its source's grid has
// finished and all its stores are visible here), then takes the signal back off the counter, so that the same
// counters serve the next call without any reset. Bounded: a source that never signals makes its thread give up
// after limit_ns with the timeout bit in the status word; nothing spins for ever and nothing traps.
__global__ void gather_wait_kernel(unsigned int* counters, int n_src, unsigned long long limit_ns, int* status) {
    const int i = threadIdx.x;
    if (i >= n_src) return;
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(counters + i) : "memory");
        if (v != 0) {
            atomicSub(counters + i, 1u);
            return;
        }
        if (globaltimer_ns() - t0 > limit_ns) {
            atomicOr(status, kDevErrBarrierTimeout);
            return;
        }
        __nanosleep(200);
    }
}

// ---- host side: tensor maps -------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
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

struct Sm100State {
    std::vector<CUtensorMap> maps;  // [layer][K/V]
    std::vector<char> built;
    float* part = nullptr;          // key-split partials, grown on demand
    size_t part_floats = 0;
    bool smem_opt_in = false;
};

}  // namespace

int launch_gather_wait(ingot_kv* kv, void* counters, int n_src, int timeout_ms, cudaStream_t stream) {
    gather_wait_kernel<<<1, 32, 0, stream>>>(static_cast<unsigned int*>(counters), n_src, (unsigned long long)timeout_ms * 1000000ull, kv->status_dev);
    INGOT_CUDA_TRY(cudaGetLastError());
    return INGOT_OK;
}

void free_prefill_sm100_state(ingot_kv* kv) {
    Sm100State* st = static_cast<Sm100State*>(kv->tmaps);
    if (st) cudaFree(st->part);
    delete st;
    kv->tmaps = nullptr;
}

int launch_attn_prefill_sm100(ingot_kv* kv, int layer, const void* q, int q_dtype, void* const* outs, int n_outs,
                              int out_dtype, int n_head, int out_n_head, int out_head0, int q_pos0, int n_tok,
                              const int32_t* block_table, void* const* signals, int src_index, cudaStream_t stream) {
    if (n_outs < 1 || n_outs > kMaxOutputs) {
        ingot_set_error("tcgen05 prefill: between 1 and 8 output buffers");
        return INGOT_ERR_INVALID;
    }
    const bool paged = kv->layout == INGOT_KV_PAGED;
    if (paged && block_table == nullptr) {
        ingot_set_error("tcgen05 prefill: a paged cache needs a block table");
        return INGOT_ERR_INVALID;
    }
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) {
        ingot_set_error("tcgen05 prefill: cuTensorMapEncodeTiled is not available from the driver");
        return INGOT_ERR_CUDA;
    }
    if (!kv->tmaps) {
        Sm100State* st = new Sm100State();
        st->maps.resize(size_t(kv->n_layer) * 2);
        st->built.assign(kv->n_layer, 0);
        kv->tmaps = st;
    }
    Sm100State* st = static_cast<Sm100State*>(kv->tmaps);
    if (!st->built[layer]) {
        for (int which = 0; which < 2; which++) {
            __half* base = (which ? kv->v : kv->k) + size_t(layer) * kv->layer_elems;
            // Contiguous: [head][position][dim] f16, dim fastest; box = 64 dims x 128 positions x 1 head.
            // Paged: [block * kv head][16 tokens][dim]; box = 64 dims x 16 tokens x 1. 128-byte swizzle.
            cuuint64_t dims[3] = {cuuint64_t(kHeadDim), cuuint64_t(paged ? kBlockTokens : kv->capacity),
                                  cuuint64_t(paged ? size_t(kv->capacity) * kv->n_head_kv : size_t(kv->n_head_kv))};
            cuuint64_t strides[2] = {cuuint64_t(kHeadDim) * 2, cuuint64_t(paged ? kBlockTokens : kv->capacity) * kHeadDim * 2};
            cuuint32_t box[3] = {64, cuuint32_t(paged ? kBlockTokens : kTileKeys), 1};
            cuuint32_t estr[3] = {1, 1, 1};
            CUresult r = encode(&st->maps[size_t(layer) * 2 + which], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, base, dims, strides,
                                box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) {
                ingot_set_error("tcgen05 prefill: cuTensorMapEncodeTiled failed with CUresult " + std::to_string(int(r)));
                return INGOT_ERR_CUDA;
            }
        }
        st->built[layer] = 1;
    }
    Sm100Params p;
    p.q = q; p.status = kv->status_dev;
    for (int i = 0; i < kMaxOutputs; i++) p.outs[i] = i < n_outs ? outs[i] : nullptr;
    p.n_outs = n_outs; p.out_n_head = out_n_head; p.out_head0 = out_head0;
    for (int i = 0; i < kMaxOutputs; i++) p.signals[i] = (signals && i < n_outs) ? static_cast<unsigned int*>(signals[i]) : nullptr;
    p.src_index = src_index;
    p.ticket = signals ? kv->status_dev + 1 : nullptr;
    p.q_dtype = q_dtype; p.out_dtype = out_dtype;
    p.n_head = n_head; p.group = n_head / kv->n_head_kv;
    p.q_pos0 = q_pos0; p.n_tok = n_tok;
    p.block_table = paged ? block_table : nullptr;
    p.capacity = kv->capacity;
    p.scale_log2 = 1.4426950408889634f / sqrtf(float(kHeadDim));
    p.q_extent = (size_t)n_tok * n_head * kHeadDim;
    p.out_extent = (size_t)n_tok * out_n_head * kHeadDim;
    p.part_extent = 0;
    // Test hook for the bounded-wait path (ingot_kv_test_stall_prefill): the producer warp issues no copies and the
    // wait limit is shortened, so every role times out, the status word gets its bit and the kernel returns
    // normally. Production: 2 s limit, producer active.
    p.test_stall_producer = kv->test_stall_ms > 0 ? 1 : 0;
    p.wait_limit_ns = kv->test_stall_ms > 0 ? (unsigned long long)kv->test_stall_ms * 1000000ull : 2000000000ull;
    if (!st->smem_opt_in) {  // function attributes belong to a device context: once per handle
        INGOT_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        st->smem_opt_in = true;
    }
    const long long n_rows = (long long)n_tok * p.group;
    const unsigned row_tiles = unsigned((n_rows + 2 * kTileRows - 1) / (2 * kTileRows));
    // Too few row tiles to fill the GPU (one CTA per SM): split the keys over grid.z and merge afterwards.
    // Only the last row tile is guaranteed to have many key tiles, so the split count is bounded by them.
    const int row_ctas = int(row_tiles) * kv->n_head_kv;
    const int kv_tiles_last = (q_pos0 + n_tok + kTileKeys - 1) / kTileKeys;
    int n_split = 1;
    if (n_outs == 1 && !signals && row_ctas * 2 <= kv->num_sms) n_split = std::max(1, std::min({kv->num_sms / row_ctas, 8, kv_tiles_last / 2}));
    p.n_split = n_split;
    p.part = nullptr;
    if (n_split > 1) {
        const size_t need = size_t(n_split) * kv->n_head_kv * n_rows * kPartStride;
        if (need > st->part_floats) {
            // Grown, never shrunk or freed before the handle goes: a graph captured earlier may point into the old
            // buffer. (Growing allocates: the first call with a larger shape must not run under stream capture.)
            float* bigger = nullptr;
            INGOT_CUDA_TRY(cudaMalloc(&bigger, need * sizeof(float)));
            if (st->part) kv->retired.push_back(st->part);
            st->part = bigger;
            st->part_floats = need;
        }
        p.part = st->part;
        p.part_extent = st->part_floats;
    }
    dim3 grid(row_tiles, kv->n_head_kv, n_split);
    INGOT_CUDA_TRY(ingot_launch_pdl(attn_prefill_sm100_kernel, grid, dim3(kThreads), size_t(kSmemBytes), stream, st->maps[size_t(layer) * 2],
                                    st->maps[size_t(layer) * 2 + 1], p));
    if (n_split > 1) {
        const long long warps = (long long)kv->n_head_kv * n_rows;
        INGOT_CUDA_TRY(ingot_launch_pdl(prefill_merge_kernel, dim3(unsigned((warps * 32 + 255) / 256)), dim3(256), 0, stream,
                                        (const float*)st->part, outs[0], out_dtype, n_split, kv->n_head_kv, int(n_rows), p.group, out_n_head,
                                        out_head0));
    }
    return INGOT_OK;
}
