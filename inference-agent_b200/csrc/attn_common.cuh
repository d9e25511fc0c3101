// Device helpers shared by the attention kernels: streaming 16-byte loads, warp-level m16n8k16
// MMA wrappers, packing, and dtype-generic query/output access.
#pragma once

#include "ingot_internal.cuh"

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

__device__ __forceinline__ uint32_t pack_half2_rn(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// Loads 8 consecutive query elements starting at element index `e` as 4 packed f16 pairs.
__device__ __forceinline__ uint4 load_q8(const void* q, int dtype, size_t e) {
    uint4 r;
    if (dtype == INGOT_F16) {
        r = __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(q) + e));
    } else if (dtype == INGOT_BF16) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(q) + e));
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; i++)  // bf16 -> f32 is a 16-bit shift; f32 -> f16 rounds to nearest
            o[i] = pack_half2_rn(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
        r = make_uint4(o[0], o[1], o[2], o[3]);
    } else {
        const float4 a = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(q) + e));
        const float4 b = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(q) + e) + 1);
        r = make_uint4(pack_half2_rn(a.x, a.y), pack_half2_rn(a.z, a.w), pack_half2_rn(b.x, b.y), pack_half2_rn(b.z, b.w));
    }
    return r;
}

__device__ __forceinline__ void store_out(void* out, int dtype, size_t e, float v) {
    if (dtype == INGOT_F32) static_cast<float*>(out)[e] = v;
    else static_cast<__half*>(out)[e] = __float2half_rn(v);
}


// Full m16n8k16 f16 MMA with f32 accumulation: d += A * B.
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
