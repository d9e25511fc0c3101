// Eight consecutive elements of a q/k/v projection row turned into eight f16 values, as the cache and the MMA
// operands hold them: four rotation pairs of ops::rope (src/ops.cpp:248-253: angle = float(pos) * inv_freq[i],
// (x0, x1) <- (x0*c - x1*s, x0*s + x1*c) on ADJACENT elements, full-range cosf / sinf) or, for V rows, just the
// rounding. One definition, so that every kernel that applies it produces the same bits.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

__device__ __forceinline__ uint32_t rope_pack_half2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// src: 8 floats (32-byte aligned); pair0: index of the first of the unit's four rotation pairs within the head.
__device__ __forceinline__ uint4 rope_pack8(const float* src, int pair0, float fpos, const float* inv_freq, bool rotate) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(src));
    const float4 b = __ldg(reinterpret_cast<const float4*>(src) + 1);
    float x[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    if (rotate) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float angle = fpos * __ldg(inv_freq + pair0 + i);
            const float c = cosf(angle), s = sinf(angle);
            const float x0 = x[2 * i], x1 = x[2 * i + 1];
            x[2 * i] = x0 * c - x1 * s;
            x[2 * i + 1] = x0 * s + x1 * c;
        }
    }
    uint4 o;
    o.x = rope_pack_half2(x[0], x[1]);
    o.y = rope_pack_half2(x[2], x[3]);
    o.z = rope_pack_half2(x[4], x[5]);
    o.w = rope_pack_half2(x[6], x[7]);
    return o;
}
