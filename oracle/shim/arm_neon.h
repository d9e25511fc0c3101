// TEST INFRASTRUCTURE (oracle build only). x86-64 stand-in for the subset of <arm_neon.h>
// that Ingot's src/ops.cpp uses, so that file compiles unmodified with g++ on Linux.
// Every intrinsic keeps NEON's lane order and rounding: vfmaq_f32 is a fused multiply-add
// per lane (fmaf), vaddvq_f32 sums lanes as (v0+v1)+(v2+v3) like AArch64 FADDP pairs, and
// f16 -> f32 widening is exact. Only the types and intrinsics named by src/ops.cpp exist.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstring>

typedef _Float16 __fp16;
typedef _Float16 float16_t;

struct float32x4_t { float v[4]; };
struct float16x4_t { _Float16 v[4]; };
struct float16x8_t { _Float16 v[8]; };
struct int8x8_t { int8_t v[8]; };
struct int8x16_t { int8_t v[16]; };
struct uint8x16_t { uint8_t v[16]; };
struct int16x4_t { int16_t v[4]; };
struct int16x8_t { int16_t v[8]; };
struct int32x4_t { int32_t v[4]; };

static inline float32x4_t vld1q_f32(const float* p) { float32x4_t r; std::memcpy(r.v, p, 16); return r; }
static inline float32x4_t vdupq_n_f32(float x) { return float32x4_t{{x, x, x, x}}; }
static inline float32x4_t vaddq_f32(float32x4_t a, float32x4_t b) {
    float32x4_t r;
    for (int i = 0; i < 4; i++) r.v[i] = a.v[i] + b.v[i];
    return r;
}
// acc + a*b, fused (single rounding) in every lane.
static inline float32x4_t vfmaq_f32(float32x4_t acc, float32x4_t a, float32x4_t b) {
    float32x4_t r;
    for (int i = 0; i < 4; i++) r.v[i] = std::fmaf(a.v[i], b.v[i], acc.v[i]);
    return r;
}
static inline float vaddvq_f32(float32x4_t a) { return (a.v[0] + a.v[1]) + (a.v[2] + a.v[3]); }

static inline float16x8_t vld1q_f16(const __fp16* p) { float16x8_t r; std::memcpy(r.v, p, 16); return r; }
static inline float16x4_t vget_low_f16(float16x8_t a) { float16x4_t r; std::memcpy(r.v, a.v, 8); return r; }
static inline float16x4_t vget_high_f16(float16x8_t a) { float16x4_t r; std::memcpy(r.v, a.v + 4, 8); return r; }
static inline float32x4_t vcvt_f32_f16(float16x4_t a) {
    float32x4_t r;
    for (int i = 0; i < 4; i++) r.v[i] = float(a.v[i]);
    return r;
}

static inline int8x16_t vld1q_s8(const int8_t* p) { int8x16_t r; std::memcpy(r.v, p, 16); return r; }
static inline uint8x16_t vld1q_u8(const uint8_t* p) { uint8x16_t r; std::memcpy(r.v, p, 16); return r; }
static inline uint8x16_t vdupq_n_u8(uint8_t x) { uint8x16_t r; std::memset(r.v, x, 16); return r; }
static inline int8x16_t vdupq_n_s8(int8_t x) { int8x16_t r; for (int i = 0; i < 16; i++) r.v[i] = x; return r; }
static inline uint8x16_t vandq_u8(uint8x16_t a, uint8x16_t b) {
    uint8x16_t r;
    for (int i = 0; i < 16; i++) r.v[i] = a.v[i] & b.v[i];
    return r;
}
#define vshrq_n_u8(a, n) ingot_neon_shim_vshrq_n_u8((a), (n))
static inline uint8x16_t ingot_neon_shim_vshrq_n_u8(uint8x16_t a, int n) {
    uint8x16_t r;
    for (int i = 0; i < 16; i++) r.v[i] = uint8_t(a.v[i] >> n);
    return r;
}
static inline int8x16_t vreinterpretq_s8_u8(uint8x16_t a) { int8x16_t r; std::memcpy(r.v, a.v, 16); return r; }
static inline int8x16_t vsubq_s8(int8x16_t a, int8x16_t b) {
    int8x16_t r;
    for (int i = 0; i < 16; i++) r.v[i] = int8_t(a.v[i] - b.v[i]);
    return r;
}
static inline int8x8_t vget_low_s8(int8x16_t a) { int8x8_t r; std::memcpy(r.v, a.v, 8); return r; }
static inline int8x8_t vget_high_s8(int8x16_t a) { int8x8_t r; std::memcpy(r.v, a.v + 8, 8); return r; }
static inline int16x8_t vmovl_s8(int8x8_t a) {
    int16x8_t r;
    for (int i = 0; i < 8; i++) r.v[i] = a.v[i];
    return r;
}
static inline int16x4_t vget_low_s16(int16x8_t a) { int16x4_t r; std::memcpy(r.v, a.v, 8); return r; }
static inline int16x4_t vget_high_s16(int16x8_t a) { int16x4_t r; std::memcpy(r.v, a.v + 4, 8); return r; }
static inline int32x4_t vmovl_s16(int16x4_t a) {
    int32x4_t r;
    for (int i = 0; i < 4; i++) r.v[i] = a.v[i];
    return r;
}
static inline float32x4_t vcvtq_f32_s32(int32x4_t a) {
    float32x4_t r;
    for (int i = 0; i < 4; i++) r.v[i] = float(a.v[i]);
    return r;
}
