/* TEST INFRASTRUCTURE — CPU restatement of the reference's GGUF block dequantisation and of its
 * dequantise-then-dot row product, used only as the checker of the CUDA weight kernels.
 *
 * Follows src/ops.cpp of the reference:
 *   oracle_dequant   <- dequant_f32/f16/bf16/q8_0/q4_0/q4_1/q6_k and the dispatch (ops.cpp:22-104)
 *   oracle_row_bytes <- row_bytes (ops.cpp:182-184) with the block sizes of src/gguf.cpp:24-47
 *   oracle_matvec    <- ops::matvec over dot_row (ops.cpp:200-225), evaluated in float64 on the dequantised
 *                       values: it is the tolerance reference for the GPU products, not a bit pattern.
 * Type codes are ggml's (src/gguf.h: F32 0, F16 1, Q4_0 2, Q4_1 3, Q8_0 8, Q6_K 14, BF16 30).
 * Pinned against the compiled reference (oracle/_ref, ref_dequant) by tests/test_oracle_quant.py and against the
 * committed fixture tests/golden/quant_golden.npz that tests/golden/make_golden_quant.py generated from it.
 * Nothing in the product links or calls this file.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

enum { T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q4_1 = 3, T_Q8_0 = 8, T_Q6_K = 14, T_BF16 = 30 };

static uint16_t load_u16(const uint8_t* p) { uint16_t v; memcpy(&v, p, 2); return v; }
static float fp16_to_f32(uint16_t h) { _Float16 v; memcpy(&v, &h, 2); return (float)v; }
static float bf16_to_f32(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }

int oracle_block_size(int type) { return type == T_Q6_K ? 256 : (type == T_F32 || type == T_F16 || type == T_BF16) ? 1 : 32; }
int oracle_block_bytes(int type) {
    switch (type) {
        case T_F32: return 4;
        case T_F16: case T_BF16: return 2;
        case T_Q4_0: return 18;
        case T_Q4_1: return 20;
        case T_Q8_0: return 34;
        case T_Q6_K: return 210;
        default: return 0;
    }
}
size_t oracle_row_bytes(int type, size_t n) { return n / (size_t)oracle_block_size(type) * (size_t)oracle_block_bytes(type); }

/* ops.cpp:22-104. n is a multiple of the block size. Returns 0, or -1 for an unsupported type. */
int oracle_dequant(int type, const uint8_t* p, float* out, size_t n) {
    switch (type) {
        case T_F32: memcpy(out, p, n * sizeof(float)); return 0;
        case T_F16: for (size_t i = 0; i < n; i++) out[i] = fp16_to_f32(load_u16(p + 2 * i)); return 0;
        case T_BF16: for (size_t i = 0; i < n; i++) out[i] = bf16_to_f32(load_u16(p + 2 * i)); return 0;
        case T_Q8_0:  /* ops.cpp:33-41: d * q */
            for (size_t b = 0; b < n / 32; b++, p += 34, out += 32) {
                const float d = fp16_to_f32(load_u16(p));
                const int8_t* q = (const int8_t*)(p + 2);
                for (int i = 0; i < 32; i++) out[i] = d * (float)q[i];
            }
            return 0;
        case T_Q4_0:  /* ops.cpp:43-54: d * (nibble - 8), low nibble = element i, high = i + 16 */
            for (size_t b = 0; b < n / 32; b++, p += 18, out += 32) {
                const float d = fp16_to_f32(load_u16(p));
                const uint8_t* q = p + 2;
                for (int i = 0; i < 16; i++) {
                    out[i] = d * (float)((int)(q[i] & 0xF) - 8);
                    out[i + 16] = d * (float)((int)(q[i] >> 4) - 8);
                }
            }
            return 0;
        case T_Q4_1:  /* ops.cpp:56-66: d * nibble + m. The reference's compilers contract this into one fused
                         multiply-add (clang on arm64 by default; g++ with -mfma for the compiled checker). */
            for (size_t b = 0; b < n / 32; b++, p += 20, out += 32) {
                const float d = fp16_to_f32(load_u16(p)), m = fp16_to_f32(load_u16(p + 2));
                const uint8_t* q = p + 4;
                for (int i = 0; i < 16; i++) {
                    out[i] = fmaf(d, (float)(q[i] & 0xF), m);
                    out[i + 16] = fmaf(d, (float)(q[i] >> 4), m);
                }
            }
            return 0;
        case T_Q6_K:  /* ops.cpp:68-91: d * scale * (q6 - 32), evaluated left to right */
            for (size_t b = 0; b < n / 256; b++, p += 210, out += 256) {
                const uint8_t* ql = p;
                const uint8_t* qh = p + 128;
                const int8_t* sc = (const int8_t*)(p + 192);
                const float d = fp16_to_f32(load_u16(p + 208));
                float* y = out;
                for (int half = 0; half < 2; half++) {
                    for (int l = 0; l < 32; l++) {
                        const int is = l / 16;
                        const int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                        const int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                        const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                        const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                        y[l] = d * (float)sc[is] * (float)q1;
                        y[l + 32] = d * (float)sc[is + 2] * (float)q2;
                        y[l + 64] = d * (float)sc[is + 4] * (float)q3;
                        y[l + 96] = d * (float)sc[is + 6] * (float)q4;
                    }
                    y += 128; ql += 64; qh += 32; sc += 8;
                }
            }
            return 0;
        default: return -1;
    }
}

/* out[r] = sum_i dequant(W)[r][i] * x[i] in float64 (tolerance reference for ops::matvec, ops.cpp:217-225).
 * scratch holds n_in floats. */
int oracle_matvec(int type, const uint8_t* w, const float* x, size_t n_in, size_t n_out, double* out, float* scratch) {
    const size_t rb = oracle_row_bytes(type, n_in);
    for (size_t r = 0; r < n_out; r++) {
        if (oracle_dequant(type, w + r * rb, scratch, n_in) != 0) return -1;
        double s = 0.0;
        for (size_t i = 0; i < n_in; i++) s += (double)scratch[i] * (double)x[i];
        out[r] = s;
    }
    return 0;
}
