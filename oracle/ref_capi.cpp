// TEST INFRASTRUCTURE — not part of the product. C entry points around the Ingot reference's
// own compiled CPU code, used only by tests/, the smoke check and bench.py's CPU-baseline legs
// as the checker / the timed baseline. It is linked with the reference's src/ops.cpp,
// src/cpu_backend.cpp, src/model.cpp, src/gguf.cpp, src/engine.cpp and src/sampler.cpp
// (compiled unmodified from the reference checkout against oracle/shim/) into
// oracle/_ref/libingot_ref.so by oracle/Makefile.
//
// What is the reference's own code here and what is restated:
//   ref_rope, ref_softmax          -> call ops::rope / ops::softmax (src/ops.cpp:243-255, 234-241)
//   ref_attend                     -> the attention lambda of CpuBackend::forward
//                                     (src/cpu_backend.cpp:27-30, 51-69) restated around the
//                                     reference's ops::parallel_for and ops::softmax, because
//                                     the lambda reads private members and cannot be called
//                                     with injected Q/K/V
//   ref_rope_inv_freq              -> src/model.cpp:59-69 restated (Model::load needs a file)
//   ref_dequant, ref_matvec        -> call ops::dequant_row / ops::matvec (src/ops.cpp:198-225) on
//                                     caller-supplied block-quantised rows
// (The end-to-end greedy check drives the reference's genuine CpuBackend through the engine library,
// backend/e2e_capi.cpp, which links the same unmodified reference sources.)
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "backend.h"
#include "cpu_backend.h"
#include "engine.h"
#include "gguf.h"
#include "metal_backend.h"
#include "model.h"
#include "ops.h"
#include "sampler.h"

// engine.cpp references the Metal factory. The CPU-only oracle library has no GPU backend;
// asking for one is an error, exactly as it is on a machine without Metal.
__attribute__((weak)) std::unique_ptr<Backend> make_metal_backend(const gguf::File&, const Model&, int, int) {
    throw std::runtime_error("metal: no GPU device");
}

static thread_local std::string g_last_error;

extern "C" {

const char* ref_last_error() { return g_last_error.c_str(); }

int ref_thread_count() { return int(ingot_dispatch_shim::Pool::get().size()); }

void ref_rope(float* x, int n_heads, int head_dim, int pos, const float* inv_freq) {
    ops::rope(x, n_heads, head_dim, pos, inv_freq);
}

void ref_softmax(float* x, size_t n) { ops::softmax(x, n); }

// src/model.cpp:59-69. factors may be null.
void ref_rope_inv_freq(float* out, int head_dim, float rope_theta, const float* factors) {
    const float theta_scale = powf(rope_theta, -2.0f / float(head_dim));
    float freq = 1.0f;
    for (int i = 0; i < head_dim / 2; i++) {
        out[i] = factors ? freq / factors[i] : freq;
        freq *= theta_scale;
    }
}

// One query token at position `pos` attending to keys 0..pos of an f32 cache laid out
// [n_ctx][n_head_kv*head_dim] like CpuBackend's (src/cpu_backend.h:23).
// q [n_head][head_dim] (already rotated), out [n_head][head_dim], scores [n_head][pos+1] scratch.
void ref_attend(const float* q, const float* kl, const float* vl, int pos, int n_head, int n_head_kv,
                int hd, float* out_all, float* scores) {
    const size_t kv_dim = size_t(n_head_kv) * hd;
    const int group = n_head / n_head_kv;
    const float scale = 1.0f / sqrtf(float(hd));
    const size_t sc_stride = size_t(pos) + 1;
    ops::parallel_for(size_t(n_head), [&](size_t h) {
        const float* qh = q + h * hd;
        const size_t kvh = h / group;
        float* sc = scores + h * sc_stride;
        for (int t = 0; t <= pos; t++) {
            const float* kt = kl + size_t(t) * kv_dim + kvh * hd;
            float s = 0;
            for (int i = 0; i < hd; i++) s += qh[i] * kt[i];
            sc[t] = s * scale;
        }
        ops::softmax(sc, size_t(pos) + 1);
        float* out = out_all + h * hd;
        std::memset(out, 0, hd * sizeof(float));
        for (int t = 0; t <= pos; t++) {
            const float* vt = vl + size_t(t) * kv_dim + kvh * hd;
            const float w = sc[t];
            for (int i = 0; i < hd; i++) out[i] += w * vt[i];
        }
    });
}

// The attention part of n consecutive CpuBackend::forward calls (what the default
// Backend::forward_batch does, src/backend.h:16-20): for token i at position pos0+i, rotate q
// and k (src/cpu_backend.cpp:43-44), append k and v rows to the f32 caches (:46-49), attend (:51-69).
// q [n][n_head*hd] and k [n][kv_dim] are rotated in place; out [n][n_head*hd].
void ref_attn_forward(float* q, float* k, const float* v, float* kcache, float* vcache, int pos0, int n,
                      int n_head, int n_head_kv, int hd, const float* inv_freq, float* out) {
    const size_t kv_dim = size_t(n_head_kv) * hd, q_dim = size_t(n_head) * hd;
    std::vector<float> scores(size_t(n_head) * (size_t(pos0) + n));
    for (int i = 0; i < n; i++) {
        const int pos = pos0 + i;
        float* qi = q + i * q_dim;
        float* ki = k + i * kv_dim;
        ops::rope(qi, n_head, hd, pos, inv_freq);
        ops::rope(ki, n_head_kv, hd, pos, inv_freq);
        std::memcpy(kcache + size_t(pos) * kv_dim, ki, kv_dim * sizeof(float));
        std::memcpy(vcache + size_t(pos) * kv_dim, v + i * kv_dim, kv_dim * sizeof(float));
        ref_attend(qi, kcache, vcache, pos, n_head, n_head_kv, hd, out + i * q_dim, scores.data());
    }
}

// ops::dequant_row (src/ops.cpp:198-200) on a caller-supplied row of `n` elements of ggml type `type`.
// Returns 0, or -1 when the reference rejects the type.
int ref_dequant(int type, const uint8_t* bytes, float* out, size_t n) {
    try {
        gguf::TensorInfo t;
        t.ne = {uint64_t(n), 1};
        t.type = gguf::TensorType(uint32_t(type));
        t.data = bytes;
        ops::dequant_row(t, 0, out);
        return 0;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return -1;
    }
}

// ops::matvec (src/ops.cpp:217-225): out[r] = dot_row(W, r, x) for a [n_out][n_in] matrix of ggml type `type`.
int ref_matvec(int type, const uint8_t* bytes, const float* x, size_t n_in, size_t n_out, float* out) {
    try {
        gguf::TensorInfo t;
        t.ne = {uint64_t(n_in), uint64_t(n_out)};
        t.type = gguf::TensorType(uint32_t(type));
        t.data = bytes;
        ops::matvec(out, t, x);
        return 0;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return -1;
    }
}

}  // extern "C"
