// CudaBackend — drop-in third implementation of Ingot's Backend (src/backend.h:9-23), beside the CPU
// reference (src/cpu_backend.cpp) and the Metal backend (src/metal_backend.mm).
//
// Per layer it runs what MetalBackend::forward_batch encodes (src/metal_backend.mm:435-455): rmsnorm,
// q/k/v projections, then the attention stage through the C ABI of libingot_cuda.so — fused RoPE + KV
// append, then split-KV decode (n == 1) or causal prefill (n > 1) — then wo (+= x), rmsnorm, gate/up,
// silu_mul, down (+= x); finally the last token's norm and the logits projection.
//
// Contracts kept from the reference backends:
//  - positions are 0-based and may be revisited in any order (src/main.cpp:295, 374-375);
//  - forward_batch returns the logits of the LAST token only (src/metal_backend.mm:456-458);
//  - the returned pointer is writable host memory owned by the backend and valid until the next call
//    (callers const_cast and edit it, src/main.cpp:238-239, src/sampler.cpp:20): a pinned buffer;
//  - the same exceptions and messages for a bad position, token id or batch size
//    (src/cpu_backend.cpp:24-25, src/metal_backend.mm:421-424);
//  - Model and gguf::File are borrowed and must outlive the backend; weights are uploaded once.
// This file also defines make_metal_backend and the four metal_* diagnostics, so that the reference's
// engine.cpp / main.cpp link against this backend without a source edit.
#include "cuda_backend.h"

#include <cuda_runtime.h>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <algorithm>
#include <vector>

#include "ingot_cuda.h"
#include "metal_backend.h"
#include "ops.h"

extern "C" {
cudaError_t ingot_support_rmsnorm(float* out, const float* x, const float* w, int n_rows, int n, float eps, cudaStream_t s);
cudaError_t ingot_support_silu_mul(float* gate, const float* up, size_t n, cudaStream_t s);
cudaError_t ingot_support_linear(float* out, const void* w, int w_is_f16, const float* x, int n_in, int n_out, int n_tok,
                                 int accumulate, cudaStream_t s);
cudaError_t ingot_support_gemv_group(float* const* outs, const void* const* ws, const int* n_out, int n_mat, int swiglu, const float* x,
                                     const float* norm_w, float eps, int n_in, int accumulate, cudaStream_t s);
// tensor-core form of the batched projections (linear_sm100.cu)
struct ingot_linear_ws;
cudaError_t ingot_linear_ws_create(ingot_linear_ws** out, int max_tok, int max_in);
void ingot_linear_ws_destroy(ingot_linear_ws* ws);
int ingot_linear_tc_supported(const ingot_linear_ws* ws, int w_is_f16, int n_in, int n_out, int n_tok);
cudaError_t ingot_linear_tc_prepare(ingot_linear_ws* ws, const float* x, int n_in, int n_tok, cudaStream_t s);
cudaError_t ingot_linear_tc_prepare_norm(ingot_linear_ws* ws, const float* x, const float* norm_w, float eps, int n_in, int n_tok,
                                         cudaStream_t s);
cudaError_t ingot_linear_tc_run_partial(ingot_linear_ws* ws, const void* w, int n_in, int n_out, int slot, cudaStream_t s);
cudaError_t ingot_linear_tc_finish_group(ingot_linear_ws* ws, float* const* outs, int count, cudaStream_t s);
cudaError_t ingot_linear_tc_finish_residual_norm(ingot_linear_ws* ws, float* x, const float* norm_w, float eps, int slot, cudaStream_t s);
cudaError_t ingot_linear_tc_finish_swiglu(ingot_linear_ws* ws, int slot_gate, int slot_up, cudaStream_t s);
cudaError_t ingot_linear_tc_run(ingot_linear_ws* ws, float* out, const void* w, int n_in, int n_out, int accumulate, cudaStream_t s);
int ingot_linear_ws_status(ingot_linear_ws* ws);
}

namespace {

void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("cuda: ") + what + ": " + cudaGetErrorString(e));
}
void ingot_check(int rc) {
    if (rc != INGOT_OK) throw std::runtime_error(ingot_last_error()[0] ? ingot_last_error() : ingot_status_string(rc));
}

struct DevWeight {
    void* data = nullptr;
    int is_f16 = 0;
    int n_in = 0, n_out = 0;
};

class CudaBackend : public Backend {
public:
    CudaBackend(const Model& m, int n_ctx, int n_batch) : m_(m), n_ctx_(n_ctx), n_batch_(n_batch) {
        const Config& c = m.cfg;
        if (n_batch < 1) throw std::runtime_error("cuda: --batch must be at least 1");
        if (c.head_dim != INGOT_HEAD_DIM) throw std::runtime_error("cuda: head_dim must be 128");
        if (c.n_head / c.n_head_kv > 8) throw std::runtime_error("cuda: more than 8 query heads per kv head not supported");
        int n_dev = 0;
        if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev < 1) throw std::runtime_error("cuda: no GPU device");
        cuda_check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
        if (profile_) {
            cuda_check(cudaEventCreate(&ev0_), "cudaEventCreate");
            cuda_check(cudaEventCreate(&ev1_), "cudaEventCreate");
        }
        ingot_check(ingot_kv_create(&kv_, INGOT_KV_CONTIGUOUS, c.n_layer, c.n_head_kv, c.head_dim, n_ctx, 1));

        layers_.resize(c.n_layer);
        for (int l = 0; l < c.n_layer; l++) {
            const Layer& L = m.layers[l];
            DevLayer& D = layers_[l];
            D.attn_norm = upload_f32(L.attn_norm);
            D.ffn_norm = upload_f32(L.ffn_norm);
            D.wq = upload(*L.wq); D.wk = upload(*L.wk); D.wv = upload(*L.wv); D.wo = upload(*L.wo);
            D.w_gate = upload(*L.w_gate); D.w_up = upload(*L.w_up); D.w_down = upload(*L.w_down);
        }
        output_norm_ = upload_f32(m.output_norm);
        output_ = upload(*m.output);
        inv_freq_ = upload_f32(m.rope_inv_freq);

        const size_t nb = size_t(n_batch);
        const size_t q_dim = size_t(c.n_head) * c.head_dim, kv_dim = size_t(c.n_head_kv) * c.head_dim;
        x_ = alloc_f32(nb * c.n_embd); h_ = alloc_f32(nb * c.n_embd);
        q_ = alloc_f32(nb * q_dim); attn_ = alloc_f32(nb * q_dim);
        k_ = alloc_f32(nb * kv_dim); v_ = alloc_f32(nb * kv_dim);
        gate_ = alloc_f32(nb * c.n_ff); up_ = alloc_f32(nb * c.n_ff);
        logits_dev_ = alloc_f32(size_t(c.n_vocab));
        cuda_check(cudaMalloc(&q_rot_, nb * q_dim * 2), "cudaMalloc(q_rot)");
        allocs_.push_back(q_rot_);
        cuda_check(cudaMalloc(&pos_dev_, 2 * sizeof(int32_t)), "cudaMalloc(pos)");
        allocs_.push_back(pos_dev_);
        cuda_check(cudaMallocHost(&pos_host_, 2 * sizeof(int32_t)), "cudaMallocHost(pos)");
        cuda_check(cudaMallocHost(&x_host_, nb * c.n_embd * sizeof(float)), "cudaMallocHost(x)");
        cuda_check(cudaMallocHost(&logits_, size_t(c.n_vocab) * sizeof(float)), "cudaMallocHost(logits)");
        // INGOT_LINEAR_TC=0 keeps the batched projections on the f32 FMA kernels (diagnostics).
        const char* tc = getenv("INGOT_LINEAR_TC");
        if (n_batch >= 16 && !(tc && atoi(tc) == 0))
            cuda_check(ingot_linear_ws_create(&lin_ws_, n_batch, std::max(c.n_embd, std::max(c.n_ff, int(q_dim)))), "linear workspace");
    }

    ~CudaBackend() override {
        cudaStreamSynchronize(stream_);
        // INGOT_PROFILE=1: GPU time against wall time per forward, as the Metal backend reports under
        // LLM_PROFILE (src/metal_backend.mm:88-93, 463-468).
        if (profile_ && calls_ > 0) {
            fprintf(stderr, "cuda: %d forwards: gpu %.3f ms, wall %.3f ms per call", calls_, gpu_ms_ / calls_, wall_ms_ / calls_);
            if (calls1_ > 0) fprintf(stderr, "; single-token: %d calls, gpu %.3f ms per call", calls1_, gpu1_ms_ / calls1_);
            fprintf(stderr, "\n");
        }
        if (ev0_) cudaEventDestroy(ev0_);
        if (ev1_) cudaEventDestroy(ev1_);
        if (decode_exec_) cudaGraphExecDestroy(decode_exec_);
        if (decode_graph_) cudaGraphDestroy(decode_graph_);
        for (void* p : allocs_) cudaFree(p);
        cudaFreeHost(pos_host_);
        cudaFreeHost(x_host_);
        cudaFreeHost(logits_);
        ingot_linear_ws_destroy(lin_ws_);
        ingot_kv_destroy(kv_);
        cudaStreamDestroy(stream_);
    }

    const float* forward(int32_t token, int pos) override { return forward_batch(&token, 1, pos); }

    const float* forward_batch(const int32_t* tokens, int n, int pos) override {
        const Config& c = m_.cfg;
        if (n < 1 || n > n_batch_) throw std::runtime_error("cuda: batch size out of range");
        if (pos < 0 || pos + n > n_ctx_) throw std::runtime_error("context window exceeded");
        for (int i = 0; i < n; i++)
            if (tokens[i] < 0 || tokens[i] >= c.n_vocab) throw std::runtime_error("token id out of range");

        // Embedding rows are dequantised on the host straight into pinned memory, as the Metal
        // backend does (src/metal_backend.mm:426-428).
        const auto wall0 = std::chrono::steady_clock::now();
        for (int i = 0; i < n; i++) ops::dequant_row(*m_.tok_embd, size_t(tokens[i]), x_host_ + size_t(i) * c.n_embd);
        if (profile_) cuda_check(cudaEventRecord(ev0_, stream_), "cudaEventRecord");
        cuda_check(cudaMemcpyAsync(x_, x_host_, size_t(n) * c.n_embd * sizeof(float), cudaMemcpyHostToDevice, stream_), "H2D x");

        if (n == 1) {
            // Single-token steps read their position and key count from device memory, so that the whole
            // step (about 370 launches) can be captured once into a CUDA graph and replayed; the Metal
            // backend likewise encodes a forward pass into one command buffer (src/metal_backend.mm:433-461).
            // The first single-token call runs eagerly (it sizes the decode scratch), the second is captured.
            pos_host_[0] = pos;
            pos_host_[1] = pos + 1;
            cuda_check(cudaMemcpyAsync(pos_dev_, pos_host_, 2 * sizeof(int32_t), cudaMemcpyHostToDevice, stream_), "H2D pos");
            if (decode_exec_) {
                cuda_check(cudaGraphLaunch(decode_exec_, stream_), "cudaGraphLaunch");
            } else if (decode_calls_++ == 0) {
                encode_layers(1, pos, true);
            } else {
                cuda_check(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
                try {
                    encode_layers(1, pos, true);
                } catch (...) {
                    cudaGraph_t dead = nullptr;
                    cudaStreamEndCapture(stream_, &dead);
                    if (dead) cudaGraphDestroy(dead);
                    throw;
                }
                cuda_check(cudaStreamEndCapture(stream_, &decode_graph_), "cudaStreamEndCapture");
                cuda_check(cudaGraphInstantiate(&decode_exec_, decode_graph_, 0), "cudaGraphInstantiate");
                cuda_check(cudaGraphLaunch(decode_exec_, stream_), "cudaGraphLaunch");
            }
        } else {
            encode_layers(n, pos, false);
        }
        cuda_check(cudaMemcpyAsync(logits_, logits_dev_, size_t(c.n_vocab) * sizeof(float), cudaMemcpyDeviceToHost, stream_), "D2H logits");
        if (profile_) cuda_check(cudaEventRecord(ev1_, stream_), "cudaEventRecord");
        cuda_check(cudaStreamSynchronize(stream_), "forward");
        if (profile_) {
            float ms = 0.f;
            cudaEventElapsedTime(&ms, ev0_, ev1_);
            gpu_ms_ += ms;
            wall_ms_ += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - wall0).count();
            calls_++;
            if (n == 1) { gpu1_ms_ += ms; calls1_++; }
        }
        int status = 0;
        ingot_check(ingot_kv_status(kv_, stream_, &status));
        if (status != 0) throw std::runtime_error("cuda: attention kernel reported status " + std::to_string(status));
        if (n > 1 && lin_ws_ && ingot_linear_ws_status(lin_ws_) != 0) throw std::runtime_error("cuda: a projection kernel gave up on a bounded wait");
        return logits_;
    }

    // Every layer plus the final norm and logits projection for n tokens at positions pos..pos+n-1, queued
    // on stream_. device_pos: single-token form whose position / key count are read from pos_dev_.
    void encode_layers(int n, int pos, bool device_pos) {
        const Config& c = m_.cfg;
        bool norm_prepared = false;  // tensor-core path: the previous layer's last kernel already normalised and split x
        for (int l = 0; l < c.n_layer; l++) {
            const DevLayer& D = layers_[l];
            const DevWeight* qkv[3] = {&D.wq, &D.wk, &D.wv};
            float* qkv_out[3] = {q_, k_, v_};
            // single token, f16 weights: the weight-streaming kernel; the norm and the projections that share it are one launch
            const bool fused = n == 1 && fuse_decode_ && streamable(D.wq) && streamable(D.wk) && streamable(D.wv) && streamable(D.wo) &&
                               streamable(D.w_gate) && streamable(D.w_up) && streamable(D.w_down);
            // batches on the tensor-core path: the norm (and below the SwiGLU product) writes the f16 hi/lo activations directly
            const bool tc_layer = n > 1 && lin_ws_ != nullptr && layer_tc_ok(D, n);
            if (fused) {
                gemv_group(qkv_out, qkv, 3, false, x_, D.attn_norm, false);
            } else if (tc_layer) {
                // Every split-k product stays in scratch as k slices; the kernel that consumes it sums them.
                if (!norm_prepared)
                    cuda_check(ingot_linear_tc_prepare_norm(lin_ws_, x_, D.attn_norm, c.rms_eps, c.n_embd, n, stream_), "rmsnorm (split)");
                for (int i = 0; i < 3; i++) tc_partial(*qkv[i], i);
                cuda_check(ingot_linear_tc_finish_group(lin_ws_, qkv_out, 3, stream_), "q/k/v (slice sum)");
            } else {
                cuda_check(ingot_support_rmsnorm(h_, x_, D.attn_norm, n, c.n_embd, c.rms_eps, stream_), "rmsnorm");
                linear_group(qkv_out, qkv, 3, h_, n, false);
            }
            ingot_check(ingot_rope_kv_append(kv_, l, q_, q_rot_, k_, v_, inv_freq_, c.n_head, pos, n,
                                             device_pos ? pos_dev_ : nullptr, nullptr, nullptr, 0, stream_));
            if (n == 1)
                ingot_check(ingot_attn_decode(kv_, l, q_rot_, INGOT_F16, attn_, INGOT_F32, c.n_head, 1,
                                              device_pos ? pos_dev_ + 1 : nullptr, device_pos ? n_ctx_ : pos + 1, nullptr, 0, 0,
                                              stream_));
            else
                ingot_check(ingot_attn_prefill(kv_, l, q_rot_, INGOT_F16, attn_, INGOT_F32, c.n_head, pos, n, nullptr, 0,
                                               stream_));
            const DevWeight* wo[1] = {&D.wo};
            if (fused) {
                gemv_group(&x_, wo, 1, false, attn_, nullptr, true);
            } else if (tc_layer) {
                cuda_check(ingot_linear_tc_prepare(lin_ws_, attn_, D.wo.n_in, n, stream_), "linear (split)");
                tc_partial(D.wo, 0);
                // x += wo product; hi/lo of rmsnorm(x; ffn_norm) for gate/up
                cuda_check(ingot_linear_tc_finish_residual_norm(lin_ws_, x_, D.ffn_norm, c.rms_eps, 0, stream_), "residual + rmsnorm (split)");
            } else {
                linear_group(&x_, wo, 1, attn_, n, true);
            }
            const DevWeight* gu[2] = {&D.w_gate, &D.w_up};
            float* gu_out[2] = {gate_, up_};
            if (fused) {
                gemv_group(gu_out, gu, 2, true, x_, D.ffn_norm, false);  // gate_ <- silu(gate) * up
            } else if (tc_layer) {
                tc_partial(D.w_gate, 0);
                tc_partial(D.w_up, 1);
                cuda_check(ingot_linear_tc_finish_swiglu(lin_ws_, 0, 1, stream_), "silu_mul (split)");
            } else {
                cuda_check(ingot_support_rmsnorm(h_, x_, D.ffn_norm, n, c.n_embd, c.rms_eps, stream_), "rmsnorm");
                linear_group(gu_out, gu, 2, h_, n, false);
                cuda_check(ingot_support_silu_mul(gate_, up_, size_t(n) * c.n_ff, stream_), "silu_mul");
            }
            const DevWeight* wd[1] = {&D.w_down};
            if (fused) gemv_group(&x_, wd, 1, false, gate_, nullptr, true);
            else if (tc_layer) {
                tc_partial(D.w_down, 0);
                // x += down product; if the next layer also takes this path, its attention norm rides along
                const bool next_tc = l + 1 < c.n_layer && layer_tc_ok(layers_[l + 1], n);
                cuda_check(ingot_linear_tc_finish_residual_norm(lin_ws_, x_, next_tc ? layers_[l + 1].attn_norm : nullptr, c.rms_eps, 0, stream_),
                           "residual (+ rmsnorm, split)");
                norm_prepared = next_tc;
            } else linear_group(&x_, wd, 1, gate_, n, true);
            if (!tc_layer) norm_prepared = false;
        }
        // Logits for the last token only.
        if (fuse_decode_ && streamable(output_)) {
            const DevWeight* wl[1] = {&output_};
            gemv_group(&logits_dev_, wl, 1, false, x_ + size_t(n - 1) * c.n_embd, output_norm_, false);
        } else {
            cuda_check(ingot_support_rmsnorm(h_, x_ + size_t(n - 1) * c.n_embd, output_norm_, 1, c.n_embd, c.rms_eps, stream_), "rmsnorm");
            linear(logits_dev_, output_, h_, 1, false);
        }
    }

    int n_ctx() const override { return n_ctx_; }
    const char* name() const override { return "cuda"; }

private:
    struct DevLayer {
        float *attn_norm = nullptr, *ffn_norm = nullptr;
        DevWeight wq, wk, wv, wo, w_gate, w_up, w_down;
    };

    float* alloc_f32(size_t n) {
        void* p = nullptr;
        cuda_check(cudaMalloc(&p, n * sizeof(float)), "cudaMalloc");
        allocs_.push_back(p);
        return static_cast<float*>(p);
    }
    float* upload_f32(const std::vector<float>& v) {
        float* p = alloc_f32(v.size());
        cuda_check(cudaMemcpy(p, v.data(), v.size() * sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy");
        return p;
    }
    // Weights are read from the mmap (src/gguf.h:56) and kept in their stored float type.
    DevWeight upload(const gguf::TensorInfo& t) {
        DevWeight w;
        if (t.type == gguf::TensorType::F16) w.is_f16 = 1;
        else if (t.type == gguf::TensorType::F32) w.is_f16 = 0;
        else throw std::runtime_error(std::string("cuda: tensor ") + t.name + " has type " + gguf::type_name(t.type) +
                                      "; this backend reads F16 and F32 weights");
        w.n_in = int(t.dim(0));
        w.n_out = int(t.dim(1));
        if (w.n_in % 8 != 0) throw std::runtime_error("cuda: tensor " + t.name + " row length must be a multiple of 8");
        cuda_check(cudaMalloc(&w.data, t.nbytes()), "cudaMalloc(weight)");
        allocs_.push_back(w.data);
        cuda_check(cudaMemcpy(w.data, t.data, t.nbytes(), cudaMemcpyHostToDevice), "cudaMemcpy(weight)");
        return w;
    }
    bool tc_group(const DevWeight* const* ws, int count, int n_tok) const {
        bool tc = lin_ws_ != nullptr;
        for (int i = 0; i < count && tc; i++)
            tc = ws[i]->n_in == ws[0]->n_in && ingot_linear_tc_supported(lin_ws_, ws[i]->is_f16, ws[i]->n_in, ws[i]->n_out, n_tok);
        return tc;
    }
    bool layer_tc_ok(const DevLayer& D, int n_tok) const {
        const DevWeight* all[7] = {&D.wq, &D.wk, &D.wv, &D.wo, &D.w_gate, &D.w_up, &D.w_down};
        for (const DevWeight* w : all)
            if (!ingot_linear_tc_supported(lin_ws_, w->is_f16, w->n_in, w->n_out, n_tok)) return false;
        return D.wq.n_in == m_.cfg.n_embd && D.w_gate.n_in == m_.cfg.n_embd && D.w_down.n_in == m_.cfg.n_ff;
    }
    void tc_partial(const DevWeight& w, int slot) {
        cuda_check(ingot_linear_tc_run_partial(lin_ws_, w.data, w.n_in, w.n_out, slot, stream_), "linear (tensor core)");
    }
    // Projections that read the same activations. Batches go to the tensor-core kernel (the activations are split
    // into f16 hi/lo parts once per group); single tokens and unsupported shapes to the f32 kernels.
    void linear_group(float* const* outs, const DevWeight* const* ws, int count, const float* x, int n_tok, bool accumulate) {
        if (!tc_group(ws, count, n_tok)) {
            for (int i = 0; i < count; i++) linear(outs[i], *ws[i], x, n_tok, accumulate);
            return;
        }
        cuda_check(ingot_linear_tc_prepare(lin_ws_, x, ws[0]->n_in, n_tok, stream_), "linear (split)");
        for (int i = 0; i < count; i++)
            cuda_check(ingot_linear_tc_run(lin_ws_, outs[i], ws[i]->data, ws[i]->n_in, ws[i]->n_out, accumulate ? 1 : 0, stream_), "linear (tensor core)");
    }
    static bool streamable(const DevWeight& w) { return w.is_f16 && w.n_in % 256 == 0 && w.n_in <= 12288; }
    void gemv_group(float* const* outs, const DevWeight* const* ws, int count, bool swiglu, const float* x, const float* norm_w,
                    bool accumulate) {
        const void* wp[3] = {};
        int rows[3] = {};
        for (int i = 0; i < count; i++) { wp[i] = ws[i]->data; rows[i] = ws[i]->n_out; }
        cuda_check(ingot_support_gemv_group(outs, wp, rows, count, swiglu ? 1 : 0, x, norm_w, m_.cfg.rms_eps, ws[0]->n_in,
                                            accumulate ? 1 : 0, stream_), "gemv");
    }
    void linear(float* out, const DevWeight& w, const float* x, int n_tok, bool accumulate) {
        cuda_check(ingot_support_linear(out, w.data, w.is_f16, x, w.n_in, w.n_out, n_tok, accumulate ? 1 : 0, stream_), "linear");
    }

    const Model& m_;
    int n_ctx_, n_batch_;
    cudaStream_t stream_ = nullptr;
    ingot_kv* kv_ = nullptr;
    ingot_linear_ws* lin_ws_ = nullptr;
    std::vector<DevLayer> layers_;
    std::vector<void*> allocs_;
    float *output_norm_ = nullptr, *inv_freq_ = nullptr;
    DevWeight output_;
    float *x_ = nullptr, *h_ = nullptr, *q_ = nullptr, *k_ = nullptr, *v_ = nullptr, *attn_ = nullptr, *gate_ = nullptr,
          *up_ = nullptr, *logits_dev_ = nullptr;
    void* q_rot_ = nullptr;
    float *x_host_ = nullptr, *logits_ = nullptr;
    int32_t* pos_dev_ = nullptr;   // [0] = position of the single-token step, [1] = its key count
    int32_t* pos_host_ = nullptr;  // pinned
    int decode_calls_ = 0;
    const bool profile_ = getenv("INGOT_PROFILE") != nullptr;
    // INGOT_DECODE_FUSED=0: separate norm / projection / SwiGLU launches in single-token steps (diagnostics)
    const bool fuse_decode_ = !(getenv("INGOT_DECODE_FUSED") && atoi(getenv("INGOT_DECODE_FUSED")) == 0);
    cudaEvent_t ev0_ = nullptr, ev1_ = nullptr;
    double gpu_ms_ = 0, wall_ms_ = 0, gpu1_ms_ = 0;
    int calls_ = 0, calls1_ = 0;
    cudaGraph_t decode_graph_ = nullptr;
    cudaGraphExec_t decode_exec_ = nullptr;
};

}  // namespace

std::unique_ptr<Backend> make_cuda_backend(const gguf::File&, const Model& model, int n_ctx, int n_batch) {
    return std::make_unique<CudaBackend>(model, n_ctx, n_batch);
}

// Link seam: engine.cpp (src/engine.cpp:9-13) knows the GPU backend as "metal".
std::unique_ptr<Backend> make_metal_backend(const gguf::File& file, const Model& model, int n_ctx, int n_batch) {
    return make_cuda_backend(file, model, n_ctx, n_batch);
}

// Diagnostics verbs of the CLI (src/metal_backend.h:17-25, src/main.cpp:417-453).
double metal_linear_bench(const gguf::File&, const Model&, const std::string&, int, int) {
    throw std::runtime_error("kbench is not available on the cuda backend");
}
void metal_linear_check(const gguf::File&, const Model&, const std::string&, int) {
    throw std::runtime_error("kcheck is not available on the cuda backend");
}
void metal_bandwidth_test(const gguf::File&, const Model&, size_t) {
    throw std::runtime_error("bwtest is not available on the cuda backend");
}

// Seconds per token spent in decode attention across all layers at position pos
// (src/metal_backend.mm:594-649): all layers' decode attention, `iters` times, timed with CUDA events.
double metal_attention_bench(const gguf::File&, const Model& model, int pos, int iters) {
    const Config& c = model.cfg;
    ingot_kv* kv = nullptr;
    ingot_check(ingot_kv_create(&kv, INGOT_KV_CONTIGUOUS, c.n_layer, c.n_head_kv, c.head_dim, pos + 1, 1));
    const size_t q_elems = size_t(c.n_layer) * c.n_head * c.head_dim;
    void *q = nullptr, *out = nullptr;
    cuda_check(cudaMalloc(&q, q_elems * 2), "cudaMalloc");
    cuda_check(cudaMalloc(&out, q_elems * 4), "cudaMalloc");
    cuda_check(cudaMemset(q, 0, q_elems * 2), "cudaMemset");
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    auto run = [&](int reps) {
        for (int i = 0; i < reps; i++)
            ingot_check(ingot_attn_decode_layers(kv, 0, c.n_layer, q, INGOT_F16, out, INGOT_F32, c.n_head, 1, nullptr, pos + 1,
                                                 nullptr, 0, 0, nullptr));
    };
    run(2);
    cudaEventRecord(e0, nullptr);
    run(iters);
    cudaEventRecord(e1, nullptr);
    cuda_check(cudaEventSynchronize(e1), "attention bench");
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(q);
    cudaFree(out);
    ingot_kv_destroy(kv);
    return double(ms) * 1e-3 / iters;
}
