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
#include "batched_backend.h"

#include <cuda_fp16.h>
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
cudaError_t ingot_support_gemv_group(float* const* outs, const void* const* ws, const void* const* scales, int fmt, const int* n_out, int n_mat,
                                     int swiglu, const float* x, const float* norm_w, float eps, int n_in, int accumulate, cudaStream_t s);
cudaError_t ingot_support_embed_rows(float* out, const void* table, int is_f16, int n_in, int n_rows_table, const int32_t* rows_dev,
                                     int n_rows, int* status_dev, cudaStream_t s);
// GGUF block-quantised weights (quant_kernels.cu); `type` is the ggml type code (gguf::TensorType)
int ingot_quant_supported(int type, int n_in);
size_t ingot_quant_planar_bytes(int type, int n_in, int n_out);
size_t ingot_quant_scale_offset(int type, int n_in, int n_out);
cudaError_t ingot_quant_repack(void* planar_dev, const void* raw_dev, int type, int n_in, int n_out, cudaStream_t s);
cudaError_t ingot_quant_dequant_rows(float* out, const void* planar_dev, int type, int n_in, int n_out, const int32_t* rows_dev, int n_rows,
                                     int* status_dev, cudaStream_t s);
cudaError_t ingot_quant_dequant_hilo(void* hi_f16, void* lo_f16, const void* planar_dev, int type, int n_in, int n_out, cudaStream_t s);
cudaError_t ingot_quant_bf16_to_f32(float* out, const void* in_bf16, size_t n, cudaStream_t s);
cudaError_t ingot_quant_gemv(float* out, const void* planar_dev, int type, const float* x, int n_in, int n_out, int accumulate, cudaStream_t s);
// tensor-core form of the batched projections (linear_sm100.cu)
struct ingot_linear_ws;
cudaError_t ingot_linear_ws_create(ingot_linear_ws** out, int max_tok, int max_in);
void ingot_linear_ws_destroy(ingot_linear_ws* ws);
int ingot_linear_tc_supported(const ingot_linear_ws* ws, int w_is_f16, int n_in, int n_out, int n_tok);
cudaError_t ingot_linear_tc_prepare(ingot_linear_ws* ws, const float* x, int n_in, int n_tok, cudaStream_t s);
cudaError_t ingot_linear_tc_prepare_norm(ingot_linear_ws* ws, const float* x, const float* norm_w, float eps, int n_in, int n_tok,
                                         cudaStream_t s);
cudaError_t ingot_linear_tc_run_partial(ingot_linear_ws* ws, const void* w, int n_in, int n_out, int slot, cudaStream_t s);
cudaError_t ingot_linear_tc_run_partial_group(ingot_linear_ws* ws, const void* const* w, int n_in, const int* n_out, int count,
                                              int first_slot, int append, cudaStream_t s);
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
    void* data = nullptr;  // f32 / f16 rows, or the repacked planes of a block-quantised matrix (quant_kernels.cu)
    int is_f16 = 0;
    int qtype = -1;        // ggml type code of a block-quantised matrix (Q8_0, Q4_0, Q4_1, Q6_K), else -1
    void* scales = nullptr;  // block-quantised: the f16 block-scale plane inside `data`
    void* planes = nullptr;  // block-quantised, optional: resident f16 hi / lo planes (2 x n_in x n_out f16) for batches
    // format code of the weight-streaming single-token kernel (support_kernels.cu): 0 f16, 1 Q8_0, 2 Q4_0, -1 none
    int stream_fmt() const { return is_f16 ? 0 : qtype == 8 ? 1 : qtype == 2 ? 2 : -1; }
    int n_in = 0, n_out = 0;
};

// Streams weights from the memory-mapped model file to the device through a small ring of pinned staging buffers:
// the CPU copy of chunk i+1 out of the page cache (where the page faults and disk reads happen) overlaps the DMA
// of chunk i, and no call blocks on a pageable copy. The Metal backend wraps the mmap without copying
// (src/metal_backend.mm:213-246); a discrete GPU has to move the bytes once, so they move as a stream.
class WeightStreamer {
public:
    WeightStreamer() {
        cuda_check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate(load)");
        for (int i = 0; i < kBufs; i++) {
            cuda_check(cudaMallocHost(&buf_[i], kChunk), "cudaMallocHost(load staging)");
            cuda_check(cudaEventCreateWithFlags(&done_[i], cudaEventDisableTiming), "cudaEventCreate");
        }
    }
    ~WeightStreamer() {
        cudaStreamSynchronize(stream_);
        for (int i = 0; i < kBufs; i++) { cudaFreeHost(buf_[i]); cudaEventDestroy(done_[i]); }
        cudaStreamDestroy(stream_);
    }
    void copy(void* dst_dev, const void* src_host, size_t bytes) {
        const char* src = static_cast<const char*>(src_host);
        char* dst = static_cast<char*>(dst_dev);
        for (size_t off = 0; off < bytes; off += kChunk) {
            const size_t n = std::min(kChunk, bytes - off);
            const int b = next_++ % kBufs;
            cuda_check(cudaEventSynchronize(done_[b]), "load staging");  // the DMA that last read this buffer is over
            memcpy(buf_[b], src + off, n);
            cuda_check(cudaMemcpyAsync(dst + off, buf_[b], n, cudaMemcpyHostToDevice, stream_), "cudaMemcpyAsync(weight)");
            cuda_check(cudaEventRecord(done_[b], stream_), "cudaEventRecord");
            bytes_ += n;
        }
    }
    cudaStream_t stream() const { return stream_; }
    void finish() { cuda_check(cudaStreamSynchronize(stream_), "weight upload"); }
    size_t bytes() const { return bytes_; }

private:
    static constexpr int kBufs = 4;
    static constexpr size_t kChunk = size_t(32) << 20;
    cudaStream_t stream_ = nullptr;
    void* buf_[kBufs] = {};
    cudaEvent_t done_[kBufs] = {};
    unsigned next_ = 0;
    size_t bytes_ = 0;
};

class CudaBackend : public Backend, public BatchedBackend {
public:
    // max_seqs > 0 builds the batched form: a paged cache for max_seqs sequences of n_ctx positions each, and n_batch
    // (the most tokens per call) equal to max_seqs.
    CudaBackend(const Model& m, int n_ctx, int n_batch, int max_seqs = 0) : m_(m), n_ctx_(n_ctx), n_batch_(n_batch), max_seqs_(max_seqs) {
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
        if (max_seqs_ > 0) {
            blocks_per_seq_ = (n_ctx + INGOT_BLOCK_TOKENS - 1) / INGOT_BLOCK_TOKENS;
            const int n_blocks = blocks_per_seq_ * max_seqs_;
            ingot_check(ingot_kv_create(&kv_, INGOT_KV_PAGED, c.n_layer, c.n_head_kv, c.head_dim, n_blocks, max_seqs_));
            block_table_.assign(size_t(max_seqs_) * blocks_per_seq_, -1);
            // Blocks are handed out in arrival order, so the sequences' blocks interleave in the pool.
            for (int b = n_blocks - 1; b >= 0; b--) free_blocks_.push_back(b);
        } else {
            ingot_check(ingot_kv_create(&kv_, INGOT_KV_CONTIGUOUS, c.n_layer, c.n_head_kv, c.head_dim, n_ctx, 1));
        }

        // Weights: streamed to the device once (see WeightStreamer); block-quantised matrices are repacked there.
        const auto load0 = std::chrono::steady_clock::now();
        WeightStreamer loader;
        loader_ = &loader;
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
        // The embedding table lives on the device too (rows are gathered / dequantised by a kernel); a model with
        // tied embeddings shares the output matrix.
        embd_ = m.tok_embd == m.output ? output_ : upload(*m.tok_embd);
        inv_freq_ = upload_f32(m.rope_inv_freq);
        loader.finish();
        loader_ = nullptr;
        if (raw_tmp_) { cudaFree(raw_tmp_); raw_tmp_ = nullptr; raw_tmp_bytes_ = 0; }
        if (profile_)
            fprintf(stderr, "cuda: %.2f GB of weights on the device in %.2f s\n", loader.bytes() / 1e9,
                    std::chrono::duration<double>(std::chrono::steady_clock::now() - load0).count());

        if (max_quant_elems_ > 0 && n_batch > 1) {
            quant_scratch_elems_ = max_quant_elems_;
            cuda_check(cudaMalloc(&quant_scratch_, 2 * quant_scratch_elems_ * sizeof(__half)), "cudaMalloc(dequantisation scratch)");
            allocs_.push_back(quant_scratch_);
        }
        // Batches (16 tokens and up) multiply with the f16 hi / lo planes of a quantised matrix. On a 180 GB part there is
        // room to keep those planes resident for the layer matrices (4 bytes per weight: 11.6 GB for a 3-billion-parameter
        // model) next to the quantised copy that single-token steps stream, which saves re-expanding every matrix in every
        // batch. They are kept only while they fit a quarter of the free memory; INGOT_QUANT_PLANES=0 keeps nothing
        // resident (the planes are then rebuilt in scratch per use).
        if (n_batch >= 16 && lin_ws_hint_planes()) {
            size_t want = 0;
            for (const DevLayer& D : layers_)
                for (const DevWeight* w : {&D.wq, &D.wk, &D.wv, &D.wo, &D.w_gate, &D.w_up, &D.w_down})
                    if (w->qtype >= 0) want += size_t(w->n_in) * w->n_out * 4;
            size_t free_b = 0, total_b = 0;
            cuda_check(cudaMemGetInfo(&free_b, &total_b), "cudaMemGetInfo");
            if (want > 0 && want <= free_b / 4) {
                for (DevLayer& D : layers_)
                    for (DevWeight* w : {&D.wq, &D.wk, &D.wv, &D.wo, &D.w_gate, &D.w_up, &D.w_down}) {
                        if (w->qtype < 0) continue;
                        const size_t elems = size_t(w->n_in) * w->n_out;
                        cuda_check(cudaMalloc(&w->planes, 2 * elems * sizeof(__half)), "cudaMalloc(f16 planes)");
                        allocs_.push_back(w->planes);
                        cuda_check(ingot_quant_dequant_hilo(w->planes, static_cast<__half*>(w->planes) + elems, w->data, w->qtype, w->n_in,
                                                            w->n_out, stream_), "dequantise (resident planes)");
                    }
                cuda_check(cudaStreamSynchronize(stream_), "resident planes");
            }
        }
        const size_t nb = size_t(n_batch);
        const size_t q_dim = size_t(c.n_head) * c.head_dim, kv_dim = size_t(c.n_head_kv) * c.head_dim;
        x_ = alloc_f32(nb * c.n_embd); h_ = alloc_f32(nb * c.n_embd);
        q_ = alloc_f32(nb * q_dim); attn_ = alloc_f32(nb * q_dim);
        k_ = alloc_f32(nb * kv_dim); v_ = alloc_f32(nb * kv_dim);
        gate_ = alloc_f32(nb * c.n_ff); up_ = alloc_f32(nb * c.n_ff);
        if (max_seqs_ == 0) logits_dev_ = alloc_f32(size_t(c.n_vocab));
        cuda_check(cudaMalloc(&q_rot_, nb * q_dim * 2), "cudaMalloc(q_rot)");
        allocs_.push_back(q_rot_);
        cuda_check(cudaMalloc(&pos_dev_, 2 * sizeof(int32_t)), "cudaMalloc(pos)");
        allocs_.push_back(pos_dev_);
        cuda_check(cudaMallocHost(&pos_host_, 2 * sizeof(int32_t)), "cudaMallocHost(pos)");
        cuda_check(cudaMalloc(&tok_dev_, nb * sizeof(int32_t)), "cudaMalloc(tokens)");
        allocs_.push_back(tok_dev_);
        cuda_check(cudaMalloc(&embd_status_, sizeof(int)), "cudaMalloc(status)");
        allocs_.push_back(embd_status_);
        cuda_check(cudaMemset(embd_status_, 0, sizeof(int)), "cudaMemset");
        cuda_check(cudaMallocHost(&tok_host_, nb * sizeof(int32_t)), "cudaMallocHost(tokens)");
        const size_t logit_rows = max_seqs_ > 0 ? size_t(max_seqs_) : 1;
        if (max_seqs_ > 0) {
            logits_dev_ = alloc_f32(logit_rows * c.n_vocab);  // one row per sequence of a step
            const size_t meta = size_t(max_seqs_) * (3 + blocks_per_seq_);  // positions, key counts, row ids, block-table rows
            cuda_check(cudaMalloc(&multi_dev_, meta * sizeof(int32_t)), "cudaMalloc(step tables)");
            allocs_.push_back(multi_dev_);
            cuda_check(cudaMallocHost(&multi_host_, meta * sizeof(int32_t)), "cudaMallocHost(step tables)");
        }
        cuda_check(cudaMallocHost(&logits_, logit_rows * c.n_vocab * sizeof(float)), "cudaMallocHost(logits)");
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
        cudaFreeHost(tok_host_);
        cudaFreeHost(multi_host_);
        cudaFreeHost(logits_);
        ingot_linear_ws_destroy(lin_ws_);
        ingot_kv_destroy(kv_);
        cudaStreamDestroy(stream_);
    }

    const float* forward(int32_t token, int pos) override { return forward_batch(&token, 1, pos); }

    const float* forward_batch(const int32_t* tokens, int n, int pos) override {
        const Config& c = m_.cfg;
        if (max_seqs_ > 0) throw std::runtime_error("cuda: this backend was built for forward_multi");
        if (n < 1 || n > n_batch_) throw std::runtime_error("cuda: batch size out of range");
        if (pos < 0 || pos + n > n_ctx_) throw std::runtime_error("context window exceeded");
        for (int i = 0; i < n; i++)
            if (tokens[i] < 0 || tokens[i] >= c.n_vocab) throw std::runtime_error("token id out of range");

        // Token ids go to the device; the embedding rows are gathered (and dequantised) there by the first kernel of
        // the pass. (The reference dequantises them on the host into the shared x buffer, src/cpu_backend.cpp:33,
        // src/metal_backend.mm:426-428.)
        const auto wall0 = std::chrono::steady_clock::now();
        // a previous call's copy out of tok_host_ is complete: every call ends with a stream synchronisation
        for (int i = 0; i < n; i++) tok_host_[i] = tokens[i];
        if (profile_) cuda_check(cudaEventRecord(ev0_, stream_), "cudaEventRecord");
        cuda_check(cudaMemcpyAsync(tok_dev_, tok_host_, size_t(n) * sizeof(int32_t), cudaMemcpyHostToDevice, stream_), "H2D tokens");

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
    // multi: the n tokens belong to n different sequences of the paged cache (forward_multi); positions, key counts,
    // row ids and block-table rows were copied to multi_dev_, max_len bounds the key counts.
    void encode_layers(int n, int pos, bool device_pos, bool multi = false, int max_len = 0) {
        const Config& c = m_.cfg;
        if (embd_.qtype >= 0)
            cuda_check(ingot_quant_dequant_rows(x_, embd_.data, embd_.qtype, embd_.n_in, embd_.n_out, tok_dev_, n, embd_status_, stream_), "embedding rows");
        else
            cuda_check(ingot_support_embed_rows(x_, embd_.data, embd_.is_f16, embd_.n_in, embd_.n_out, tok_dev_, n, embd_status_, stream_), "embedding rows");
        bool norm_prepared = false;  // tensor-core path: the previous layer's last kernel already normalised and split x
        for (int l = 0; l < c.n_layer; l++) {
            const DevLayer& D = layers_[l];
            const DevWeight* qkv[3] = {&D.wq, &D.wk, &D.wv};
            float* qkv_out[3] = {q_, k_, v_};
            // single token, f16 weights: the weight-streaming kernel; the norm and the projections that share it are one launch
            const bool fused = n == 1 && fuse_decode_ && streamable(D.wq) && streamable(D.wk) && streamable(D.wv) && streamable(D.wo) &&
                               streamable(D.w_gate) && streamable(D.w_up) && streamable(D.w_down) && same_fmt(D.wq, D.wk) &&
                               same_fmt(D.wq, D.wv) && same_fmt(D.w_gate, D.w_up);
            // batches on the tensor-core path: the norm (and below the SwiGLU product) writes the f16 hi/lo activations directly
            const bool tc_layer = n > 1 && lin_ws_ != nullptr && layer_tc_ok(D, n);
            if (fused) {
                gemv_group(qkv_out, qkv, 3, false, x_, D.attn_norm, false);
            } else if (tc_layer) {
                // Every split-k product stays in scratch as k slices; the kernel that consumes it sums them.
                if (!norm_prepared)
                    cuda_check(ingot_linear_tc_prepare_norm(lin_ws_, x_, D.attn_norm, c.rms_eps, c.n_embd, n, stream_), "rmsnorm (split)");
                tc_partial_group(qkv, 3);  // one launch, slots 0..2
                cuda_check(ingot_linear_tc_finish_group(lin_ws_, qkv_out, 3, stream_), "q/k/v (slice sum)");
            } else {
                cuda_check(ingot_support_rmsnorm(h_, x_, D.attn_norm, n, c.n_embd, c.rms_eps, stream_), "rmsnorm");
                linear_group(qkv_out, qkv, 3, h_, n, false);
            }
            if (multi) {
                const int32_t* positions = multi_dev_;
                const int32_t* key_counts = multi_dev_ + max_seqs_;
                const int32_t* row_ids = multi_dev_ + 2 * size_t(max_seqs_);
                const int32_t* tables = multi_dev_ + 3 * size_t(max_seqs_);
                ingot_check(ingot_rope_kv_append(kv_, l, q_, q_rot_, k_, v_, inv_freq_, c.n_head, 0, n, positions, row_ids, tables,
                                                 blocks_per_seq_, stream_));
                ingot_check(ingot_attn_decode(kv_, l, q_rot_, INGOT_F16, attn_, INGOT_F32, c.n_head, n, key_counts, max_len, tables,
                                              blocks_per_seq_, 0, stream_));
            } else if (n == 1 && append_fused_) {
                // one token: RoPE, cache append and attention in one launch (bit-identical to the two calls below)
                ingot_check(ingot_rope_append_decode(kv_, l, q_, k_, v_, inv_freq_, attn_, INGOT_F32, c.n_head,
                                                     device_pos ? pos_dev_ + 1 : nullptr, pos, device_pos ? n_ctx_ : pos + 1, stream_));
            } else {
                ingot_check(ingot_rope_kv_append(kv_, l, q_, q_rot_, k_, v_, inv_freq_, c.n_head, pos, n,
                                                 device_pos ? pos_dev_ : nullptr, nullptr, nullptr, 0, stream_));
                if (n == 1)
                    ingot_check(ingot_attn_decode(kv_, l, q_rot_, INGOT_F16, attn_, INGOT_F32, c.n_head, 1,
                                                  device_pos ? pos_dev_ + 1 : nullptr, device_pos ? n_ctx_ : pos + 1, nullptr, 0, 0,
                                                  stream_));
                else
                    ingot_check(ingot_attn_prefill(kv_, l, q_rot_, INGOT_F16, attn_, INGOT_F32, c.n_head, pos, n, nullptr, 0,
                                                   stream_));
            }
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
                tc_partial_group(gu, 2);  // one launch, slots 0 and 1
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
        if (multi) {  // logits for every row: each belongs to another sequence
            cuda_check(ingot_support_rmsnorm(h_, x_, output_norm_, n, c.n_embd, c.rms_eps, stream_), "rmsnorm");
            const DevWeight* wl[1] = {&output_};
            if (n < 16 && output_.qtype >= 0) {  // few rows of a quantised matrix: one dequantise-in-GEMV pass per row
                for (int i = 0; i < n; i++) linear(logits_dev_ + size_t(i) * c.n_vocab, output_, h_ + size_t(i) * c.n_embd, 1, false);
            } else if (n == 1) {
                linear(logits_dev_, output_, h_, 1, false);
            } else {
                linear_group(&logits_dev_, wl, 1, h_, n, false);
            }
            return;
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

    // ---- BatchedBackend ----
    const float* forward_multi(const int32_t* tokens, const int32_t* seq_ids, const int32_t* positions, int n) override {
        const Config& c = m_.cfg;
        if (max_seqs_ == 0) throw std::runtime_error("cuda: this backend was built for single-sequence calls");
        if (n < 1 || n > max_seqs_) throw std::runtime_error("cuda: batch size out of range");
        std::vector<char> seen(size_t(max_seqs_), 0);
        int max_len = 1;
        int32_t* pos_h = multi_host_;
        int32_t* len_h = multi_host_ + max_seqs_;
        int32_t* row_h = multi_host_ + 2 * size_t(max_seqs_);
        int32_t* tab_h = multi_host_ + 3 * size_t(max_seqs_);
        for (int i = 0; i < n; i++) {
            if (tokens[i] < 0 || tokens[i] >= c.n_vocab) throw std::runtime_error("token id out of range");
            if (seq_ids[i] < 0 || seq_ids[i] >= max_seqs_) throw std::runtime_error("cuda: sequence id out of range");
            if (seen[seq_ids[i]]++) throw std::runtime_error("cuda: a sequence appears twice in one forward_multi call");
            if (positions[i] < 0 || positions[i] >= n_ctx_) throw std::runtime_error("context window exceeded");
        }
        for (int i = 0; i < n; i++) {
            // the block that holds this position is taken from the pool when the sequence first reaches it
            int32_t* row = block_table_.data() + size_t(seq_ids[i]) * blocks_per_seq_;
            const int blk = positions[i] / INGOT_BLOCK_TOKENS;
            for (int b = 0; b <= blk; b++) {  // a sequence may start beyond position 0 only over blocks it owns
                if (row[b] >= 0) continue;
                if (free_blocks_.empty()) throw std::runtime_error("context window exceeded");
                row[b] = free_blocks_.back();
                free_blocks_.pop_back();
            }
            tok_host_[i] = tokens[i];
            pos_h[i] = positions[i];
            len_h[i] = positions[i] + 1;
            row_h[i] = i;
            std::copy(row, row + blocks_per_seq_, tab_h + size_t(i) * blocks_per_seq_);
            max_len = std::max(max_len, positions[i] + 1);
        }
        cuda_check(cudaMemcpyAsync(tok_dev_, tok_host_, size_t(n) * sizeof(int32_t), cudaMemcpyHostToDevice, stream_), "H2D tokens");
        cuda_check(cudaMemcpyAsync(multi_dev_, multi_host_, (3 * size_t(max_seqs_) + size_t(n) * blocks_per_seq_) * sizeof(int32_t),
                                   cudaMemcpyHostToDevice, stream_), "H2D step tables");
        encode_layers(n, 0, false, true, max_len);
        cuda_check(cudaMemcpyAsync(logits_, logits_dev_, size_t(n) * c.n_vocab * sizeof(float), cudaMemcpyDeviceToHost, stream_), "D2H logits");
        cuda_check(cudaStreamSynchronize(stream_), "forward_multi");
        int status = 0;
        ingot_check(ingot_kv_status(kv_, stream_, &status));
        if (status != 0) throw std::runtime_error("cuda: attention kernel reported status " + std::to_string(status));
        return logits_;
    }
    void release_sequence(int seq_id) override {
        if (seq_id < 0 || seq_id >= max_seqs_) throw std::runtime_error("cuda: sequence id out of range");
        int32_t* row = block_table_.data() + size_t(seq_id) * blocks_per_seq_;
        for (int b = 0; b < blocks_per_seq_; b++)
            if (row[b] >= 0) { free_blocks_.push_back(row[b]); row[b] = -1; }
    }
    int max_seqs() const override { return max_seqs_; }
    int n_ctx_per_seq() const override { return n_ctx_; }

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
    // Weights are read from the mmap (src/gguf.h:56). F16 and F32 matrices keep their stored type; BF16 is widened
    // to F32 on the device (exact); Q8_0 / Q4_0 / Q4_1 / Q6_K keep their bits and are repacked into aligned planes
    // on the device (quant_kernels.cu). The types are those ops::type_supported accepts (src/ops.cpp:186-192).
    DevWeight upload(const gguf::TensorInfo& t) {
        DevWeight w;
        w.n_in = int(t.dim(0));
        w.n_out = int(t.dim(1));
        const int type = int(uint32_t(t.type));
        const bool quant = ingot_quant_supported(type, w.n_in) != 0;
        if (t.type == gguf::TensorType::F16) w.is_f16 = 1;
        else if (t.type == gguf::TensorType::F32 || t.type == gguf::TensorType::BF16) w.is_f16 = 0;
        else if (quant) w.qtype = type;
        else throw std::runtime_error(std::string("cuda: tensor ") + t.name + " has type " + gguf::type_name(t.type) +
                                      ", which this backend does not read (row length " + std::to_string(w.n_in) + ")");
        if (w.n_in % 8 != 0) throw std::runtime_error("cuda: tensor " + t.name + " row length must be a multiple of 8");
        if (quant || t.type == gguf::TensorType::BF16) {
            // file bytes -> device staging -> converted on the device (in stream order behind the copy)
            if (t.nbytes() > raw_tmp_bytes_) {
                loader_->finish();  // a conversion may still be reading the old staging buffer
                if (raw_tmp_) cudaFree(raw_tmp_);
                raw_tmp_ = nullptr;
                cuda_check(cudaMalloc(&raw_tmp_, t.nbytes()), "cudaMalloc(weight staging)");
                raw_tmp_bytes_ = t.nbytes();
            }
            const size_t out_bytes = quant ? ingot_quant_planar_bytes(type, w.n_in, w.n_out) : size_t(w.n_in) * w.n_out * sizeof(float);
            cuda_check(cudaMalloc(&w.data, out_bytes), "cudaMalloc(weight)");
            allocs_.push_back(w.data);
            loader_->copy(raw_tmp_, t.data, t.nbytes());
            if (quant) {
                cuda_check(ingot_quant_repack(w.data, raw_tmp_, type, w.n_in, w.n_out, loader_->stream()), "repack");
                w.scales = static_cast<char*>(w.data) + ingot_quant_scale_offset(type, w.n_in, w.n_out);
            }
            else cuda_check(ingot_quant_bf16_to_f32(static_cast<float*>(w.data), raw_tmp_, size_t(w.n_in) * w.n_out, loader_->stream()), "bf16 -> f32");
            // the output / embedding matrix is expanded only by the batched form with at least 16 rows per step
            const bool layer_matrix = &t != m_.output && &t != m_.tok_embd;
            if (quant && w.n_in * size_t(w.n_out) > max_quant_elems_ && (layer_matrix || max_seqs_ >= 16)) max_quant_elems_ = w.n_in * size_t(w.n_out);
            return w;
        }
        cuda_check(cudaMalloc(&w.data, t.nbytes()), "cudaMalloc(weight)");
        allocs_.push_back(w.data);
        loader_->copy(w.data, t.data, t.nbytes());
        return w;
    }
    bool tc_group(const DevWeight* const* ws, int count, int n_tok) const {
        bool tc = lin_ws_ != nullptr;
        for (int i = 0; i < count && tc; i++)
            tc = ws[i]->n_in == ws[0]->n_in &&
                 ingot_linear_tc_supported(lin_ws_, ws[i]->is_f16 || ws[i]->qtype >= 0, ws[i]->n_in, ws[i]->n_out, n_tok);
        return tc;
    }
    // f16 matrices, or block-quantised ones whose f16 hi/lo planes are resident (two products into the same slices)
    bool layer_tc_ok(const DevLayer& D, int n_tok) const {
        const DevWeight* all[7] = {&D.wq, &D.wk, &D.wv, &D.wo, &D.w_gate, &D.w_up, &D.w_down};
        for (const DevWeight* w : all)
            if (!ingot_linear_tc_supported(lin_ws_, w->is_f16 || (w->qtype >= 0 && w->planes), w->n_in, w->n_out, n_tok)) return false;
        if ((D.wq.planes != nullptr) != (D.wk.planes != nullptr) || (D.wq.planes != nullptr) != (D.wv.planes != nullptr) ||
            (D.w_gate.planes != nullptr) != (D.w_up.planes != nullptr))
            return false;  // a group is one launch per plane
        return D.wq.n_in == m_.cfg.n_embd && D.w_gate.n_in == m_.cfg.n_embd && D.w_down.n_in == m_.cfg.n_ff;
    }
    // Products of count matrices that read the prepared activations, left as k slices in slots first_slot.. for the consumer
    // kernels. A quantised matrix is its hi plane and then its lo plane (hi + lo = w exactly), the second launch adding slices.
    void tc_partial_group(const DevWeight* const* ws, int count, int first_slot = 0) {
        const void* wp[3] = {};
        int rows[3] = {};
        const bool planes = ws[0]->planes != nullptr;
        for (int i = 0; i < count; i++) { wp[i] = planes ? ws[i]->planes : ws[i]->data; rows[i] = ws[i]->n_out; }
        cuda_check(ingot_linear_tc_run_partial_group(lin_ws_, wp, ws[0]->n_in, rows, count, first_slot, 0, stream_), "linear (tensor core, grouped)");
        if (!planes) return;
        for (int i = 0; i < count; i++) wp[i] = static_cast<const __half*>(ws[i]->planes) + size_t(ws[i]->n_in) * ws[i]->n_out;
        cuda_check(ingot_linear_tc_run_partial_group(lin_ws_, wp, ws[0]->n_in, rows, count, first_slot, 1, stream_), "linear (tensor core, grouped, lo plane)");
    }
    void tc_partial(const DevWeight& w, int slot) {
        const DevWeight* one[1] = {&w};
        tc_partial_group(one, 1, slot);
    }
    // Projections that read the same activations. Batches go to the tensor-core kernel (the activations are split
    // into f16 hi/lo parts once per group); single tokens and unsupported shapes to the f32 kernels.
    void linear_group(float* const* outs, const DevWeight* const* ws, int count, const float* x, int n_tok, bool accumulate) {
        if (!tc_group(ws, count, n_tok)) {
            for (int i = 0; i < count; i++) linear(outs[i], *ws[i], x, n_tok, accumulate);
            return;
        }
        cuda_check(ingot_linear_tc_prepare(lin_ws_, x, ws[0]->n_in, n_tok, stream_), "linear (split)");
        for (int i = 0; i < count; i++) {
            const DevWeight& w = *ws[i];
            if (w.qtype < 0) {
                cuda_check(ingot_linear_tc_run(lin_ws_, outs[i], w.data, w.n_in, w.n_out, accumulate ? 1 : 0, stream_), "linear (tensor core)");
                continue;
            }
            // Block-quantised matrix: two f16 planes hi + lo = w (exact), each a tensor-core GEMM into the same output.
            // The planes are resident when memory allows (see the constructor), else rebuilt in scratch per use.
            __half* hi = w.planes ? static_cast<__half*>(w.planes) : quant_scratch(size_t(w.n_in) * w.n_out);
            __half* lo = hi + size_t(w.n_in) * w.n_out;
            if (!w.planes) cuda_check(ingot_quant_dequant_hilo(hi, lo, w.data, w.qtype, w.n_in, w.n_out, stream_), "dequantise (hi/lo)");
            cuda_check(ingot_linear_tc_run(lin_ws_, outs[i], hi, w.n_in, w.n_out, accumulate ? 1 : 0, stream_), "linear (tensor core, hi)");
            cuda_check(ingot_linear_tc_run(lin_ws_, outs[i], lo, w.n_in, w.n_out, 1, stream_), "linear (tensor core, lo)");
        }
    }
    static bool lin_ws_hint_planes() {
        const char* e = getenv("INGOT_QUANT_PLANES");
        return !(e && atoi(e) == 0);
    }
    // Scratch for the f16 hi/lo planes (or, for the f32 fallback, the f32 copy) of one block-quantised matrix: sized at
    // construction for the largest layer matrix, so nothing is allocated inside a forward pass.
    __half* quant_scratch(size_t elems) {
        if (elems > quant_scratch_elems_) throw std::runtime_error("cuda: quantised matrix larger than the dequantisation scratch");
        return static_cast<__half*>(quant_scratch_);
    }
    // what ingot_support_gemv_group takes: f16, Q8_0 or Q4_0 rows whose length is a multiple of one warp-wide load
    static bool streamable(const DevWeight& w) {
        const int fmt = w.stream_fmt();
        return fmt >= 0 && w.n_in % (fmt == 0 ? 256 : fmt == 1 ? 512 : 1024) == 0 && w.n_in <= 12032;
    }
    static bool same_fmt(const DevWeight& a, const DevWeight& b) { return a.stream_fmt() == b.stream_fmt(); }
    void gemv_group(float* const* outs, const DevWeight* const* ws, int count, bool swiglu, const float* x, const float* norm_w,
                    bool accumulate) {
        const void* wp[3] = {};
        const void* sp[3] = {};
        int rows[3] = {};
        for (int i = 0; i < count; i++) { wp[i] = ws[i]->data; sp[i] = ws[i]->scales; rows[i] = ws[i]->n_out; }
        cuda_check(ingot_support_gemv_group(outs, wp, sp, ws[0]->stream_fmt(), rows, count, swiglu ? 1 : 0, x, norm_w, m_.cfg.rms_eps,
                                            ws[0]->n_in, accumulate ? 1 : 0, stream_), "gemv");
    }
    void linear(float* out, const DevWeight& w, const float* x, int n_tok, bool accumulate) {
        if (w.qtype >= 0) {
            if (n_tok == 1) {  // dequantise-in-GEMV: reads the quantised bytes once
                cuda_check(ingot_quant_gemv(out, w.data, w.qtype, x, w.n_in, w.n_out, accumulate ? 1 : 0, stream_), "gemv (quantised)");
                return;
            }
            // few tokens (below the tensor-core kernel's minimum): f32 copy of the matrix, then the f32 kernels
            float* wf = reinterpret_cast<float*>(quant_scratch(size_t(w.n_in) * w.n_out));
            cuda_check(ingot_quant_dequant_rows(wf, w.data, w.qtype, w.n_in, w.n_out, nullptr, w.n_out, nullptr, stream_), "dequantise (f32)");
            cuda_check(ingot_support_linear(out, wf, 0, x, w.n_in, w.n_out, n_tok, accumulate ? 1 : 0, stream_), "linear");
            return;
        }
        cuda_check(ingot_support_linear(out, w.data, w.is_f16, x, w.n_in, w.n_out, n_tok, accumulate ? 1 : 0, stream_), "linear");
    }

    const Model& m_;
    int n_ctx_, n_batch_;
    int max_seqs_ = 0, blocks_per_seq_ = 0;       // batched form: paged cache shared by max_seqs_ sequences
    std::vector<int32_t> block_table_;            // [max_seqs_][blocks_per_seq_], -1 = not allocated
    std::vector<int32_t> free_blocks_;
    int32_t *multi_dev_ = nullptr, *multi_host_ = nullptr;  // per step: positions, key counts, row ids [max_seqs_ each], block-table rows
    cudaStream_t stream_ = nullptr;
    ingot_kv* kv_ = nullptr;
    ingot_linear_ws* lin_ws_ = nullptr;
    std::vector<DevLayer> layers_;
    std::vector<void*> allocs_;
    float *output_norm_ = nullptr, *inv_freq_ = nullptr;
    DevWeight output_, embd_;
    WeightStreamer* loader_ = nullptr;        // alive during construction only
    void* raw_tmp_ = nullptr;                 // device staging for tensors that are converted on the device at load
    size_t raw_tmp_bytes_ = 0;
    size_t max_quant_elems_ = 0;              // largest block-quantised layer matrix
    void* quant_scratch_ = nullptr;           // 2 x max_quant_elems_ f16 (= max_quant_elems_ f32)
    size_t quant_scratch_elems_ = 0;
    int32_t *tok_dev_ = nullptr, *tok_host_ = nullptr;
    int* embd_status_ = nullptr;
    float *x_ = nullptr, *h_ = nullptr, *q_ = nullptr, *k_ = nullptr, *v_ = nullptr, *attn_ = nullptr, *gate_ = nullptr,
          *up_ = nullptr, *logits_dev_ = nullptr;
    void* q_rot_ = nullptr;
    float* logits_ = nullptr;
    int32_t* pos_dev_ = nullptr;   // [0] = position of the single-token step, [1] = its key count
    int32_t* pos_host_ = nullptr;  // pinned
    int decode_calls_ = 0;
    const bool profile_ = getenv("INGOT_PROFILE") != nullptr;
    // INGOT_DECODE_FUSED=0: separate norm / projection / SwiGLU launches in single-token steps (diagnostics)
    const bool fuse_decode_ = !(getenv("INGOT_DECODE_FUSED") && atoi(getenv("INGOT_DECODE_FUSED")) == 0);
    // one launch for RoPE + append + attention of a single token (ingot_rope_append_decode): same bits, same speed as the two
    // launches it replaces (tg32 586 against 589 tok/s), so it is opt-in
    const bool append_fused_ = getenv("INGOT_APPEND_FUSED") && atoi(getenv("INGOT_APPEND_FUSED")) != 0;
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

std::unique_ptr<BatchedBackend> make_cuda_batched_backend(const gguf::File&, const Model& model, int n_ctx_per_seq, int max_seqs) {
    if (max_seqs < 1 || n_ctx_per_seq < 1) throw std::runtime_error("cuda: the batched backend needs at least one sequence and one position");
    return std::make_unique<CudaBackend>(model, n_ctx_per_seq, max_seqs, max_seqs);
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
// `bwtest` (src/metal_backend.mm:533-592): read bandwidth over growing read sizes. The Metal version reads a
// private buffer, the shared KV cache and the no-copy model file; a discrete GPU has one kind of device memory,
// so there is one row, from sizes that fit the L2 up to `bytes` (sizes beyond the 126 MB L2 measure HBM).
void metal_bandwidth_test(const gguf::File&, const Model&, size_t bytes) {
    std::vector<size_t> sizes = {size_t(4e6), size_t(16e6), size_t(64e6), size_t(256e6)};
    if (bytes > sizes.back()) sizes.push_back(bytes);
    fprintf(stderr, "%-22s", "read size ->");
    for (size_t n : sizes) fprintf(stderr, " %7zu MB", n / 1000000);
    fprintf(stderr, "\n-- 16-byte streaming loads\n%-22s", "device memory");
    for (size_t n : sizes) {
        double secs = 0.0;
        ingot_check(ingot_hbm_read_probe(n, 5, &secs, nullptr));
        fprintf(stderr, " %5.0f GB/s", double(n / 16 * 16) / secs / 1e9);
    }
    fprintf(stderr, "\n");
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
