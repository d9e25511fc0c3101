// Batched extension of the compute boundary: one forward step for many independent sequences.
//
// This interface has no counterpart in the reference, whose Backend runs one sequence (one token or one chunk
// of it per call) and whose server handles one connection at a time. It exists so that the paged KV cache and
// the multi-sequence decode kernel of libingot_cuda.so (ingot_attn_decode with n_seq > 1, ingot_rope_kv_append
// with per-token positions and sequence ids) have a caller that a serving loop can drive: continuous batching
// is "call forward_multi with whatever sequences have a token ready".
//
// Semantics follow the single-sequence Backend: a sequence's cache is a pure function of (sequence, position),
// positions may be revisited, and the returned logits live in writable host memory owned by the backend until
// the next call.
#pragma once

#include <cstdint>
#include <memory>
#include <string>

#include "gguf.h"
#include "model.h"

class BatchedBackend {
public:
    virtual ~BatchedBackend() = default;
    // One token for each of n DIFFERENT sequences: tokens[i] of sequence seq_ids[i] (0 <= id < max_seqs()) sits at
    // position positions[i], is written to that sequence's cache and attends to its keys 0..positions[i].
    // Returns n rows of n_vocab logits, row i for tokens[i]. Throws std::runtime_error with the reference's
    // messages for a bad token id ("token id out of range") or position ("context window exceeded"), and for a
    // repeated or out-of-range sequence id.
    virtual const float* forward_multi(const int32_t* tokens, const int32_t* seq_ids, const int32_t* positions, int n) = 0;
    // Gives a sequence's cache blocks back to the pool (its id can then serve a new request).
    virtual void release_sequence(int seq_id) = 0;
    virtual int max_seqs() const = 0;
    virtual int n_ctx_per_seq() const = 0;
};

// max_seqs sequences of up to n_ctx_per_seq positions each share one paged cache (16-token blocks handed out on
// demand). Throws like make_cuda_backend.
std::unique_ptr<BatchedBackend> make_cuda_batched_backend(const gguf::File& file, const Model& model, int n_ctx_per_seq, int max_seqs);

// The batched interface over a named backend. "cuda" (or "metal", the name the reference's engine knows its GPU
// backend by) is make_cuda_batched_backend. Any other name the reference's make_backend accepts ("cpu") gets one
// single-sequence backend instance per sequence slot, stepped one after another: no sharing of launches, but the
// same interface and the same results, e.g. to run a serving loop written against forward_multi without a GPU.
std::unique_ptr<BatchedBackend> make_batched_backend(const std::string& name, const gguf::File& file, const Model& model,
                                                     int n_ctx_per_seq, int max_seqs);
