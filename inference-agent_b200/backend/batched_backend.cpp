// make_batched_backend: the batched interface over a named backend (see batched_backend.h).
#include "batched_backend.h"

#include <cstring>
#include <stdexcept>
#include <vector>

#include "backend.h"
#include "engine.h"

namespace {

// One single-sequence Backend (src/backend.h:9-23) per sequence slot. A slot's cache is its backend's own, so
// release_sequence has nothing to hand back: the next request simply starts again at position 0.
class PerSequenceBackends : public BatchedBackend {
public:
    PerSequenceBackends(const std::string& name, const gguf::File& file, const Model& model, int n_ctx_per_seq, int max_seqs)
        : n_vocab_(model.cfg.n_vocab), n_ctx_(n_ctx_per_seq) {
        if (max_seqs < 1 || n_ctx_per_seq < 1) throw std::runtime_error("batched backend: needs at least one sequence and one position");
        for (int s = 0; s < max_seqs; s++) seqs_.push_back(make_backend(name, file, model, n_ctx_per_seq, 1));
        logits_.resize(size_t(max_seqs) * size_t(n_vocab_));
    }
    const float* forward_multi(const int32_t* tokens, const int32_t* seq_ids, const int32_t* positions, int n) override {
        if (n < 1 || n > int(seqs_.size())) throw std::runtime_error("batched backend: batch size out of range");
        std::vector<char> seen(seqs_.size(), 0);
        for (int i = 0; i < n; i++) {
            if (seq_ids[i] < 0 || seq_ids[i] >= int(seqs_.size())) throw std::runtime_error("batched backend: sequence id out of range");
            if (seen[size_t(seq_ids[i])]++) throw std::runtime_error("batched backend: a sequence appears twice in one forward_multi call");
        }
        for (int i = 0; i < n; i++) {
            const float* row = seqs_[size_t(seq_ids[i])]->forward(tokens[i], positions[i]);  // throws the reference's own messages
            std::memcpy(logits_.data() + size_t(i) * size_t(n_vocab_), row, size_t(n_vocab_) * sizeof(float));
        }
        return logits_.data();
    }
    void release_sequence(int seq_id) override {
        if (seq_id < 0 || seq_id >= int(seqs_.size())) throw std::runtime_error("batched backend: sequence id out of range");
    }
    int max_seqs() const override { return int(seqs_.size()); }
    int n_ctx_per_seq() const override { return n_ctx_; }

private:
    int n_vocab_, n_ctx_;
    std::vector<std::unique_ptr<Backend>> seqs_;
    std::vector<float> logits_;
};

}  // namespace

std::unique_ptr<BatchedBackend> make_batched_backend(const std::string& name, const gguf::File& file, const Model& model,
                                                     int n_ctx_per_seq, int max_seqs) {
    if (name == "cuda" || name == "metal") return make_cuda_batched_backend(file, model, n_ctx_per_seq, max_seqs);
    return std::make_unique<PerSequenceBackends>(name, file, model, n_ctx_per_seq, max_seqs);
}
