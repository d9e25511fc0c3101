// Continuous batching on top of BatchedBackend: many generation requests share the forward steps of one backend.
//
// The reference serves one request at a time: tokenise, prefill, then sample / forward until a stop token or the
// token limit (src/server.cpp:139-140, 164-184). This scheduler runs that same per-request loop for up to
// max_seqs() requests at once. Every step() makes ONE forward_multi call that carries one token of each running
// request - the next token of its prompt while it is still being read in, afterwards the token it sampled last -
// so requests that arrive at different times and are at different phases ride in the same launches. A finished
// request gives its cache blocks back (release_sequence) and its slot goes to the next queued request.
//
// Per request the observable behaviour is the reference loop's: the same Sampler (src/sampler.h) over the
// request's own history (prompt + reply), the stop token is not part of the reply, the token limit is clamped to
// the context window the same way, and the last token of a reply that ends on the limit is never fed back.
// A request's reply does not depend on what else is running: each sequence only ever sees its own cache.
#pragma once

#include <algorithm>
#include <cstdint>
#include <deque>
#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "batched_backend.h"
#include "sampler.h"

class BatchScheduler {
public:
    struct Request {
        std::vector<int32_t> prompt;
        int max_tokens = 128;
        SamplerParams sampling;                  // temperature 0 = greedy (the default)
        std::function<bool(int32_t)> is_stop;    // empty: the reply only ends on the token limit
        std::function<void(int32_t)> on_token;   // empty, or called for every token as it joins the reply
    };
    struct Result {
        std::vector<int32_t> tokens;             // the reply so far
        const char* finish = nullptr;            // nullptr while queued or running, then "stop", "length" or "cancelled"
    };

    BatchScheduler(BatchedBackend& backend, int n_vocab)
        : backend_(backend), n_vocab_(n_vocab), slots_(size_t(backend.max_seqs())) {
        if (n_vocab < 1) throw std::runtime_error("scheduler: vocabulary size must be positive");
    }

    // Queues a request and returns its id. Rejects what the reference server rejects before it starts
    // (src/server.cpp:139) with the same text, and token ids the backend would refuse in the middle of a step.
    int submit(Request r) {
        const int n_ctx = backend_.n_ctx_per_seq();
        if (r.prompt.empty()) throw std::runtime_error("scheduler: empty prompt");
        if (int(r.prompt.size()) + 1 >= n_ctx)
            throw std::runtime_error("prompt is " + std::to_string(r.prompt.size()) + " tokens, context is " + std::to_string(n_ctx));
        for (int32_t t : r.prompt)
            if (t < 0 || t >= n_vocab_) throw std::runtime_error("token id out of range");
        r.max_tokens = std::min(r.max_tokens, n_ctx - int(r.prompt.size()) - 1);  // src/server.cpp:140
        const int id = int(results_.size());
        results_.emplace_back();
        requests_.push_back(std::move(r));
        if (requests_[size_t(id)].max_tokens <= 0) results_[size_t(id)].finish = "length";  // nothing to generate
        else queue_.push_back(id);
        return id;
    }

    // One forward step over every running request (queued ones are admitted into free slots first).
    // Returns false, without calling the backend, when nothing is queued or running.
    bool step() {
        for (size_t s = 0; s < slots_.size() && !queue_.empty(); s++) {
            if (slots_[s].request >= 0) continue;
            Slot& slot = slots_[s];
            slot = Slot();
            slot.request = queue_.front();
            queue_.pop_front();
            const Request& r = requests_[size_t(slot.request)];
            slot.history = r.prompt;
            slot.sampler = std::make_unique<Sampler>(r.sampling, n_vocab_);
        }
        tok_.clear(); seq_.clear(); pos_.clear();
        for (size_t s = 0; s < slots_.size(); s++) {
            const Slot& slot = slots_[s];
            if (slot.request < 0) continue;
            const Request& r = requests_[size_t(slot.request)];
            tok_.push_back(slot.fed < int(r.prompt.size()) ? r.prompt[size_t(slot.fed)] : slot.next);
            seq_.push_back(int32_t(s));
            pos_.push_back(slot.fed);
        }
        if (tok_.empty()) return false;
        const float* logits = backend_.forward_multi(tok_.data(), seq_.data(), pos_.data(), int(tok_.size()));
        steps_++;
        rows_ += tok_.size();
        for (size_t i = 0; i < seq_.size(); i++) {
            Slot& slot = slots_[size_t(seq_[i])];
            const Request& r = requests_[size_t(slot.request)];
            Result& out = results_[size_t(slot.request)];
            slot.fed++;
            if (slot.fed < int(r.prompt.size())) continue;  // still inside the prompt: these logits are not sampled
            // the backend's logits are writable host memory (the sampler edits them in place, as in the reference)
            float* row = const_cast<float*>(logits) + i * size_t(n_vocab_);
            const int32_t next = slot.sampler->sample(row, slot.history);
            if (r.is_stop && r.is_stop(next)) {
                finish(slot, out, "stop");
                continue;
            }
            slot.history.push_back(next);
            out.tokens.push_back(next);
            if (r.on_token) r.on_token(next);
            if (int(out.tokens.size()) >= r.max_tokens) finish(slot, out, "length");  // the last token is not fed back
            else slot.next = next;
        }
        return true;
    }

    void run() { while (step()) {} }

    // Ends a request between steps (its client went away): a queued one never starts, a running one gives its slot
    // and cache blocks back. What it has generated so far stays readable; finish becomes "cancelled".
    void cancel(int id) {
        Result& out = results_.at(size_t(id));
        if (out.finish) return;
        for (auto it = queue_.begin(); it != queue_.end(); ++it)
            if (*it == id) { queue_.erase(it); out.finish = "cancelled"; return; }
        for (Slot& slot : slots_)
            if (slot.request == id) { finish(slot, out, "cancelled"); return; }
    }

    const Result& result(int id) const { return results_.at(size_t(id)); }
    int queued() const { return int(queue_.size()); }
    int running() const {
        int n = 0;
        for (const Slot& s : slots_) n += s.request >= 0;
        return n;
    }
    long long steps() const { return steps_; }   // forward_multi calls so far
    long long rows() const { return rows_; }     // tokens those calls carried

private:
    struct Slot {
        int request = -1;             // -1: free
        int fed = 0;                  // tokens of this request the backend has seen = position of the next one
        int32_t next = 0;             // sampled and not yet fed
        std::vector<int32_t> history; // prompt + reply, what the sampler's repetition penalty looks at
        std::unique_ptr<Sampler> sampler;
    };

    void finish(Slot& slot, Result& out, const char* why) {
        out.finish = why;
        backend_.release_sequence(int(&slot - slots_.data()));
        slot.request = -1;
        slot.sampler.reset();
    }

    BatchedBackend& backend_;
    int n_vocab_;
    std::vector<Slot> slots_;
    std::deque<Request> requests_;   // deques: references stay valid when a callback submits a new request
    std::deque<Result> results_;
    std::deque<int> queue_;
    std::vector<int32_t> tok_, seq_, pos_;
    long long steps_ = 0, rows_ = 0;
};
