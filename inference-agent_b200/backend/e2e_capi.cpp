// C entry point that drives greedy generation through the reference's own glue (make_backend, prefill,
// Sampler; src/engine.cpp:9-23, src/sampler.cpp:14-51) on a named backend: "cpu" is the reference's
// CpuBackend, "metal" resolves to the CUDA backend in this build (see cuda_backend.cpp). Used by the
// end-to-end parity test; token ids are fed directly, so the GGUF needs no tokenizer arrays.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "batch_scheduler.h"
#include "batched_backend.h"
#include "engine.h"
#include "metal_backend.h"
#include "gguf.h"
#include "model.h"
#include "sampler.h"

static thread_local std::string g_err;

extern "C" {

const char* ingot_e2e_last_error() { return g_err.c_str(); }

// Writes n_gen greedy token ids to out_ids and the top-1 minus top-2 logit margin of every step to
// out_margin (may be null). Returns 0, or -1 with ingot_e2e_last_error() set.
int ingot_e2e_greedy(const char* gguf_path, const char* backend_name, const int32_t* prompt, int n_prompt, int n_gen,
                     int n_batch, int32_t* out_ids, float* out_margin) {
    try {
        gguf::File f = gguf::File::open(gguf_path);
        Model model = Model::load(f);
        auto backend = make_backend(backend_name, f, model, n_prompt + n_gen + 8, n_batch);
        SamplerParams sp;
        sp.temperature = 0.0f;
        Sampler sampler(sp, model.cfg.n_vocab);
        std::vector<int32_t> ids(prompt, prompt + n_prompt);
        int pos = 0;
        const float* logits = prefill(*backend, ids, pos, n_batch);
        for (int i = 0; i < n_gen; i++) {
            if (out_margin) {
                float a = -INFINITY, b = -INFINITY;
                for (int t = 0; t < model.cfg.n_vocab; t++) {
                    const float x = logits[t];
                    if (x > a) { b = a; a = x; } else if (x > b) { b = x; }
                }
                out_margin[i] = a - b;
            }
            const int32_t next = sampler.sample(const_cast<float*>(logits), ids);
            out_ids[i] = next;
            ids.push_back(next);
            if (i + 1 < n_gen) logits = backend->forward(next, pos++);
        }
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

// The measurement `ingot bench -p N -n M -r R` makes (src/main.cpp:340-399) with the prompt given as token
// ids: warm-up (one batched and one single-token forward), then R times { prefill in n_batch chunks, M
// greedy decode steps }, wall-clock. out[0] = mean prompt tokens/s, out[1] = mean generated tokens/s.
int ingot_e2e_bench(const char* gguf_path, const char* backend_name, const int32_t* prompt, int n_prompt, int n_gen,
                    int n_batch, int reps, double* out) {
    try {
        gguf::File f = gguf::File::open(gguf_path);
        Model model = Model::load(f);
        auto backend = make_backend(backend_name, f, model, n_prompt + n_gen + 8, n_batch);
        using clock = std::chrono::steady_clock;
        auto secs = [](clock::time_point a, clock::time_point b) { return std::chrono::duration<double>(b - a).count(); };
        backend->forward_batch(prompt, std::min(n_batch, n_prompt), 0);
        backend->forward(prompt[0], 0);
        double pp = 0, tg = 0;
        for (int r = 0; r < reps; r++) {
            int pos = 0;
            const auto t0 = clock::now();
            const float* logits = nullptr;
            for (int i = 0; i < n_prompt; i += n_batch) {
                const int n = std::min(n_batch, n_prompt - i);
                logits = backend->forward_batch(prompt + i, n, pos);
                pos += n;
            }
            const auto t1 = clock::now();
            for (int i = 0; i < n_gen; i++) {
                const int32_t next = int32_t(std::max_element(logits, logits + model.cfg.n_vocab) - logits);
                logits = backend->forward(next, pos++);
            }
            const auto t2 = clock::now();
            pp += n_prompt / secs(t0, t1);
            tg += n_gen / secs(t1, t2);
        }
        out[0] = pp / reps;
        out[1] = tg / reps;
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

// Greedy generation for n_seq sequences at once through BatchedBackend::forward_multi, the way a continuous-batching
// loop would drive it: at every step each unfinished sequence contributes one token - the next token of its
// prompt while it is still being prefilled, afterwards the token it generated last - so sequences of different
// prompt lengths are at different phases in the same call. prompts holds the prompts back to back, prompt_lens
// their lengths. out_ids receives n_gen tokens per sequence ([n_seq][n_gen]). Returns 0, or -1 with
// ingot_e2e_last_error() set.
int ingot_e2e_multi_greedy(const char* gguf_path, const int32_t* prompts, const int32_t* prompt_lens, int n_seq, int n_gen,
                           int n_ctx_per_seq, int32_t* out_ids) {
    try {
        gguf::File f = gguf::File::open(gguf_path);
        Model model = Model::load(f);
        auto backend = make_cuda_batched_backend(f, model, n_ctx_per_seq, n_seq);
        const int n_vocab = model.cfg.n_vocab;
        std::vector<const int32_t*> prompt(n_seq);
        std::vector<int> fed(n_seq, 0), made(n_seq, 0);   // tokens fed so far / generated so far
        std::vector<int32_t> last(n_seq, 0);
        for (int s = 0, off = 0; s < n_seq; off += prompt_lens[s], s++) prompt[s] = prompts + off;
        std::vector<int32_t> tok, seq, pos;
        for (;;) {
            tok.clear(); seq.clear(); pos.clear();
            for (int s = 0; s < n_seq; s++) {
                if (made[s] >= n_gen) continue;
                tok.push_back(fed[s] < prompt_lens[s] ? prompt[s][fed[s]] : last[s]);
                seq.push_back(s);
                pos.push_back(fed[s]);
            }
            if (tok.empty()) break;
            const float* logits = backend->forward_multi(tok.data(), seq.data(), pos.data(), int(tok.size()));
            for (size_t i = 0; i < tok.size(); i++) {
                const int s = seq[i];
                fed[s]++;
                if (fed[s] < prompt_lens[s]) continue;  // still inside the prompt: these logits are not sampled
                const float* row = logits + i * size_t(n_vocab);
                last[s] = int32_t(std::max_element(row, row + n_vocab) - row);
                out_ids[size_t(s) * n_gen + made[s]++] = last[s];
                if (made[s] >= n_gen) backend->release_sequence(s);
            }
        }
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

// sampling: null for greedy defaults, else {temperature, top_k, top_p, repeat_penalty, repeat_last_n, seed} (src/sampler.h:8-15).
static SamplerParams sampler_params(const double* sampling) {
    SamplerParams sp;
    sp.temperature = 0.0f;
    if (sampling) {
        sp.temperature = float(sampling[0]);
        sp.top_k = int(sampling[1]);
        sp.top_p = float(sampling[2]);
        sp.repeat_penalty = float(sampling[3]);
        sp.repeat_last_n = int(sampling[4]);
        sp.seed = uint64_t(sampling[5]);
    }
    return sp;
}

// One request the way the reference's server runs it (src/server.cpp:164-184): prefill, then sample from the logits with
// the request's own Sampler over prompt + reply, stop before stop_token (-1: none), at most max_tokens tokens, the last
// one not fed back. Writes the reply to out_ids (room for max_tokens) and returns its length, or -1 with
// ingot_e2e_last_error() set.
int ingot_e2e_generate(const char* gguf_path, const char* backend_name, const int32_t* prompt, int n_prompt, int max_tokens,
                       int n_batch, const double* sampling, int stop_token, int32_t* out_ids) {
    try {
        gguf::File f = gguf::File::open(gguf_path);
        Model model = Model::load(f);
        auto backend = make_backend(backend_name, f, model, n_prompt + max_tokens + 8, n_batch);
        Sampler sampler(sampler_params(sampling), model.cfg.n_vocab);
        std::vector<int32_t> history(prompt, prompt + n_prompt);
        int pos = 0;
        const float* logits = prefill(*backend, history, pos, n_batch);
        int generated = 0;
        while (generated < max_tokens) {
            const int32_t next = sampler.sample(const_cast<float*>(logits), history);
            if (next == stop_token) break;
            history.push_back(next);
            out_ids[generated++] = next;
            if (generated < max_tokens) logits = backend->forward(next, pos++);
        }
        return generated;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

// Generation of n_req requests through BatchScheduler on a backend with max_seqs sequence slots ("cpu": one
// reference CpuBackend per slot; "metal" / "cuda": the paged CUDA backend). Request r is submitted before step
// arrival_step[r] (null: all at the start), so later requests join while earlier ones are running and take over the
// slots of finished ones. A reply ends before stop_token (pass -1 for none) or after max_tokens[r] tokens.
// A negative max_tokens[r] = -(k + 1) stands for a client that goes away: no limit of its own, cancelled before step k.
// out_ids [n_req][max_out] receives the replies, out_counts their lengths, out_finish 0 for "length", 1 for "stop"
// and 2 for "cancelled"; stats (may be null) receives the number of forward_multi calls and the tokens they carried;
// sampling (may be null: greedy) is what ingot_e2e_generate takes.
// Returns 0, or -1 with ingot_e2e_last_error() set.
int ingot_e2e_sched_greedy(const char* gguf_path, const char* backend_name, const int32_t* prompts, const int32_t* prompt_lens,
                           const int32_t* max_tokens, const int32_t* arrival_step, int n_req, int max_seqs, int n_ctx_per_seq,
                           int stop_token, int32_t* out_ids, int max_out, int32_t* out_counts, int32_t* out_finish, long long* stats,
                           const double* sampling) {
    try {
        gguf::File f = gguf::File::open(gguf_path);
        Model model = Model::load(f);
        auto backend = make_batched_backend(backend_name, f, model, n_ctx_per_seq, max_seqs);
        BatchScheduler sched(*backend, model.cfg.n_vocab);
        std::vector<int> id(static_cast<size_t>(n_req), -1);
        std::vector<const int32_t*> prompt(static_cast<size_t>(n_req), nullptr);
        for (int r = 0, off = 0; r < n_req; off += prompt_lens[r], r++) prompt[size_t(r)] = prompts + off;
        int submitted = 0;
        for (long long step = 0;; step++) {
            for (int r = 0; r < n_req; r++) {
                if (id[size_t(r)] >= 0 || (arrival_step && arrival_step[r] > step)) continue;
                BatchScheduler::Request q;
                q.prompt.assign(prompt[size_t(r)], prompt[size_t(r)] + prompt_lens[r]);
                q.max_tokens = max_tokens[r] < 0 ? (1 << 20) : max_tokens[r];
                q.is_stop = [stop_token](int32_t t) { return t == stop_token; };
                q.sampling = sampler_params(sampling);  // every request seeds its own sampler, as every server request does
                id[size_t(r)] = sched.submit(std::move(q));
                submitted++;
            }
            // a negative max_tokens[r] = -(k + 1) means: limit 1 << 20, and the client of request r goes away after step k
            for (int r = 0; r < n_req; r++)
                if (id[size_t(r)] >= 0 && max_tokens[r] < 0 && step == -(max_tokens[r] + 1)) sched.cancel(id[size_t(r)]);
            if (!sched.step() && submitted == n_req) break;  // idle steps while waiting for an arrival cost nothing
        }
        for (int r = 0; r < n_req; r++) {
            const BatchScheduler::Result& res = sched.result(id[size_t(r)]);
            if (!res.finish) throw std::runtime_error("scheduler: a request was left unfinished");
            if (int(res.tokens.size()) > max_out) throw std::runtime_error("scheduler: reply longer than the output rows");
            out_counts[r] = int32_t(res.tokens.size());
            out_finish[r] = std::string(res.finish) == "stop" ? 1 : std::string(res.finish) == "cancelled" ? 2 : 0;
            std::copy(res.tokens.begin(), res.tokens.end(), out_ids + size_t(r) * size_t(max_out));
        }
        if (stats) { stats[0] = sched.steps(); stats[1] = sched.rows(); }
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

// The reference CLI's `abench` and `bwtest` verbs (src/main.cpp:441-455) as C calls: seconds per token of decode
// attention over all layers at position `pos` (metal_attention_bench), and the read-bandwidth table on stderr
// (metal_bandwidth_test) - both resolve to the CUDA backend of this build.
int ingot_e2e_abench(const char* gguf_path, int pos, int iters, double* secs_per_token, double* kv_bytes) {
    try {
        gguf::File f = gguf::File::open(gguf_path);
        Model model = Model::load(f);
        *secs_per_token = metal_attention_bench(f, model, pos, iters);
        *kv_bytes = 2.0 * model.cfg.n_layer * double(pos + 1) * model.cfg.n_head_kv * model.cfg.head_dim * 2;  // src/main.cpp:446
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

int ingot_e2e_bwtest(const char* gguf_path, double megabytes) {
    try {
        gguf::File f = gguf::File::open(gguf_path);
        Model model = Model::load(f);
        metal_bandwidth_test(f, model, size_t(megabytes * 1e6));
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

}  // extern "C"
