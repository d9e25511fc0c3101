// C entry point that drives greedy generation through the reference's own glue (make_backend, prefill,
// Sampler; src/engine.cpp:9-23, src/sampler.cpp:14-51) on a named backend: "cpu" is the reference's
// CpuBackend, "metal" resolves to the CUDA backend in this build (see cuda_backend.cpp). Used by the
// end-to-end parity test; token ids are fed directly, so the GGUF needs no tokenizer arrays.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <string>
#include <vector>

#include "engine.h"
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

}  // extern "C"
