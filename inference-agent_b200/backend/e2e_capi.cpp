// C entry point that drives greedy generation through the reference's own glue (make_backend, prefill,
// Sampler; src/engine.cpp:9-23, src/sampler.cpp:14-51) on a named backend: "cpu" is the reference's
// CpuBackend, "metal" resolves to the CUDA backend in this build (see cuda_backend.cpp). Used by the
// end-to-end parity test; token ids are fed directly, so the GGUF needs no tokenizer arrays.
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

}  // extern "C"
