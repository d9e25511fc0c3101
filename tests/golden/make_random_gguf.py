"""Writes a seeded random-init Llama-architecture F16 GGUF for the end-to-end greedy check.

    python tests/golden/make_random_gguf.py OUT.gguf [--layers 28] [--vocab 128256] [--seed 0]

Defaults are the Llama-3.2-3B shape: d_model 3072, 24 query / 8 KV heads of 128, FFN 8192, RMSNorm
eps 1e-5, RoPE theta 500000. Matrices are N(0, 0.02) in F16 (ggml layout ne = [n_in, n_out], i.e.
numpy shape [n_out, n_in]); norm gains are 1 (F32). The vocabulary is a placeholder list of the right
length; token ids are fed to the engine directly.
"""
import argparse

import numpy as np


def write(path, n_layer=28, n_vocab=128256, seed=0, n_embd=3072, n_head=24, n_head_kv=8, n_ff=8192, n_ctx=8192):
    import gguf
    rng = np.random.default_rng(seed)
    w = gguf.GGUFWriter(path, "llama")
    w.add_block_count(n_layer)
    w.add_embedding_length(n_embd)
    w.add_head_count(n_head)
    w.add_head_count_kv(n_head_kv)
    w.add_feed_forward_length(n_ff)
    w.add_context_length(n_ctx)
    w.add_rope_freq_base(500000.0)
    w.add_layer_norm_rms_eps(1e-5)
    w.add_vocab_size(n_vocab)
    # Model::load evaluates the tokenizer array's size even when llama.vocab_size is present
    # (src/model.cpp:47), so a placeholder vocabulary of the right length is written.
    w.add_token_list([f"<{i}>" for i in range(n_vocab)])
    head_dim = n_embd // n_head
    q_dim, kv_dim = n_head * head_dim, n_head_kv * head_dim

    def mat(name, n_in, n_out):
        a = (rng.standard_normal((n_out, n_in), dtype=np.float32) * np.float32(0.02)).astype(np.float16)
        w.add_tensor(name, a)

    mat("token_embd.weight", n_embd, n_vocab)
    w.add_tensor("output_norm.weight", np.ones(n_embd, dtype=np.float32))
    mat("output.weight", n_embd, n_vocab)
    for l in range(n_layer):
        p = f"blk.{l}."
        w.add_tensor(p + "attn_norm.weight", np.ones(n_embd, dtype=np.float32))
        w.add_tensor(p + "ffn_norm.weight", np.ones(n_embd, dtype=np.float32))
        mat(p + "attn_q.weight", n_embd, q_dim)
        mat(p + "attn_k.weight", n_embd, kv_dim)
        mat(p + "attn_v.weight", n_embd, kv_dim)
        mat(p + "attn_output.weight", q_dim, n_embd)
        mat(p + "ffn_gate.weight", n_embd, n_ff)
        mat(p + "ffn_up.weight", n_embd, n_ff)
        mat(p + "ffn_down.weight", n_ff, n_embd)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("out")
    ap.add_argument("--layers", type=int, default=28)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    write(a.out, a.layers, a.vocab, a.seed)
