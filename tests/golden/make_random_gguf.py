"""Writes a seeded random-init Llama-architecture GGUF for the end-to-end greedy check.

    python tests/golden/make_random_gguf.py OUT.gguf [--layers 28] [--vocab 128256] [--seed 0]
                                            [--type F16|Q8_0|Q4_0|Q4_1|Q6_K] [--output-type ...]

Defaults are the Llama-3.2-3B shape: d_model 3072, 24 query / 8 KV heads of 128, FFN 8192, RMSNorm
eps 1e-5, RoPE theta 500000. F16 matrices are N(0, 0.02) (ggml layout ne = [n_in, n_out], i.e.
numpy shape [n_out, n_in]). Block-quantised matrices are written directly in their block format
(src/ops.cpp:33-91 of the reference describes the layouts): uniformly random quants and per-block f16
scales chosen so that the decoded weights have a standard deviation of about 0.02 - no float matrix
is quantised, which keeps a 3-billion-parameter file a matter of seconds. --output-type sets the type
of token_embd / output (llama.cpp's Q4_0 files keep them in Q6_K). Norm gains are 1 (F32). The
vocabulary is a placeholder list of the right length; token ids are fed to the engine directly.
"""
import argparse

import numpy as np

BLOCK = {"Q8_0": (32, 34), "Q4_0": (32, 18), "Q4_1": (32, 20), "Q6_K": (256, 210)}


def random_quant_matrix(rng, qtype, n_out, n_in, std=0.02):
    """uint8 [n_out, n_in / block * block_bytes] in the GGUF block layout of `qtype`."""
    elems, nbytes = BLOCK[qtype]
    nb = n_in // elems
    raw = rng.integers(0, 256, size=(n_out, nb, nbytes), dtype=np.uint8)
    jitter = (0.75 + 0.5 * rng.random((n_out, nb), dtype=np.float32))  # scales differ from block to block

    def put_f16(col, values):
        raw[:, :, col:col + 2] = values.astype(np.float16).view(np.uint8).reshape(n_out, nb, 2)

    # Quants are drawn from ranges that are symmetric about zero after decoding, so that the weights have zero mean
    # (a common offset in every weight would make the random model emit one token regardless of its input).
    if qtype == "Q8_0":      # d * q, q uniform in [-127, 127]: std 73.3 d
        raw[:, :, 2:34] = rng.integers(-127, 128, size=(n_out, nb, 32), dtype=np.int8).view(np.uint8)
        put_f16(0, std / 73.3 * jitter)
    elif qtype == "Q4_0":    # d * (nibble - 8), nibbles uniform in [1, 15]: std 4.32 d
        nib = rng.integers(1, 16, size=(n_out, nb, 32), dtype=np.uint8)
        raw[:, :, 2:18] = nib[:, :, :16] | (nib[:, :, 16:] << 4)
        put_f16(0, std / 4.32 * jitter)
    elif qtype == "Q4_1":    # d * nibble + m with m = -7.5 d: uniform in [-7.5 d, 7.5 d], std 4.61 d
        d = (std / 4.61 * jitter).astype(np.float16).astype(np.float32)
        put_f16(0, d)
        put_f16(2, -7.5 * d)
    else:                    # Q6_K: d * scale * (q6 - 32), q6 uniform in [1, 63]: std 18.2; scales of either sign
        q6 = rng.integers(1, 64, size=(n_out, nb, 256), dtype=np.uint8).reshape(n_out, nb, 2, 4, 32)  # [half][k][l]
        lo4, hi2 = q6 & 0xF, q6 >> 4
        ql = np.empty((n_out, nb, 2, 2, 32), dtype=np.uint8)   # [half][which 32 of the half's 64 bytes][l]
        ql[:, :, :, 0] = lo4[:, :, :, 0] | (lo4[:, :, :, 2] << 4)
        ql[:, :, :, 1] = lo4[:, :, :, 1] | (lo4[:, :, :, 3] << 4)
        qh = hi2[:, :, :, 0] | (hi2[:, :, :, 1] << 2) | (hi2[:, :, :, 2] << 4) | (hi2[:, :, :, 3] << 6)  # [half][l]
        raw[:, :, 0:128] = ql.reshape(n_out, nb, 128)
        raw[:, :, 128:192] = qh.reshape(n_out, nb, 64)
        sc = rng.integers(16, 64, size=(n_out, nb, 16), dtype=np.int8) * rng.choice(np.array([-1, 1], dtype=np.int8), size=(n_out, nb, 16))
        raw[:, :, 192:208] = sc.view(np.uint8)
        put_f16(208, std / (18.2 * 42.0) * jitter)
    return raw.reshape(n_out, nb * nbytes)


def write(path, n_layer=28, n_vocab=128256, seed=0, n_embd=3072, n_head=24, n_head_kv=8, n_ff=8192, n_ctx=8192,
          wtype="F16", output_type=None):
    import gguf
    rng = np.random.default_rng(seed)
    output_type = output_type or wtype
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

    def mat(name, n_in, n_out, t=None):
        t = t or wtype
        if t == "F16":
            a = (rng.standard_normal((n_out, n_in), dtype=np.float32) * np.float32(0.02)).astype(np.float16)
            w.add_tensor(name, a)
        else:
            w.add_tensor(name, random_quant_matrix(rng, t, n_out, n_in), raw_dtype=getattr(gguf.GGMLQuantizationType, t))

    mat("token_embd.weight", n_embd, n_vocab, output_type)
    w.add_tensor("output_norm.weight", np.ones(n_embd, dtype=np.float32))
    mat("output.weight", n_embd, n_vocab, output_type)
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
    ap.add_argument("--type", default="F16", choices=["F16", "Q8_0", "Q4_0", "Q4_1", "Q6_K"])
    ap.add_argument("--output-type", default=None, choices=["F16", "Q8_0", "Q4_0", "Q4_1", "Q6_K"])
    a = ap.parse_args()
    write(a.out, a.layers, a.vocab, a.seed, wtype=a.type, output_type=a.output_type)
