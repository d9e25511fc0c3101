/* ingot_cuda.h — C ABI of the B200 (sm_100a) attention path for the Ingot inference engine.
 *
 * The library replaces, for a Backend implementation, the per-layer attention stage that sits
 * between the Q/K/V projections and the output projection of Ingot's forward pass:
 *     rope(q), rope(k) -> KV-cache append -> causal GQA attention
 * (CPU reference: src/cpu_backend.cpp:43-69; Metal reference: src/metal_backend.mm:443-445).
 *
 * Conventions
 *   - Every entry point returns an int status (INGOT_OK == 0); nothing throws or aborts.
 *   - Pointers named *_dev are device pointers on the device the cache was created on; pointers
 *     named *_host are host pointers. `stream` is a cudaStream_t passed as void* (NULL = default
 *     stream). Calls are asynchronous on `stream` unless stated otherwise.
 *   - head_dim is 128 (the reference's flash kernels are specialised the same way,
 *     src/metal_backend.mm:340,361). Query heads are grouped onto KV heads as h / (n_head / n_head_kv)
 *     (src/cpu_backend.cpp:29,53).
 *   - Query / output activations are row-major [token][head][128].
 *   - The KV cache is f16 (as the Metal reference's, src/metal_backend.mm:197-198). Layouts:
 *       contiguous: K and V each [n_layer][n_head_kv][n_ctx][128]            (one sequence)
 *       paged:      K and V each [n_layer][n_blocks][n_head_kv][16][128]     (16-token blocks,
 *                   any number of sequences, each described by a row of a block table)
 *   - The cache is a pure function of (layer, position): positions may be rewritten in any order
 *     and the caller owns the notion of sequence length (src/main.cpp:295,374-375 rewind `pos`
 *     without telling the backend).
 *   - Scratch. The decode, prefill and host-buffer calls keep scratch on the handle, sized on first use and
 *     grown when a later call needs more (nothing is ever freed before ingot_kv_destroy). Growing
 *     allocates device memory, which is not allowed while a stream is being captured: run a call once
 *     eagerly with the largest shape before capturing it into a CUDA graph. Graphs captured earlier stay
 *     valid across a later growth.
 *   - A handle belongs to the device that was current at ingot_kv_create; calls with another device
 *     current are rejected with INGOT_ERR_INVALID.
 */
#ifndef INGOT_CUDA_H
#define INGOT_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    INGOT_OK = 0,
    INGOT_ERR_INVALID = 1,      /* bad argument (null pointer, range, unsupported shape) */
    INGOT_ERR_CUDA = 2,         /* a CUDA runtime/driver call failed; see ingot_last_error() */
    INGOT_ERR_UNSUPPORTED = 3,  /* shape or dtype outside what the kernels are built for */
    INGOT_ERR_NOMEM = 4,
    INGOT_ERR_DEVICE = 5        /* a kernel reported a problem through its status word */
};

enum { INGOT_F32 = 0, INGOT_F16 = 1, INGOT_BF16 = 2 };
enum { INGOT_KV_CONTIGUOUS = 0, INGOT_KV_PAGED = 1 };
#define INGOT_BLOCK_TOKENS 16
#define INGOT_HEAD_DIM 128

typedef struct ingot_kv ingot_kv;

/* Human-readable text for a status code / for the last failure on the calling thread. */
const char* ingot_status_string(int status);
const char* ingot_last_error(void);
/* Library build: compiled architecture string, e.g. "sm_100a". */
const char* ingot_build_arch(void);
/* Build variant: "" for the production library, "bounds-check" for the build whose kernels range-check every
 * offset they compute (see ingot_kv_test_shrink_extent). */
const char* ingot_build_flags(void);

/* ---- KV cache ------------------------------------------------------------------------------
 * Replaces the cache the reference backends own (src/backend.h:1; CPU: src/cpu_backend.h:23,
 * src/cpu_backend.cpp:18-19; Metal: src/metal_backend.mm:197-198).
 * capacity = n_ctx positions (contiguous) or number of 16-token blocks (paged).
 * max_seqs = most sequences one decode call will carry (sizes the split-KV scratch); 1 for a
 * single-sequence backend. Allocates on the current device. Synchronous. */
int ingot_kv_create(ingot_kv** out, int layout, int n_layer, int n_head_kv, int head_dim, int capacity,
                    int max_seqs);
void ingot_kv_destroy(ingot_kv* kv);
/* Device base pointers of one layer's K / V storage (layouts above), e.g. to import a cache. */
void* ingot_kv_k_dev(ingot_kv* kv, int layer);
void* ingot_kv_v_dev(ingot_kv* kv, int layer);
size_t ingot_kv_layer_bytes(const ingot_kv* kv);
/* Reads and clears the device status word (0 = no kernel reported a problem). Synchronises `stream`. */
int ingot_kv_status(ingot_kv* kv, void* stream, int* status_out);
/* TEST HOOK (no reference counterpart): with stall_ms > 0 the tcgen05 prefill kernel launched for this handle
 * issues no K/V copies and bounds its waits at stall_ms milliseconds, so that every wait runs out, the kernel
 * returns normally and status bit 4 is raised; 0 restores normal operation. Lets a test exercise the
 * bounded-wait exit without hanging or faulting anything. */
int ingot_kv_test_stall_prefill(ingot_kv* kv, int stall_ms);
/* TEST HOOK of the bounds-check build (no reference counterpart; no effect in the production library): the
 * kernels' range checks treat each cache layer as only `elems` f16 elements long (0 restores the real extent).
 * Accesses beyond that - which are inside the real allocation - are then skipped and raise status bit 8, which
 * shows that the checks are live without any access ever leaving a buffer. */
int ingot_kv_test_shrink_extent(ingot_kv* kv, size_t elems);

/* ---- K1: fused RoPE + K/V append -------------------------------------------------------------
 * Replaces ops::rope on q and k plus the cache memcpy (src/ops.cpp:243-255,
 * src/cpu_backend.cpp:43-49); on Metal: rope + rope_k_to_cache + to_half
 * (shaders/kernels.metal:256-282,779-782; src/metal_backend.mm:324-334,395-409).
 * For each token t in [0, n_tok): position p = positions_dev ? positions_dev[t] : pos0 + t.
 *   q_dev  [n_tok][n_head][128]   f32, may be NULL (no query work);  rotated q is written as f16
 *          to q_out_dev [n_tok][n_head][128].
 *   k_dev, v_dev [n_tok][n_head_kv][128] f32; rotated k and raw v are written as f16 into the cache
 *          at position p.
 *   inv_freq_dev [64] f32: Model::rope_inv_freq (src/model.cpp:59-69). Rotation is on adjacent
 *          pairs (x[2i], x[2i+1]) by angle float(p) * inv_freq[i], in f32.
 * Paged caches: token t belongs to sequence s = seq_ids_dev ? seq_ids_dev[t] : 0 and its block is
 * block_tables_dev[s * max_blocks_per_seq + p / 16]. Contiguous caches ignore those arguments. */
int ingot_rope_kv_append(ingot_kv* kv, int layer, const float* q_dev, void* q_out_dev, const float* k_dev,
                         const float* v_dev, const float* inv_freq_dev, int n_head, int pos0, int n_tok,
                         const int32_t* positions_dev, const int32_t* seq_ids_dev,
                         const int32_t* block_tables_dev, int max_blocks_per_seq, void* stream);

/* Import of already-rotated f16 K/V rows [n_tok][n_head_kv][128] into the cache at positions
 * pos0..pos0+n_tok-1 of one sequence (block_table_dev: that sequence's row, paged only).
 * No reference counterpart on the CPU path (its cache is f32); mirrors the layout transform of
 * the Metal KV store (src/metal_backend.mm:395-409) without the arithmetic. */
int ingot_kv_import_f16(ingot_kv* kv, int layer, const void* k_f16_dev, const void* v_f16_dev, int pos0,
                        int n_tok, const int32_t* block_table_dev, void* stream);

/* ---- K3: split-KV flash decoding -------------------------------------------------------------
 * Replaces the attention lambda for one-token queries (src/cpu_backend.cpp:51-69) and Metal's
 * attn_decode_g3 + attn_combine (shaders/kernels.metal:428-516; src/metal_backend.mm:340-360).
 * n_seq sequences, one query token each:
 *   q_dev   [n_seq][n_head][128]  q_dtype in {F32, F16, BF16}, already rotated
 *   out_dev [n_seq][n_head][128]  out_dtype in {F32, F16}
 *   seq_lens_dev [n_seq] int32: keys 0..len-1 of each sequence are attended (len >= 1).
 *          NULL with n_seq == 1 means the single length max_seq_len.
 *   max_seq_len: host-side upper bound of every length (sizes the launch grid).
 *   block_tables_dev [n_seq][max_blocks_per_seq]: paged caches only.
 * chunk_keys: keys per split (multiple of 16), or 0 to let the library choose. */
int ingot_attn_decode(ingot_kv* kv, int layer, const void* q_dev, int q_dtype, void* out_dev, int out_dtype,
                      int n_head, int n_seq, const int32_t* seq_lens_dev, int max_seq_len,
                      const int32_t* block_tables_dev, int max_blocks_per_seq, int chunk_keys, void* stream);

/* The same for `layer_count` consecutive layers in one call, with the same lengths and block tables:
 * q_dev [layer_count][n_seq][n_head][128], out_dev likewise. This is the shape of the reference's
 * decode-attention microbenchmark, which encodes every layer's attention for one token into one
 * command buffer (src/metal_backend.mm:594-649, src/main.cpp:441-449). The layers are independent, so the
 * split CTAs of all of them form ONE grid (no launch boundary between layers) and a second launch merges the
 * split partials; ingot_attn_decode is the same with layer_count 1. */
int ingot_attn_decode_layers(ingot_kv* kv, int layer_begin, int layer_count, const void* q_dev, int q_dtype,
                             void* out_dev, int out_dtype, int n_head, int n_seq, const int32_t* seq_lens_dev,
                             int max_seq_len, const int32_t* block_tables_dev, int max_blocks_per_seq,
                             int chunk_keys, void* stream);

/* Decode for callers that cannot allocate device memory (no counterpart in the reference).
 * Meant for code that lives inside somebody else's memory budget: a plugin that is only ever handed
 * pre-allocated buffers, a component of a serving loop where cudaMalloc/cudaFree are banned because
 * they synchronise the device, or a process whose allocator is a fixed pool. This entry point takes
 * raw device pointers, needs no ingot_kv handle, and calls no cudaMalloc, cudaFree or allocating
 * library routine: the split-KV partials go to a fixed 2.06 MiB array that is part of the library
 * image (each GPU that loads the library holds it until the process exits).
 *   k_dev, v_dev  one layer of a contiguous f16 cache, [n_head_kv][n_ctx][128] (the caller's memory)
 *   q_dev   [n_head][128]  q_dtype in {F32, F16, BF16}, already rotated;  out_dev [n_head][128] F32 or F16
 *   n_keys  keys 0..n_keys-1 are attended (1 <= n_keys <= n_ctx); one sequence per call
 * Limits: n_head <= 64 and n_head / n_head_kv <= 8; larger calls are rejected with INGOT_ERR_INVALID
 * (use ingot_attn_decode). The first call on each device resolves the array's device address; make
 * that call before starting any stream capture. All calls on a device share the one array and it keeps
 * the previous call's contents (nothing in it needs clearing: every partial a call reads was written by
 * that same call), so two calls whose kernels can overlap on the GPU — different streams without an
 * ordering between them — race; keep them in one stream or order them with events. */
int ingot_attn_decode_noalloc(const void* k_dev, const void* v_dev, int n_ctx, int n_head_kv, const void* q_dev,
                              int q_dtype, void* out_dev, int out_dtype, int n_head, int n_keys, int chunk_keys,
                              void* stream);

/* ---- K2: causal GQA flash-attention prefill / chunked prefill -----------------------------------
 * Replaces n_tok iterations of the attention lambda (src/backend.h:16-20 + src/cpu_backend.cpp:51-69)
 * and Metal's attn_prefill (shaders/kernels.metal:518-633; src/metal_backend.mm:361-372).
 * Query token i (0 <= i < n_tok) sits at position q_pos0 + i and attends to keys 0..q_pos0+i, which
 * must already be in the cache (append first).
 *   q_dev   [n_tok][n_head][128]  q_dtype in {F32, F16, BF16}, already rotated
 *   out_dev [n_tok][n_head][128]  out_dtype in {F32, F16}
 *   block_table_dev: the sequence's block-table row (paged caches), else NULL.
 * impl: 0 = library's choice, 1 = force the warp-MMA kernel, 2 = force the tcgen05/TMEM/TMA kernel. */
int ingot_attn_prefill(ingot_kv* kv, int layer, const void* q_dev, int q_dtype, void* out_dev, int out_dtype,
                       int n_head, int q_pos0, int n_tok, const int32_t* block_table_dev, int impl,
                       void* stream);

/* K2 with the gather of head outputs fused into its epilogue, for a prefill sharded by KV head over
 * the GPUs of one NVLink/NVSwitch box (no counterpart in the reference, which is single-device; it
 * replaces "attn_prefill, then an all-gather of the head outputs"). This GPU's cache holds n_head_kv / N
 * KV heads and q_dev its n_head query heads [n_tok][n_head][128]. Every output row is written, by
 * plain stores from the kernel's epilogue, to each of the n_out (<= 8) buffers in out_ptrs — this GPU's
 * own and its peers' (peer-mapped device pointers, e.g. from symmetric memory) — in the token-major
 * layout [n_tok][out_n_head][128] at head index out_head0 + local head. When every rank has run it
 * and the ranks have synchronised (a barrier on the stream), each buffer holds all heads. tcgen05
 * kernel, contiguous caches only. out_ptrs is a host array read during the call. */
int ingot_attn_prefill_gather(ingot_kv* kv, int layer, const void* q_dev, int q_dtype, void* const* out_ptrs, int n_out,
                              int out_dtype, int n_head, int out_n_head, int out_head0, int q_pos0, int n_tok,
                              void* stream);

/* The same with completion signalling, so that no collective is needed as the cross-GPU barrier. Each GPU owns an
 * array of 32-bit counters, zero-initialised, one per source GPU, mapped into every peer (symmetric memory).
 * signal_ptrs[i] is the counter array that lives beside out_ptrs[i]; src_index is this GPU's slot in those arrays.
 * When the last CTA of this call's grid has finished - all stores to all destinations issued and fenced at
 * system scope - it adds 1 to counter src_index of every destination (red.release.sys). The consumer side is
 * ingot_gather_wait on the destination GPU: a one-CTA kernel on `stream` that waits until each of its n_src
 * counters is non-zero, takes the signal back off (so the counters need no reset between calls) and returns;
 * work queued behind it on the stream then sees every source's rows. The wait is bounded by timeout_ms: a source
 * that never signals raises status bit 4 (read it with ingot_kv_status) instead of hanging the GPU.
 * The destination buffers of call n+1 must not be reused before the consumers of call n are done with them
 * (alternate two buffers, or order the calls otherwise): the signal only says "written", not "read".
 * No counterpart in the reference. tcgen05 kernel, contiguous caches only. */
int ingot_attn_prefill_gather_signal(ingot_kv* kv, int layer, const void* q_dev, int q_dtype, void* const* out_ptrs,
                                     void* const* signal_ptrs, int n_out, int src_index, int out_dtype, int n_head,
                                     int out_n_head, int out_head0, int q_pos0, int n_tok, void* stream);
int ingot_gather_wait(ingot_kv* kv, void* counters_dev, int n_src, int timeout_ms, void* stream);

/* ---- Several GPUs from one process (no counterpart in the reference, which is single-device) ---------------
 * A handle that shards a long prefill by KV head over the first n_dev GPUs of this machine: it enables peer
 * access, creates on every GPU a cache shard with n_head_kv / n_dev heads (ingot_mg_kv(dev): fill it with
 * ingot_rope_kv_append / ingot_kv_import_f16 with that device current, that GPU's heads only), a token-major
 * destination buffer [n_ctx][n_head][128] (ingot_mg_out(dev)) and a counter array, and a stream (ingot_mg_stream).
 * ingot_mg_prefill runs ingot_attn_prefill_gather_signal on every GPU (q_dev[d]: GPU d's query heads
 * [n_tok][n_head / n_dev][128], on GPU d) and the bounded ingot_gather_wait behind it, synchronises, and returns
 * INGOT_OK when every GPU's buffer holds all heads of rows q_pos0..q_pos0+n_tok-1 (stored from row 0 of the buffer),
 * or INGOT_ERR_DEVICE if a wait for a peer ran out after timeout_ms. Needs peer access between all pairs. */
typedef struct ingot_mg ingot_mg;
int ingot_mg_create(ingot_mg** out, int n_dev, int n_layer, int n_head, int n_head_kv, int n_ctx, int out_dtype);
void ingot_mg_destroy(ingot_mg* mg);
ingot_kv* ingot_mg_kv(ingot_mg* mg, int dev);
void* ingot_mg_out(ingot_mg* mg, int dev);
void* ingot_mg_stream(ingot_mg* mg, int dev);
int ingot_mg_prefill(ingot_mg* mg, int layer, const void* const* q_dev, int q_dtype, int q_pos0, int n_tok, int timeout_ms);
/* One token of the one sequence of a CONTIGUOUS cache, K1 and K3 in one launch: q_dev [n_head][128], k_dev and v_dev
 * [n_head_kv][128] are the f32 projections of the token at position `pos`; the kernel rotates q and k
 * (src/ops.cpp:243-255), writes the K/V row of that position to the cache and attends over keys 0..pos
 * (src/cpu_backend.cpp:43-69 for one token), out_dev [n_head][128] f32 or f16. Bit-identical to ingot_rope_kv_append
 * followed by ingot_attn_decode. key_count_dev: null, or a device int32 holding pos + 1 (then `pos` is ignored and
 * max_seq_len bounds it, for CUDA graphs that are replayed at growing positions). */
int ingot_rope_append_decode(ingot_kv* kv, int layer, const float* q_dev, const float* k_dev, const float* v_dev,
                             const float* inv_freq_dev, void* out_dev, int out_dtype, int n_head, const int32_t* key_count_dev,
                             int pos, int max_seq_len, void* stream);

/* Prefill attention with the queries and the output in HOST memory and the cache resident on the device (the keys of
 * positions 0 .. q_pos0+n_tok-1 are in the cache already, e.g. after ingot_rope_kv_append or ingot_kv_import_f16):
 * q_host [n_tok][n_head][128] (f32, f16 or bf16) in, out_host [n_tok][n_head][128] (f32 or f16) out. The rows are
 * processed in chunks of chunk_tokens tokens (0: three full waves of CTAs, 4693 tokens at 24/8 heads) so that the copy of the next chunk in, the attention of the
 * current one and the copy of the previous one out overlap (copy streams of the handle's own; the caller's stream
 * carries the kernels and, at the end, waits for the last copy out). Asynchronous: synchronise `stream` before
 * reading out_host. Host buffers should be pinned. Not capturable into a CUDA graph. block_table_dev as for
 * ingot_attn_prefill. Replaces: a host-side loop over src/cpu_backend.cpp:51-69 for a block of tokens whose q rows
 * live in host memory. */
int ingot_attn_prefill_host(ingot_kv* kv, int layer, const void* q_host, int q_dtype, void* out_host, int out_dtype,
                            int n_head, int q_pos0, int n_tok, const int32_t* block_table_dev, int chunk_tokens,
                            void* stream);

/* Length-balanced assignment of n_seq sequences (key counts lens[]) to n_ranks GPUs for the sequence-sharded
 * batched decode: longest first, each to the least loaded rank (ties to the lower rank). rank_of_seq[i] receives
 * the rank of sequence i. Pure host code. */
int ingot_lpt_assign(const int32_t* lens, int n_seq, int n_ranks, int32_t* rank_of_seq);

/* ---- Host-buffer convenience call ---------------------------------------------------------------
 * One layer of the reference's attention stage with HOST inputs/outputs, as a CPU-side caller sees
 * it (q,k,v from the projections in; attention output for the wo projection out):
 * copies q/k/v f32 rows host->device, runs K1 then K3 (n_tok == 1) or K2 (n_tok > 1) on a contiguous
 * cache at positions pos0..pos0+n_tok-1, copies the f32 output device->host. All on `stream`,
 * asynchronous: call ingot_stream_sync (or cudaStreamSynchronize) before reading out_host.
 * Host buffers should be pinned for the copies to overlap. inv_freq_dev is a device pointer. */
int ingot_attn_layer_host(ingot_kv* kv, int layer, const float* q_host, const float* k_host, const float* v_host,
                          float* out_host, const float* inv_freq_dev, int n_head, int pos0, int n_tok,
                          void* stream);
/* The same for `layer_count` consecutive layers starting at `layer_begin` in one call, as the
 * reference's attention microbenchmark drives its backend (every layer's attention for one step,
 * src/metal_backend.mm:594-649): host arrays are [layer_count][n_tok][heads][128], one slice per layer.
 * If k_host directly follows q_host and v_host directly follows k_host in memory, the three arrays travel in one copy. */
int ingot_attn_layers_host(ingot_kv* kv, int layer_begin, int layer_count, const float* q_host, const float* k_host,
                           const float* v_host, float* out_host, const float* inv_freq_dev, int n_head, int pos0,
                           int n_tok, void* stream);
int ingot_stream_sync(void* stream);

/* ---- Diagnostics ----------------------------------------------------------------------------------
 * HBM read-bandwidth probe: what the reference's `bwtest` verb measures (src/main.cpp:450-455,
 * MetalBackend::bandwidth_test src/metal_backend.mm:533-592 with the bw_fill / bw_sum kernels,
 * shaders/kernels.metal:949-991). Allocates `bytes` on the current device, fills them, then times a kernel
 * that only reads them with 16-byte streaming loads, `reps` times; *best_seconds receives the fastest pass
 * (bandwidth = bytes / *best_seconds). Synchronous. Sizes beyond the L2 (126 MB) measure HBM. */
int ingot_hbm_read_probe(size_t bytes, int reps, double* best_seconds, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* INGOT_CUDA_H */
