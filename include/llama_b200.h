/* llama_b200.h — a Llama decode driver on top of the ggml backend plug-in of libggml-b200.so.
 *
 * It plays the part of the reference's DecodeContext for the llama architecture: weights in device
 * buffers (crates/llama/src/context.rs:4511-4560 enable_gpu), one unified F16 KV cache
 * (crates/llama/src/kv_cache.rs:1887-1917), per-step inputs (context.rs:6565-6640 step_inputs_pos_rows),
 * the node list of crates/llama/src/graph_arch.rs:106-248 build_llama_forward with the flash-attention
 * branch of attn_kv_cached (:1173-1240), and graph_compute through the backend vtable
 * (context.rs:4611-4646 run_graph).  Every tensor operation goes through the plug-in face declared in
 * ggml_b200_backend.h — the driver holds no kernels of its own — so it doubles as an executable
 * description of the graphs the backend has to serve.
 */
#ifndef LLAMA_B200_H
#define LLAMA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* crates/llama/src/graph.rs:24-60 AttnParams + the llama.* GGUF keys they come from */
struct b200_llama_hparams {
    int32_t n_vocab;
    int32_t n_embd;
    int32_t n_head;
    int32_t n_head_kv;
    int32_t n_embd_head;      /* key and value head size */
    int32_t n_ff;
    int32_t n_layer;
    int32_t n_ctx_train;      /* rope n_ctx_orig */
    int32_t rope_mode;        /* 0 = NORMAL (llama), 2 = NEOX */
    float norm_rms_eps;
    float rope_freq_base;
    float rope_freq_scale;
};

typedef struct b200_llama b200_llama;

/* All functions return a b200_status (0 = success); b200_last_error() has the message. */

/* device: CUDA device index.  n_ctx: KV cache cells.  n_batch: most tokens one decode call may carry.
 * cpu_threads: the CPU thread count whose attention arithmetic is reproduced (see ggml_b200_backend.h). */
int b200_llama_new(const struct b200_llama_hparams *hp, int device, int32_t n_ctx, int32_t n_batch, int32_t cpu_threads,
                   b200_llama **out);
void b200_llama_free(b200_llama *ctx);

/* ---- tensor parallelism across the GPUs of one node (one process per GPU) ------------------------------
 * The reference has no multi-device path; this is the row-split of BASELINE's 70B configuration: attn_q/k/v,
 * ffn_gate/up and output by rows (whole heads, FFN rows, vocabulary rows), attn_output and ffn_down by K with
 * an all-reduce of the partial sums, norms and token_embd replicated, logits all-gathered.  Collectives of up
 * to 131072 floats per rank (every collective of a decode step) run as one kernel of this library over
 * peer-mapped memory, with the partial sums added in rank order; larger ones (prompt batches) go to NCCL.
 *
 * b200_tp_unique_id: rank 0 fills 128 bytes (an ncclUniqueId) that the host passes to every rank.
 * b200_llama_new_tp: as b200_llama_new, for rank tp_rank of tp_size (n_head_kv, n_ff and n_vocab must divide).
 *   b200_llama_set_tensor then takes the WHOLE tensor on every rank and keeps this rank's shard.
 * b200_tp_shard_shape / b200_tp_shard_tensor: the cut itself, on host memory (split: 0 replicated, 1 rows,
 *   2 K), for hosts that shard while loading and for tests. */
int b200_tp_unique_id(void *id128);
/* A rank whose collectives are carried out by the host instead of by NCCL / peer memory, for tests that play
 * several ranks on one GPU (one thread per rank): the driver calls the hook with its stream drained.
 *   kind 0, all-reduce: dev_buf holds `count` floats, this rank's partial sums; on return it must hold the sum over
 *           the ranks, added in rank order.
 *   kind 1, all-gather: dev_buf holds rows x n_local floats (count of them); dev_dst [rows][n_local * size] must
 *           receive every rank's slice of every row, rank r's at column r * n_local.
 * A non-zero return fails the decode call.  No counterpart in the reference (which has no multi-device path). */
typedef int (*b200_tp_hook_fn)(void *user, int kind, int rank, int size, float *dev_buf, int64_t count, float *dev_dst,
                               int64_t n_local, int64_t rows);
int b200_llama_new_tp_hook(const struct b200_llama_hparams *hp, int device, int32_t n_ctx, int32_t n_batch, int32_t cpu_threads,
                           int32_t tp_rank, int32_t tp_size, b200_tp_hook_fn hook, void *user, b200_llama **out);
/* How the group's small collectives travel: 1 = the library's single-kernel exchange over peer-mapped memory,
 * 0 = NCCL (a rank could not map a peer's buffer, or B200_TP_LL=0), -1 = not a tensor-parallel driver / hook. */
int b200_llama_tp_exchange_kind(const b200_llama *ctx);
int b200_llama_new_tp(const struct b200_llama_hparams *hp, int device, int32_t n_ctx, int32_t n_batch, int32_t cpu_threads,
                      int32_t tp_rank, int32_t tp_size, const void *id128, b200_llama **out);
int b200_tp_shard_shape(const char *name, int type, int64_t ne0, int64_t ne1, int32_t tp_size, int32_t *split, int64_t *ne0_local,
                        int64_t *ne1_local);
int b200_tp_shard_tensor(const char *name, int type, int64_t ne0, int64_t ne1, const void *data, int32_t tp_rank, int32_t tp_size,
                         void *out, size_t out_nbytes);
/* b200_llama_set_tensor for a rank that cut the tensor itself: data is this rank's shard, ne0 / ne1 its local shape. */
int b200_llama_set_tensor_shard(b200_llama *ctx, const char *name, int type, int64_t ne0, int64_t ne1, const void *data, size_t nbytes);

/* A llama-architecture GGUF file straight into a driver (Gguf::open + LlamaHparams::from_gguf + the tensor
 * loop of crates/llama/src/model.rs): reads general.architecture, llama.block_count, embedding_length,
 * feed_forward_length, attention.head_count(_kv), attention.key_length, attention.layer_norm_rms_epsilon,
 * rope.freq_base, context_length, takes n_vocab from token_embd.weight, and sets every tensor.  The _tp form
 * loads rank tp_rank's shards.  b200_llama_get_hparams reports what a driver was built with. */
int b200_llama_load_gguf(const char *path, int device, int32_t n_ctx, int32_t n_batch, int32_t cpu_threads, b200_llama **out);
int b200_llama_load_gguf_tp(const char *path, int device, int32_t n_ctx, int32_t n_batch, int32_t cpu_threads, int32_t tp_rank,
                            int32_t tp_size, const void *id128, b200_llama **out);
int b200_llama_get_hparams(const b200_llama *ctx, struct b200_llama_hparams *out);

/* One model tensor under its GGUF name (crates/llama/src/model.rs: token_embd.weight, output_norm.weight,
 * output.weight, blk.N.{attn_norm,attn_q,attn_k,attn_v,attn_output,ffn_norm,ffn_gate,ffn_up,ffn_down}.weight).
 * data: ggml blocks of `type`, ne1 rows of ne0 elements, in host memory.  output.weight may be left out
 * when the model ties it to token_embd.weight. */
int b200_llama_set_tensor(b200_llama *ctx, const char *name, int type, int64_t ne0, int64_t ne1, const void *data, size_t nbytes);

/* DecodeContext::decode (crates/llama/src/context.rs:4648-4680): n_tokens tokens of one sequence at the
 * given positions are appended to the cache; logits (host, n_vocab floats, may be null) receives the last
 * token's row, argmax (may be null) the index of its largest logit computed on the device
 * (last index among equals, crates/ggml/src/compute.rs:4208-4228). */
int b200_llama_decode(b200_llama *ctx, const int32_t *tokens, const int32_t *pos, int32_t n_tokens, float *logits, int32_t *argmax);

/* The batched form: tokens of several sequences in one step (one token each while generating, or one
 * sequence's prompt).  seq_ids[i] names token i's sequence (null = all 0); the cache is the reference's
 * unified one: every token takes the next free cell, a query sees the cells of its own sequence at positions
 * up to its own (llama-kv-cache's mask rule as ported in crates/llama/src/graph.rs:592-724).  out_rows: the
 * n_out batch rows whose logits are wanted (crates/llama/src/graph.rs:308-313 out_rows); logits receives
 * n_out rows of n_vocab floats, argmax n_out indices. */
int b200_llama_decode_seqs(b200_llama *ctx, const int32_t *tokens, const int32_t *pos, const int32_t *seq_ids, int32_t n_tokens,
                           const int32_t *out_rows, int32_t n_out, float *logits, int32_t *argmax);

/* Forget every cached position (DecodeContext::kv_clear). */
int b200_llama_kv_clear(b200_llama *ctx);
/* Cells in use, and the padded cell count the next step's attention would span. */
int32_t b200_llama_kv_used(const b200_llama *ctx);

/* Reads back a tensor of the last decode call's graph by name (the last one of that name; a layer's
 * intermediates share memory with the next layer's, so only the last layer's survive): "inp_tokens",
 * "attn_norm", "Kcur", "Kcur_rope", "Vcur", "Qcur", "Qcur_rope", "kqv_out", "attn_out", "ffn_inp",
 * "ffn_norm", "ffn_gate", "ffn_up", "ffn_gate_par", "ffn_out", "l_out", "result_norm",
 * "result_output".  For node-by-node comparisons in the manner of the reference's decode dumps
 * (parity/ref_decode_dump.c). */
int b200_llama_read_node(b200_llama *ctx, const char *name, void *out, size_t nbytes);

/* Re-runs the graph of the last decode call `reps` times on the backend's stream with the inputs that
 * are already on the device, timed with events on that stream; *ms receives the total.  For measuring
 * the device-side cost of a step without the input upload and the logits read-back. */
int b200_llama_replay(b200_llama *ctx, int32_t reps, float *ms);

#ifdef __cplusplus
}
#endif
#endif /* LLAMA_B200_H */
