/*
 * kiln_cuda.h — C ABI of libkiln_cuda.so: the sm_100a replacement for the
 * kiln-mlx device layer on kiln's speculative-decoding verify path.
 *
 * What this boundary replaces in the reference (paths inside ikematta/kiln):
 *   - crates/kiln-engine/src/step.rs:85-96      trait StepModel::forward_step
 *   - crates/kiln-engine/src/paged.rs:90-386    PagedKv (pools, write, copy_block,
 *                                               read_block_bytes / write_block_bytes)
 *   - crates/kiln-engine/src/engine.rs:879-901  sample_from_row (greedy lane)
 *   - crates/kiln-engine/src/engine.rs:2336-2383 the verify settle walk
 *   - crates/kiln-mlx/src/lib.rs:16-57          init / error / leak-counter surface
 *
 * Conventions kept from kiln-mlx (crates/kiln-mlx/src/error.rs:1-16, 54-72;
 * crates/kiln-mlx/src/debug.rs): every fallible call returns a status and
 * records a thread-local message; nothing here calls exit() or abort(); every
 * *_create / *_load has exactly one *_destroy / *_free and a process-wide live
 * object counter is exported. All device work of one kc_ctx must come from one
 * host thread (crates/kiln-mlx/src/stream.rs:1-19); kc_live_objects and
 * kc_last_error may be called from any thread.
 *
 * Plain C: pointers and sizes only. No torch, no C++ types.
 */
#ifndef KILN_CUDA_H
#define KILN_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KC_API __attribute__((visibility("default")))

/* ---- status codes ------------------------------------------------------ */
enum {
  KC_OK = 0,
  KC_ERR_INVALID = 1,     /* rejected argument / malformed step batch            */
  KC_ERR_CUDA = 2,        /* a CUDA runtime or driver call failed                */
  KC_ERR_OOM = 3,         /* device allocation failed                            */
  KC_ERR_UNSUPPORTED = 4, /* geometry outside what the kernels are built for     */
  KC_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up (status word set)*/
  KC_ERR_CAPACITY = 6     /* block pool exhausted (host scheduler)               */
};

/* Element dtype tags. Numbers follow the reference's stable on-disk tags
 * (crates/kiln-engine/src/engine.rs:2706-2717). */
enum {
  KC_BOOL = 1, KC_U8 = 2, KC_U16 = 3, KC_U32 = 4, KC_I32 = 5,
  KC_F16 = 6, KC_BF16 = 7, KC_F32 = 8
};

/* Architectures of the shared trunk (crates/kiln-models/src/{llama,qwen2,gemma2}.rs). */
enum { KC_ARCH_LLAMA = 0, KC_ARCH_QWEN2 = 1, KC_ARCH_GEMMA2 = 2 };

/* rope_scaling kinds (crates/kiln-models/src/nn.rs:1409-1477). */
enum { KC_ROPE_DEFAULT = 0, KC_ROPE_LINEAR = 1, KC_ROPE_LLAMA3 = 2 };

typedef struct kc_ctx* kc_ctx_t;
typedef struct kc_model* kc_model_t;
typedef struct kc_kv* kc_kv_t;

/* ---- process / context (replaces kiln_mlx::init, Stream::gpu) ----------- */

/* Creates a context bound to CUDA device `device` with its own stream.
 * Replaces kiln_mlx::init + Stream::gpu (crates/kiln-mlx/src/stream.rs:30-43). */
KC_API int kc_ctx_create(int device, kc_ctx_t* out);
KC_API void kc_ctx_destroy(kc_ctx_t ctx);

/* Thread-local message of the last failing call on this thread
 * (crates/kiln-mlx/src/error.rs:54-72). Never NULL. */
KC_API const char* kc_last_error(void);

/* Live handles (contexts + models + kv pools): the leak gate of
 * crates/kiln-mlx/src/debug.rs. */
KC_API int64_t kc_live_objects(void);

/* Blocks until all work queued on the context's stream has finished
 * (the `eval` boundary, crates/kiln-engine/src/engine.rs:2302-2310). Returns KC_ERR_TIMEOUT, and clears
 * the device status word, when a kernel of that work gave up a bounded wait: results queued since the
 * previous synchronisation are then not valid. kc_verify_step and kc_draft_chain, which synchronise
 * themselves, report the same way. */
KC_API int kc_sync(kc_ctx_t ctx);

/* The context's CUDA stream as a cudaStream_t, for callers that time with
 * CUDA events or enqueue their own copies. */
KC_API void* kc_ctx_stream(kc_ctx_t ctx);

/* Device status word: 0 when no kernel has recorded a bounded-wait failure
 * since the last call; otherwise a code naming the kernel and the wait that
 * gave up. Reading clears it. */
KC_API int kc_device_status(kc_ctx_t ctx, uint32_t* status);

/* Kernel launches issued through this context since it was created (every kernel of this library
 * is counted where it is launched). No counterpart in the reference. */
KC_API int64_t kc_launch_count(kc_ctx_t ctx);

/* Device time of the most recent kc_verify_step on this context, in milliseconds: CUDA events on the
 * context's stream, from just before the step's metadata copy is queued (after the host has packed it)
 * to just after its result copy. */
KC_API double kc_last_step_ms(kc_ctx_t ctx);

/* Optional per-class device timing: while enabled, every launch is bracketed by CUDA events on the
 * context's stream. kc_profile_read synchronises, returns milliseconds and launch counts per class
 * since the previous read, and clears them. Classes: 0 quantised GEMM, 1 split-K reduction,
 * 2 paged attention (partial + combine), 3 row-wise ops (embed, norms, rope + KV write, GLU,
 * softcap, block copy), 4 sampling (greedy rows, acceptance walk). ms_out / launches_out: 5 entries.
 * The reference's counterpart is its in-line timers (crates/kiln-engine/src/engine.rs:2377-2379). */
KC_API int kc_profile_enable(kc_ctx_t ctx, int32_t on);
KC_API int kc_profile_read(kc_ctx_t ctx, double* ms_out, int64_t* launches_out);

/* ---- model ------------------------------------------------------------- */

/* Geometry and switches; field meaning follows mlx-lm config.json as parsed by
 * crates/kiln-models/src/config.rs. */
typedef struct {
  int32_t arch;              /* KC_ARCH_*                                        */
  int32_t hidden_size;
  int32_t num_layers;
  int32_t num_heads;
  int32_t num_kv_heads;
  int32_t head_dim;
  int32_t intermediate_size;
  int32_t vocab_size;
  int32_t bits;              /* 4 or 8   (config.rs:138-148)                     */
  int32_t group_size;        /* 32, 64 or 128                                    */
  float   rms_norm_eps;
  float   rope_theta;
  int32_t rope_traditional;  /* 0 = split-halves pairing, 1 = interleaved        */
  int32_t rope_scaling;      /* KC_ROPE_*                                        */
  float   rope_factor;
  float   rope_low_freq_factor;
  float   rope_high_freq_factor;
  float   rope_original_max_position;
  int32_t tie_word_embeddings;
  /* Gemma-2 only (crates/kiln-models/src/gemma2.rs:46-95); 0 elsewhere. */
  float   attn_logit_softcapping;
  float   final_logit_softcapping;
  float   query_pre_attn_scalar;
  int32_t sliding_window;    /* 0 = every layer global. >0: even layers attend the
                                last `sliding_window` keys (no reference behaviour:
                                the reference ignores the field, gemma2.rs:12-14)  */
  /* Step envelope the device buffers are sized for. */
  int32_t max_step_tokens;   /* largest n of one forward_step                    */
  int32_t max_step_seqs;     /* largest number of sequences in one step          */
  /* Tensor parallel slice this process holds (1 GPU: rank 0 of 1). */
  int32_t tp_rank;
  int32_t tp_world;
} kc_model_desc;

/* One named tensor in mlx-lm naming (crates/kiln-models/src/nn.rs:1092-1115):
 * "model.embed_tokens.{weight,scales,biases}", "model.layers.N.self_attn.
 * {q,k,v,o}_proj.{weight,scales,biases[,bias]}", "model.layers.N.mlp.
 * {gate,up,down}_proj.*", "model.layers.N.{input,post_attention,pre_feedforward,
 * post_feedforward}_layernorm.weight", "model.norm.weight", "lm_head.*".
 * Quantised weights are mlx affine: u32 [out, in*bits/32], element j of a row in
 * bits [bits*(j%(32/bits)), +bits) of word j/(32/bits); scales/biases bf16
 * [out, in/group]; w = q*scale + bias. */
typedef struct {
  const char* name;
  const void* data;     /* host or device pointer                              */
  int32_t dtype;        /* KC_U32 for packed weights, KC_BF16 otherwise        */
  int32_t ndim;
  int64_t shape[4];
  int32_t on_device;    /* 1 if `data` is a device pointer on the ctx's device */
} kc_tensor_view;

/* Copies (and re-tiles) the tensors to the device; the caller keeps ownership
 * of its memory. Replaces AnyModel::load + CausalLm::load
 * (crates/kiln-models/src/model.rs:36, nn.rs:1081-1139). Missing or unconsumed
 * tensors fail the load like nn.rs:1118-1128. */
KC_API int kc_model_load(kc_ctx_t ctx, const kc_model_desc* desc,
                         const kc_tensor_view* tensors, size_t n_tensors,
                         kc_model_t* out);
KC_API void kc_model_free(kc_model_t model);

/* The speculation envelope as a backend property. Replaces the constants the
 * reference derives from MLX's kernel dispatch: speculative_gamma_bound
 * (crates/kiln-models/src/model.rs:169-253), VERIFY_MAX_KEY_LEN
 * (crates/kiln-engine/src/engine.rs:213) and calibrate_deterministic_width
 * (crates/kiln-models/src/nn.rs:1190-1248). max_key_len = 0 means unbounded. */
KC_API int kc_envelope(kc_model_t model, int32_t* max_gamma, int32_t* max_key_len,
                       int32_t* det_width);

/* Switches the weight-streaming lane on or off for this model: forwards of at most 8 rows (a draft model's chained
 * decode steps, crates/kiln-models/src/draft.rs:354-388) then read every weight straight from global memory into
 * registers instead of going through the tensor-core pipeline, whose set-up dominates such a step. on = 1: weights of
 * at least 24 MB (8B-class layers, every head) stream, smaller ones take the small-weight kernel of the same arithmetic
 * (kc_quantized_matmul_gemv) where their shape fits it; on = 2: every weight streams; on = 0: off. Off by default,
 * and meant for draft models: a row's bits differ between the two lanes, so a target model whose decode steps
 * (few rows) and verify steps (more than 8 rows) must agree bit for bit keeps it off. Not available on a
 * tensor-parallel slice. */
KC_API int kc_model_set_stream_lane(kc_model_t model, int32_t on);

/* Bytes of quantised weight storage held on the device. */
KC_API int64_t kc_model_weight_bytes(kc_model_t model);

/* ---- paged KV pools (crates/kiln-engine/src/paged.rs) ------------------- */

/* Per-layer K and V pools, each [num_blocks, kv_heads, block_size, head_dim],
 * zero-filled (paged.rs:7-15, 165-172). dtype must be KC_BF16; block_size a
 * power of two in 16..128. */
KC_API int kc_kv_create(kc_ctx_t ctx, int32_t layers, int32_t kv_heads, int32_t head_dim,
                        int32_t num_blocks, int32_t block_size, int32_t dtype, kc_kv_t* out);
KC_API void kc_kv_free(kc_kv_t kv);
/* Copy-on-write: block `src` into `dst` in every layer (paged.rs:230-250). */
KC_API int kc_kv_copy_block(kc_kv_t kv, uint32_t src, uint32_t dst);
/* One block serialised as, per layer, the K rows then the V rows
 * (paged.rs:280-304); n must equal kc_kv_block_bytes. Synchronous. */
KC_API int kc_kv_read_block(kc_kv_t kv, uint32_t block, void* dst, size_t n);
KC_API int kc_kv_write_block(kc_kv_t kv, uint32_t block, const void* src, size_t n);
KC_API int64_t kc_kv_block_bytes(kc_kv_t kv);      /* KvSpec::bytes_per_block, paged.rs:51-58 */
KC_API int64_t kc_kv_allocated_bytes(kc_kv_t kv);  /* paged.rs:358-365 */
/* Zero-fills the pools (engine fault recovery, paged.rs:381-385). */
KC_API int kc_kv_reset(kc_kv_t kv);

/* ---- one forward pass (crates/kiln-engine/src/step.rs:14-75) ------------ */

/* One sequence's contribution to a step: SeqStep without the fields that are a
 * function of the others. `writes` (paged.rs:61-75) is derivable from (offset,
 * len, blocks, block_size) exactly as engine.rs:2757-2769 derives it, and
 * `paged_attn` is an MLX-dispatch artefact. */
typedef struct {
  int32_t len;            /* tokens fed this step                               */
  int32_t offset;         /* tokens already in KV = RoPE offset                 */
  int32_t sample_rows;    /* trailing positions whose logits are returned       */
  int32_t n_blocks;
  const uint32_t* blocks; /* all blocks backing the sequence through this step  */
} kc_seq_step;

/* StepModel::forward_step (step.rs:85-96; CausalLm::forward_step, nn.rs:1303-1388).
 * token_ids: n host u32. Writes this step's post-RoPE K/V into `kv`, returns a
 * device pointer to bf16 logits [n_sampled, vocab] owned by the model and valid
 * until its next call; *logits_dev = NULL and *n_sampled = 0 when no sequence
 * samples. Validation mirrors nn.rs:1309-1337. pad_rows must be 0: the
 * kernel-class padding of ADR 0002 has no purpose on row-invariant kernels.
 * Asynchronous on the context stream. */
KC_API int kc_forward_step(kc_model_t model, kc_kv_t kv, const uint32_t* token_ids, int32_t n,
                           const kc_seq_step* seqs, int32_t n_seqs, int32_t pad_rows,
                           void** logits_dev, int32_t* n_sampled);

/* Greedy token per logits row. normalize=1 is the target lane: argmax over
 * bf16(logit - bf16(logsumexp(row))) with the lowest index winning ties
 * (engine.rs:899-900, sampler.rs:100-104). normalize=0 is the draft lane:
 * argmax of the raw row (crates/kiln-models/src/draft.rs:379-381).
 * tokens_out_dev: device u32 [rows]. */
KC_API int kc_greedy_rows(kc_ctx_t ctx, const void* logits_dev, int32_t rows, int32_t vocab,
                          int32_t normalize, uint32_t* tokens_out_dev);

/* Device form of the settle walk (engine.rs:2336-2383) for n_seqs verify
 * segments. Row tokens of segment i start at seq_row_offsets[i] and number
 * draft_len[i]+1; draft tokens start at draft_offsets[i]. Outputs per segment:
 * n_committed (accepted + 1), n_accepted, and the committed tokens packed at
 * i*max_commit. All pointers are device pointers. The host walk stays
 * authoritative for early finish (engine.rs:2343-2345). */
KC_API int kc_verify_accept(kc_ctx_t ctx, const uint32_t* row_tokens_dev,
                            const int32_t* seq_row_offsets_dev, const uint32_t* draft_dev,
                            const int32_t* draft_offsets_dev, const int32_t* draft_len_dev,
                            int32_t n_seqs, int32_t max_commit, uint32_t* committed_out_dev,
                            int32_t* n_committed_out_dev, int32_t* n_accepted_out_dev);

/* The whole verify round in one call with HOST buffers — forward_step over the
 * batch, target-lane greedy on every sampled row, the settle walk, one
 * device→host copy of the result, one synchronisation. This is what
 * Engine::run_iteration does between "FORWARD" and "SETTLE"
 * (engine.rs:2240-2271, 2302-2310, 2336-2366) for all speculating and plainly
 * decoding sequences of the step at once. draft_len[i] = sample_rows-1 tokens
 * of sequence i's input after its first are its proposal; sequences with
 * sample_rows = 0 (replay / prefill) produce nothing.
 * Host outputs: row_tokens [n_sampled] (greedy token of every sampled row),
 * n_committed [n_seqs], n_accepted [n_seqs]. */
KC_API int kc_verify_step(kc_model_t model, kc_kv_t kv, const uint32_t* token_ids, int32_t n,
                          const kc_seq_step* seqs, int32_t n_seqs,
                          uint32_t* row_tokens_out, int32_t* n_committed_out,
                          int32_t* n_accepted_out);

/* Pipelined plain decode (crates/kiln-engine/src/engine.rs:1428-1455 pipelined_turn, 1656-1744 build_pipelined,
 * 1748-1766 apply_inflight). kc_decode_launch queues ONE decode forward — every segment feeds one row and samples it,
 * greedy over normalised logits as in kc_verify_step — and returns at once with a ticket. feed[i] >= 0 takes
 * sequence i's input id from row feed[i] of the PREVIOUS launch's sampled tokens, which are still on the device
 * (StepInput::Lazy, step.rs:45-56); feed[i] < 0 takes token_ids[i]. kc_decode_collect blocks until the launch with
 * that ticket has finished and copies its n tokens out (Array::item_u32 of the deferred rows); only the two most
 * recent launches can be collected, and a launch that is never collected costs nothing. A bounded wait that gave up
 * in that launch makes collect return KC_ERR_TIMEOUT. The caller must not reuse a block a launch writes to for
 * another sequence except through later calls on the same context, which are ordered behind it on the stream. */
KC_API int kc_decode_launch(kc_model_t model, kc_kv_t kv, const uint32_t* token_ids, const int32_t* feed,
                            const kc_seq_step* seqs, int32_t n_seqs, uint64_t* ticket_out);
KC_API int kc_decode_collect(kc_model_t model, uint64_t ticket, uint32_t* row_tokens_out, int32_t n);

/* The draft lane of DraftModel::propose (draft.rs:354-388): `gamma` chained
 * single-token decode forwards for ONE sequence, each feeding the previous raw
 * argmax without a host round trip. blocks must already cover offset+gamma
 * slots. proposal_out: host u32 [gamma]. Synchronous. */
KC_API int kc_draft_chain(kc_model_t model, kc_kv_t kv, uint32_t first_token, int32_t offset,
                          const uint32_t* blocks, int32_t n_blocks, int32_t gamma,
                          uint32_t* proposal_out);

/* Accounting of the draft lane on this context: wall-clock milliseconds spent inside kc_draft_chain (launches,
 * the device work and the read-back of the proposal), tokens proposed and calls, since the context was created or
 * the last reset. The reference's counterpart is the per-request spec_tokens_proposed counter plus its perf lane
 * (crates/kiln-models/tests/spec_throughput.rs:106-147). */
KC_API int kc_draft_stats(kc_ctx_t ctx, double* ms_out, int64_t* tokens_out, int64_t* calls_out, int32_t reset);

/* ---- single ops, exported for parity tests and for callers composing their
 *      own graphs (the kiln_mlx::ops / fast call sites of nn.rs) ------------ */

/* ops::quantized_matmul(x, w, scales, biases, transpose=true, group, bits)
 * (crates/kiln-mlx/src/ops.rs:362-388; Linear::forward nn.rs:79-102).
 * Handle to one re-tiled quantised weight. */
typedef struct kc_qweight* kc_qweight_t;
KC_API int kc_qweight_create(kc_ctx_t ctx, const uint32_t* w, const void* scales, const void* biases,
                             int32_t out_features, int32_t in_features, int32_t bits,
                             int32_t group_size, int32_t on_device, kc_qweight_t* out);
KC_API void kc_qweight_free(kc_qweight_t w);
/* y[m, out] (bf16, device) = x[m, in] (bf16, device) · dequant(W)ᵀ. */
KC_API int kc_quantized_matmul(kc_ctx_t ctx, kc_qweight_t w, const void* x_dev, int32_t m,
                               void* y_dev);

/* The same product for at most 8 rows through the weight-streaming lane: the kernels a model runs for its decode
 * forwards once kc_model_set_stream_lane switched the lane on. MLX likewise serves small batches with its own
 * row-vector kernels (quantized_matmul dispatches qmv below a row threshold), and this lane computes in their
 * arithmetic class: per group, scale * sum(x q) + bias * sum(x) in fp32, no weight rounded to bf16. As there, the two
 * lanes agree to rounding, not bit for bit. */
KC_API int kc_quantized_matmul_stream(kc_ctx_t ctx, kc_qweight_t w, const void* x_dev, int32_t m,
                                      void* y_dev);

/* The same arithmetic for weights of a few MB (the layers of a 1B-class draft model), where a launch is a chain of
 * latencies rather than a stream: one CTA per (128-row tile, run of k-blocks) asks for all of its records at once,
 * before it waits for the kernel ahead of it, and works through them resident; a tile's k-blocks are cut into at most
 * 8 runs whose fp32 partials are summed in order. A model with the weight-streaming lane on takes this kernel for the
 * weights below the streaming threshold. KC_ERR_UNSUPPORTED when the weight's shape does not fit the lane. */
KC_API int kc_quantized_matmul_gemv(kc_ctx_t ctx, kc_qweight_t w, const void* x_dev, int32_t m,
                                    void* y_dev);

/* kc_quantized_matmul without any allocation behind it. No counterpart in the
 * reference (MLX owns every buffer there); added for callers that cannot let a
 * library allocate: the split-K fp32 partials go to a fixed 16 MiB device array
 * that is part of this library's image instead of a cudaMalloc'ed buffer owned
 * by the weight handle, and the call itself makes no device or pinned-host
 * allocation. Same kernels, same bits as kc_quantized_matmul.
 *  - splits x min(m, 512) x out_features x 4 bytes must fit
 *    kc_static_scratch_bytes(); a larger request fails with KC_ERR_UNSUPPORTED
 *    before anything is launched (weights that are not split along K need no
 *    scratch and always fit).
 *  - The first call on a device looks the array up (this loads the library's
 *    module on that device if nothing has yet) and sets the kernel attributes:
 *    make it before any stream capture starts.
 *  - The array is shared by all contexts and weights on a device and keeps the
 *    last call's partials; calls overlapping in time on one device race on it. */
KC_API int kc_quantized_matmul_static(kc_ctx_t ctx, kc_qweight_t w, const void* x_dev, int32_t m,
                                      void* y_dev);
/* Size of that array in bytes (a compile-time constant of the library). */
KC_API int64_t kc_static_scratch_bytes(void);

/* fast::rms_norm (crates/kiln-mlx/src/fast.rs:36-41): bf16 [rows, dim]. */
KC_API int kc_rms_norm(kc_ctx_t ctx, const void* x_dev, const void* weight_dev, int32_t rows,
                       int32_t dim, float eps, void* y_dev);

/* Paged multi-query attention over the pools for an already-built step: q is
 * bf16 [n, num_heads, head_dim] post-RoPE, this step's K/V already written.
 * Replaces PagedKv::gather + fast::scaled_dot_product_attention
 * (paged.rs:191-225, nn.rs:800-817) and the Metal kernels of
 * crates/kiln-engine/src/paged_attn.rs:59-303. softcap = 0 disables capping;
 * window = 0 is global. out: bf16 [n, num_heads*head_dim]. */
KC_API int kc_paged_attention(kc_ctx_t ctx, kc_kv_t kv, int32_t layer, const void* q_dev,
                              int32_t n, int32_t num_heads, const kc_seq_step* seqs,
                              int32_t n_seqs, float scale, float softcap, int32_t window,
                              void* out_dev);

/* RoPE at per-sequence offsets fused with PagedKv::write (nn.rs:760-769,
 * paged.rs:147-187): qkv bf16 [n, (num_heads+2*kv_heads)*head_dim] →
 * q_out bf16 [n, num_heads, head_dim] and the layer's pool rows. inv_freq:
 * device f32 [head_dim/2]. qkv_bias may be NULL. */
KC_API int kc_rope_kv_write(kc_ctx_t ctx, kc_kv_t kv, int32_t layer, const void* qkv_dev,
                            const void* qkv_bias_dev, const float* inv_freq_dev, int32_t n,
                            int32_t num_heads, int32_t traditional, const kc_seq_step* seqs,
                            int32_t n_seqs, void* q_out_dev);

/* ---- tensor parallel (no counterpart in the reference, which has no
 *      collective of any kind: docs/SPEC.md:70-75) ------------------------ */

/* Joins an NCCL communicator of `world` ranks. After o_proj and down_proj the
 * ranks' bf16 outputs are all-gathered and summed in rank order (fp32, one
 * rounding) by the next kernel. unique_id: the 128 bytes of an ncclUniqueId
 * from rank 0. */
KC_API int kc_tp_init(kc_ctx_t ctx, const void* unique_id, int32_t rank, int32_t world);

/* The tensor-parallel exchange over peer memory instead of NCCL. After kc_model_load on every rank (one process per
 * GPU): kc_tp_export writes this rank's KC_TP_EXPORT_BYTES of inter-process memory handles (its two output buffers
 * and its flag array); the caller brings every rank's bytes to every rank (rank order, world x KC_TP_EXPORT_BYTES)
 * and passes them to kc_tp_attach, which maps the peers' buffers. From then on the model's o_proj / down_proj
 * outputs are not copied at all: a one-warp kernel publishes "exchange e done" into every rank's flag array and the
 * consumer kernel (residual add + RMSNorm) reads every rank's rows where they were written, in rank order — plain
 * peer loads over NVLink, no multicast. The consumer's wait for the flags is bounded like every wait of the library
 * (KC_ERR_TIMEOUT at the next synchronisation if a rank never publishes). From 4 ranks on the exchange takes two
 * phases (each rank first sums its column slice of all ranks' rows, the consumer then gathers the summed slices:
 * fewer bytes over NVLink, the same bits); the environment variable KILN_TP_TWO_PHASE = 0 / 1, read by kc_tp_attach,
 * forces one form. Without these two calls the exchange is an NCCL all-gather. All ranks must run the same sequence
 * of forwards. */
#define KC_TP_EXPORT_BYTES 192
KC_API int kc_tp_export(kc_model_t model, void* handles_out);
KC_API int kc_tp_attach(kc_model_t model, const void* handles_all);
KC_API int kc_tp_unique_id(void* unique_id_out_128);

#ifdef __cplusplus
}
#endif
#endif /* KILN_CUDA_H */
