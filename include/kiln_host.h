/*
 * kiln_host.h — C ABI of libkiln_host.so: the host-side scheduler pieces of kiln's
 * speculative-decoding path (no CUDA dependency; the device sits behind function
 * tables, so a fake model can drive every entry point on a CPU-only machine).
 *
 * What each group replaces in the reference (paths inside ikematta/kiln):
 *   kh_bm_* / kh_bt_*      crates/kiln-engine/src/block.rs:88-426   BlockManager, BlockTable
 *   kh_radix_*             crates/kiln-engine/src/radix.rs:92-457   RadixCache
 *   kh_spec_gamma_at_width crates/kiln-engine/src/drafter.rs:62-70
 *   kh_canonical_prefill_len crates/kiln-engine/src/engine.rs:167-179
 *   kh_engine_*            crates/kiln-engine/src/engine.rs:1006-1407, 2035-2417  Engine
 *   kh_scripted_* / kh_draft_model_*  the Drafter trait (drafter.rs:125-147) and
 *                          DraftModel (crates/kiln-models/src/draft.rs:258-412)
 * Every call returns 0 on success; kh_last_error() holds the message otherwise.
 */
#ifndef KILN_HOST_H
#define KILN_HOST_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KH_API __attribute__((visibility("default")))

KH_API const char* kh_last_error(void);

/* BlockError kinds (block.rs:39-64), as return codes of kh_bm_* / kh_bt_*. */
enum {
  KH_OK = 0, KH_OUT_OF_BLOCKS = 1, KH_NOT_ALLOCATED = 2, KH_REFCOUNT_OVERFLOW = 3, KH_INVALID_BLOCK_SIZE = 4,
  KH_INVALID_CAPACITY = 5, KH_TOKEN_COUNT_OVERFLOW = 6, KH_MISALIGNED_ADOPTION = 7, KH_ERR_MODEL = 20, KH_ERR_ARG = 21
};

typedef struct kh_bm* kh_bm_t;
typedef struct kh_bt* kh_bt_t;

/* ---- BlockManager (block.rs:88-203) ---- */
KH_API int kh_bm_create(uint64_t capacity, uint64_t block_size, kh_bm_t* out);
KH_API void kh_bm_free(kh_bm_t bm);
KH_API uint64_t kh_bm_block_size(kh_bm_t bm);
KH_API uint64_t kh_bm_capacity(kh_bm_t bm);
KH_API uint64_t kh_bm_num_free(kh_bm_t bm);
KH_API int64_t kh_bm_refcount(kh_bm_t bm, uint32_t id);              /* -1: id not from this pool */
KH_API int kh_bm_allocate(kh_bm_t bm, uint32_t* id_out);
KH_API int kh_bm_retain(kh_bm_t bm, uint32_t id);
KH_API int kh_bm_release(kh_bm_t bm, uint32_t id);
/* copied_out = 0: sole owner, write in place; 1: ownership moved to *dst_out, copy src's rows first. */
KH_API int kh_bm_copy_on_write(kh_bm_t bm, uint32_t id, int32_t* copied_out, uint32_t* src_out, uint32_t* dst_out);
/* The LIFO free list, top of stack last (the next allocation pops the last entry). */
KH_API uint64_t kh_bm_free_list(kh_bm_t bm, uint32_t* out, uint64_t cap);
/* Fields of the last OutOfBlocks error on this thread: capacity, needed. */
KH_API void kh_last_out_of_blocks(uint64_t* capacity, uint64_t* needed);

/* ---- BlockTable (block.rs:223-426) ---- */
KH_API int kh_bt_create(kh_bt_t* out);
KH_API void kh_bt_free(kh_bt_t bt);                                   /* does NOT release blocks (block.rs:219-222) */
KH_API uint64_t kh_bt_num_tokens(kh_bt_t bt);
KH_API uint64_t kh_bt_blocks(kh_bt_t bt, uint32_t* out, uint64_t cap); /* returns the block count */
/* AppendPlan: has_cow/cow_src/cow_dst and the appended ids (appended_out may be NULL). */
KH_API int kh_bt_append_tokens(kh_bt_t bt, kh_bm_t bm, uint64_t n, int32_t* has_cow, uint32_t* cow_src, uint32_t* cow_dst,
                               uint32_t* appended_out, uint64_t appended_cap, uint64_t* n_appended);
KH_API int kh_bt_push_full_block(kh_bt_t bt, uint32_t id, uint64_t block_size);
KH_API int kh_bt_push_partial_block(kh_bt_t bt, uint32_t id, uint64_t rows, uint64_t block_size);
KH_API int kh_bt_truncate(kh_bt_t bt, kh_bm_t bm, uint64_t keep_tokens);   /* the rollback, block.rs:381-396 */
KH_API int kh_bt_fork(kh_bt_t bt, kh_bm_t bm, kh_bt_t* out);
KH_API int kh_bt_release(kh_bt_t bt, kh_bm_t bm);

/* ---- pure functions ---- */
KH_API uint64_t kh_spec_gamma_at_width(uint64_t gamma, uint64_t spec_max_batch, uint64_t width);
KH_API uint64_t kh_canonical_prefill_len(uint64_t at, uint64_t limit, uint64_t prefill_chunk, uint64_t fine);

/* ---- RadixCache (radix.rs:92-457); node 0 is the root ---- */
typedef struct kh_radix* kh_radix_t;
KH_API int kh_radix_create(uint64_t block_size, const uint8_t seed[32], kh_radix_t* out);
KH_API void kh_radix_free(kh_radix_t r);
KH_API int64_t kh_radix_child(kh_radix_t r, uint64_t node, const uint32_t* chunk, uint64_t n);   /* -1 if absent */
KH_API void kh_radix_chain_hash_of(kh_radix_t r, uint64_t node, const uint32_t* chunk, uint64_t n, uint8_t out[32]);
KH_API void kh_radix_node_hash(kh_radix_t r, uint64_t node, uint8_t out[32]);
KH_API int64_t kh_radix_node_block(kh_radix_t r, uint64_t node);                                 /* -1 if not resident */
KH_API uint64_t kh_radix_node_rows(kh_radix_t r, uint64_t node);
KH_API int32_t kh_radix_node_is_partial(kh_radix_t r, uint64_t node);
KH_API uint64_t kh_radix_node_generation(kh_radix_t r, uint64_t node);
KH_API int32_t kh_radix_is_live(kh_radix_t r, uint64_t node, uint64_t generation);
KH_API uint64_t kh_radix_insert_child(kh_radix_t r, uint64_t parent, const uint32_t* chunk, uint64_t n);
KH_API uint64_t kh_radix_insert_partial_child(kh_radix_t r, uint64_t parent, const uint32_t* tokens, uint64_t n);
KH_API int64_t kh_radix_upgrade_partial(kh_radix_t r, uint64_t node, const uint32_t* tokens, uint64_t n, uint32_t block);
KH_API void kh_radix_set_resident(kh_radix_t r, uint64_t node, uint32_t block);
KH_API void kh_radix_touch(kh_radix_t r, uint64_t node);
/* The cold-tier flag of a node (radix.rs: set_on_ssd / node_on_ssd): an evicted node that has it stays in the tree
 * without a block, so a later walk can find and reload it. The slab files themselves are not part of this library. */
KH_API void kh_radix_set_on_ssd(kh_radix_t r, uint64_t node);
KH_API int32_t kh_radix_node_on_ssd(kh_radix_t r, uint64_t node);
KH_API int64_t kh_radix_evict_candidate(kh_radix_t r, kh_bm_t bm);
KH_API int64_t kh_radix_evict(kh_radix_t r, kh_bm_t bm, uint64_t node);
KH_API void kh_radix_prune_subtree(kh_radix_t r, kh_bm_t bm, uint64_t node);
KH_API uint64_t kh_radix_resident_blocks(kh_radix_t r);
KH_API void kh_radix_reset(kh_radix_t r);

/* ---- the StepModel / Drafter seams ---- */

/* Same layout as kc_seq_step (include/kiln_cuda.h). */
typedef struct {
  int32_t len, offset, sample_rows, n_blocks;
  const uint32_t* blocks;
} kh_seq_step;

/* verify_step has exactly the signature of kc_verify_step; copy_block that of kc_kv_copy_block. */
typedef struct {
  void* model;
  void* kv;
  int (*verify_step)(void* model, void* kv, const uint32_t* ids, int32_t n, const kh_seq_step* seqs, int32_t n_seqs,
                     uint32_t* row_tokens, int32_t* n_committed, int32_t* n_accepted);
  int (*copy_block)(void* kv, uint32_t src, uint32_t dst);
  int32_t vocab;
} kh_step_model;

/* The pipelined plain-decode seam (engine.rs:1428-1475, 1656-1766: pipelined_turn, build_pipelined, apply_inflight).
 * launch queues one decode forward (one sampled row per sequence) without waiting and returns a ticket; feed[i] >= 0
 * takes sequence i's input id from row feed[i] of the previous launch, still on the device (StepInput::Lazy,
 * step.rs:45-56); feed[i] < 0 takes ids[i]. collect blocks until that launch's tokens are on the host. launch has
 * the signature of kc_decode_launch, collect of kc_decode_collect; model and kv are those of the step model. */
typedef struct {
  int (*launch)(void* model, void* kv, const uint32_t* ids, const int32_t* feed, const kh_seq_step* seqs, int32_t n_seqs,
                uint64_t* ticket);
  int (*collect)(void* model, uint64_t ticket, uint32_t* row_tokens, int32_t n);
} kh_decode_pipeline;

/* DrafterMemory (drafter.rs:88-102): summed into the worker's memory report. */
typedef struct { uint64_t weights_bytes, kv_allocated_bytes, kv_used_bytes; } kh_drafter_memory;

/* trait Drafter (drafter.rs:125-147). A non-zero return from begin/propose is a DraftError: never fatal to the request.
 * memory may be NULL (a drafter with no footprint of its own: all zeros). */
typedef struct {
  void* user;
  int (*begin)(void* user, uint64_t seq, const uint32_t* prompt, int32_t n);
  int (*propose)(void* user, uint64_t seq, const uint32_t* committed, int32_t n_committed, int32_t gamma, uint32_t* out,
                 int32_t* n_out);
  void (*release)(void* user, uint64_t seq);
  void (*memory)(void* user, kh_drafter_memory* out);
} kh_drafter;

/* EngineConfig (engine.rs:239-306) plus the envelope the backend provides (kc_envelope). */
typedef struct {
  int32_t block_size, num_blocks, max_batch_tokens, prefill_chunk, prefill_fine_chunk, prefix_cache;
  int32_t deterministic_decode_width, gamma, spec_max_batch;
  double spec_min_acceptance;
  int32_t max_key_len;    /* VERIFY_MAX_KEY_LEN (engine.rs:213) = 1023 in the reference; 0 = unbounded */
  int32_t batch_verify;   /* 1: every segment of an iteration rides one forward (row-invariant backend);
                             0: the reference's grouping (engine.rs:2170-2271) */
} kh_engine_config;

typedef struct {  /* SpecStats (engine.rs:811-830) */
  uint64_t rounds_total, proposed_total, accepted_total, rollback_rounds_total, rollback_tokens_total,
      rollback_nanos_total, draft_errors_total, standdowns_total;
} kh_spec_stats;

typedef struct kh_engine* kh_engine_t;
KH_API void kh_engine_default_config(kh_engine_config* out);   /* EngineConfig::default() */
KH_API int kh_engine_create(const kh_engine_config* cfg, const kh_step_model* model, kh_engine_t* out);
KH_API void kh_engine_free(kh_engine_t e);
KH_API int kh_engine_set_drafter(kh_engine_t e, const kh_drafter* d);
/* Engine::drafter_memory (engine.rs:1128-1132): 1 and the attached drafter's footprint, or 0 (and zeros) when
 * speculation is not configured. */
KH_API int kh_engine_drafter_memory(kh_engine_t e, kh_drafter_memory* out);
/* Without this call the engine never pipelines (every step is read back before the next is built). p = NULL turns
 * pipelining off again; a step already in flight is read back at the next kh_engine_step. */
KH_API int kh_engine_set_pipeline(kh_engine_t e, const kh_decode_pipeline* p);
KH_API uint64_t kh_engine_pipelined_steps(kh_engine_t e);    /* Engine::pipelined_steps (engine.rs:1160-1163) */
/* Engine::submit (engine.rs:1294-1363); greedy requests only. */
KH_API int kh_engine_submit(kh_engine_t e, const uint32_t* prompt, uint64_t n, uint64_t max_tokens, const uint32_t* stop_tokens,
                            uint64_t n_stop, uint64_t* arrival_out);
KH_API int kh_engine_cancel(kh_engine_t e, uint64_t arrival);
KH_API int kh_engine_step(kh_engine_t e);                     /* Engine::step (engine.rs:1367-1407) */
KH_API uint64_t kh_engine_num_running(kh_engine_t e);
KH_API uint64_t kh_engine_num_waiting(kh_engine_t e);
KH_API uint64_t kh_engine_iterations(kh_engine_t e);
KH_API uint64_t kh_engine_forwards(kh_engine_t e);
KH_API const char* kh_engine_last_error(kh_engine_t e);     /* message of the last failed step */
/* Tokens emitted since the last call (SeqEvent::Token), plus the terminal state. finish_kind: 0 running,
 * 1 stop, 2 length, 3 error, 4 cancelled. */
KH_API int kh_engine_take_output(kh_engine_t e, uint64_t arrival, uint32_t* out, uint64_t cap, uint64_t* n_out,
                                 int32_t* finish_kind);
/* Per-request view for parity tests: table blocks, KV tokens, generated count, speculation counters. */
KH_API int kh_engine_seq_state(kh_engine_t e, uint64_t arrival, uint32_t* blocks_out, uint64_t cap, uint64_t* n_blocks,
                               uint64_t* num_tokens, uint64_t* generated, uint32_t* spec_proposed, uint32_t* spec_accepted,
                               int32_t* standdown, uint32_t* cached_tokens);
KH_API void kh_engine_spec_stats(kh_engine_t e, kh_spec_stats* out);
KH_API kh_bm_t kh_engine_block_manager(kh_engine_t e);        /* borrowed; do not free */
KH_API void kh_engine_cache_stats(kh_engine_t e, uint64_t* hits, uint64_t* tokens_reused, uint64_t* resident_blocks);

/* ---- SSD cold tier (crates/kiln-engine/src/ssd.rs; engine hooks engine.rs:601-690, 1412-1426, 1868-2033, 2559-2704) ---- */

typedef struct { uint32_t layers, kv_heads, head_dim, block_size; } kh_slab_geometry;   /* SlabGeometry (ssd.rs:61-66) */
/* Block IO of the pool: read has the signature of kc_kv_read_block, write of kc_kv_write_block (payload per layer: K
 * rows then V rows, paged.rs:280-304). dtype_tag is the stable on-disk tag (engine.rs:2707-2718: 7 = bfloat16). */
typedef struct {
  int (*read)(void* kv, uint32_t block, void* dst, size_t n);
  int (*write)(void* kv, uint32_t block, const void* src, size_t n);
  uint32_t dtype_tag, dtype_size;
} kh_block_io;
typedef struct {  /* SsdCounters (ssd.rs:94-99) + the store's totals + the engine's flush queue and SSD-served prefix hits */
  uint64_t blocks_stored, bytes_stored, reads_total, writes_total, writes_failed_total, fingerprint_rejects_total, flush_queue_depth,
      ssd_hits_total;
} kh_ssd_stats;
typedef struct { uint64_t node, generation; uint8_t hash[32]; int32_t ok; } kh_flush_ack;   /* FlushAck (ssd.rs:135-140) */

/* Attaches the tier to an engine with a prefix cache: blocks donated at finish are written behind the steps
 * (FLUSH_BATCH captures per synchronous or idle step, none during a pipelined turn), evicted blocks stay discoverable,
 * and a new engine over the same directory finds them hash-first on its prefix walks. fingerprint: 32 bytes binding
 * weights, architecture, dtype and block geometry; slabs that fail it are skipped with a counter. */
KH_API int kh_engine_set_ssd(kh_engine_t e, const char* dir, const uint8_t* fingerprint, const kh_slab_geometry* g, uint64_t max_bytes,
                             const kh_block_io* io);
KH_API void kh_engine_ssd_sync(kh_engine_t e);                 /* Engine::sync_ssd (engine.rs:1220-1235): shutdown and tests */
KH_API void kh_engine_ssd_stats(kh_engine_t e, kh_ssd_stats* out);

/* The slab store on its own (SsdStore, ssd.rs:159-586). */
typedef struct kh_ssd* kh_ssd_t;
KH_API int kh_ssd_open(const char* dir, const uint8_t* fingerprint, const kh_slab_geometry* g, uint64_t max_bytes, kh_ssd_t* out);
KH_API void kh_ssd_close(kh_ssd_t s);                          /* joins the writer thread: queued writes land first */
KH_API int kh_ssd_contains(kh_ssd_t s, const uint8_t* hash);
KH_API int kh_ssd_enqueue_write(kh_ssd_t s, uint64_t node, uint64_t generation, const uint8_t* hash, const uint32_t* tokens,
                                uint64_t n_tokens, const uint8_t* payload, uint64_t n_payload, uint32_t dtype_tag, uint32_t dtype_size);
KH_API uint64_t kh_ssd_drain_acks(kh_ssd_t s, kh_flush_ack* out, uint64_t cap);
KH_API uint64_t kh_ssd_sync(kh_ssd_t s, kh_flush_ack* out, uint64_t cap);
/* Returns the payload size, -1 when the slot is missing or fails verification (the index entry is then dropped),
 * -2 when `cap` is too small. pool_dtype_tag < 0 accepts the slab's dtype. */
KH_API int64_t kh_ssd_read(kh_ssd_t s, const uint8_t* hash, const uint32_t* expected_tokens, uint64_t n_tokens, int64_t pool_dtype_tag,
                           uint8_t* out, uint64_t cap, uint32_t* dtype_tag);
KH_API void kh_ssd_get_stats(kh_ssd_t s, kh_ssd_stats* out);

/* ---- drafters ---- */

/* Scripted drafter with seeded acceptance injection: proposal position j equals the registered continuation
 * with probability p, else a uniform-random id (the reference tests' OracleDrafter/AdversarialDrafter shape,
 * crates/kiln-models/tests/spec_decode.rs:147-198). */
typedef struct kh_scripted* kh_scripted_t;
KH_API int kh_scripted_create(double p, uint64_t seed, uint32_t vocab, kh_scripted_t* out);
KH_API void kh_scripted_free(kh_scripted_t d);
KH_API int kh_scripted_set_continuation(kh_scripted_t d, uint64_t seq, const uint32_t* tokens, uint64_t n);
KH_API void kh_scripted_vtable(kh_scripted_t d, kh_drafter* out);

/* DraftModel (draft.rs:109-122, 258-412). forward has the signature of kc_verify_step, chain of kc_draft_chain. */
typedef struct {
  void* model;
  void* kv;
  int (*forward)(void* model, void* kv, const uint32_t* ids, int32_t n, const kh_seq_step* seqs, int32_t n_seqs,
                 uint32_t* row_tokens, int32_t* n_committed, int32_t* n_accepted);
  int (*chain)(void* model, void* kv, uint32_t first_token, int32_t offset, const uint32_t* blocks, int32_t n_blocks,
               int32_t gamma, uint32_t* proposal);
  int32_t max_chunk;
  /* For Drafter::memory (draft.rs:259-266): kc_model_weight_bytes, kc_kv_allocated_bytes and kc_kv_block_bytes of the
   * draft model and its pool; kv_used_bytes is live blocks x kv_block_bytes. Zeros where unknown. */
  uint64_t weights_bytes, kv_allocated_bytes, kv_block_bytes;
} kh_draft_backend;
typedef struct kh_draft_model* kh_draft_model_t;
KH_API int kh_draft_model_create(const kh_draft_backend* b, uint64_t num_blocks, uint64_t block_size, kh_draft_model_t* out);
KH_API void kh_draft_model_free(kh_draft_model_t d);
KH_API void kh_draft_model_vtable(kh_draft_model_t d, kh_drafter* out);
KH_API kh_bm_t kh_draft_model_block_manager(kh_draft_model_t d);   /* borrowed */
KH_API uint64_t kh_draft_model_live_sequences(kh_draft_model_t d);

#ifdef __cplusplus
}
#endif
#endif /* KILN_HOST_H */
