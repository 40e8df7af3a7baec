// C ABI of the engine and the drafters (declared in include/kiln_host.h).
#include "../../../include/kiln_host.h"

#include <cstring>
#include <memory>
#include <string>

#include "engine.hpp"

using namespace kh;

struct kh_bm { BlockManager* p; bool owned; };  // same layout as in kh_api.cpp

static thread_local std::string g_eng_err;
extern "C" const char* kh_last_error(void);

struct kh_engine {
  Engine* e;
  kh_bm bm_view;
};
struct kh_scripted { ScriptedDrafter* d; };
struct kh_draft_model {
  DraftModel* d;
  kh_bm bm_view;
};

static_assert(sizeof(kh_seq_step) == sizeof(SeqStepC), "seq step layout");
static_assert(sizeof(kh_drafter_memory) == sizeof(DrafterMemory), "drafter memory layout");

extern "C" {

void kh_engine_default_config(kh_engine_config* out) {
  EngineConfig c;
  out->block_size = c.block_size; out->num_blocks = c.num_blocks; out->max_batch_tokens = c.max_batch_tokens;
  out->prefill_chunk = c.prefill_chunk; out->prefill_fine_chunk = c.prefill_fine_chunk; out->prefix_cache = c.prefix_cache;
  out->deterministic_decode_width = c.deterministic_decode_width; out->gamma = c.gamma; out->spec_max_batch = c.spec_max_batch;
  out->spec_min_acceptance = c.spec_min_acceptance; out->max_key_len = c.max_key_len; out->batch_verify = c.batch_verify;
}

int kh_engine_create(const kh_engine_config* cfg, const kh_step_model* model, kh_engine_t* out) {
  if (!cfg || !model || !out || !model->verify_step || !model->copy_block) return KH_ERR_ARG;
  BlockStatus st = BlockManager::validate(cfg->num_blocks, cfg->block_size);
  if (!st.ok()) return (int)st.err;
  EngineConfig c;
  c.block_size = cfg->block_size; c.num_blocks = cfg->num_blocks; c.max_batch_tokens = cfg->max_batch_tokens;
  c.prefill_chunk = cfg->prefill_chunk; c.prefill_fine_chunk = cfg->prefill_fine_chunk; c.prefix_cache = cfg->prefix_cache;
  c.deterministic_decode_width = cfg->deterministic_decode_width; c.gamma = cfg->gamma; c.spec_max_batch = cfg->spec_max_batch;
  c.spec_min_acceptance = cfg->spec_min_acceptance; c.max_key_len = cfg->max_key_len; c.batch_verify = cfg->batch_verify;
  if (c.prefill_chunk < 1 || c.max_batch_tokens < 1) return KH_ERR_ARG;
  StepModelVT vt;
  vt.model = model->model; vt.kv = model->kv; vt.vocab = model->vocab;
  vt.verify_step = reinterpret_cast<decltype(vt.verify_step)>(model->verify_step);
  vt.copy_block = model->copy_block;
  kh_engine* h = new kh_engine;
  h->e = new Engine(c, vt);
  h->bm_view = kh_bm{&h->e->block_manager(), false};
  *out = h;
  return KH_OK;
}
void kh_engine_free(kh_engine_t e) { if (e) { delete e->e; delete e; } }

int kh_engine_set_drafter(kh_engine_t e, const kh_drafter* d) {
  if (!e || !d || !d->begin || !d->propose || !d->release) return KH_ERR_ARG;
  DrafterVT vt{d->user, d->begin, d->propose, d->release};
  vt.memory = reinterpret_cast<decltype(vt.memory)>(d->memory);
  e->e->set_drafter(vt);
  return KH_OK;
}
int kh_engine_drafter_memory(kh_engine_t e, kh_drafter_memory* out) {
  if (!e || !out) return 0;
  DrafterMemory m;
  const bool has = e->e->drafter_memory(&m);
  out->weights_bytes = m.weights_bytes; out->kv_allocated_bytes = m.kv_allocated_bytes; out->kv_used_bytes = m.kv_used_bytes;
  return has ? 1 : 0;
}
int kh_engine_set_pipeline(kh_engine_t e, const kh_decode_pipeline* p) {
  if (!e) return KH_ERR_ARG;
  if (!p) { e->e->clear_pipeline(); return KH_OK; }
  if (!p->launch || !p->collect) return KH_ERR_ARG;
  DecodePipelineVT vt;
  vt.launch = reinterpret_cast<decltype(vt.launch)>(p->launch);
  vt.collect = p->collect;
  e->e->set_pipeline(vt);
  return KH_OK;
}
uint64_t kh_engine_pipelined_steps(kh_engine_t e) { return e->e->pipelined_steps(); }

static ChainHash hash_of(const uint8_t* p) {
  ChainHash h;
  memcpy(h.data(), p, 32);
  return h;
}
int kh_engine_set_ssd(kh_engine_t e, const char* dir, const uint8_t* fingerprint, const kh_slab_geometry* g, uint64_t max_bytes,
                      const kh_block_io* io) {
  if (!e || !dir || !fingerprint || !g || !io || !io->read || !io->write || io->dtype_size == 0 || io->dtype_size > 8) return KH_ERR_ARG;
  SlabGeometry sg;
  sg.layers = g->layers; sg.kv_heads = g->kv_heads; sg.head_dim = g->head_dim; sg.block_size = g->block_size;
  BlockIoVT vt;
  vt.read = io->read; vt.write = io->write; vt.dtype_tag = io->dtype_tag; vt.dtype_size = io->dtype_size;
  return e->e->set_ssd(dir, hash_of(fingerprint), sg, max_bytes, vt) ? KH_OK : KH_ERR_ARG;
}
void kh_engine_ssd_sync(kh_engine_t e) { e->e->ssd_sync(); }
void kh_engine_ssd_stats(kh_engine_t e, kh_ssd_stats* out) {
  memset(out, 0, sizeof *out);
  SsdStore* s = e->e->ssd();
  if (!s) return;
  out->blocks_stored = s->blocks_stored(); out->bytes_stored = s->bytes_stored();
  out->reads_total = s->counters().reads_total; out->writes_total = s->counters().writes_total;
  out->writes_failed_total = s->counters().writes_failed_total; out->fingerprint_rejects_total = s->counters().fingerprint_rejects_total;
  out->flush_queue_depth = e->e->flush_queue_depth();
  out->ssd_hits_total = e->e->cache_stats().ssd_hits_total;
}

// ---- the slab store on its own (ssd.rs unit tests drive it like this) ----
struct kh_ssd { std::unique_ptr<SsdStore> s; };
int kh_ssd_open(const char* dir, const uint8_t* fingerprint, const kh_slab_geometry* g, uint64_t max_bytes, kh_ssd_t* out) {
  if (!dir || !fingerprint || !g || !out) return KH_ERR_ARG;
  SlabGeometry sg;
  sg.layers = g->layers; sg.kv_heads = g->kv_heads; sg.head_dim = g->head_dim; sg.block_size = g->block_size;
  std::unique_ptr<SsdStore> s = SsdStore::open(dir, hash_of(fingerprint), sg, max_bytes);
  if (!s) return KH_ERR_ARG;
  *out = new kh_ssd{std::move(s)};
  return KH_OK;
}
void kh_ssd_close(kh_ssd_t s) { delete s; }
int kh_ssd_contains(kh_ssd_t s, const uint8_t* hash) { return s->s->contains(hash_of(hash)) ? 1 : 0; }
int kh_ssd_enqueue_write(kh_ssd_t s, uint64_t node, uint64_t generation, const uint8_t* hash, const uint32_t* tokens, uint64_t n_tokens,
                         const uint8_t* payload, uint64_t n_payload, uint32_t dtype_tag, uint32_t dtype_size) {
  if (!s || !hash || !payload || dtype_size == 0) return KH_ERR_ARG;
  s->s->enqueue_write(FlushTicket{(size_t)node, generation, hash_of(hash)}, tokens, n_tokens, std::vector<uint8_t>(payload, payload + n_payload),
                      dtype_tag, dtype_size);
  return KH_OK;
}
static uint64_t copy_acks(const std::vector<FlushAck>& acks, kh_flush_ack* out, uint64_t cap) {
  uint64_t n = 0;
  for (const FlushAck& a : acks) {
    if (n >= cap) break;
    out[n].node = a.node; out[n].generation = a.generation; out[n].ok = a.ok ? 1 : 0;
    memcpy(out[n].hash, a.hash.data(), 32);
    ++n;
  }
  return n;
}
uint64_t kh_ssd_drain_acks(kh_ssd_t s, kh_flush_ack* out, uint64_t cap) { return copy_acks(s->s->drain_acks(), out, cap); }
uint64_t kh_ssd_sync(kh_ssd_t s, kh_flush_ack* out, uint64_t cap) { return copy_acks(s->s->sync(), out, cap); }
int64_t kh_ssd_read(kh_ssd_t s, const uint8_t* hash, const uint32_t* expected_tokens, uint64_t n_tokens, int64_t pool_dtype_tag, uint8_t* out,
                    uint64_t cap, uint32_t* dtype_tag) {
  std::vector<uint8_t> payload;
  uint32_t tag = 0;
  if (!s->s->read(hash_of(hash), expected_tokens, n_tokens, pool_dtype_tag, &payload, &tag)) return -1;
  if (payload.size() > cap) return -2;
  memcpy(out, payload.data(), payload.size());
  if (dtype_tag) *dtype_tag = tag;
  return (int64_t)payload.size();
}
void kh_ssd_get_stats(kh_ssd_t s, kh_ssd_stats* out) {
  memset(out, 0, sizeof *out);
  out->blocks_stored = s->s->blocks_stored(); out->bytes_stored = s->s->bytes_stored();
  out->reads_total = s->s->counters().reads_total; out->writes_total = s->s->counters().writes_total;
  out->writes_failed_total = s->s->counters().writes_failed_total; out->fingerprint_rejects_total = s->s->counters().fingerprint_rejects_total;
}
int kh_engine_submit(kh_engine_t e, const uint32_t* prompt, uint64_t n, uint64_t max_tokens, const uint32_t* stop_tokens,
                     uint64_t n_stop, uint64_t* arrival_out) {
  if (!e || (!prompt && n)) return KH_ERR_ARG;
  const uint64_t a = e->e->submit(prompt, n, max_tokens, stop_tokens, n_stop);
  if (arrival_out) *arrival_out = a;
  return KH_OK;
}
int kh_engine_cancel(kh_engine_t e, uint64_t arrival) { e->e->cancel(arrival); return KH_OK; }
int kh_engine_step(kh_engine_t e) {
  const int rc = e->e->step();
  return rc == 0 ? KH_OK : KH_ERR_MODEL;
}
uint64_t kh_engine_num_running(kh_engine_t e) { return e->e->num_running(); }
uint64_t kh_engine_num_waiting(kh_engine_t e) { return e->e->num_waiting(); }
uint64_t kh_engine_iterations(kh_engine_t e) { return e->e->iterations(); }
uint64_t kh_engine_forwards(kh_engine_t e) { return e->e->forwards(); }
const char* kh_engine_last_error(kh_engine_t e) { return e->e->last_error().c_str(); }

int kh_engine_take_output(kh_engine_t e, uint64_t arrival, uint32_t* out, uint64_t cap, uint64_t* n_out, int32_t* finish_kind) {
  Seq* s = e->e->find(arrival);
  if (!s) return KH_ERR_ARG;
  uint64_t n = 0;
  while (s->taken < s->emitted.size() && n < cap) out[n++] = s->emitted[s->taken++];
  if (n_out) *n_out = n;
  if (finish_kind) *finish_kind = (s->finished && s->taken == s->emitted.size()) ? s->finish_kind : FINISH_NONE;
  return KH_OK;
}
int kh_engine_seq_state(kh_engine_t e, uint64_t arrival, uint32_t* blocks_out, uint64_t cap, uint64_t* n_blocks,
                        uint64_t* num_tokens, uint64_t* generated, uint32_t* spec_proposed, uint32_t* spec_accepted,
                        int32_t* standdown, uint32_t* cached_tokens) {
  Seq* s = e->e->find(arrival);
  if (!s) return KH_ERR_ARG;
  const auto& b = s->table.blocks();
  if (blocks_out) for (uint64_t i = 0; i < b.size() && i < cap; ++i) blocks_out[i] = b[i];
  if (n_blocks) *n_blocks = b.size();
  if (num_tokens) *num_tokens = s->table.num_tokens();
  if (generated) *generated = s->generated;
  if (spec_proposed) *spec_proposed = s->spec_proposed;
  if (spec_accepted) *spec_accepted = s->spec_accepted;
  if (standdown) *standdown = s->draft_standdown ? 1 : (s->draft_dead ? 2 : 0);
  if (cached_tokens) *cached_tokens = s->cached_tokens;
  return KH_OK;
}
void kh_engine_spec_stats(kh_engine_t e, kh_spec_stats* out) {
  const SpecStats& s = e->e->spec_stats();
  out->rounds_total = s.rounds_total; out->proposed_total = s.proposed_total; out->accepted_total = s.accepted_total;
  out->rollback_rounds_total = s.rollback_rounds_total; out->rollback_tokens_total = s.rollback_tokens_total;
  out->rollback_nanos_total = s.rollback_nanos_total; out->draft_errors_total = s.draft_errors_total;
  out->standdowns_total = s.standdowns_total;
}
kh_bm_t kh_engine_block_manager(kh_engine_t e) {
  e->bm_view.p = &e->e->block_manager();  // the manager is rebuilt after a failed step
  return &e->bm_view;
}
void kh_engine_cache_stats(kh_engine_t e, uint64_t* hits, uint64_t* tokens_reused, uint64_t* resident_blocks) {
  PrefixCacheStats s = e->e->cache_stats();
  if (hits) *hits = s.hits_total;
  if (tokens_reused) *tokens_reused = s.tokens_reused_total;
  if (resident_blocks) *resident_blocks = s.resident_blocks;
}

// ---- drafters ----
int kh_scripted_create(double p, uint64_t seed, uint32_t vocab, kh_scripted_t* out) {
  if (!out || vocab == 0) return KH_ERR_ARG;
  *out = new kh_scripted{new ScriptedDrafter(p, seed, vocab)};
  return KH_OK;
}
void kh_scripted_free(kh_scripted_t d) { if (d) { delete d->d; delete d; } }
int kh_scripted_set_continuation(kh_scripted_t d, uint64_t seq, const uint32_t* tokens, uint64_t n) {
  d->d->set_continuation(seq, tokens, n);
  return KH_OK;
}
void kh_scripted_vtable(kh_scripted_t d, kh_drafter* out) {
  DrafterVT v = d->d->vtable();
  out->user = v.user; out->begin = v.begin; out->propose = v.propose; out->release = v.release;
  out->memory = nullptr;   // a scripted drafter holds no weights and no pool
}

int kh_draft_model_create(const kh_draft_backend* b, uint64_t num_blocks, uint64_t block_size, kh_draft_model_t* out) {
  if (!b || !out || !b->forward || !b->chain) return KH_ERR_ARG;
  BlockStatus st = BlockManager::validate(num_blocks, block_size);
  if (!st.ok()) return (int)st.err;
  DraftModelVT vt;
  vt.model = b->model; vt.kv = b->kv; vt.max_chunk = b->max_chunk > 0 ? b->max_chunk : 2048;
  vt.weights_bytes = b->weights_bytes; vt.kv_allocated_bytes = b->kv_allocated_bytes; vt.kv_block_bytes = b->kv_block_bytes;
  vt.forward = reinterpret_cast<decltype(vt.forward)>(b->forward);
  vt.chain = b->chain;
  kh_draft_model* h = new kh_draft_model;
  h->d = new DraftModel(vt, num_blocks, block_size);
  h->bm_view = kh_bm{&h->d->block_manager(), false};
  *out = h;
  return KH_OK;
}
void kh_draft_model_free(kh_draft_model_t d) { if (d) { delete d->d; delete d; } }
void kh_draft_model_vtable(kh_draft_model_t d, kh_drafter* out) {
  DrafterVT v = d->d->vtable();
  out->user = v.user; out->begin = v.begin; out->propose = v.propose; out->release = v.release;
  out->memory = reinterpret_cast<decltype(out->memory)>(v.memory);
}
kh_bm_t kh_draft_model_block_manager(kh_draft_model_t d) { return &d->bm_view; }
uint64_t kh_draft_model_live_sequences(kh_draft_model_t d) { return d->d->live_sequences(); }

}  // extern "C"
