// C ABI of libkiln_host.so (declared in include/kiln_host.h) over the C++ scheduler pieces.
#include "../../../include/kiln_host.h"

#include <cstring>
#include <string>
#include <vector>

#include "block.hpp"
#include "engine.hpp"
#include "radix.hpp"

using namespace kh;

static thread_local std::string g_err;
static thread_local uint64_t g_oob_capacity = 0, g_oob_needed = 0;

static int status(const BlockStatus& st) {
  if (st.ok()) return KH_OK;
  g_err = st.message();
  if (st.err == BlockErr::OutOfBlocks) { g_oob_capacity = st.a; g_oob_needed = st.b; }
  return (int)st.err;  // BlockErr values are the KH_* codes
}

struct kh_bm { BlockManager* p; bool owned; };
struct kh_bt { BlockTable t; };
struct kh_radix { RadixCache* p; };

extern "C" {

const char* kh_last_error(void) { return g_err.c_str(); }
void kh_last_out_of_blocks(uint64_t* capacity, uint64_t* needed) {
  if (capacity) *capacity = g_oob_capacity;
  if (needed) *needed = g_oob_needed;
}

// ---- BlockManager ----
int kh_bm_create(uint64_t capacity, uint64_t block_size, kh_bm_t* out) {
  BlockStatus st = BlockManager::validate(capacity, block_size);
  if (!st.ok()) return status(st);
  *out = new kh_bm{new BlockManager(capacity, block_size), true};
  return KH_OK;
}
void kh_bm_free(kh_bm_t bm) {
  if (!bm) return;
  if (bm->owned) delete bm->p;
  delete bm;
}
uint64_t kh_bm_block_size(kh_bm_t bm) { return bm->p->block_size(); }
uint64_t kh_bm_capacity(kh_bm_t bm) { return bm->p->capacity(); }
uint64_t kh_bm_num_free(kh_bm_t bm) { return bm->p->num_free(); }
int64_t kh_bm_refcount(kh_bm_t bm, uint32_t id) { return bm->p->refcount(id); }
int kh_bm_allocate(kh_bm_t bm, uint32_t* id_out) { return status(bm->p->allocate(id_out)); }
int kh_bm_retain(kh_bm_t bm, uint32_t id) { return status(bm->p->retain(id)); }
int kh_bm_release(kh_bm_t bm, uint32_t id) { return status(bm->p->release(id)); }
int kh_bm_copy_on_write(kh_bm_t bm, uint32_t id, int32_t* copied_out, uint32_t* src_out, uint32_t* dst_out) {
  CowOutcome oc;
  BlockStatus st = bm->p->copy_on_write(id, &oc);
  if (!st.ok()) return status(st);
  if (copied_out) *copied_out = oc.copied ? 1 : 0;
  if (src_out) *src_out = oc.src;
  if (dst_out) *dst_out = oc.dst;
  return KH_OK;
}
uint64_t kh_bm_free_list(kh_bm_t bm, uint32_t* out, uint64_t cap) {
  const auto& f = bm->p->free_list();
  for (uint64_t i = 0; i < f.size() && i < cap; ++i) out[i] = f[i];
  return f.size();
}

// ---- BlockTable ----
int kh_bt_create(kh_bt_t* out) { *out = new kh_bt; return KH_OK; }
void kh_bt_free(kh_bt_t bt) { delete bt; }
uint64_t kh_bt_num_tokens(kh_bt_t bt) { return bt->t.num_tokens(); }
uint64_t kh_bt_blocks(kh_bt_t bt, uint32_t* out, uint64_t cap) {
  const auto& b = bt->t.blocks();
  for (uint64_t i = 0; i < b.size() && i < cap; ++i) out[i] = b[i];
  return b.size();
}
int kh_bt_append_tokens(kh_bt_t bt, kh_bm_t bm, uint64_t n, int32_t* has_cow, uint32_t* cow_src, uint32_t* cow_dst,
                        uint32_t* appended_out, uint64_t appended_cap, uint64_t* n_appended) {
  AppendPlan plan;
  BlockStatus st = bt->t.append_tokens(*bm->p, n, &plan);
  if (!st.ok()) return status(st);
  if (has_cow) *has_cow = plan.has_cow ? 1 : 0;
  if (cow_src) *cow_src = plan.cow_src;
  if (cow_dst) *cow_dst = plan.cow_dst;
  if (n_appended) *n_appended = plan.appended.size();
  if (appended_out)
    for (uint64_t i = 0; i < plan.appended.size() && i < appended_cap; ++i) appended_out[i] = plan.appended[i];
  return KH_OK;
}
int kh_bt_push_full_block(kh_bt_t bt, uint32_t id, uint64_t block_size) { return status(bt->t.push_full_block(id, block_size)); }
int kh_bt_push_partial_block(kh_bt_t bt, uint32_t id, uint64_t rows, uint64_t block_size) {
  return status(bt->t.push_partial_block(id, rows, block_size));
}
int kh_bt_truncate(kh_bt_t bt, kh_bm_t bm, uint64_t keep_tokens) { return status(bt->t.truncate(*bm->p, keep_tokens)); }
int kh_bt_fork(kh_bt_t bt, kh_bm_t bm, kh_bt_t* out) {
  kh_bt* f = new kh_bt;
  BlockStatus st = bt->t.fork(*bm->p, &f->t);
  if (!st.ok()) { delete f; return status(st); }
  *out = f;
  return KH_OK;
}
int kh_bt_release(kh_bt_t bt, kh_bm_t bm) { return status(bt->t.release(*bm->p)); }

// ---- pure functions ----
uint64_t kh_spec_gamma_at_width(uint64_t gamma, uint64_t spec_max_batch, uint64_t width) {
  return spec_gamma_at_width(gamma, spec_max_batch, width);
}
uint64_t kh_canonical_prefill_len(uint64_t at, uint64_t limit, uint64_t prefill_chunk, uint64_t fine) {
  return canonical_prefill_len(at, limit, prefill_chunk, fine);
}

// ---- RadixCache ----
int kh_radix_create(uint64_t block_size, const uint8_t seed[32], kh_radix_t* out) {
  ChainHash h{};
  if (seed) memcpy(h.data(), seed, 32);
  *out = new kh_radix{new RadixCache(block_size, h)};
  return KH_OK;
}
void kh_radix_free(kh_radix_t r) { if (r) { delete r->p; delete r; } }
static std::vector<uint32_t> vec(const uint32_t* p, uint64_t n) { return std::vector<uint32_t>(p, p + n); }
int64_t kh_radix_child(kh_radix_t r, uint64_t node, const uint32_t* chunk, uint64_t n) { return r->p->child(node, vec(chunk, n)); }
void kh_radix_chain_hash_of(kh_radix_t r, uint64_t node, const uint32_t* chunk, uint64_t n, uint8_t out[32]) {
  ChainHash h = r->p->chain_hash_of(node, chunk, n);
  memcpy(out, h.data(), 32);
}
void kh_radix_node_hash(kh_radix_t r, uint64_t node, uint8_t out[32]) { memcpy(out, r->p->node_hash(node).data(), 32); }
int64_t kh_radix_node_block(kh_radix_t r, uint64_t node) { return r->p->node_block(node); }
uint64_t kh_radix_node_rows(kh_radix_t r, uint64_t node) { return r->p->node_rows(node); }
int32_t kh_radix_node_is_partial(kh_radix_t r, uint64_t node) { return r->p->node_is_partial(node) ? 1 : 0; }
uint64_t kh_radix_node_generation(kh_radix_t r, uint64_t node) { return r->p->node_generation(node); }
int32_t kh_radix_is_live(kh_radix_t r, uint64_t node, uint64_t generation) { return r->p->is_live(node, generation) ? 1 : 0; }
uint64_t kh_radix_insert_child(kh_radix_t r, uint64_t parent, const uint32_t* chunk, uint64_t n) {
  return r->p->insert_child(parent, vec(chunk, n));
}
uint64_t kh_radix_insert_partial_child(kh_radix_t r, uint64_t parent, const uint32_t* tokens, uint64_t n) {
  return r->p->insert_partial_child(parent, vec(tokens, n));
}
int64_t kh_radix_upgrade_partial(kh_radix_t r, uint64_t node, const uint32_t* tokens, uint64_t n, uint32_t block) {
  return r->p->upgrade_partial(node, vec(tokens, n), block);
}
void kh_radix_set_resident(kh_radix_t r, uint64_t node, uint32_t block) { r->p->set_resident(node, block); }
void kh_radix_touch(kh_radix_t r, uint64_t node) { r->p->touch(node); }
void kh_radix_set_on_ssd(kh_radix_t r, uint64_t node) { r->p->set_on_ssd(node); }
int32_t kh_radix_node_on_ssd(kh_radix_t r, uint64_t node) { return r->p->node_on_ssd(node) ? 1 : 0; }
int64_t kh_radix_evict_candidate(kh_radix_t r, kh_bm_t bm) { return r->p->evict_candidate(*bm->p); }
int64_t kh_radix_evict(kh_radix_t r, kh_bm_t bm, uint64_t node) { return r->p->evict(*bm->p, node); }
void kh_radix_prune_subtree(kh_radix_t r, kh_bm_t bm, uint64_t node) { r->p->prune_subtree(*bm->p, node); }
uint64_t kh_radix_resident_blocks(kh_radix_t r) { return r->p->resident_blocks(); }
void kh_radix_reset(kh_radix_t r) { r->p->reset(); }

}  // extern "C"
