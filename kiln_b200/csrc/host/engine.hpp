// The speculative scheduler step on the host: plan -> verify forward -> settle
// walk -> rollback -> stand-down, with chunked prefill, admission, the radix
// prefix cache and the two drafters. C++ equivalent of the reference's
//   crates/kiln-engine/src/engine.rs   Engine::{submit, step, admit, run_iteration,
//                                      collect_proposal, maybe_stand_down}, build_seq_step,
//                                      settle_sampled, finish, CacheState::donate,
//                                      match_head_prefix (1294-1363, 1367-1407, 1508-1634,
//                                      1802-2033, 2035-2417, 2736-2796, 601-778, 907-963),
//                                      pipelined_turn, pipeline_ok, build_pipelined,
//                                      apply_inflight (1428-1475, 1656-1766); cache_io_tick,
//                                      resolve_chunk, load_from_ssd, flush_entries, apply_ack
//                                      (1412-1426, 2559-2704) over the slab store of ssd.hpp
//   crates/kiln-engine/src/drafter.rs  spec_gamma_at_width, trait Drafter (62-70, 125-147)
//   crates/kiln-models/src/draft.rs    DraftModel::{begin, propose, release} (268-411)
// The model and the drafter sit behind C function tables (the StepModel / Drafter
// trait seams, step.rs:85-96, drafter.rs:125-147), so tests drive the engine with
// fake models exactly as the reference's engine tests do.
//
// One deliberate difference, a property of the backend and not of the algorithm:
// because every kernel of libkiln_cuda.so is row-invariant, all decode and verify
// segments of an iteration (and its prefill chunk) ride ONE forward when
// `batch_verify` is set, where the reference issues one forward per verify segment
// (engine.rs:2164-2172, 2240-2271). With batch_verify = 0 the reference's grouping
// is reproduced. The envelope constants the reference derives from MLX's kernel
// dispatch (VERIFY_MAX_KEY_LEN, deterministic width, per-model gamma) are inputs here.
//
// Out of scope (not on the verify path): preemption under pool exhaustion, priorities,
// cancellation tokens, penalties, grammars, stochastic samplers. A step
// that cannot get blocks for a plain decode slot returns a capacity error.
#pragma once

#include <algorithm>
#include <cstdint>
#include <deque>
#include <map>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "block.hpp"
#include "radix.hpp"
#include "ssd.hpp"

namespace kh {

// Same layout as kc_seq_step (include/kiln_cuda.h).
struct SeqStepC {
  int32_t len, offset, sample_rows, n_blocks;
  const uint32_t* blocks;
};

// StepModel seam. verify_step has the signature of kc_verify_step, copy_block of kc_kv_copy_block.
struct StepModelVT {
  void* model;
  void* kv;
  int (*verify_step)(void* model, void* kv, const uint32_t* ids, int32_t n, const SeqStepC* seqs, int32_t n_seqs,
                     uint32_t* row_tokens, int32_t* n_committed, int32_t* n_accepted);
  int (*copy_block)(void* kv, uint32_t src, uint32_t dst);
  int32_t vocab;
};

// The pipelined-decode seam: launch queues one decode forward (one sampled row per sequence) without waiting for it and
// returns a ticket; feed[i] >= 0 takes sequence i's input id from row feed[i] of the previous launch, still on the device
// (StepInput::Lazy, step.rs:45-56), feed[i] < 0 takes ids[i]. collect blocks until that launch's tokens are on the host
// (Array::item_u32 after async_eval). launch has the signature of kc_decode_launch, collect of kc_decode_collect.
struct DecodePipelineVT {
  int (*launch)(void* model, void* kv, const uint32_t* ids, const int32_t* feed, const SeqStepC* seqs, int32_t n_seqs,
                uint64_t* ticket);
  int (*collect)(void* model, uint64_t ticket, uint32_t* row_tokens, int32_t n);
};

// Block IO for the SSD tier: read has the signature of kc_kv_read_block, write of kc_kv_write_block (the payload order
// of PagedKv::read_block_bytes, paged.rs:280-304); kv is the step model's pool.
struct BlockIoVT {
  int (*read)(void* kv, uint32_t block, void* dst, size_t n);
  int (*write)(void* kv, uint32_t block, const void* src, size_t n);
  uint32_t dtype_tag = 7, dtype_size = 2;   // stable on-disk tags (engine.rs:2707-2718): 7 = bfloat16
};

// Drafter seam (drafter.rs:125-147). propose writes at most `gamma` ids; a non-zero return is a DraftError.
// DrafterMemory (drafter.rs:88-102): what a drafter adds to the worker's memory report.
struct DrafterMemory { uint64_t weights_bytes = 0, kv_allocated_bytes = 0, kv_used_bytes = 0; };

struct DrafterVT {
  void* user;
  int (*begin)(void* user, uint64_t seq, const uint32_t* prompt, int32_t n);
  int (*propose)(void* user, uint64_t seq, const uint32_t* committed, int32_t n_committed, int32_t gamma, uint32_t* out,
                 int32_t* n_out);
  void (*release)(void* user, uint64_t seq);
  void (*memory)(void* user, DrafterMemory* out) = nullptr;   // Drafter::memory (drafter.rs:127); null = all zeros
};

// drafter.rs:26-50 and engine.rs:133-213 defaults.
constexpr int DEFAULT_GAMMA = 4;
constexpr int DEFAULT_SPEC_MAX_BATCH = 4;
constexpr double DEFAULT_SPEC_MIN_ACCEPTANCE = 0.125;
constexpr uint32_t SPEC_ACCEPTANCE_WARMUP_PROPOSED = 16;
constexpr int DEFAULT_BLOCK_SIZE = 32;
constexpr int DEFAULT_NUM_BLOCKS = 512;
constexpr int DEFAULT_MAX_BATCH_TOKENS = 8192;
constexpr int DEFAULT_PREFILL_CHUNK = 2048;
constexpr int DEFAULT_PREFILL_FINE_CHUNK = 128;
constexpr int DEFAULT_DETERMINISTIC_DECODE_WIDTH = 4;
constexpr int VERIFY_MAX_KEY_LEN = 1023;

inline size_t spec_gamma_at_width(size_t gamma, size_t spec_max_batch, size_t width) {  // drafter.rs:62-70
  width = std::max<size_t>(width, 1);
  if (gamma == 0 || width > spec_max_batch) return 0;
  return (gamma * (spec_max_batch + 1 - width) + spec_max_batch - 1) / spec_max_batch;
}

inline size_t canonical_prefill_len(size_t at, size_t limit, size_t prefill_chunk, size_t fine) {  // engine.rs:167-179
  fine = std::min(std::max<size_t>(fine, 1), prefill_chunk);
  const size_t tail_start = limit / prefill_chunk * prefill_chunk;
  if (at < tail_start) return prefill_chunk - at % prefill_chunk;
  return std::min(fine - at % fine, limit - at);
}

struct EngineConfig {  // engine.rs:239-306, plus the backend-provided envelope
  int32_t block_size = DEFAULT_BLOCK_SIZE;
  int32_t num_blocks = DEFAULT_NUM_BLOCKS;
  int32_t max_batch_tokens = DEFAULT_MAX_BATCH_TOKENS;
  int32_t prefill_chunk = DEFAULT_PREFILL_CHUNK;
  int32_t prefill_fine_chunk = DEFAULT_PREFILL_FINE_CHUNK;
  int32_t prefix_cache = 1;
  int32_t deterministic_decode_width = DEFAULT_DETERMINISTIC_DECODE_WIDTH;
  int32_t gamma = DEFAULT_GAMMA;
  int32_t spec_max_batch = DEFAULT_SPEC_MAX_BATCH;
  double spec_min_acceptance = DEFAULT_SPEC_MIN_ACCEPTANCE;
  int32_t max_key_len = VERIFY_MAX_KEY_LEN;  // 0 = the backend has no key-length bound
  int32_t batch_verify = 0;                  // 1 = all segments of an iteration in one forward
};

struct SpecStats {  // engine.rs:811-830
  uint64_t rounds_total = 0, proposed_total = 0, accepted_total = 0, rollback_rounds_total = 0, rollback_tokens_total = 0,
           rollback_nanos_total = 0, draft_errors_total = 0, standdowns_total = 0;
};

enum FinishKind : int32_t { FINISH_NONE = 0, FINISH_STOP = 1, FINISH_LENGTH = 2, FINISH_ERROR = 3, FINISH_CANCELLED = 4 };

struct Seq {  // engine.rs:470-527 (the fields this path uses)
  std::vector<uint32_t> prompt;
  size_t max_tokens = 0;
  std::vector<uint32_t> stop_tokens;
  uint64_t arrival = 0;
  BlockTable table;
  size_t processed = 0;
  std::vector<uint32_t> history;
  size_t fed = 0;
  uint32_t generated = 0;
  bool cache_checked = false;
  uint32_t cached_tokens = 0;
  bool draft_begun = false;
  size_t draft_committed = 0;
  bool draft_dead = false, draft_standdown = false;
  uint32_t spec_proposed = 0, spec_accepted = 0;
  bool finished = false;
  bool cancel = false;
  int32_t finish_kind = FINISH_NONE;
  std::string error;
  std::vector<uint32_t> emitted;   // SeqEvent::Token stream
  size_t taken = 0;                // emitted tokens already handed to the caller

  bool decoding() const { return processed + 1 >= prompt.size(); }        // engine.rs:531-533
  bool spec_eligible() const { return !draft_dead && !draft_standdown; }  // greedy, no penalties/grammar: engine.rs:548-554
  size_t admission_blocks(size_t bs) const {                              // engine.rs:563-565
    return (prompt.size() - 1 - processed + std::max<size_t>(history.size(), 1) + bs - 1) / bs;
  }
};

struct PrefixCacheStats { uint64_t hits_total = 0, tokens_reused_total = 0, resident_blocks = 0, ssd_hits_total = 0; };

constexpr size_t FLUSH_BATCH = 8;   // blocks captured for the SSD writer per synchronous step (engine.rs:225-228)

class Engine {
 public:
  Engine(const EngineConfig& cfg, const StepModelVT& model)
      : cfg_(cfg), model_(model), mgr_(cfg.num_blocks, cfg.block_size) {
    if (cfg.prefix_cache) radix_.reset(new RadixCache(cfg.block_size, ChainHash{}));
  }
  void set_drafter(const DrafterVT& d) { drafter_ = d; has_drafter_ = true; }
  // Engine::drafter_memory (engine.rs:1128-1132): false when speculation is not configured.
  bool drafter_memory(DrafterMemory* out) const {
    *out = DrafterMemory{};
    if (!has_drafter_) return false;
    if (drafter_.memory) drafter_.memory(drafter_.user, out);
    return true;
  }
  // Attaches the SSD tier (engine.rs:1053-1076): donated blocks are written behind the steps, evicted ones stay
  // discoverable, and a fresh engine over the same directory finds them again hash-first. Needs the prefix cache.
  bool set_ssd(const std::string& dir, const ChainHash& fingerprint, const SlabGeometry& g, uint64_t max_bytes, const BlockIoVT& io) {
    if (!radix_) return false;
    store_ = SsdStore::open(dir, fingerprint, g, max_bytes);
    io_ = io;
    slab_geometry_ = g;
    return store_ != nullptr;
  }
  SsdStore* ssd() { return store_.get(); }
  size_t flush_queue_depth() const { return store_ ? flush_queue_.size() : 0; }
  // Blocks until every queued write has landed and applies the acks (shutdown and tests; engine.rs:1220-1235).
  void ssd_sync() {
    if (!store_) return;
    while (!flush_queue_.empty()) flush_entries(flush_queue_.size());
    for (const FlushAck& a : store_->sync()) apply_ack(a);
  }
  void set_pipeline(const DecodePipelineVT& p) { pipe_ = p; has_pipe_ = true; }
  void clear_pipeline() { has_pipe_ = false; }  // a step already in flight is still read back at the next turn
  uint64_t pipelined_steps() const { return pipelined_total_; }  // engine.rs:1160-1163
  const SpecStats& spec_stats() const { return spec_; }
  BlockManager& block_manager() { return mgr_; }
  RadixCache* radix() { return radix_.get(); }
  PrefixCacheStats cache_stats() const {
    PrefixCacheStats s = cache_stats_;
    s.resident_blocks = radix_ ? radix_->resident_blocks() : 0;
    return s;
  }
  size_t num_running() const { return running_.size(); }
  size_t num_waiting() const { return waiting_.size(); }
  uint64_t iterations() const { return iterations_; }
  uint64_t forwards() const { return forwards_; }
  const std::string& last_error() const { return err_; }

  // Engine::submit (engine.rs:1294-1363). Returns the arrival number; errors finish the request in-band.
  uint64_t submit(const uint32_t* prompt, size_t n, size_t max_tokens, const uint32_t* stops, size_t n_stops) {
    auto seq = std::make_shared<Seq>();
    seq->prompt.assign(prompt, prompt + n);
    seq->max_tokens = max_tokens;
    seq->stop_tokens.assign(stops, stops + n_stops);
    seq->arrival = next_arrival_++;
    all_[seq->arrival] = seq;
    std::string error;
    if (n == 0) error = "empty prompt";
    else if (max_tokens == 0) error = "max_tokens must be >= 1";
    else if (n + max_tokens > (size_t)cfg_.num_blocks * cfg_.block_size)
      error = "prompt (" + std::to_string(n) + ") + max_tokens (" + std::to_string(max_tokens) + ") exceeds the KV pool (" +
              std::to_string((size_t)cfg_.num_blocks * cfg_.block_size) + " tokens)";
    if (!error.empty()) {
      seq->error = error;
      finish(*seq, FINISH_ERROR, false);
      return seq->arrival;
    }
    if (n == 1) seq->history.push_back(seq->prompt[0]);  // a 1-token prompt decodes immediately
    waiting_.push_back(seq);
    return seq->arrival;
  }
  void cancel(uint64_t arrival) {
    auto it = all_.find(arrival);
    if (it != all_.end()) it->second->cancel = true;
  }
  Seq* find(uint64_t arrival) {
    auto it = all_.find(arrival);
    return it == all_.end() ? nullptr : it->second.get();
  }
  void forget(uint64_t arrival) {
    auto it = all_.find(arrival);
    if (it != all_.end() && it->second->finished) all_.erase(it);
  }

  // One iteration (engine.rs:1367-1407). 0 on success; on a model error every request is failed and the pools reset.
  int step() {
    if (has_inflight_) {
      InFlight prev = std::move(inflight_);
      has_inflight_ = false;
      bool still = false;
      int rc = pipelined_turn(prev, &still);
      if (rc != 0) { fail_all(err_); return rc; }
      if (still) { cache_io_tick(0); return 0; }  // a new step is in flight: only the (cheap) write acks are applied
    }
    sweep_cancelled();
    admit();
    if (running_.empty()) {
      cache_io_tick(FLUSH_BATCH);   // idle: write-behind progress never depends on new traffic
      return 0;
    }
    int rc = run_iteration();
    if (rc != 0) fail_all(err_);
    else if (!has_inflight_) cache_io_tick(FLUSH_BATCH);
    return rc;
  }

 private:
  typedef std::shared_ptr<Seq> SeqP;

  // A decode step that has been queued on the device and not read back (engine.rs:790-793): per row the request it
  // belongs to; the row index doubles as the feed index of the next launch.
  struct InFlight {
    uint64_t ticket = 0;
    size_t width = 0;                                  // rows the launch sampled
    std::vector<std::pair<uint64_t, int32_t>> rows;    // (arrival, row of the launch)
  };

  struct DecodePlan {  // engine.rs:795-803
    size_t seq;
    bool sample;
    size_t len, offset;
    std::vector<uint32_t> blocks;
    bool has_draft = false;
    std::vector<uint32_t> draft;
  };

  void sweep_cancelled() {  // engine.rs:1771-1789
    for (auto& s : waiting_) if (s->cancel) finish(*s, FINISH_CANCELLED, true);
    for (auto& s : running_) if (s->cancel) finish(*s, FINISH_CANCELLED, true);
    release_finished_drafts();
    retain_unfinished(waiting_);
    running_.erase(std::remove_if(running_.begin(), running_.end(), [](const SeqP& s) { return s->finished; }), running_.end());
  }
  static void retain_unfinished(std::deque<SeqP>& q) {
    q.erase(std::remove_if(q.begin(), q.end(), [](const SeqP& s) { return s->finished; }), q.end());
  }

  // engine.rs:1802-1848 without priorities/preemption: admit while the head's projection fits, evicting cache-only blocks first.
  void admit() {
    for (;;) {
      bool mid_prefill = false;
      for (auto& s : running_) if (!s->finished && !s->decoding()) mid_prefill = true;
      if (mid_prefill || running_.size() >= (size_t)cfg_.max_batch_tokens) return;
      match_head_prefix();
      if (waiting_.empty()) return;
      Seq& head = *waiting_.front();
      const size_t needed = head.admission_blocks(mgr_.block_size());
      while (mgr_.num_free() < needed) {
        if (!evict_one()) return;
      }
      running_.push_back(waiting_.front());
      waiting_.pop_front();
    }
  }
  bool evict_one() {  // engine.rs:584-589
    if (!radix_) return false;
    const int64_t node = radix_->evict_candidate(mgr_);
    if (node < 0) return false;
    return radix_->evict(mgr_, (size_t)node) >= 0;
  }

  // engine.rs:1868-2033 minus the SSD tier.
  void match_head_prefix() {
    if (!radix_ || waiting_.empty()) return;
    Seq& seq = *waiting_.front();
    if (seq.cache_checked) return;
    seq.cache_checked = true;
    if (seq.processed != 0 || !seq.table.blocks().empty()) return;
    const size_t bs = mgr_.block_size();
    const size_t limit = seq.prompt.size() - 1;  // the last prompt token is always computed
    size_t cur = RADIX_ROOT;
    std::vector<uint32_t> walked;
    bool from_ssd = false;
    while ((walked.size() + 1) * bs <= limit) {
      const size_t at = walked.size() * bs;
      std::vector<uint32_t> chunk(seq.prompt.begin() + at, seq.prompt.begin() + at + bs);
      const int64_t node = resolve_chunk(cur, chunk, &from_ssd);
      if (node < 0) break;
      const int64_t block = radix_->node_block((size_t)node);
      if (block < 0) break;
      radix_->touch((size_t)node);
      walked.push_back((uint32_t)block);
      cur = (size_t)node;
    }
    const size_t d_full = walked.size() * bs;
    const size_t r = limit - d_full;
    bool has_tail = false;
    uint32_t tail = 0;
    if (r > 0 && r < bs) {  // containment probe (engine.rs:1918-1964)
      const std::vector<uint32_t> want(seq.prompt.begin() + d_full, seq.prompt.begin() + limit);
      auto starts_with = [&](const std::vector<uint32_t>& t) { return t.size() >= want.size() && std::equal(want.begin(), want.end(), t.begin()); };
      int64_t cand = -1;
      for (size_t node : radix_->full_children(cur)) if (starts_with(radix_->node_tokens(node))) { cand = (int64_t)node; break; }
      if (cand < 0)
        for (size_t node : radix_->partial_children(cur)) if (starts_with(radix_->node_tokens(node))) { cand = (int64_t)node; break; }
      if (cand < 0 && store_ && seq.prompt.size() >= d_full + bs) {
        // hash-first discovery needs a full chunk's tokens, which the request has when exactly one position is left
        const std::vector<uint32_t> chunk(seq.prompt.begin() + d_full, seq.prompt.begin() + d_full + bs);
        if (store_->contains(radix_->chain_hash_of(cur, chunk.data(), chunk.size()))) {
          cand = (int64_t)radix_->insert_child(cur, chunk);
          radix_->set_on_ssd((size_t)cand);
        }
      }
      if (cand >= 0 && radix_->node_block((size_t)cand) < 0 && !radix_->node_is_partial((size_t)cand) && radix_->node_on_ssd((size_t)cand) && store_) {
        const std::vector<uint32_t> toks = radix_->node_tokens((size_t)cand);
        if (load_from_ssd((size_t)cand, toks)) from_ssd = true;
        else cand = -1;   // the node was pruned
      }
      if (cand >= 0 && radix_->node_block((size_t)cand) >= 0) {
        radix_->touch((size_t)cand);
        tail = (uint32_t)radix_->node_block((size_t)cand);
        has_tail = true;
      }
    }
    size_t serve_full, serve_tail_rows;
    if (r == 0 || has_tail) {
      serve_full = walked.size();
      serve_tail_rows = r;
    } else {  // trim to a resumable boundary of the canonical schedule (engine.rs:1975-1985)
      const size_t pc = cfg_.prefill_chunk;
      const size_t fine = std::min(std::max<size_t>(cfg_.prefill_fine_chunk, 1), pc);
      const size_t tail_start = limit / pc * pc;
      const size_t m = d_full >= tail_start ? std::max(tail_start, d_full / fine * fine) : d_full / pc * pc;
      has_tail = (m % bs) != 0;
      if (has_tail) tail = walked[m / bs];
      serve_full = m / bs;
      serve_tail_rows = m % bs;
    }
    size_t served = 0;
    for (size_t i = 0; i < serve_full; ++i) {
      if (!mgr_.retain(walked[i]).ok()) break;
      if (!seq.table.push_full_block(walked[i], bs).ok()) { mgr_.release(walked[i]); break; }
      served += bs;
    }
    if (served == serve_full * bs && serve_tail_rows > 0 && has_tail && mgr_.retain(tail).ok()) {
      if (seq.table.push_partial_block(tail, serve_tail_rows, bs).ok()) served += serve_tail_rows;
      else mgr_.release(tail);
    }
    if (served == 0) return;
    seq.processed = served;
    if (seq.processed + 1 == seq.prompt.size() && seq.history.empty()) seq.history.push_back(seq.prompt[seq.processed]);
    seq.cached_tokens = std::max<uint32_t>(seq.cached_tokens, (uint32_t)served);
    cache_stats_.hits_total++;
    cache_stats_.tokens_reused_total += served;
    if (from_ssd) cache_stats_.ssd_hits_total++;
  }

  // engine.rs:1412-1426: apply writer acks, capture up to `captures` queued blocks.
  void cache_io_tick(size_t captures) {
    if (!store_) return;
    for (const FlushAck& a : store_->drain_acks()) apply_ack(a);
    if (captures > 0) flush_entries(captures);
  }
  void apply_ack(const FlushAck& ack) {  // engine.rs:2693-2704
    if (!radix_->is_live(ack.node, ack.generation) || radix_->node_hash(ack.node) != ack.hash) return;
    if (ack.ok) radix_->set_on_ssd(ack.node);
    else radix_->clear_flush_pending(ack.node);   // a later donation may retry
  }
  size_t flush_entries(size_t max) {  // engine.rs:2645-2690
    size_t flushed = 0;
    while (flushed < max && !flush_queue_.empty()) {
      const auto [node, generation] = flush_queue_.front();
      flush_queue_.pop_front();
      if (!radix_->is_live(node, generation) || radix_->node_on_ssd(node) || radix_->flush_pending(node)) continue;
      const int64_t block = radix_->node_block(node);
      if (block < 0) continue;
      std::vector<uint8_t> payload(slab_geometry_.payload_bytes(io_.dtype_size));
      if (!io_.read || io_.read(model_.kv, (uint32_t)block, payload.data(), payload.size()) != 0) continue;   // silent skip
      const auto& toks = radix_->node_tokens(node);
      store_->enqueue_write(FlushTicket{node, generation, radix_->node_hash(node)}, toks.data(), toks.size(), std::move(payload), io_.dtype_tag,
                            io_.dtype_size);
      radix_->set_flush_pending(node);
      flushed++;
    }
    return flushed;
  }
  // engine.rs:2596-2640: pulls one persisted block into the pool for a non-resident node; failures are silent.
  bool load_from_ssd(size_t node, const std::vector<uint32_t>& chunk) {
    std::vector<uint8_t> payload;
    uint32_t tag = 0;
    if (!store_->read(radix_->node_hash(node), chunk.data(), chunk.size(), (int64_t)io_.dtype_tag, &payload, &tag)) {
      radix_->prune_subtree(mgr_, node);   // the store dropped its entry: drop the dead subtree too
      return false;
    }
    uint32_t block = 0;
    if (!mgr_.allocate(&block).ok()) {
      if (!evict_one() || !mgr_.allocate(&block).ok()) return false;   // the pool is full of live requests: a miss
    }
    if (!io_.write || io_.write(model_.kv, block, payload.data(), payload.size()) != 0) {
      mgr_.release(block);
      return false;
    }
    radix_->set_resident(node, block);
    return true;
  }
  // engine.rs:2559-2594: the child of `cur` keyed by `chunk` for a match walk — an existing node, or hash-first discovery
  // from the SSD index — made resident; -1 stops the walk.
  int64_t resolve_chunk(size_t cur, const std::vector<uint32_t>& chunk, bool* from_ssd) {
    int64_t node = radix_->child(cur, chunk);
    if (node < 0) {
      if (!store_ || !store_->contains(radix_->chain_hash_of(cur, chunk.data(), chunk.size()))) return -1;
      node = (int64_t)radix_->insert_child(cur, chunk);
      radix_->set_on_ssd((size_t)node);
    }
    if (radix_->node_block((size_t)node) < 0) {
      if (!radix_->node_on_ssd((size_t)node) || !store_) { radix_->prune_subtree(mgr_, (size_t)node); return -1; }
      if (!load_from_ssd((size_t)node, chunk)) return -1;
      *from_ssd = true;
    }
    return node;
  }

  int find_running(uint64_t arrival) const {
    for (size_t i = 0; i < running_.size(); ++i) if (running_[i]->arrival == arrival) return (int)i;
    return -1;
  }

  // engine.rs:1482-1500: would the next synchronous step run (or be able to run) a verify round?
  bool spec_would_engage() const {
    if (!has_drafter_ || cfg_.deterministic_decode_width <= 1) return false;
    if (spec_gamma_at_width(cfg_.gamma, cfg_.spec_max_batch, running_.size()) == 0) return false;
    for (auto& s : running_) {
      const size_t remaining = s->max_tokens > s->generated ? s->max_tokens - s->generated : 0;
      if (s->spec_eligible() && remaining >= 2 && (cfg_.max_key_len <= 0 || s->processed + s->fed + 2 <= (size_t)cfg_.max_key_len))
        return true;
    }
    return false;
  }

  // engine.rs:1456-1475: the pipeline spans steady-state decode only. Penalties and grammars do not exist on this path.
  // With the reference's forward grouping (batch_verify = 0) a step wider than the deterministic width is several
  // forwards; that case stays on the synchronous path, which reproduces the grouping.
  bool pipeline_ok() const {
    if (!has_pipe_ || spec_would_engage() || !waiting_.empty()) return false;
    if (!cfg_.batch_verify && running_.size() > (size_t)std::max(cfg_.deterministic_decode_width, 1)) return false;
    for (auto& s : running_) if (!s->decoding() || s->cancel) return false;
    return true;
  }

  // engine.rs:1434-1455.
  int pipelined_turn(InFlight& prev, bool* still) {
    InFlight next;
    bool has_next = false;
    if (pipeline_ok()) {
      int rc = build_pipelined(prev, &next, &has_next);
      if (rc != 0) return rc;
    }
    int rc = apply_inflight(prev);
    if (rc != 0) return rc;
    if (!has_next) { *still = false; return 0; }
    // A sequence that stopped or was cancelled at the apply has one speculative row in flight: it is dropped unread.
    // Its KV write went to blocks the sequence owned when the step was built; only settled rows are ever donated.
    next.rows.erase(std::remove_if(next.rows.begin(), next.rows.end(),
                                   [&](const std::pair<uint64_t, int32_t>& r) { return find_running(r.first) < 0; }),
                    next.rows.end());
    if (!next.rows.empty()) {
      pipelined_total_++;
      inflight_ = std::move(next);
      has_inflight_ = true;
    }
    *still = true;
    return 0;
  }

  // engine.rs:1656-1744: the next decode step, fed from prev's unread tokens.
  int build_pipelined(const InFlight& prev, InFlight* out, bool* built) {
    *built = false;
    const size_t bs = mgr_.block_size();
    std::vector<std::pair<size_t, int32_t>> included;  // (index into running_, row of prev)
    size_t new_blocks = 0;
    for (auto& r : prev.rows) {
      const int i = find_running(r.first);
      if (i < 0) return 0;
      Seq& seq = *running_[i];
      if ((size_t)seq.generated + 1 >= seq.max_tokens) continue;  // its final token is in prev
      if (seq.table.num_tokens() == seq.table.blocks().size() * bs) new_blocks++;
      included.push_back({(size_t)i, r.second});
    }
    if (included.empty() || mgr_.num_free() < new_blocks) return 0;  // preemption/eviction stay synchronous decisions
    iterations_++;
    std::vector<DecodePlan> plans(included.size());
    std::vector<SeqStepC> seqs;
    std::vector<uint32_t> ids(included.size(), 0);
    std::vector<int32_t> feed;
    for (size_t j = 0; j < included.size(); ++j) {
      Seq& seq = *running_[included[j].first];
      int rc = build_seq_step(seq, 1, &plans[j]);
      if (rc < 0) return rc;
      if (rc == 0) { err_ = "pipelined append exceeded the precounted pool"; return -1; }
      feed.push_back(included[j].second);
      out->rows.push_back({seq.arrival, (int32_t)j});
    }
    for (auto& p : plans) seqs.push_back(SeqStepC{1, (int32_t)p.offset, 1, (int32_t)p.blocks.size(), p.blocks.data()});
    forwards_++;
    int rc = pipe_.launch(model_.model, model_.kv, ids.data(), feed.data(), seqs.data(), (int32_t)seqs.size(), &out->ticket);
    if (rc != 0) { err_ = "pipelined decode launch failed with status " + std::to_string(rc); return rc; }
    out->width = included.size();
    *built = true;
    return 0;
  }

  // engine.rs:1748-1766: read a scheduled step back and settle it.
  int apply_inflight(const InFlight& prev) {
    std::vector<uint32_t> tokens(std::max<size_t>(prev.width, 1));
    int rc = pipe_.collect(model_.model, prev.ticket, tokens.data(), (int32_t)prev.width);
    if (rc != 0) { err_ = "pipelined decode collect failed with status " + std::to_string(rc); return rc; }
    for (auto& r : prev.rows) {
      const int i = find_running(r.first);
      if (i < 0) continue;
      settle_sampled(*running_[i], tokens[r.second]);
    }
    release_finished_drafts();
    running_.erase(std::remove_if(running_.begin(), running_.end(), [](const SeqP& s) { return s->finished; }), running_.end());
    return 0;
  }

  // engine.rs:1508-1596.
  bool collect_proposal(size_t i, std::vector<uint32_t>* out) {
    if (!has_drafter_ || !logits_vocab_known_) return false;
    const size_t width_gamma = spec_gamma_at_width(cfg_.gamma, cfg_.spec_max_batch, running_.size());
    if (width_gamma == 0) return false;
    Seq& seq = *running_[i];
    if (!seq.spec_eligible()) return false;
    const size_t remaining = seq.max_tokens > seq.generated ? seq.max_tokens - seq.generated : 0;
    const size_t offset = seq.processed + seq.fed;
    size_t gamma = std::min(width_gamma, (size_t)std::max(cfg_.deterministic_decode_width - 1, 0));
    gamma = std::min(gamma, remaining > 0 ? remaining - 1 : 0);
    if (cfg_.max_key_len > 0) {
      const size_t room = (size_t)cfg_.max_key_len > offset + 1 ? (size_t)cfg_.max_key_len - (offset + 1) : 0;
      gamma = std::min(gamma, room);
    }
    if (gamma == 0) return false;
    int rc = 0;
    std::vector<uint32_t> proposal(gamma);
    int32_t n_out = 0;
    if (!seq.draft_begun) {
      rc = drafter_.begin(drafter_.user, seq.arrival, seq.prompt.data(), (int32_t)seq.prompt.size());
      if (rc == 0) { seq.draft_begun = true; seq.draft_committed = 0; }
    }
    if (rc == 0) {
      // history[0] is the last prompt token; everything after it the drafter has not seen is newly committed
      const uint32_t* committed = seq.history.data() + 1 + seq.draft_committed;
      const size_t n_committed = seq.history.size() - 1 - seq.draft_committed;
      rc = drafter_.propose(drafter_.user, seq.arrival, committed, (int32_t)n_committed, (int32_t)gamma, proposal.data(), &n_out);
      if (rc == 0) seq.draft_committed = seq.history.size() - 1;
    }
    if (rc != 0) {  // a draft fault never fails a generation (engine.rs:1586-1594)
      spec_.draft_errors_total++;
      seq.draft_dead = true;
      if (seq.draft_begun) { drafter_.release(drafter_.user, seq.arrival); seq.draft_begun = false; }
      return false;
    }
    proposal.resize(std::min<size_t>(std::max(n_out, 0), gamma));
    for (size_t k = 0; k < proposal.size(); ++k)
      if ((int64_t)proposal[k] >= (int64_t)model_.vocab) { proposal.resize(k); break; }  // engine.rs:1580-1582
    if (proposal.empty()) return false;
    *out = proposal;
    return true;
  }

  void maybe_stand_down(size_t i) {  // engine.rs:1607-1634
    Seq& seq = *running_[i];
    if (cfg_.spec_min_acceptance <= 0.0 || seq.finished || seq.draft_standdown || seq.draft_dead ||
        seq.spec_proposed < SPEC_ACCEPTANCE_WARMUP_PROPOSED ||
        (double)seq.spec_accepted >= cfg_.spec_min_acceptance * (double)seq.spec_proposed)
      return;
    seq.draft_standdown = true;
    spec_.standdowns_total++;
    if (seq.draft_begun && has_drafter_) { drafter_.release(drafter_.user, seq.arrival); seq.draft_begun = false; }
  }

  void release_finished_drafts() {  // engine.rs:1640-1649
    if (!has_drafter_) return;
    for (auto& s : waiting_) if (s->finished && s->draft_begun) { drafter_.release(drafter_.user, s->arrival); s->draft_begun = false; }
    for (auto& s : running_) if (s->finished && s->draft_begun) { drafter_.release(drafter_.user, s->arrival); s->draft_begun = false; }
  }

  // build_seq_step (engine.rs:2736-2796): append slots, execute the copy-on-write, snapshot the blocks.
  // Returns 1 when planned, 0 when the pool is exhausted, -1 on a model error.
  int build_seq_step(Seq& seq, size_t len, DecodePlan* plan) {
    const size_t offset = seq.table.num_tokens();
    AppendPlan ap;
    BlockStatus st = seq.table.append_tokens(mgr_, len, &ap);
    if (st.err == BlockErr::OutOfBlocks) return 0;
    if (!st.ok()) { err_ = st.message(); return -1; }
    if (ap.has_cow && model_.copy_block(model_.kv, ap.cow_src, ap.cow_dst) != 0) { err_ = "copy_block failed"; return -1; }
    plan->len = len;
    plan->offset = offset;
    plan->blocks = seq.table.blocks();
    return 1;
  }

  // plan_step (engine.rs:2424-...): here only cache eviction can make room; preemption is out of scope.
  int plan_step(size_t i, size_t len, DecodePlan* plan) {
    for (;;) {
      int rc = build_seq_step(*running_[i], len, plan);
      if (rc != 0) return rc;
      if (!evict_one()) {
        err_ = "block pool exhausted and nothing evictable (preemption is not part of this path)";
        return -2;
      }
    }
  }

  // settle_sampled (engine.rs:907-963).
  void settle_sampled(Seq& seq, uint32_t token) {
    if (seq.finished) return;
    seq.generated += 1;
    seq.history.push_back(token);
    seq.fed += 1;
    if (seq.cancel) { finish(seq, FINISH_CANCELLED, true); return; }
    if (std::find(seq.stop_tokens.begin(), seq.stop_tokens.end(), token) != seq.stop_tokens.end()) {
      finish(seq, FINISH_STOP, true);  // counted in usage, not emitted
      return;
    }
    seq.emitted.push_back(token);
    if (seq.generated >= seq.max_tokens) finish(seq, FINISH_LENGTH, true);
  }

  // finish (engine.rs:736-778): donate the settled blocks to the prefix cache on clean finishes, release otherwise.
  void finish(Seq& seq, int32_t kind, bool donate_ok) {
    if (seq.finished) return;
    seq.finished = true;
    seq.finish_kind = kind;
    if (radix_ && donate_ok && kind != FINISH_ERROR) donate(seq);
    else seq.table.release(mgr_);
  }

  // CacheState::donate (engine.rs:601-689). Every request on this path is greedy, i.e. deterministic.
  void donate(Seq& seq) {
    const size_t bs = radix_->block_size();
    const size_t settled = seq.processed + seq.fed;
    std::vector<uint32_t> blocks = seq.table.into_blocks();
    const size_t full = std::min(settled / bs, blocks.size());
    auto token_at = [&](size_t pos) { return pos < seq.processed ? seq.prompt[pos] : seq.history[pos - seq.processed]; };
    size_t cur = RADIX_ROOT;
    std::vector<uint32_t> chunk;
    for (size_t i = 0; i < blocks.size(); ++i) {
      const uint32_t block = blocks[i];
      if (i > full || (i == full && settled % bs == 0)) { mgr_.release(block); continue; }
      chunk.clear();
      for (size_t pos = i * bs; pos < std::min((i + 1) * bs, settled); ++pos) chunk.push_back(token_at(pos));
      if (i == full) { donate_partial(cur, block, chunk); continue; }
      const int64_t found = radix_->child(cur, chunk);
      if (found >= 0) {
        if (radix_->node_block((size_t)found) >= 0) mgr_.release(block);  // already resident: drop the duplicate ref
        else radix_->set_resident((size_t)found, block);
        radix_->touch((size_t)found);
        cur = (size_t)found;
      } else {
        const size_t node = radix_->insert_child(cur, chunk);
        radix_->set_resident(node, block);
        if (store_ && store_->contains(radix_->node_hash(node))) radix_->set_on_ssd(node);   // a previous run persisted it
        std::vector<size_t> covered;
        for (size_t partial : radix_->partial_children(cur)) {
          const auto& t = radix_->node_tokens(partial);
          if (t.size() <= chunk.size() && std::equal(t.begin(), t.end(), chunk.begin())) covered.push_back(partial);
        }
        for (size_t partial : covered) radix_->prune_subtree(mgr_, partial);
        cur = node;
      }
      if (store_ && !radix_->node_on_ssd(cur) && !radix_->flush_pending(cur)) flush_queue_.push_back({cur, radix_->node_generation(cur)});
    }
  }
  void donate_partial(size_t parent, uint32_t block, const std::vector<uint32_t>& tokens) {  // engine.rs:694-731
    auto starts_with = [](const std::vector<uint32_t>& a, const std::vector<uint32_t>& prefix) {
      return a.size() >= prefix.size() && std::equal(prefix.begin(), prefix.end(), a.begin());
    };
    for (size_t node : radix_->full_children(parent))
      if (radix_->node_block(node) >= 0 && starts_with(radix_->node_tokens(node), tokens)) { mgr_.release(block); return; }
    const std::vector<size_t> partials = radix_->partial_children(parent);
    for (size_t node : partials) {
      if (starts_with(radix_->node_tokens(node), tokens)) { mgr_.release(block); return; }
      if (starts_with(tokens, radix_->node_tokens(node))) {
        const int64_t old = radix_->upgrade_partial(node, tokens, block);
        if (old >= 0) mgr_.release((uint32_t)old);
        return;
      }
    }
    const size_t node = radix_->insert_partial_child(parent, tokens);
    radix_->set_resident(node, block);
  }

  // One forward over `plans` (+ optionally the prefill segment). Fills rows per plan.
  int forward(const std::vector<DecodePlan*>& plans, const DecodePlan* prefill, const std::vector<uint32_t>* prefill_tokens,
              std::vector<std::vector<uint32_t>>* rows_out) {
    std::vector<uint32_t> ids;
    std::vector<SeqStepC> seqs;
    size_t n_sampled = 0;
    for (DecodePlan* p : plans) {
      Seq& seq = *running_[p->seq];
      ids.push_back(seq.history[seq.fed]);
      ids.insert(ids.end(), p->draft.begin(), p->draft.end());
      seqs.push_back(SeqStepC{(int32_t)p->len, (int32_t)p->offset, p->sample ? (int32_t)p->len : 0, (int32_t)p->blocks.size(), p->blocks.data()});
      if (p->sample) n_sampled += p->len;
    }
    if (prefill) {
      ids.insert(ids.end(), prefill_tokens->begin(), prefill_tokens->end());
      seqs.push_back(SeqStepC{(int32_t)prefill->len, (int32_t)prefill->offset, 0, (int32_t)prefill->blocks.size(), prefill->blocks.data()});
    }
    if (seqs.empty()) return 0;
    std::vector<uint32_t> row_tokens(std::max<size_t>(n_sampled, 1));
    std::vector<int32_t> ncom(seqs.size()), nacc(seqs.size());
    forwards_++;
    int rc = model_.verify_step(model_.model, model_.kv, ids.data(), (int32_t)ids.size(), seqs.data(), (int32_t)seqs.size(),
                                row_tokens.data(), ncom.data(), nacc.data());
    if (rc != 0) { err_ = "model forward failed with status " + std::to_string(rc); return rc; }
    size_t at = 0;
    for (DecodePlan* p : plans) {
      std::vector<uint32_t> r;
      if (p->sample) { r.assign(row_tokens.begin() + at, row_tokens.begin() + at + p->len); at += p->len; }
      rows_out->push_back(r);
    }
    return 0;
  }

  // run_iteration (engine.rs:2035-2417).
  int run_iteration() {
    iterations_++;
    std::vector<DecodePlan> plans;
    plans.reserve(running_.size());
    for (size_t i = 0; i < running_.size(); ++i) {
      Seq& seq = *running_[i];
      if (seq.finished || !seq.decoding()) continue;
      const bool sample = seq.fed + 1 == seq.history.size();
      DecodePlan plan;
      plan.seq = i;
      plan.sample = sample;
      std::vector<uint32_t> proposal;
      if (sample && collect_proposal(i, &proposal)) {
        // Speculation never evicts or preempts: if the pool cannot cover the wider segment, fall back (engine.rs:2081-2104).
        int rc = build_seq_step(seq, 1 + proposal.size(), &plan);
        if (rc < 0) return rc;
        if (rc == 1) {
          plan.has_draft = true;
          plan.draft = proposal;
          plans.push_back(plan);
          continue;
        }
      }
      int rc = plan_step(i, 1, &plan);
      if (rc < 0) return rc;
      plans.push_back(plan);
    }
    // at most one prefill chunk per iteration (engine.rs:2114-2162); no kernel-class pad rows on this backend
    bool has_prefill = false;
    DecodePlan prefill_plan;
    std::vector<uint32_t> prefill_tokens;
    size_t prefill_seq = 0;
    for (size_t i = 0; i < running_.size(); ++i) {
      Seq& seq = *running_[i];
      if (seq.finished || seq.decoding()) continue;
      size_t used = 0;
      for (auto& p : plans) used += p.len;
      const size_t budget = (size_t)cfg_.max_batch_tokens > used ? (size_t)cfg_.max_batch_tokens - used : 0;
      const size_t at = seq.processed;
      const size_t chunk = std::min(canonical_prefill_len(at, seq.prompt.size() - 1, cfg_.prefill_chunk, cfg_.prefill_fine_chunk), budget);
      if (chunk > 0) {
        prefill_plan.seq = i;
        prefill_plan.sample = false;
        int rc = plan_step(i, chunk, &prefill_plan);
        if (rc < 0) return rc;
        prefill_tokens.assign(seq.prompt.begin() + at, seq.prompt.begin() + at + chunk);
        has_prefill = true;
        prefill_seq = i;
      }
      break;
    }

    // Pipeline entry (engine.rs:2272-2297): a steady-state pure-decode step defers its read-back; the next step is built
    // from its still-unread tokens at the start of the next step() call, while the device executes this one.
    {
      bool all_plain = !has_prefill && plans.size() == running_.size() && !plans.empty();
      for (auto& p : plans) all_plain = all_plain && p.sample && !p.has_draft;
      if (all_plain && pipeline_ok()) {
        std::vector<uint32_t> ids;
        std::vector<int32_t> feed(plans.size(), -1);
        std::vector<SeqStepC> seqs;
        InFlight f;
        for (size_t j = 0; j < plans.size(); ++j) {
          Seq& seq = *running_[plans[j].seq];
          ids.push_back(seq.history[seq.fed]);
          seqs.push_back(SeqStepC{1, (int32_t)plans[j].offset, 1, (int32_t)plans[j].blocks.size(), plans[j].blocks.data()});
          f.rows.push_back({seq.arrival, (int32_t)j});
        }
        forwards_++;
        int rc = pipe_.launch(model_.model, model_.kv, ids.data(), feed.data(), seqs.data(), (int32_t)seqs.size(), &f.ticket);
        if (rc != 0) { err_ = "pipelined decode launch failed with status " + std::to_string(rc); return rc; }
        f.width = plans.size();
        logits_vocab_known_ = true;
        pipelined_total_++;
        inflight_ = std::move(f);
        has_inflight_ = true;
        return 0;
      }
    }

    // FORWARD. Reference grouping: prefill first, then plain-decode groups of at most deterministic_decode_width rows,
    // then one forward per verify segment (engine.rs:2170-2271). Row-invariant backend: everything in one forward.
    std::vector<std::vector<uint32_t>> rows(plans.size());
    if (cfg_.batch_verify) {
      std::vector<DecodePlan*> all;
      for (auto& p : plans) all.push_back(&p);
      std::vector<std::vector<uint32_t>> out;
      int rc = forward(all, has_prefill ? &prefill_plan : nullptr, &prefill_tokens, &out);
      if (rc != 0) return rc;
      rows = out;
    } else {
      if (has_prefill) {
        std::vector<std::vector<uint32_t>> out;
        int rc = forward({}, &prefill_plan, &prefill_tokens, &out);
        if (rc != 0) return rc;
      }
      std::vector<size_t> plain;
      for (size_t j = 0; j < plans.size(); ++j) if (!plans[j].has_draft) plain.push_back(j);
      const size_t width = std::max(cfg_.deterministic_decode_width, 1);
      for (size_t g0 = 0; g0 < plain.size(); g0 += width) {
        std::vector<DecodePlan*> group;
        for (size_t g = g0; g < std::min(plain.size(), g0 + width); ++g) group.push_back(&plans[plain[g]]);
        std::vector<std::vector<uint32_t>> out;
        int rc = forward(group, nullptr, nullptr, &out);
        if (rc != 0) return rc;
        for (size_t g = 0; g < group.size(); ++g) rows[plain[g0 + g]] = out[g];
      }
      for (size_t j = 0; j < plans.size(); ++j) {
        if (!plans[j].has_draft) continue;
        std::vector<std::vector<uint32_t>> out;
        int rc = forward({&plans[j]}, nullptr, nullptr, &out);
        if (rc != 0) return rc;
        rows[j] = out[0];
      }
    }
    bool any_sampled = false;
    for (auto& p : plans) any_sampled |= p.sample;
    if (any_sampled) logits_vocab_known_ = true;  // speculation waits for the first sampled forward (engine.rs:2226)

    // SETTLE: plain rows first, then replay, then verify rounds (engine.rs:2313-2383).
    for (size_t j = 0; j < plans.size(); ++j) {
      DecodePlan& p = plans[j];
      if (p.has_draft) continue;
      if (p.sample) settle_sampled(*running_[p.seq], rows[j][0]);
      else running_[p.seq]->fed += 1;
    }
    for (size_t j = 0; j < plans.size(); ++j) {
      DecodePlan& p = plans[j];
      if (!p.has_draft) continue;
      Seq& seq = *running_[p.seq];
      spec_.rounds_total++;
      spec_.proposed_total += p.draft.size();
      seq.spec_proposed += (uint32_t)p.draft.size();
      size_t accepted = 0, committed = 0;
      for (size_t r = 0; r < rows[j].size(); ++r) {
        if (seq.finished) break;
        const uint32_t token = rows[j][r];
        const bool agrees = r < p.draft.size() && token == p.draft[r];
        if (agrees) { accepted++; seq.spec_accepted++; }
        settle_sampled(seq, token);
        committed++;
        if (!agrees) break;
      }
      spec_.accepted_total += accepted;
      const size_t stale = 1 + p.draft.size() > committed ? 1 + p.draft.size() - committed : 0;
      if (stale > 0) {
        spec_.rollback_rounds_total++;
        spec_.rollback_tokens_total += stale;
        if (!seq.finished) {
          BlockStatus st = seq.table.truncate(mgr_, seq.processed + seq.fed);  // ROLLBACK (block.rs:381-396)
          if (!st.ok()) { err_ = st.message(); return -1; }
        }
      }
      maybe_stand_down(p.seq);
    }
    if (has_prefill) {  // engine.rs:2387-2393
      Seq& seq = *running_[prefill_seq];
      seq.processed += prefill_tokens.size();
      if (seq.processed + 1 == seq.prompt.size() && seq.history.empty()) seq.history.push_back(seq.prompt[seq.processed]);
    }
    release_finished_drafts();
    running_.erase(std::remove_if(running_.begin(), running_.end(), [](const SeqP& s) { return s->finished; }), running_.end());
    return 0;
  }

  void fail_all(const std::string& why) {  // engine.rs:2519-2553
    for (auto& s : running_) { s->error = why; finish(*s, FINISH_ERROR, false); }
    for (auto& s : waiting_) { s->error = why; finish(*s, FINISH_ERROR, false); }
    release_finished_drafts();
    running_.clear();
    waiting_.clear();
    has_inflight_ = false;  // engine.rs:2521
    flush_queue_.clear();
    mgr_ = BlockManager(cfg_.num_blocks, cfg_.block_size);
    if (radix_) radix_->reset();
  }

  EngineConfig cfg_;
  StepModelVT model_;
  DrafterVT drafter_{};
  bool has_drafter_ = false;
  std::unique_ptr<SsdStore> store_;
  BlockIoVT io_{};
  SlabGeometry slab_geometry_{};
  std::deque<std::pair<size_t, uint64_t>> flush_queue_;   // (node, generation) awaiting capture
  DecodePipelineVT pipe_{};
  bool has_pipe_ = false, has_inflight_ = false;
  InFlight inflight_;
  uint64_t pipelined_total_ = 0;
  BlockManager mgr_;
  std::unique_ptr<RadixCache> radix_;
  std::deque<SeqP> waiting_;
  std::vector<SeqP> running_;
  std::map<uint64_t, SeqP> all_;
  SpecStats spec_;
  PrefixCacheStats cache_stats_;
  bool logits_vocab_known_ = false;
  uint64_t next_arrival_ = 0, iterations_ = 0, forwards_ = 0;
  std::string err_;
};

// ---------------------------------------------------------------------------
// Drafters
// ---------------------------------------------------------------------------

// A scripted drafter with seeded acceptance injection: position j of a proposal equals the
// target's known greedy continuation with probability p, else a uniform-random id. Same shape
// as the reference tests' OracleDrafter / AdversarialDrafter (crates/kiln-models/tests/spec_decode.rs:147-198).
class ScriptedDrafter {
 public:
  ScriptedDrafter(double p, uint64_t seed, uint32_t vocab) : p_(p), seed_(seed), vocab_(vocab) {}
  void set_continuation(uint64_t seq, const uint32_t* toks, size_t n) { cont_[seq].assign(toks, toks + n); }
  int begin(uint64_t seq, const uint32_t*, int32_t) { done_[seq] = 0; return 0; }
  int propose(uint64_t seq, const uint32_t*, int32_t n_committed, int32_t gamma, uint32_t* out, int32_t* n_out) {
    auto it = done_.find(seq);
    if (it == done_.end()) return 1;  // DraftError::UnknownSeq
    it->second += (size_t)n_committed;
    const size_t done = it->second;
    const std::vector<uint32_t>& c = cont_[seq];
    int32_t n = 0;
    for (int32_t j = 0; j < gamma; ++j) {
      const size_t pos = done + j;
      const uint64_t r = mix(seed_ ^ mix(seq * 0x9E3779B97F4A7C15ull + pos));
      const double u = (double)(r >> 11) * (1.0 / 9007199254740992.0);
      uint32_t tok;
      if (pos < c.size() && u < p_) tok = c[pos];
      else tok = (uint32_t)(mix(r) % vocab_);
      out[n++] = tok;
    }
    *n_out = n;
    return 0;
  }
  void release(uint64_t seq) { done_.erase(seq); }
  DrafterVT vtable() {
    return DrafterVT{this,
                     [](void* u, uint64_t s, const uint32_t* p, int32_t n) { return ((ScriptedDrafter*)u)->begin(s, p, n); },
                     [](void* u, uint64_t s, const uint32_t* c, int32_t nc, int32_t g, uint32_t* o, int32_t* no) {
                       return ((ScriptedDrafter*)u)->propose(s, c, nc, g, o, no);
                     },
                     [](void* u, uint64_t s) { ((ScriptedDrafter*)u)->release(s); }};
  }

 private:
  static uint64_t mix(uint64_t z) {  // splitmix64 finaliser
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
  double p_;
  uint64_t seed_;
  uint32_t vocab_;
  std::map<uint64_t, std::vector<uint32_t>> cont_;
  std::map<uint64_t, size_t> done_;
};

// The draft-model seam: forward has the signature of kc_verify_step, chain of kc_draft_chain.
struct DraftModelVT {
  void* model;
  void* kv;
  uint64_t weights_bytes = 0, kv_allocated_bytes = 0, kv_block_bytes = 0;   // for Drafter::memory (draft.rs:259-266)
  int (*forward)(void* model, void* kv, const uint32_t* ids, int32_t n, const SeqStepC* seqs, int32_t n_seqs, uint32_t* row_tokens,
                 int32_t* n_committed, int32_t* n_accepted);
  int (*chain)(void* model, void* kv, uint32_t first_token, int32_t offset, const uint32_t* blocks, int32_t n_blocks, int32_t gamma,
               uint32_t* proposal);
  int32_t max_chunk;  // tokens per catch-up forward (DRAFT_PREFILL_CHUNK = 2048 in the reference, draft.rs:51)
};

// DraftModel: Drafter (draft.rs:95-122, 258-412): own block manager and tables over the draft's own pool.
class DraftModel {
 public:
  DraftModel(const DraftModelVT& vt, size_t num_blocks, size_t block_size) : vt_(vt), mgr_(num_blocks, block_size) {}
  BlockManager& block_manager() { return mgr_; }
  size_t live_sequences() const { return seqs_.size(); }
  DrafterMemory memory() const {  // draft.rs:259-266
    DrafterMemory m;
    m.weights_bytes = vt_.weights_bytes;
    m.kv_allocated_bytes = vt_.kv_allocated_bytes;
    m.kv_used_bytes = (uint64_t)(mgr_.capacity() - mgr_.num_free()) * vt_.kv_block_bytes;
    return m;
  }

  int begin(uint64_t seq, const uint32_t* prompt, int32_t n) {  // draft.rs:268-284
    auto it = seqs_.find(seq);
    if (it != seqs_.end()) { it->second.table.release(mgr_); seqs_.erase(it); }
    DraftSeq s;
    s.context.assign(prompt, prompt + n);
    seqs_[seq] = std::move(s);
    return 0;
  }
  int propose(uint64_t seq, const uint32_t* committed, int32_t n_committed, int32_t gamma, uint32_t* out, int32_t* n_out) {
    *n_out = 0;
    auto it = seqs_.find(seq);
    if (it == seqs_.end()) return 1;  // DraftError::UnknownSeq
    DraftSeq& st = it->second;
    // reconcile (draft.rs:296-324)
    const size_t base = std::min(st.context.size(), st.fed.size());
    st.context.insert(st.context.end(), committed, committed + n_committed);
    size_t keep = base;
    while (keep < st.fed.size() && keep < st.context.size() && st.fed[keep] == st.context[keep]) keep++;
    if (keep < st.fed.size()) {
      if (!st.table.truncate(mgr_, keep).ok()) return 2;
      st.fed.resize(keep);
    }
    if (st.table.num_tokens() != st.fed.size() && !st.table.truncate(mgr_, st.fed.size()).ok()) return 2;
    const size_t len = st.context.size();
    if (gamma == 0 || len == 0 || st.fed.size() >= len) return 0;  // a legal "no speculation this round"
    // catch up (draft.rs:333-352)
    const size_t last = len - 1;
    size_t at = st.fed.size();
    while (at < last) {
      const size_t chunk = std::min(last - at, (size_t)std::max(vt_.max_chunk, 1));
      const size_t offset = st.table.num_tokens();
      AppendPlan ap;
      if (!st.table.append_tokens(mgr_, chunk, &ap).ok()) return 3;  // DraftError::Capacity
      SeqStepC s{(int32_t)chunk, (int32_t)offset, 0, (int32_t)st.table.blocks().size(), st.table.blocks().data()};
      int32_t nc = 0, na = 0;
      uint32_t dummy = 0;
      if (vt_.forward(vt_.model, vt_.kv, st.context.data() + at, (int32_t)chunk, &s, 1, &dummy, &nc, &na) != 0) return 4;
      st.fed.insert(st.fed.end(), st.context.begin() + at, st.context.begin() + at + chunk);
      at += chunk;
    }
    // propose gamma tokens greedily, each argmax feeding the next forward on the device (draft.rs:354-388)
    const size_t offset = st.table.num_tokens();
    AppendPlan ap;
    if (!st.table.append_tokens(mgr_, (size_t)gamma, &ap).ok()) return 3;
    st.fed.push_back(st.context[last]);
    if (vt_.chain(vt_.model, vt_.kv, st.context[last], (int32_t)offset, st.table.blocks().data(), (int32_t)st.table.blocks().size(), gamma, out) != 0)
      return 4;
    *n_out = gamma;
    st.fed.insert(st.fed.end(), out, out + gamma - 1);  // all but the final proposed token were fed (draft.rs:401-402)
    return 0;
  }
  void release(uint64_t seq) {  // draft.rs:406-411
    auto it = seqs_.find(seq);
    if (it != seqs_.end()) { it->second.table.release(mgr_); seqs_.erase(it); }
  }
  DrafterVT vtable() {
    return DrafterVT{this,
                     [](void* u, uint64_t s, const uint32_t* p, int32_t n) { return ((DraftModel*)u)->begin(s, p, n); },
                     [](void* u, uint64_t s, const uint32_t* c, int32_t nc, int32_t g, uint32_t* o, int32_t* no) {
                       return ((DraftModel*)u)->propose(s, c, nc, g, o, no);
                     },
                     [](void* u, uint64_t s) { ((DraftModel*)u)->release(s); },
                     [](void* u, DrafterMemory* o) { *o = ((DraftModel*)u)->memory(); }};
  }

 private:
  struct DraftSeq {  // draft.rs:95-107
    std::vector<uint32_t> context, fed;
    BlockTable table;
  };
  DraftModelVT vt_;
  BlockManager mgr_;
  std::map<uint64_t, DraftSeq> seqs_;
};

}  // namespace kh
