// Paged-KV block bookkeeping: a fixed pool of refcounted blocks with copy-on-write
// and the per-request block tables. C++ equivalent of the reference's
// crates/kiln-engine/src/block.rs:88-426 with the same semantics, including the
// LIFO free list (block.rs:110-111, 167-169) that makes block placement — and so
// the next allocations after a rollback — reproducible.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace kh {

enum class BlockErr : int {
  Ok = 0,
  OutOfBlocks,         // block.rs:43
  NotAllocated,        // block.rs:47
  RefcountOverflow,    // block.rs:50
  InvalidBlockSize,    // block.rs:53
  InvalidCapacity,     // block.rs:56
  TokenCountOverflow,  // block.rs:59
  MisalignedAdoption,  // block.rs:63
};

struct BlockStatus {
  BlockErr err = BlockErr::Ok;
  uint64_t a = 0, b = 0;  // OutOfBlocks: capacity, needed. NotAllocated / RefcountOverflow: id.
  bool ok() const { return err == BlockErr::Ok; }
  std::string message() const {
    switch (err) {
      case BlockErr::Ok: return "ok";
      case BlockErr::OutOfBlocks:
        return "block pool exhausted: " + std::to_string(b) + " free block(s) needed, pool capacity " + std::to_string(a);
      case BlockErr::NotAllocated: return "block " + std::to_string(a) + " is not allocated";
      case BlockErr::RefcountOverflow: return "refcount overflow on block " + std::to_string(a);
      case BlockErr::InvalidBlockSize: return "invalid block size " + std::to_string(a) + ": must be a nonzero power of two";
      case BlockErr::InvalidCapacity: return "invalid pool capacity " + std::to_string(a) + ": must be in 1..=u32::MAX";
      case BlockErr::TokenCountOverflow: return "token count overflow";
      case BlockErr::MisalignedAdoption: return "table is not block-aligned for full-block adoption";
    }
    return "?";
  }
};

struct CowOutcome {
  bool copied = false;  // false: sole owner, write in place (src == dst)
  uint32_t src = 0, dst = 0;
};

class BlockManager {
 public:
  static BlockStatus validate(uint64_t capacity, uint64_t block_size) {
    if (block_size == 0 || (block_size & (block_size - 1)) != 0) return {BlockErr::InvalidBlockSize, block_size, 0};
    if (capacity == 0 || capacity > 0xFFFFFFFFull) return {BlockErr::InvalidCapacity, capacity, 0};
    return {};
  }
  BlockManager(size_t capacity, size_t block_size) : block_size_(block_size), refcounts_(capacity, 0) {
    free_.reserve(capacity);
    for (size_t i = capacity; i-- > 0;) free_.push_back((uint32_t)i);  // first issued in 0, 1, 2, ... order
  }
  size_t block_size() const { return block_size_; }
  size_t capacity() const { return refcounts_.size(); }
  size_t num_free() const { return free_.size(); }
  const std::vector<uint32_t>& free_list() const { return free_; }
  // -1: the id is not from this pool.
  int64_t refcount(uint32_t id) const { return id < refcounts_.size() ? (int64_t)refcounts_[id] : -1; }

  BlockStatus allocate(uint32_t* out) {
    if (free_.empty()) return {BlockErr::OutOfBlocks, capacity(), 1};
    const uint32_t id = free_.back();
    free_.pop_back();
    refcounts_[id] = 1;
    *out = id;
    return {};
  }
  BlockStatus retain(uint32_t id) {
    if (id >= refcounts_.size() || refcounts_[id] == 0) return {BlockErr::NotAllocated, id, 0};
    if (refcounts_[id] == 0xFFFFFFFFu) return {BlockErr::RefcountOverflow, id, 0};
    ++refcounts_[id];
    return {};
  }
  BlockStatus release(uint32_t id) {
    if (id >= refcounts_.size() || refcounts_[id] == 0) return {BlockErr::NotAllocated, id, 0};
    if (--refcounts_[id] == 0) free_.push_back(id);
    return {};
  }
  // block.rs:181-196: the copy target is allocated first so exhaustion leaves the pool untouched.
  BlockStatus copy_on_write(uint32_t id, CowOutcome* out) {
    const int64_t rc = refcount(id);
    if (rc <= 0) return {BlockErr::NotAllocated, id, 0};
    if (rc == 1) { *out = {false, id, id}; return {}; }
    uint32_t dst;
    BlockStatus st = allocate(&dst);
    if (!st.ok()) return st;
    release(id);
    *out = {true, id, dst};
    return {};
  }

 private:
  size_t block_size_;
  std::vector<uint32_t> refcounts_;
  std::vector<uint32_t> free_;  // LIFO
};

struct AppendPlan {
  bool has_cow = false;
  uint32_t cow_src = 0, cow_dst = 0;
  std::vector<uint32_t> appended;
};

class BlockTable {
 public:
  const std::vector<uint32_t>& blocks() const { return blocks_; }
  size_t num_tokens() const { return num_tokens_; }

  // block.rs:253-312. Atomic on failure.
  BlockStatus append_tokens(BlockManager& mgr, size_t n, AppendPlan* plan) {
    *plan = AppendPlan{};
    if (n == 0) return {};
    const size_t bs = mgr.block_size();
    if (num_tokens_ + n < num_tokens_) return {BlockErr::TokenCountOverflow, 0, 0};
    const size_t new_total = num_tokens_ + n;
    bool cow = false;
    uint32_t cow_src = 0;
    if (num_tokens_ % bs != 0 && !blocks_.empty() && mgr.refcount(blocks_.back()) > 1) { cow = true; cow_src = blocks_.back(); }
    const size_t want = (new_total + bs - 1) / bs;
    const size_t fresh = want > blocks_.size() ? want - blocks_.size() : 0;
    const size_t needed = fresh + (cow ? 1 : 0);
    if (mgr.num_free() < needed) return {BlockErr::OutOfBlocks, mgr.capacity(), needed};
    if (cow) {
      CowOutcome oc;
      BlockStatus st = mgr.copy_on_write(cow_src, &oc);
      if (!st.ok()) return st;
      if (oc.copied) { blocks_.back() = oc.dst; plan->has_cow = true; plan->cow_src = oc.src; plan->cow_dst = oc.dst; }
    }
    for (size_t i = 0; i < fresh; ++i) {
      uint32_t id;
      BlockStatus st = mgr.allocate(&id);
      if (!st.ok()) return st;  // unreachable: the free list covers `needed`
      blocks_.push_back(id);
      plan->appended.push_back(id);
    }
    num_tokens_ = new_total;
    return {};
  }
  BlockStatus push_full_block(uint32_t id, size_t block_size) {  // block.rs:319-332
    if (num_tokens_ % block_size != 0) return {BlockErr::MisalignedAdoption, 0, 0};
    num_tokens_ += block_size;
    blocks_.push_back(id);
    return {};
  }
  BlockStatus push_partial_block(uint32_t id, size_t rows, size_t block_size) {  // block.rs:339-354
    if (rows == 0 || rows >= block_size || num_tokens_ % block_size != 0) return {BlockErr::MisalignedAdoption, 0, 0};
    num_tokens_ += rows;
    blocks_.push_back(id);
    return {};
  }
  // The rollback (block.rs:381-396): blocks past ceil(keep / BS) are released in table order.
  BlockStatus truncate(BlockManager& mgr, size_t keep_tokens) {
    if (keep_tokens > num_tokens_) return {BlockErr::TokenCountOverflow, 0, 0};
    const size_t keep_blocks = (keep_tokens + mgr.block_size() - 1) / mgr.block_size();
    for (size_t i = std::min(keep_blocks, blocks_.size()); i < blocks_.size(); ++i) {
      BlockStatus st = mgr.release(blocks_[i]);
      if (!st.ok()) return st;
    }
    if (keep_blocks < blocks_.size()) blocks_.resize(keep_blocks);
    num_tokens_ = keep_tokens;
    return {};
  }
  BlockStatus fork(BlockManager& mgr, BlockTable* out) const {  // block.rs:401-416
    for (size_t i = 0; i < blocks_.size(); ++i) {
      BlockStatus st = mgr.retain(blocks_[i]);
      if (!st.ok()) {
        for (size_t j = 0; j < i; ++j) mgr.release(blocks_[j]);
        return st;
      }
    }
    out->blocks_ = blocks_;
    out->num_tokens_ = num_tokens_;
    return {};
  }
  BlockStatus release(BlockManager& mgr) {  // block.rs:420-425 (consumes the table)
    BlockStatus first;
    for (uint32_t id : blocks_) {
      BlockStatus st = mgr.release(id);
      if (!st.ok() && first.ok()) first = st;
    }
    blocks_.clear();
    num_tokens_ = 0;
    return first;
  }
  // Finish-time donation path (block.rs:360-362): hands the blocks over without releasing them.
  std::vector<uint32_t> into_blocks() {
    std::vector<uint32_t> b;
    b.swap(blocks_);
    num_tokens_ = 0;
    return b;
  }

 private:
  std::vector<uint32_t> blocks_;
  size_t num_tokens_ = 0;
};

}  // namespace kh
