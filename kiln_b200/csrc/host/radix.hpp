// Radix prefix cache: a tree keyed on token ids in block-sized chunks, one node
// per full KV block (plus partial leaves for settled tails), mapping prefixes of
// finished requests to pool blocks. C++ equivalent of the reference's
// crates/kiln-engine/src/radix.rs:92-457 with the same node API, the same
// chained SHA-256 digests (radix.rs:145-152) and the same LRU leaf eviction.
// The SSD tier's flags are kept so the API matches; nothing here does IO.
#pragma once

#include <array>
#include <cstdint>
#include <cstring>
#include <map>
#include <vector>

#include "block.hpp"

namespace kh {

typedef std::array<uint8_t, 32> ChainHash;

// SHA-256 (FIPS 180-4), written out here because the digest is part of the
// cache's identity contract (a child's hash = sha256(parent hash || tokens as LE u32)).
class Sha256 {
 public:
  Sha256() { reset(); }
  void reset() {
    static const uint32_t iv[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    memcpy(h_, iv, sizeof iv);
    len_ = 0; fill_ = 0;
  }
  void update(const uint8_t* p, size_t n) {
    len_ += n;
    while (n) {
      const size_t take = std::min(n, (size_t)64 - fill_);
      memcpy(buf_ + fill_, p, take);
      fill_ += take; p += take; n -= take;
      if (fill_ == 64) { block(buf_); fill_ = 0; }
    }
  }
  ChainHash finish() {
    const uint64_t bits = len_ * 8;
    uint8_t pad = 0x80;
    update(&pad, 1);
    pad = 0;
    while (fill_ != 56) update(&pad, 1);
    uint8_t lenb[8];
    for (int i = 0; i < 8; ++i) lenb[i] = (uint8_t)(bits >> (56 - 8 * i));
    update(lenb, 8);
    ChainHash out;
    for (int i = 0; i < 8; ++i)
      for (int j = 0; j < 4; ++j) out[4 * i + j] = (uint8_t)(h_[i] >> (24 - 8 * j));
    return out;
  }

 private:
  static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void block(const uint8_t* p) {
    static const uint32_t k[64] = {
        0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
        0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
        0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
        0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
        0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
        0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
        0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i) w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h_[0], b = h_[1], c = h_[2], d = h_[3], e = h_[4], f = h_[5], g = h_[6], h = h_[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t t1 = h + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + k[i] + w[i];
      const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
      h = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h_[0] += a; h_[1] += b; h_[2] += c; h_[3] += d; h_[4] += e; h_[5] += f; h_[6] += g; h_[7] += h;
  }
  uint32_t h_[8];
  uint64_t len_;
  uint8_t buf_[64];
  size_t fill_;
};

constexpr size_t RADIX_ROOT = 0;

class RadixCache {
 public:
  RadixCache(size_t block_size, const ChainHash& seed) : block_size_(block_size) {
    Node root;
    root.chain_hash = seed;
    nodes_.push_back(root);
  }
  size_t block_size() const { return block_size_; }
  size_t resident_blocks() const { return resident_; }
  size_t num_slots() const { return nodes_.size(); }

  // The child of `node` labelled with exactly `chunk`; -1 if absent (radix.rs:140-142).
  int64_t child(size_t node, const std::vector<uint32_t>& chunk) const {
    auto it = nodes_[node].children.find(chunk);
    return it == nodes_[node].children.end() ? -1 : (int64_t)it->second;
  }
  ChainHash chain_hash_of(size_t node, const uint32_t* chunk, size_t n) const {  // radix.rs:145-152
    Sha256 h;
    h.update(nodes_[node].chain_hash.data(), 32);
    for (size_t i = 0; i < n; ++i) {
      const uint8_t le[4] = {(uint8_t)chunk[i], (uint8_t)(chunk[i] >> 8), (uint8_t)(chunk[i] >> 16), (uint8_t)(chunk[i] >> 24)};
      h.update(le, 4);
    }
    return h.finish();
  }
  uint64_t node_generation(size_t node) const { return nodes_[node].generation; }
  const ChainHash& node_hash(size_t node) const { return nodes_[node].chain_hash; }
  int64_t node_block(size_t node) const { return nodes_[node].has_block ? (int64_t)nodes_[node].block : -1; }
  const std::vector<uint32_t>& node_tokens(size_t node) const { return nodes_[node].tokens; }
  size_t node_rows(size_t node) const { return nodes_[node].tokens.size(); }
  bool node_is_partial(size_t node) const { return nodes_[node].partial; }
  std::vector<size_t> full_children(size_t node) const {
    std::vector<size_t> out;
    for (auto& kv : nodes_[node].children) out.push_back(kv.second);
    return out;
  }
  const std::vector<size_t>& partial_children(size_t node) const { return nodes_[node].partials; }
  bool node_on_ssd(size_t node) const { return nodes_[node].ssd; }
  void set_on_ssd(size_t node) { nodes_[node].ssd = true; nodes_[node].flush_pending = false; }
  bool flush_pending(size_t node) const { return nodes_[node].flush_pending; }
  void set_flush_pending(size_t node) { nodes_[node].flush_pending = true; }
  void clear_flush_pending(size_t node) { nodes_[node].flush_pending = false; }
  bool is_live(size_t node, uint64_t generation) const {  // radix.rs:275-279
    return node < nodes_.size() && nodes_[node].generation == generation && (node == RADIX_ROOT || !nodes_[node].tokens.empty());
  }
  void touch(size_t node) { nodes_[node].last_hit = ++clock_; }

  size_t insert_child(size_t parent, const std::vector<uint32_t>& chunk) {  // radix.rs:288-320
    Node n = fresh(parent, chunk, false);
    const size_t index = place(n);
    nodes_[parent].children[chunk] = index;
    return index;
  }
  size_t insert_partial_child(size_t parent, const std::vector<uint32_t>& tokens) {  // radix.rs:193-225
    Node n = fresh(parent, tokens, true);
    const size_t index = place(n);
    nodes_[parent].partials.push_back(index);
    return index;
  }
  // Re-keys a partial leaf with a longer settled tail; returns the old block or -1 (radix.rs:230-249).
  int64_t upgrade_partial(size_t node, const std::vector<uint32_t>& tokens, uint32_t block) {
    const size_t parent = nodes_[node].parent;
    const ChainHash h = chain_hash_of(parent, tokens.data(), tokens.size());
    const int64_t old = node_block(node);
    nodes_[node].has_block = true;
    nodes_[node].block = block;
    if (old < 0) { nodes_[parent].resident_children++; resident_++; }
    nodes_[node].tokens = tokens;
    nodes_[node].chain_hash = h;
    touch(node);
    return old;
  }
  void set_resident(size_t node, uint32_t block) {  // radix.rs:324-330
    nodes_[node].has_block = true;
    nodes_[node].block = block;
    nodes_[nodes_[node].parent].resident_children++;
    resident_++;
  }
  // LRU among resident nodes with no resident children whose block the cache solely owns (radix.rs:335-349).
  int64_t evict_candidate(const BlockManager& mgr) const {
    int64_t best = -1;
    uint64_t best_hit = ~0ull;
    for (size_t i = 1; i < nodes_.size(); ++i) {
      const Node& n = nodes_[i];
      if (n.tokens.empty() || n.resident_children != 0 || !n.has_block || mgr.refcount(n.block) != 1) continue;
      if (n.last_hit < best_hit) { best_hit = n.last_hit; best = (int64_t)i; }
    }
    return best;
  }
  // Drops residency, releasing the cache's reference; returns the freed block or -1 (radix.rs:355-366).
  int64_t evict(BlockManager& mgr, size_t node) {
    if (!nodes_[node].has_block) return -1;
    const uint32_t block = nodes_[node].block;
    nodes_[node].has_block = false;
    mgr.release(block);
    nodes_[nodes_[node].parent].resident_children--;
    resident_--;
    if (!nodes_[node].ssd) prune(node);
    return block;
  }
  void prune_subtree(BlockManager& mgr, size_t node) {  // radix.rs:373-395
    if (node == RADIX_ROOT) return;
    const size_t parent = nodes_[node].parent;
    if (nodes_[node].has_block) nodes_[parent].resident_children--;
    detach(parent, node);
    std::vector<size_t> stack{node};
    while (!stack.empty()) {
      const size_t i = stack.back();
      stack.pop_back();
      if (nodes_[i].has_block) { mgr.release(nodes_[i].block); nodes_[i].has_block = false; resident_--; }
      for (auto& kv : nodes_[i].children) stack.push_back(kv.second);
      for (size_t p : nodes_[i].partials) stack.push_back(p);
      recycle(i);
    }
  }
  void reset() {  // radix.rs:448-456
    const ChainHash seed = nodes_[RADIX_ROOT].chain_hash;
    const uint64_t clock = clock_, gens = generations_ + 1;
    nodes_.clear(); free_slots_.clear(); resident_ = 0;
    Node root;
    root.chain_hash = seed;
    nodes_.push_back(root);
    clock_ = clock; generations_ = gens;
  }

 private:
  struct Node {
    uint64_t generation = 0;
    size_t parent = RADIX_ROOT;
    std::vector<uint32_t> tokens;
    bool partial = false;
    std::map<std::vector<uint32_t>, size_t> children;
    std::vector<size_t> partials;
    bool has_block = false;
    uint32_t block = 0;
    ChainHash chain_hash{};
    bool ssd = false, flush_pending = false;
    uint64_t last_hit = 0;
    uint32_t resident_children = 0;
  };
  Node fresh(size_t parent, const std::vector<uint32_t>& tokens, bool partial) {
    Node n;
    n.chain_hash = chain_hash_of(parent, tokens.data(), tokens.size());
    n.generation = ++generations_;
    n.parent = parent;
    n.tokens = tokens;
    n.partial = partial;
    n.last_hit = ++clock_;
    return n;
  }
  size_t place(const Node& n) {
    if (!free_slots_.empty()) {
      const size_t slot = free_slots_.back();
      free_slots_.pop_back();
      nodes_[slot] = n;
      return slot;
    }
    nodes_.push_back(n);
    return nodes_.size() - 1;
  }
  void detach(size_t parent, size_t node) {  // radix.rs:417-424
    if (nodes_[node].partial) {
      auto& v = nodes_[parent].partials;
      for (size_t i = 0; i < v.size();) { if (v[i] == node) v.erase(v.begin() + i); else ++i; }
    } else {
      nodes_[parent].children.erase(nodes_[node].tokens);
      nodes_[node].tokens.clear();
    }
  }
  void prune(size_t node) {  // radix.rs:397-414
    detach(nodes_[node].parent, node);
    std::vector<size_t> stack;
    for (auto& kv : nodes_[node].children) stack.push_back(kv.second);
    for (size_t p : nodes_[node].partials) stack.push_back(p);
    recycle(node);
    while (!stack.empty()) {
      const size_t i = stack.back();
      stack.pop_back();
      for (auto& kv : nodes_[i].children) stack.push_back(kv.second);
      for (size_t p : nodes_[i].partials) stack.push_back(p);
      recycle(i);
    }
  }
  void recycle(size_t node) {  // radix.rs:426-443
    Node blank;
    blank.generation = ++generations_;
    nodes_[node] = blank;
    free_slots_.push_back(node);
  }

  size_t block_size_;
  std::vector<Node> nodes_;
  std::vector<size_t> free_slots_;
  uint64_t clock_ = 0, generations_ = 0;
  size_t resident_ = 0;
};

}  // namespace kh
