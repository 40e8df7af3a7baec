// SSD cold tier for KV blocks: fixed-layout slab files under a per-model directory, index rebuilt at start-up by
// scanning slab headers. C++ equivalent of the reference's crates/kiln-engine/src/ssd.rs (SlabGeometry 61-91,
// SsdStore::{open 185-217, read 244-300, enqueue_write 303-409, drain_acks 411-418, commit 420-446, drop_file 448-455,
// sync 457-466, scan 494-586}, file_header 609-630, writer_main 635-676).
//
// Layout (little-endian), file `slab-<8-digit id>.kiln`:
//   header (128 bytes): magic "KILNSLB1" | version u32 | layers u32 | kv_heads u32 | head_dim u32 | block_size u32
//                       | dtype_tag u32 | slots u32 | fingerprint [32] | dtype_size u32 | zero padding
//   slot:               used u8 | pad [7] | chain_hash [32] | payload_sha256 [32] | token_ids [block_size * u32] | payload
//   payload:            per layer K rows then V rows (what kc_kv_read_block returns)
// Writes go through a dedicated writer thread; a block counts as stored (readable, index entry inserted) only once
// its write has been acknowledged and the engine has drained the ack. Failure policy: a fingerprint or geometry
// mismatch, a torn slot or an IO error is a silent skip plus a counter, never an error surfaced to a request.
#pragma once

#include <algorithm>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <dirent.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include "radix.hpp"

namespace kh {

constexpr uint32_t SLAB_VERSION = 1;
constexpr size_t SLAB_HEADER_BYTES = 128;
constexpr uint32_t SLOTS_PER_FILE = 64;   // one file per group of 64 blocks

struct SlabGeometry {  // ssd.rs:61-91
  uint32_t layers = 0, kv_heads = 0, head_dim = 0, block_size = 0;
  uint64_t payload_bytes(uint32_t dtype_size) const {
    return (uint64_t)layers * 2 * kv_heads * block_size * head_dim * dtype_size;
  }
  uint64_t slot_header_bytes() const { return 8 + 32 + 32 + (uint64_t)block_size * 4; }
  uint64_t slot_stride(uint32_t dtype_size) const { return slot_header_bytes() + payload_bytes(dtype_size); }
  uint64_t slot_offset(uint32_t dtype_size, uint32_t slot) const { return SLAB_HEADER_BYTES + (uint64_t)slot * slot_stride(dtype_size); }
};

struct SsdCounters { uint64_t reads_total = 0, writes_total = 0, writes_failed_total = 0, fingerprint_rejects_total = 0; };

struct FlushTicket { size_t node; uint64_t generation; ChainHash hash; };
struct FlushAck { size_t node; uint64_t generation; ChainHash hash; bool ok; };

inline ChainHash sha256_of(const uint8_t* p, size_t n) {
  Sha256 h;
  h.update(p, n);
  return h.finish();
}

class SsdStore {
 public:
  // Opens (creating if needed) the slab directory and scans it into the index. Returns null when the directory
  // cannot be created or read.
  static std::unique_ptr<SsdStore> open(const std::string& dir, const ChainHash& fingerprint, const SlabGeometry& g, uint64_t max_bytes) {
    ::mkdir(dir.c_str(), 0755);
    struct stat st;
    if (::stat(dir.c_str(), &st) != 0 || !S_ISDIR(st.st_mode)) return nullptr;
    std::unique_ptr<SsdStore> s(new SsdStore(dir, fingerprint, g, max_bytes));
    if (!s->scan()) return nullptr;
    s->writer_ = std::thread([p = s.get()] { p->writer_main(); });
    return s;
  }
  ~SsdStore() {
    {
      std::lock_guard<std::mutex> lk(mu_);
      closing_ = true;
    }
    cv_.notify_all();
    if (writer_.joinable()) writer_.join();   // queued writes land before the store goes away
    for (auto& kv : handles_) ::close(kv.second);
  }

  const SsdCounters& counters() const { return counters_; }
  uint64_t blocks_stored() const { return index_.size(); }
  uint64_t bytes_stored() const { return bytes_; }
  bool contains(const ChainHash& h) const { return index_.count(h) != 0; }

  // Reads and verifies the payload of `hash`. Any mismatch or IO failure removes the index entry (ssd.rs:244-300).
  bool read(const ChainHash& hash, const uint32_t* expected_tokens, size_t n_tokens, int64_t pool_dtype_tag, std::vector<uint8_t>* payload,
            uint32_t* dtype_tag) {
    auto it = index_.find(hash);
    if (it == index_.end()) return false;
    const SlotRef slot = it->second;
    if (read_verified(slot, hash, expected_tokens, n_tokens, pool_dtype_tag, payload)) {
      counters_.reads_total++;
      clock_++;
      auto f = files_.find(slot.file);
      if (f != files_.end()) f->second.last_touch = clock_;
      *dtype_tag = slot.dtype_tag;
      return true;
    }
    counters_.fingerprint_rejects_total++;
    index_.erase(hash);
    return false;
  }

  // Queues one block for the writer thread; not readable until its ack has been drained (ssd.rs:303-409).
  void enqueue_write(const FlushTicket& ticket, const uint32_t* tokens, size_t n_tokens, std::vector<uint8_t> payload, uint32_t dtype_tag,
                     uint32_t dtype_size) {
    const SlabGeometry& g = geometry_;
    const uint64_t stride = g.slot_stride(dtype_size);
    // byte cap: drop least-recently-hit slabs, never the one this write lands in nor one with writes in flight
    const bool starts_new_file = !(has_open_ && open_used_ < SLOTS_PER_FILE);
    const uint64_t incoming = stride + (starts_new_file ? SLAB_HEADER_BYTES : 0);
    while (bytes_ + incoming > max_bytes_) {
      int64_t victim = -1;
      uint64_t best = ~0ull;
      for (auto& kv : files_) {
        if (!starts_new_file && has_open_ && kv.first == open_file_) continue;
        if (kv.second.pending_slots != 0) continue;
        if (kv.second.last_touch < best) { best = kv.second.last_touch; victim = kv.first; }
      }
      if (victim < 0) break;
      drop_file((uint32_t)victim);
      if (has_open_ && open_file_ == (uint32_t)victim) has_open_ = false;
    }
    uint32_t file, slot;
    if (has_open_ && open_used_ < SLOTS_PER_FILE) {
      file = open_file_; slot = open_used_;
    } else {
      file = next_file_++;
      Job j; j.kind = Job::Create; j.file = file; j.bytes = file_header(dtype_tag, dtype_size);
      push(std::move(j));
      bytes_ += SLAB_HEADER_BYTES;
      FileMeta m; m.bytes = SLAB_HEADER_BYTES; m.last_touch = clock_;
      files_[file] = m;
      slot = 0;
    }
    has_open_ = true; open_file_ = file; open_used_ = slot + 1;

    std::vector<uint8_t> bytes;
    bytes.reserve(stride);
    bytes.push_back(1);
    bytes.insert(bytes.end(), 7, 0);
    bytes.insert(bytes.end(), ticket.hash.begin(), ticket.hash.end());
    const ChainHash digest = sha256_of(payload.data(), payload.size());
    bytes.insert(bytes.end(), digest.begin(), digest.end());
    for (size_t i = 0; i < g.block_size; ++i) {
      const uint32_t t = i < n_tokens ? tokens[i] : 0;
      for (int b = 0; b < 4; ++b) bytes.push_back((uint8_t)(t >> (8 * b)));
    }
    bytes.insert(bytes.end(), payload.begin(), payload.end());

    bytes_ += stride;
    files_[file].pending_slots++;
    files_[file].pending_bytes += stride;
    inflight_[{file, slot}] = ticket.hash;
    Job j; j.kind = Job::Write; j.file = file; j.offset = g.slot_offset(dtype_size, slot); j.bytes = std::move(bytes);
    j.ack = FlushAck{ticket.node, ticket.generation, ticket.hash, true};
    j.slot = SlotRef{file, slot, dtype_tag, dtype_size};
    j.close_after = slot + 1 == SLOTS_PER_FILE;   // the file is full: the writer gives its descriptor back
    push(std::move(j));
  }

  // Applies completed writes and returns their acks (ssd.rs:411-446).
  std::vector<FlushAck> drain_acks() {
    std::vector<Done> done;
    {
      std::lock_guard<std::mutex> lk(mu_);
      done.swap(acks_);
    }
    std::vector<FlushAck> acks;
    acks.reserve(done.size());
    for (const Done& d : done) { commit(d.ack, d.slot); acks.push_back(d.ack); }
    return acks;
  }

  // Blocks until everything queued so far has been written, then commits the acks (shutdown and tests only).
  std::vector<FlushAck> sync() {
    std::unique_lock<std::mutex> lk(mu_);
    const uint64_t want = pushed_;
    done_cv_.wait(lk, [&] { return done_ >= want; });
    lk.unlock();
    return drain_acks();
  }

 private:
  struct SlotRef { uint32_t file, slot, dtype_tag, dtype_size; };
  struct FileMeta { uint32_t slots_used = 0; uint64_t bytes = 0, last_touch = 0; uint32_t pending_slots = 0; uint64_t pending_bytes = 0; };
  struct Job {
    enum Kind { Create, Write, Delete } kind = Create;
    uint32_t file = 0;
    uint64_t offset = 0;
    std::vector<uint8_t> bytes;
    FlushAck ack{};
    SlotRef slot{};
    bool close_after = false;
  };
  struct Done { FlushAck ack; SlotRef slot; };

  SsdStore(const std::string& dir, const ChainHash& fp, const SlabGeometry& g, uint64_t max_bytes)
      : dir_(dir), fingerprint_(fp), geometry_(g), max_bytes_(max_bytes) {}

  static std::string file_name(uint32_t id) {
    char buf[32];
    snprintf(buf, sizeof buf, "slab-%08u.kiln", id);
    return buf;
  }
  static bool parse_file_name(const char* name, uint32_t* id) {
    if (strlen(name) != 5 + 8 + 5 || strncmp(name, "slab-", 5) != 0 || strcmp(name + 13, ".kiln") != 0) return false;
    uint32_t v = 0;
    for (int i = 5; i < 13; ++i) {
      if (name[i] < '0' || name[i] > '9') return false;
      v = v * 10 + (uint32_t)(name[i] - '0');
    }
    *id = v;
    return true;
  }
  std::vector<uint8_t> file_header(uint32_t dtype_tag, uint32_t dtype_size) const {  // ssd.rs:609-630
    std::vector<uint8_t> h;
    h.insert(h.end(), {'K', 'I', 'L', 'N', 'S', 'L', 'B', '1'});
    const uint32_t vals[7] = {SLAB_VERSION, geometry_.layers, geometry_.kv_heads, geometry_.head_dim, geometry_.block_size, dtype_tag, SLOTS_PER_FILE};
    for (uint32_t v : vals) for (int b = 0; b < 4; ++b) h.push_back((uint8_t)(v >> (8 * b)));
    h.insert(h.end(), fingerprint_.begin(), fingerprint_.end());
    for (int b = 0; b < 4; ++b) h.push_back((uint8_t)(dtype_size >> (8 * b)));
    h.resize(SLAB_HEADER_BYTES, 0);
    return h;
  }

  bool read_verified(const SlotRef& slot, const ChainHash& hash, const uint32_t* expected_tokens, size_t n_tokens, int64_t pool_dtype_tag,
                     std::vector<uint8_t>* payload) const {
    if (pool_dtype_tag >= 0 && (uint32_t)pool_dtype_tag != slot.dtype_tag) return false;
    const SlabGeometry& g = geometry_;
    const int fd = ::open((dir_ + "/" + file_name(slot.file)).c_str(), O_RDONLY);
    if (fd < 0) return false;
    bool ok = false;
    const uint64_t offset = g.slot_offset(slot.dtype_size, slot.slot);
    std::vector<uint8_t> header(g.slot_header_bytes());
    if (::pread(fd, header.data(), header.size(), (off_t)offset) == (ssize_t)header.size() && header[0] == 1 &&
        memcmp(header.data() + 8, hash.data(), 32) == 0) {
      bool tokens_ok = true;
      for (size_t i = 0; i < n_tokens && tokens_ok; ++i) {
        uint32_t t = 0;
        for (int b = 0; b < 4; ++b) t |= (uint32_t)header[72 + i * 4 + b] << (8 * b);
        tokens_ok = t == expected_tokens[i];
      }
      if (tokens_ok) {
        payload->resize(g.payload_bytes(slot.dtype_size));
        if (::pread(fd, payload->data(), payload->size(), (off_t)(offset + g.slot_header_bytes())) == (ssize_t)payload->size()) {
          const ChainHash digest = sha256_of(payload->data(), payload->size());
          ok = memcmp(digest.data(), header.data() + 40, 32) == 0;   // a torn write fails here
        }
      }
    }
    ::close(fd);
    return ok;
  }

  // Writes in flight are keyed by their slot, not by their hash: a block that is queued twice before the first
  // acknowledgement arrives owns two slots, and each acknowledgement must settle its own.
  void commit(const FlushAck& ack, const SlotRef& slot) {  // ssd.rs:420-446
    auto it = inflight_.find({slot.file, slot.slot});
    if (it == inflight_.end()) return;   // the slab was evicted while the write was queued
    inflight_.erase(it);
    const uint64_t stride = geometry_.slot_stride(slot.dtype_size);
    auto f = files_.find(slot.file);
    if (f == files_.end()) return;
    FileMeta& meta = f->second;
    meta.pending_slots = meta.pending_slots ? meta.pending_slots - 1 : 0;
    meta.pending_bytes = meta.pending_bytes >= stride ? meta.pending_bytes - stride : 0;
    if (ack.ok) {
      counters_.writes_total++;
      clock_++;
      meta.slots_used++;
      meta.bytes += stride;
      meta.last_touch = clock_;
      index_[ack.hash] = slot;
    } else {
      counters_.writes_failed_total++;
      bytes_ = bytes_ >= stride ? bytes_ - stride : 0;
    }
  }

  void drop_file(uint32_t file) {  // ssd.rs:448-455
    auto f = files_.find(file);
    if (f != files_.end()) {
      const uint64_t b = f->second.bytes + f->second.pending_bytes;
      bytes_ = bytes_ >= b ? bytes_ - b : 0;
      files_.erase(f);
    }
    for (auto it = index_.begin(); it != index_.end();) it = it->second.file == file ? index_.erase(it) : std::next(it);
    for (auto it = inflight_.begin(); it != inflight_.end();) it = it->first.first == file ? inflight_.erase(it) : std::next(it);
    Job j; j.kind = Job::Delete; j.file = file;
    push(std::move(j));
  }

  // Start-up index scan: trust nothing but slab headers (ssd.rs:494-586).
  bool scan() {
    DIR* d = ::opendir(dir_.c_str());
    if (!d) return false;
    std::vector<uint32_t> ids;
    while (struct dirent* e = ::readdir(d)) {
      uint32_t id;
      if (parse_file_name(e->d_name, &id)) ids.push_back(id);
    }
    ::closedir(d);
    std::sort(ids.begin(), ids.end());
    for (uint32_t id : ids) {
      next_file_ = std::max(next_file_, id + 1);
      if (!scan_file(id)) counters_.fingerprint_rejects_total++;
    }
    return true;
  }
  bool scan_file(uint32_t id) {
    const int fd = ::open((dir_ + "/" + file_name(id)).c_str(), O_RDONLY);
    if (fd < 0) return false;
    uint8_t header[SLAB_HEADER_BYTES];
    bool ok = ::pread(fd, header, sizeof header, 0) == (ssize_t)sizeof header;
    auto u32_at = [&](size_t at) { return (uint32_t)header[at] | (uint32_t)header[at + 1] << 8 | (uint32_t)header[at + 2] << 16 | (uint32_t)header[at + 3] << 24; };
    const SlabGeometry& g = geometry_;
    ok = ok && memcmp(header, "KILNSLB1", 8) == 0 && u32_at(8) == SLAB_VERSION && u32_at(12) == g.layers && u32_at(16) == g.kv_heads &&
         u32_at(20) == g.head_dim && u32_at(24) == g.block_size && u32_at(32) == SLOTS_PER_FILE && memcmp(header + 36, fingerprint_.data(), 32) == 0;
    const uint32_t dtype_tag = ok ? u32_at(28) : 0, dtype_size = ok ? u32_at(68) : 0;
    ok = ok && dtype_size != 0 && dtype_size <= 8;
    if (!ok) { ::close(fd); return false; }
    struct stat st;
    const uint64_t file_len = ::fstat(fd, &st) == 0 ? (uint64_t)st.st_size : 0;
    uint32_t slots_used = 0;
    std::vector<uint8_t> slot_header(g.slot_header_bytes());
    for (uint32_t slot = 0; slot < SLOTS_PER_FILE; ++slot) {
      const uint64_t offset = g.slot_offset(dtype_size, slot);
      if (offset + g.slot_stride(dtype_size) > file_len) break;
      if (::pread(fd, slot_header.data(), slot_header.size(), (off_t)offset) != (ssize_t)slot_header.size()) break;
      if (slot_header[0] != 1) continue;
      ChainHash hash;
      memcpy(hash.data(), slot_header.data() + 8, 32);
      slots_used++;
      index_[hash] = SlotRef{id, slot, dtype_tag, dtype_size};   // later files win on duplicates
    }
    ::close(fd);
    clock_++;
    FileMeta m; m.slots_used = slots_used; m.bytes = file_len; m.last_touch = clock_;
    files_[id] = m;
    bytes_ += file_len;
    return true;
  }

  void push(Job&& j) {
    {
      std::lock_guard<std::mutex> lk(mu_);
      jobs_.push_back(std::move(j));
      pushed_++;
    }
    cv_.notify_one();
  }
  // The writer thread: owns the file handles, performs creates, writes and deletes in order, acknowledges every write;
  // IO failures are acknowledged with ok = false (ssd.rs:635-676).
  void writer_main() {
    for (;;) {
      Job j;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return closing_ || !jobs_.empty(); });
        if (jobs_.empty()) return;
        j = std::move(jobs_.front());
        jobs_.pop_front();
      }
      const std::string path = dir_ + "/" + file_name(j.file);
      if (j.kind == Job::Create) {
        const int fd = ::open(path.c_str(), O_CREAT | O_TRUNC | O_RDWR, 0644);
        if (fd >= 0) {
          if (::pwrite(fd, j.bytes.data(), j.bytes.size(), 0) != (ssize_t)j.bytes.size()) { /* writes to this file fail their acks */ }
          handles_[j.file] = fd;
        }
      } else if (j.kind == Job::Write) {
        auto h = handles_.find(j.file);
        j.ack.ok = h != handles_.end() && ::pwrite(h->second, j.bytes.data(), j.bytes.size(), (off_t)j.offset) == (ssize_t)j.bytes.size();
        if (j.close_after && h != handles_.end()) { ::close(h->second); handles_.erase(h); }
        std::lock_guard<std::mutex> lk(mu_);
        acks_.push_back(Done{j.ack, j.slot});
      } else {
        auto h = handles_.find(j.file);
        if (h != handles_.end()) { ::close(h->second); handles_.erase(h); }
        ::unlink(path.c_str());
      }
      {
        std::lock_guard<std::mutex> lk(mu_);
        done_++;
      }
      done_cv_.notify_all();
    }
  }

  std::string dir_;
  ChainHash fingerprint_;
  SlabGeometry geometry_;
  uint64_t max_bytes_;
  std::map<ChainHash, SlotRef> index_;
  std::map<std::pair<uint32_t, uint32_t>, ChainHash> inflight_;   // (file, slot) of every write not yet acknowledged
  std::map<uint32_t, FileMeta> files_;
  uint64_t bytes_ = 0, clock_ = 0;
  uint32_t next_file_ = 0, open_file_ = 0, open_used_ = 0;
  bool has_open_ = false;
  SsdCounters counters_;
  // shared with the writer thread
  std::mutex mu_;
  std::condition_variable cv_, done_cv_;
  std::deque<Job> jobs_;
  std::vector<Done> acks_;
  uint64_t pushed_ = 0, done_ = 0;
  bool closing_ = false;
  std::map<uint32_t, int> handles_;   // writer thread only (and the destructor after the join)
  std::thread writer_;
};

}  // namespace kh
