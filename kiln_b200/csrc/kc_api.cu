// C ABI of libkiln_cuda.so (declared in include/kiln_cuda.h): contexts, model
// loading, paged KV pools, forward_step and the verify round.
//
// The forward restates CausalLm::forward_step (crates/kiln-models/src/nn.rs:1303-1388)
// as a fixed sequence of kernel launches on one stream; nothing here computes on
// the host. Errors never abort: every entry point returns a status and leaves a
// thread-local message (crates/kiln-mlx/src/error.rs:54-72).
#include "../../include/kiln_cuda.h"

#include <nccl.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "kc_attn.cuh"
#include "kc_fused.cuh"
#include "kc_internal.cuh"
#include "kc_qlinear.cuh"

using namespace kc;

namespace kc {
bool make_tmap_bf16_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint32_t box_inner,
                       uint32_t box_outer, const char** err);
bool make_tmap_kv_4d(CUtensorMap* map, const void* pool, uint32_t head_dim, uint64_t plane_rows, uint64_t planes,
                     const char** err);
}

// ---------------------------------------------------------------------------
// errors, live counter
// ---------------------------------------------------------------------------

static thread_local std::string g_err = "";
static std::atomic<int64_t> g_live{0};

static int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}
#define CK(call)                                                                             \
  do {                                                                                       \
    cudaError_t e__ = (call);                                                                \
    if (e__ != cudaSuccess)                                                                  \
      return fail(e__ == cudaErrorMemoryAllocation ? KC_ERR_OOM : KC_ERR_CUDA, "%s: %s", #call, \
                  cudaGetErrorString(e__));                                                  \
  } while (0)

#define RC(call) do { int r__ = (call); if (r__) return r__; } while (0)

enum { KC_PROF_GEMM = 0, KC_PROF_GEMM_REDUCE = 1, KC_PROF_ATTN = 2, KC_PROF_ROWWISE = 3, KC_PROF_SAMPLE = 4, KC_PROFILE_CLASSES = 5 };

extern "C" const char* kc_last_error(void) { return g_err.c_str(); }
extern "C" int64_t kc_live_objects(void) { return g_live.load(); }

// ---------------------------------------------------------------------------
// handles
// ---------------------------------------------------------------------------

struct kc_ctx {
  int device = 0;
  int sm_count = 148;
  cudaStream_t stream = nullptr;
  uint32_t* status = nullptr;  // device status word
  uint32_t* status_host = nullptr;  // pinned copy, filled by the copy that precedes a synchronisation
  ncclComm_t comm = nullptr;
  int tp_rank = 0, tp_world = 1;
  // launch accounting and optional per-class timing (kc_profile_*)
  int64_t launches = 0;
  int profile = 0;
  cudaEvent_t step_a = nullptr, step_b = nullptr;   // device span of the last kc_verify_step
  float last_step_ms = 0.f;
  struct Span { cudaEvent_t a, b; int cls; };
  std::vector<Span> spans;
  std::vector<cudaEvent_t> event_pool;
  int64_t class_launches[KC_PROFILE_CLASSES] = {0, 0, 0, 0, 0};
  // draft lane accounting (kc_draft_chain): host wall time of the calls and tokens proposed
  double draft_ms = 0.0;
  int64_t draft_tokens = 0, draft_calls = 0;
  cudaEvent_t take_event() {
    if (!event_pool.empty()) { cudaEvent_t e = event_pool.back(); event_pool.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
  }
};

// Runs `call` (a cudaError_t expression that launches `n` kernels of class `cls`); under kc_profile_enable the
// launch is bracketed by events on the context's stream.
#define LAUNCH(c, cls, n, call)                                                       \
  do {                                                                                \
    kc_ctx* c__ = (c);                                                                \
    c__->launches += (n);                                                             \
    c__->class_launches[cls] += (n);                                                  \
    if (c__->profile) {                                                               \
      kc_ctx::Span sp__{c__->take_event(), c__->take_event(), (cls)};                 \
      cudaEventRecord(sp__.a, c__->stream);                                           \
      CK(call);                                                                       \
      cudaEventRecord(sp__.b, c__->stream);                                           \
      c__->spans.push_back(sp__);                                                     \
    } else {                                                                          \
      CK(call);                                                                       \
    }                                                                                 \
  } while (0)

struct kc_kv {
  kc_ctx* ctx = nullptr;
  int device = 0;
  int layers = 0, kv_heads = 0, head_dim = 0, num_blocks = 0, block_size = 0;
  bf16* pool = nullptr;        // [layers][2][num_blocks][kv_heads][block_size][head_dim]
  size_t block_elems = 0;      // kv_heads * block_size * head_dim
  size_t bytes = 0;
  CUtensorMap map;             // all pool rows x head_dim, box {64, 16}, 128-byte swizzle; or, with map4d, the 4-D
  bool map4d = false;          // map whose box is the K and the V tile of a layer (make_tmap_kv_4d)
};

struct kc_qweight {
  kc_ctx* ctx = nullptr;
  int device = 0;
  QWeight w;
  float* partial = nullptr;
  ActOperand op;               // bound lazily to the caller's x buffer
  const void* op_ptr = nullptr;
  int op_rows = 0;
};

namespace kc {
CtxView ctx_view(kc_ctx* c) { return CtxView{c->device, c->stream, c->status}; }
const QWeight* qweight_view(kc_qweight* q) { return &q->w; }
kc_ctx* qweight_owner(kc_qweight* q) { return q->ctx; }
void ctx_count_launches(kc_ctx* c, int cls, int n) { c->launches += n; c->class_launches[cls] += n; }
int api_fail(int code, const char* msg) { return fail(code, "%s", msg); }
}  // namespace kc

struct Layer {
  QWeight qkv, o, gate_up, down;
  bf16* qkv_bias = nullptr;    // qwen2
  bf16 *input_ln = nullptr, *post_attn_ln = nullptr, *pre_ffw_ln = nullptr, *post_ffw_ln = nullptr;
};

// Per-step metadata, packed on the host and copied to the device in one transfer.
struct MetaLayout {
  size_t tokens, token_pos, kv_slot, sampled, tables, work, v_row_off, v_draft_off, v_draft_len, v_draft, feed, total;
};

struct kc_model {
  kc_ctx* ctx = nullptr;
  int device = 0;
  kc_model_desc d{};
  int Hq = 0, Hkv = 0;                 // local (tensor-parallel) head counts
  int F = 0;                           // local intermediate size
  bool stream_lane = false;            // forwards of at most QL_STREAM_MAX_M rows take the weight-streaming kernels
  size_t stream_min_bytes = QL_STREAM_MIN_BYTES;   // ... for weights of at least this many bytes of records
  bool glu_interleaved = false;        // gate_up rows alternate gate / up in blocks of 128 (so the GEMM can fuse the activation)
  int n_qkv = 0;
  std::vector<Layer> layers;
  // embedding table in mlx layout (gather) and the head as GEMM records
  uint32_t* emb_w = nullptr; bf16 *emb_s = nullptr, *emb_b = nullptr;
  QWeight head;
  bf16* final_norm = nullptr;
  float* inv_freq = nullptr;
  float embed_scale = 0.f;
  float attn_scale = 0.f;
  int64_t weight_bytes = 0;
  // activations
  int max_rows = 0, max_seqs = 0, logit_rows = 0;
  bf16 *h = nullptr, *normed = nullptr, *qkv = nullptr, *q_rot = nullptr, *attn = nullptr, *proj = nullptr, *proj_ranks = nullptr,
       *gu = nullptr, *act = nullptr, *hs = nullptr, *logits = nullptr;
  ActOperand op_normed, op_attn, op_act, op_hs;
  float* partial = nullptr; size_t partial_bytes = 0;
  float* argmax_scratch = nullptr;     // per-CTA bests + counter of the fused reduction / arg-max of a streamed head
  float* partial_gu = nullptr;         // gate_up's fp32 partials while a gated down projection reads them (stream lane on)
  float* attn_ws = nullptr; size_t attn_ws_bytes = 0;
  float* tp_buf = nullptr;             // fp32 staging for the tensor-parallel all-reduce
  // Tensor-parallel exchange over peer memory (kc_tp_export / kc_tp_attach): the o_proj / down_proj output of exchange e
  // goes to tp_out[e & 1]; tp_flags[r] = the last exchange rank r has published. peer_* = every rank's buffers as
  // mapped into this process (this rank's own pointers at index tp_rank).
  bf16* tp_out[2] = {nullptr, nullptr};
  uint32_t* tp_flags = nullptr;
  bf16* peer_out[2][KC_MAX_TP] = {};
  uint32_t* peer_flags[KC_MAX_TP] = {};
  bool tp_p2p = false;
  // Two-phase exchange (from 4 ranks on): each tp_out buffer is followed by a second region of the same size that
  // holds this rank's summed column slice [rows][H / world]; the second half of the flag array belongs to that phase.
  bool tp_two_phase = false;
  size_t tp_sum_off = 0;              // elements from tp_out[b] to the slice region
  uint32_t tp_epoch = 0;
  // step metadata
  uint8_t* meta_dev = nullptr; size_t meta_cap = 0;
  static constexpr int kStaging = 4;
  uint8_t* meta_host[kStaging] = {nullptr, nullptr, nullptr, nullptr};
  cudaEvent_t meta_ev[kStaging] = {nullptr, nullptr, nullptr, nullptr};
  int meta_next = 0;
  // verify results
  uint32_t* row_tokens = nullptr; int32_t *n_committed = nullptr, *n_accepted = nullptr; uint32_t* committed = nullptr;
  uint8_t* result_host = nullptr;      // pinned
  // pipelined decode: launch k keeps its sampled tokens in slot k % 2 until launch k + 2 reuses it
  uint32_t* pipe_tokens[2] = {nullptr, nullptr};   // device [max_seqs]
  uint32_t* pipe_host[2] = {nullptr, nullptr};     // pinned [max_seqs + 1]: tokens, then the device status word
  cudaEvent_t pipe_ev[2] = {nullptr, nullptr};
  int pipe_n[2] = {0, 0};
  uint64_t pipe_ticket = 0;                        // of the most recent launch; 0 = none yet
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Live contexts. A handle that outlives its context (the convention is the other order, but a garbage-collected host
// language does not promise one) must not touch the context's stream when it is freed: it then synchronises the
// device instead.
static std::mutex g_ctx_mu;
static std::vector<kc_ctx*> g_ctxs;
static void quiesce(kc_ctx* c, int device) {
  cudaSetDevice(device);
  bool alive;
  {
    std::lock_guard<std::mutex> lk(g_ctx_mu);
    alive = std::find(g_ctxs.begin(), g_ctxs.end(), c) != g_ctxs.end();
  }
  if (alive) cudaStreamSynchronize(c->stream);
  else cudaDeviceSynchronize();
}

// ---------------------------------------------------------------------------
// context
// ---------------------------------------------------------------------------

extern "C" int kc_ctx_create(int device, kc_ctx_t* out) {
  if (!out) return fail(KC_ERR_INVALID, "kc_ctx_create: out is NULL");
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return fail(KC_ERR_CUDA, "kc_ctx_create: no CUDA device (%s)", cudaGetErrorString(e));
  if (device < 0 || device >= count) return fail(KC_ERR_INVALID, "kc_ctx_create: device %d of %d", device, count);
  CK(cudaSetDevice(device));
  cudaDeviceProp prop;
  CK(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(KC_ERR_UNSUPPORTED, "kc_ctx_create: device is sm_%d%d; this library is built for sm_100a only",
                prop.major, prop.minor);
  kc_ctx* c = new kc_ctx;
  c->device = device;
  c->sm_count = prop.multiProcessorCount;
  if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaMalloc(&c->status, sizeof(uint32_t)) != cudaSuccess ||
      cudaMallocHost(&c->status_host, sizeof(uint32_t)) != cudaSuccess ||
      cudaMemsetAsync(c->status, 0, sizeof(uint32_t), c->stream) != cudaSuccess) {
    if (c->stream) cudaStreamDestroy(c->stream);
    cudaFree(c->status);
    if (c->status_host) cudaFreeHost(c->status_host);
    delete c;
    return fail(KC_ERR_CUDA, "kc_ctx_create: stream/status allocation failed");
  }
  cudaEventCreate(&c->step_a);
  cudaEventCreate(&c->step_b);
  g_live++;
  {
    std::lock_guard<std::mutex> lk(g_ctx_mu);
    g_ctxs.push_back(c);
  }
  *out = c;
  return KC_OK;
}

extern "C" void kc_ctx_destroy(kc_ctx_t c) {
  if (!c) return;
  {
    std::lock_guard<std::mutex> lk(g_ctx_mu);
    g_ctxs.erase(std::remove(g_ctxs.begin(), g_ctxs.end(), c), g_ctxs.end());
  }
  cudaSetDevice(c->device);
  cudaStreamSynchronize(c->stream);
  for (auto& sp : c->spans) { cudaEventDestroy(sp.a); cudaEventDestroy(sp.b); }
  for (auto e : c->event_pool) cudaEventDestroy(e);
  cudaEventDestroy(c->step_a);
  cudaEventDestroy(c->step_b);
  if (c->comm) ncclCommDestroy(c->comm);
  cudaFree(c->status);
  cudaFreeHost(c->status_host);
  cudaStreamDestroy(c->stream);
  delete c;
  g_live--;
}

// Queues the copy of the status word into the context's pinned word; the caller synchronises the stream and then
// calls status_verdict. A bounded wait that gave up therefore never passes as success: every entry point that
// synchronises returns KC_ERR_TIMEOUT when a kernel of the queue before it abandoned its work.
static cudaError_t status_fetch(kc_ctx* c) {
  return cudaMemcpyAsync(c->status_host, c->status, sizeof(uint32_t), cudaMemcpyDeviceToHost, c->stream);
}
static int status_verdict(kc_ctx* c, const char* where) {
  const uint32_t st = *c->status_host;
  if (!st) return KC_OK;
  *c->status_host = 0;
  cudaMemsetAsync(c->status, 0, sizeof(uint32_t), c->stream);
  return fail(KC_ERR_TIMEOUT, "%s: device status 0x%x: a bounded wait gave up (kernel 0x%x, wait %u); the results of the "
              "calls since the last synchronisation are not valid", where, st, st & 0xff00u, st & 0xffu);
}

extern "C" int kc_sync(kc_ctx_t c) {
  if (!c) return fail(KC_ERR_INVALID, "kc_sync: ctx is NULL");
  CK(cudaSetDevice(c->device));
  CK(status_fetch(c));
  CK(cudaStreamSynchronize(c->stream));
  return status_verdict(c, "kc_sync");
}

extern "C" void* kc_ctx_stream(kc_ctx_t c) { return c ? (void*)c->stream : nullptr; }

extern "C" int kc_device_status(kc_ctx_t c, uint32_t* status) {
  if (!c || !status) return fail(KC_ERR_INVALID, "kc_device_status: NULL argument");
  CK(cudaSetDevice(c->device));
  CK(status_fetch(c));
  CK(cudaStreamSynchronize(c->stream));
  *status = *c->status_host;
  return status_verdict(c, "kc_device_status");
}

extern "C" int64_t kc_launch_count(kc_ctx_t c) { return c ? c->launches : 0; }
extern "C" double kc_last_step_ms(kc_ctx_t c) { return c ? (double)c->last_step_ms : 0.0; }

extern "C" int kc_profile_enable(kc_ctx_t c, int32_t on) {
  if (!c) return fail(KC_ERR_INVALID, "kc_profile_enable: NULL");
  c->profile = on ? 1 : 0;
  return KC_OK;
}

extern "C" int kc_profile_read(kc_ctx_t c, double* ms_out, int64_t* launches_out) {
  if (!c || !ms_out || !launches_out) return fail(KC_ERR_INVALID, "kc_profile_read: NULL argument");
  CK(cudaStreamSynchronize(c->stream));
  for (int i = 0; i < KC_PROFILE_CLASSES; ++i) { ms_out[i] = 0.0; launches_out[i] = c->class_launches[i]; c->class_launches[i] = 0; }
  for (auto& sp : c->spans) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, sp.a, sp.b) == cudaSuccess) ms_out[sp.cls] += ms;
    c->event_pool.push_back(sp.a);
    c->event_pool.push_back(sp.b);
  }
  c->spans.clear();
  return KC_OK;
}

extern "C" int kc_draft_stats(kc_ctx_t c, double* ms_out, int64_t* tokens_out, int64_t* calls_out, int32_t reset) {
  if (!c) return fail(KC_ERR_INVALID, "kc_draft_stats: NULL");
  if (ms_out) *ms_out = c->draft_ms;
  if (tokens_out) *tokens_out = c->draft_tokens;
  if (calls_out) *calls_out = c->draft_calls;
  if (reset) { c->draft_ms = 0.0; c->draft_tokens = 0; c->draft_calls = 0; }
  return KC_OK;
}

extern "C" int kc_tp_unique_id(void* out128) {
  if (!out128) return fail(KC_ERR_INVALID, "kc_tp_unique_id: NULL");
  ncclUniqueId id;
  if (ncclGetUniqueId(&id) != ncclSuccess) return fail(KC_ERR_CUDA, "ncclGetUniqueId failed");
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId size");
  memcpy(out128, &id, 128);
  return KC_OK;
}

extern "C" int kc_tp_init(kc_ctx_t c, const void* unique_id, int32_t rank, int32_t world) {
  if (!c || !unique_id) return fail(KC_ERR_INVALID, "kc_tp_init: NULL argument");
  if (world < 1 || rank < 0 || rank >= world) return fail(KC_ERR_INVALID, "kc_tp_init: rank %d of %d", rank, world);
  CK(cudaSetDevice(c->device));
  ncclUniqueId id;
  memcpy(&id, unique_id, 128);
  ncclResult_t r = ncclCommInitRank(&c->comm, world, id, rank);
  if (r != ncclSuccess) return fail(KC_ERR_CUDA, "ncclCommInitRank: %s", ncclGetErrorString(r));
  c->tp_rank = rank; c->tp_world = world;
  return KC_OK;
}

// ---------------------------------------------------------------------------
// KV pools
// ---------------------------------------------------------------------------

extern "C" int kc_kv_create(kc_ctx_t c, int32_t layers, int32_t kv_heads, int32_t head_dim, int32_t num_blocks,
                            int32_t block_size, int32_t dtype, kc_kv_t* out) {
  if (!c || !out) return fail(KC_ERR_INVALID, "kc_kv_create: NULL argument");
  if (dtype != KC_BF16) return fail(KC_ERR_UNSUPPORTED, "kc_kv_create: pools are bf16 (dtype tag %d given)", dtype);
  if (layers < 1 || kv_heads < 1 || num_blocks < 1) return fail(KC_ERR_INVALID, "kc_kv_create: empty geometry");
  if (head_dim != 64 && head_dim != 128 && head_dim != 256)
    return fail(KC_ERR_UNSUPPORTED, "kc_kv_create: head_dim %d (64, 128 or 256)", head_dim);
  if (block_size < 16 || block_size > 128 || (block_size & (block_size - 1)))
    return fail(KC_ERR_UNSUPPORTED, "kc_kv_create: block_size %d (a power of two in 16..128)", block_size);
  const size_t rows = (size_t)layers * 2 * num_blocks * kv_heads * block_size;
  if (rows > 0x7fffffffull) return fail(KC_ERR_UNSUPPORTED, "kc_kv_create: %zu pool rows overflow i32 addressing", rows);
  CK(cudaSetDevice(c->device));
  kc_kv* kv = new kc_kv;
  kv->ctx = c; kv->device = c->device; kv->layers = layers; kv->kv_heads = kv_heads; kv->head_dim = head_dim;
  kv->num_blocks = num_blocks; kv->block_size = block_size;
  kv->block_elems = (size_t)kv_heads * block_size * head_dim;
  kv->bytes = rows * head_dim * sizeof(bf16);
  cudaError_t e = cudaMalloc(&kv->pool, kv->bytes);
  if (e != cudaSuccess) { delete kv; return fail(KC_ERR_OOM, "kc_kv_create: %zu bytes: %s", kv->bytes, cudaGetErrorString(e)); }
  e = cudaMemsetAsync(kv->pool, 0, kv->bytes, c->stream);
  const char* terr = "";
  if (e == cudaSuccess && !getenv("KILN_KV_MAP_2D")) {   // KILN_KV_MAP_2D=1 keeps the 2-D map (4 operations per tile pair)
    const char* e4 = "";
    kv->map4d = make_tmap_kv_4d(&kv->map, kv->pool, head_dim, (uint64_t)num_blocks * kv_heads * block_size, (uint64_t)layers * 2, &e4);
  }
  if (e != cudaSuccess || (!kv->map4d && !make_tmap_bf16_2d(&kv->map, kv->pool, head_dim, rows, 64, 16, &terr))) {
    cudaFree(kv->pool); delete kv;
    return fail(KC_ERR_CUDA, "kc_kv_create: %s", e != cudaSuccess ? cudaGetErrorString(e) : terr);
  }
  g_live++;
  *out = kv;
  return KC_OK;
}

extern "C" void kc_kv_free(kc_kv_t kv) {
  if (!kv) return;
  quiesce(kv->ctx, kv->device);
  cudaFree(kv->pool);
  delete kv;
  g_live--;
}

extern "C" int64_t kc_kv_block_bytes(kc_kv_t kv) {
  return kv ? (int64_t)(kv->block_elems * sizeof(bf16) * 2 * kv->layers) : 0;
}
extern "C" int64_t kc_kv_allocated_bytes(kc_kv_t kv) { return kv ? (int64_t)kv->bytes : 0; }

extern "C" int kc_kv_reset(kc_kv_t kv) {
  if (!kv) return fail(KC_ERR_INVALID, "kc_kv_reset: NULL");
  CK(cudaMemsetAsync(kv->pool, 0, kv->bytes, kv->ctx->stream));
  return KC_OK;
}

extern "C" int kc_kv_copy_block(kc_kv_t kv, uint32_t src, uint32_t dst) {
  if (!kv) return fail(KC_ERR_INVALID, "kc_kv_copy_block: NULL");
  if (src >= (uint32_t)kv->num_blocks || dst >= (uint32_t)kv->num_blocks)
    return fail(KC_ERR_INVALID, "kc_kv_copy_block: block %u -> %u of %d", src, dst, kv->num_blocks);
  if (src == dst) return KC_OK;
  LAUNCH(kv->ctx, KC_PROF_ROWWISE, 1, launch_copy_block(kv->pool, kv->layers, kv->num_blocks, kv->block_elems, src, dst, kv->ctx->stream));
  return KC_OK;
}

static int kv_block_io(kc_kv_t kv, uint32_t block, void* host, size_t n, bool read) {
  if (!kv || !host) return fail(KC_ERR_INVALID, "kc_kv_%s_block: NULL argument", read ? "read" : "write");
  if (block >= (uint32_t)kv->num_blocks) return fail(KC_ERR_INVALID, "block %u of %d", block, kv->num_blocks);
  const size_t plane = kv->block_elems * sizeof(bf16);
  if (n != plane * 2 * kv->layers)
    return fail(KC_ERR_INVALID, "block payload of %zu bytes does not match the pool geometry (%zu expected)", n,
                plane * 2 * kv->layers);
  for (int l = 0; l < kv->layers; ++l)
    for (int s = 0; s < 2; ++s) {
      uint8_t* dev = reinterpret_cast<uint8_t*>(kv->pool) + (((size_t)l * 2 + s) * kv->num_blocks + block) * plane;
      uint8_t* h = static_cast<uint8_t*>(host) + ((size_t)l * 2 + s) * plane;
      if (read) CK(cudaMemcpyAsync(h, dev, plane, cudaMemcpyDeviceToHost, kv->ctx->stream));
      else CK(cudaMemcpyAsync(dev, h, plane, cudaMemcpyHostToDevice, kv->ctx->stream));
    }
  CK(cudaStreamSynchronize(kv->ctx->stream));
  return KC_OK;
}
extern "C" int kc_kv_read_block(kc_kv_t kv, uint32_t block, void* dst, size_t n) {
  return kv_block_io(kv, block, dst, n, true);
}
extern "C" int kc_kv_write_block(kc_kv_t kv, uint32_t block, const void* src, size_t n) {
  return kv_block_io(kv, block, const_cast<void*>(src), n, false);
}

// ---------------------------------------------------------------------------
// GEMM dispatch
// ---------------------------------------------------------------------------

// y = x . dequant(W)^T for M rows. When `fused` is given and the weight is split along K, the reduction is left
// to the consumer kernel: *fused then describes the fp32 partials instead of y (one launch and one round trip
// through memory less). Rows beyond one 512-row slab always go through the reduction kernel.
static int run_qlinear(kc_ctx* c, const QWeight& w, const ActOperand& x, int M, bf16* y, int ldy, float* partial,
                       SublayerOut* fused = nullptr) {
  const bool defer = fused && w.splits > 1 && M <= QL_MAX_M;
  for (int row0 = 0; row0 < M; row0 += QL_MAX_M) {
    QLinearLaunch l;
    l.w = &w; l.x = &x; l.row0 = row0; l.M = std::min(QL_MAX_M, M - row0);
    l.y = y; l.ldy = ldy; l.partial = partial; l.status = c->status;
    LAUNCH(c, KC_PROF_GEMM, qlinear_launches(w, l.M), qlinear_umma(l, c->stream));
    if (w.splits > 1 && !defer)
      LAUNCH(c, KC_PROF_GEMM_REDUCE, 1, qlinear_reduce_splits(partial, w.splits, l.M, w.N, y + (size_t)row0 * ldy, ldy, c->stream));
  }
  if (fused) *fused = defer ? SublayerOut::partials(partial, w.splits, (size_t)M, w.N) : SublayerOut::dense(y, ldy);
  return KC_OK;
}

// act[M, F] = activation(x . Wgate^T) * (x . Wup^T) for a gate_up weight whose tiles alternate gate / up. Row slabs
// whose GEMM launch owns whole tile pairs get the activation in the GEMM's epilogue; the others write the
// interleaved [M, 2F] product and run the element-wise kernel on it. Both ways round at the same points.
static int run_gated(kc_ctx* c, const QWeight& w, const ActOperand& x, int M, bf16* gu, int F, int gelu, bool interleaved,
                     bf16* act, float* partial) {
  for (int row0 = 0; row0 < M; row0 += QL_MAX_M) {
    const int rows = std::min(QL_MAX_M, M - row0);
    int done = 0;
    QLinearLaunch l;
    l.w = &w; l.x = &x; l.row0 = row0; l.M = rows;
    l.y = gu; l.ldy = 2 * F; l.partial = partial; l.status = c->status;
    if (interleaved) { l.glu = gelu ? 2 : 1; l.act = act; l.ld_act = F; l.glu_done = &done; }
    LAUNCH(c, KC_PROF_GEMM, qlinear_launches(w, rows), qlinear_umma(l, c->stream));
    if (done) continue;
    if (w.splits > 1)
      LAUNCH(c, KC_PROF_GEMM_REDUCE, 1, qlinear_reduce_splits(partial, w.splits, rows, w.N, gu + (size_t)row0 * 2 * F, 2 * F, c->stream));
    LAUNCH(c, KC_PROF_ROWWISE, 1, launch_glu(gu + (size_t)row0 * 2 * F, rows, F, gelu, interleaved ? 1 : 0, act + (size_t)row0 * F, c->stream));
  }
  return KC_OK;
}

// The weight-streaming lane for at most QL_STREAM_MAX_M rows: *out describes where the result is (bf16 y, or the
// fp32 partials of the lane for the consumer kernel to sum); without `out` they are reduced into y here.
static int run_stream(kc_ctx* c, const QWeight& w, const bf16* x, int M, bf16* y, int ldy, float* partial, SublayerOut* out) {
  const int pieces = qlinear_stream_pieces(w);
  LAUNCH(c, KC_PROF_GEMM, 1, qlinear_stream(w, x, w.K, M, partial, c->status, c->stream));
  if (!out) LAUNCH(c, KC_PROF_GEMM_REDUCE, 1, qlinear_reduce_splits(partial, pieces, M, w.N, y, ldy, c->stream));
  else *out = SublayerOut::partials(partial, pieces, (size_t)M, w.N);
  return KC_OK;
}

// The small-weight lane (qlinear_gemv): same contract as run_stream.
static int run_gemv(kc_ctx* c, const QWeight& w, const bf16* x, int M, bf16* y, int ldy, float* partial, SublayerOut* out) {
  const int pieces = qlinear_gemv_pieces(w);
  LAUNCH(c, KC_PROF_GEMM, 1, qlinear_gemv(w, x, w.K, M, partial, c->status, c->stream));
  if (!out) LAUNCH(c, KC_PROF_GEMM_REDUCE, 1, qlinear_reduce_splits(partial, pieces, M, w.N, y, ldy, c->stream));
  else *out = SublayerOut::partials(partial, pieces, (size_t)M, w.N);
  return KC_OK;
}

// ---------------------------------------------------------------------------
// stand-alone quantised weight (parity tests / composed graphs)
// ---------------------------------------------------------------------------

static int upload(kc_ctx* c, const void* src, size_t bytes, int on_device, void** out) {
  CK(cudaMalloc(out, std::max<size_t>(bytes, 16)));
  CK(cudaMemcpyAsync(*out, src, bytes, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, c->stream));
  return KC_OK;
}

static int check_quant(int bits, int group, int in_features, const char* what) {
  if (bits != 4 && bits != 8) return fail(KC_ERR_UNSUPPORTED, "%s: bits %d (4 or 8)", what, bits);
  if (group != 32 && group != 64 && group != 128) return fail(KC_ERR_UNSUPPORTED, "%s: group_size %d (32, 64 or 128)", what, group);
  if (in_features % 64 || in_features % group)
    return fail(KC_ERR_UNSUPPORTED, "%s: in_features %d must be a multiple of 64 and of the group size", what, in_features);
  return KC_OK;
}

extern "C" int kc_qweight_create(kc_ctx_t c, const uint32_t* w, const void* scales, const void* biases,
                                 int32_t out_features, int32_t in_features, int32_t bits, int32_t group_size,
                                 int32_t on_device, kc_qweight_t* out) {
  if (!c || !w || !scales || !biases || !out) return fail(KC_ERR_INVALID, "kc_qweight_create: NULL argument");
  if (out_features < 1) return fail(KC_ERR_INVALID, "kc_qweight_create: out_features %d", out_features);
  int rc = check_quant(bits, group_size, in_features, "kc_qweight_create");
  if (rc) return rc;
  CK(cudaSetDevice(c->device));
  void *dw = nullptr, *ds = nullptr, *db = nullptr;
  const size_t wb = (size_t)out_features * in_features * bits / 8;
  const size_t sb = (size_t)out_features * (in_features / group_size) * 2;
  if ((rc = upload(c, w, wb, on_device, &dw)) || (rc = upload(c, scales, sb, on_device, &ds)) ||
      (rc = upload(c, biases, sb, on_device, &db))) {
    cudaFree(dw); cudaFree(ds); cudaFree(db);
    return rc;
  }
  kc_qweight* q = new kc_qweight;
  q->ctx = c; q->device = c->device;
  cudaError_t e = qweight_build(&q->w, (const uint32_t*)dw, (const bf16*)ds, (const bf16*)db, out_features,
                                in_features, bits, group_size, c->sm_count, c->stream);
  if (e == cudaSuccess) {
    const size_t need = std::max({(size_t)(q->w.splits > 1 ? q->w.splits : 0) * QL_MAX_M * q->w.N,
                                  (size_t)qlinear_stream_pieces(q->w) * QL_STREAM_MAX_M * q->w.N,
                                  (size_t)qlinear_gemv_pieces(q->w) * QL_STREAM_MAX_M * q->w.N});
    if (need) e = cudaMalloc(&q->partial, need * sizeof(float));
  }
  cudaStreamSynchronize(c->stream);
  cudaFree(dw); cudaFree(ds); cudaFree(db);
  if (e != cudaSuccess) { qweight_free(&q->w); delete q; return fail(KC_ERR_CUDA, "kc_qweight_create: %s", cudaGetErrorString(e)); }
  g_live++;
  *out = q;
  return KC_OK;
}

extern "C" void kc_qweight_free(kc_qweight_t q) {
  if (!q) return;
  quiesce(q->ctx, q->device);
  qweight_free(&q->w);
  cudaFree(q->partial);
  delete q;
  g_live--;
}

extern "C" int kc_quantized_matmul(kc_ctx_t c, kc_qweight_t q, const void* x_dev, int32_t m, void* y_dev) {
  if (!c || !q || !x_dev || !y_dev) return fail(KC_ERR_INVALID, "kc_quantized_matmul: NULL argument");
  if (m < 1) return fail(KC_ERR_INVALID, "kc_quantized_matmul: m = %d", m);
  if ((uintptr_t)x_dev % 16) return fail(KC_ERR_INVALID, "kc_quantized_matmul: x must be 16-byte aligned");
  if (q->ctx != c) return fail(KC_ERR_INVALID, "kc_quantized_matmul: the weight was created on another context");
  CK(cudaSetDevice(c->device));
  // x must be readable for round_up(m, 16) rows; rows past m may hold anything.
  const int rows = (m + 15) & ~15;
  if (q->op_ptr != x_dev || q->op_rows != rows) {
    const char* terr = "";
    if (!act_operand_init(&q->op, (const bf16*)x_dev, rows, q->w.K, &terr)) return fail(KC_ERR_CUDA, "kc_quantized_matmul: %s", terr);
    q->op_ptr = x_dev; q->op_rows = rows;
  }
  RC(run_qlinear(c, q->w, q->op, m, (bf16*)y_dev, q->w.N, q->partial));
  return KC_OK;
}

// The weight-streaming lane on its own (at most 8 rows): what a model with the lane switched on runs for its decode
// forwards (kc_model_set_stream_lane).
extern "C" int kc_quantized_matmul_stream(kc_ctx_t c, kc_qweight_t q, const void* x_dev, int32_t m, void* y_dev) {
  if (!c || !q || !x_dev || !y_dev) return fail(KC_ERR_INVALID, "kc_quantized_matmul_stream: NULL argument");
  if (m < 1 || m > QL_STREAM_MAX_M) return fail(KC_ERR_INVALID, "kc_quantized_matmul_stream: m = %d (1..%d)", m, QL_STREAM_MAX_M);
  if ((uintptr_t)x_dev % 16) return fail(KC_ERR_INVALID, "kc_quantized_matmul_stream: x must be 16-byte aligned");
  if (q->ctx != c) return fail(KC_ERR_INVALID, "kc_quantized_matmul_stream: the weight was created on another context");
  CK(cudaSetDevice(c->device));
  LAUNCH(c, KC_PROF_GEMM, 1, qlinear_stream(q->w, (const bf16*)x_dev, q->w.K, m, q->partial, c->status, c->stream));
  LAUNCH(c, KC_PROF_GEMM_REDUCE, 1, qlinear_reduce_splits(q->partial, qlinear_stream_pieces(q->w), m, q->w.N, (bf16*)y_dev, q->w.N, c->stream));
  return KC_OK;
}

extern "C" int kc_quantized_matmul_gemv(kc_ctx_t c, kc_qweight_t q, const void* x_dev, int32_t m, void* y_dev) {
  if (!c || !q || !x_dev || !y_dev) return fail(KC_ERR_INVALID, "kc_quantized_matmul_gemv: NULL argument");
  if (m < 1 || m > QL_STREAM_MAX_M) return fail(KC_ERR_INVALID, "kc_quantized_matmul_gemv: m = %d (1..%d)", m, QL_STREAM_MAX_M);
  if ((uintptr_t)x_dev % 16) return fail(KC_ERR_INVALID, "kc_quantized_matmul_gemv: x must be 16-byte aligned");
  if (q->ctx != c) return fail(KC_ERR_INVALID, "kc_quantized_matmul_gemv: the weight was created on another context");
  if (qlinear_gemv_pieces(q->w) == 0)
    return fail(KC_ERR_UNSUPPORTED, "kc_quantized_matmul_gemv: a weight of %d x %d does not fit the small-weight lane", q->w.N, q->w.K);
  CK(cudaSetDevice(c->device));
  RC(run_gemv(c, q->w, (const bf16*)x_dev, m, (bf16*)y_dev, q->w.N, q->partial, nullptr));
  return KC_OK;
}

extern "C" int kc_rms_norm(kc_ctx_t c, const void* x_dev, const void* weight_dev, int32_t rows, int32_t dim, float eps,
                           void* y_dev) {
  if (!c || !x_dev || !weight_dev || !y_dev) return fail(KC_ERR_INVALID, "kc_rms_norm: NULL argument");
  if (rows < 1 || dim < 2 || dim % 2 || dim > 12288) return fail(KC_ERR_INVALID, "kc_rms_norm: [%d, %d]", rows, dim);
  CK(cudaSetDevice(c->device));
  LAUNCH(c, KC_PROF_ROWWISE, 1, launch_add_rmsnorm((const bf16*)x_dev, SublayerOut::none(), nullptr, (const bf16*)weight_dev, nullptr, rows, dim, eps, nullptr,
                        (bf16*)y_dev, c->stream));
  return KC_OK;
}

// ---------------------------------------------------------------------------
// model loading
// ---------------------------------------------------------------------------

namespace {

struct TensorIndex {
  std::map<std::string, const kc_tensor_view*> m;
  std::map<std::string, bool> used;
  const kc_tensor_view* take(const std::string& name) {
    auto it = m.find(name);
    if (it == m.end()) return nullptr;
    used[name] = true;
    return it->second;
  }
};

// Copies rows [r0, r1) x byte columns [c0, c1) of a row-major tensor into dst (device), row pitch = c1 - c0.
int copy_slice(kc_ctx* c, const kc_tensor_view* t, size_t row_bytes, int64_t r0, int64_t r1, size_t c0, size_t c1,
               uint8_t* dst) {
  const uint8_t* src = static_cast<const uint8_t*>(t->data) + (size_t)r0 * row_bytes + c0;
  CK(cudaMemcpy2DAsync(dst, c1 - c0, src, row_bytes, c1 - c0, (size_t)(r1 - r0),
                       t->on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, c->stream));
  return KC_OK;
}

struct Part { std::string prefix; int64_t r0, r1; };  // one source linear and the output rows taken from it

// Builds one QWeight from the row-concatenation of `parts`, taking input columns [k0, k1).
int build_linear(kc_model* m, TensorIndex& idx, const std::vector<Part>& parts, int K_full, int k0, int k1, QWeight* out,
                 bf16** bias_out) {
  kc_ctx* c = m->ctx;
  const int bits = m->d.bits, group = m->d.group_size;
  const int K = k1 - k0;
  int64_t N = 0;
  for (auto& p : parts) N += p.r1 - p.r0;
  const size_t wrow = (size_t)K * bits / 8, srow = (size_t)(K / group) * 2;
  uint8_t *dw = nullptr, *ds = nullptr, *db = nullptr;
  bf16* dbias = nullptr;
  CK(cudaMalloc(&dw, N * wrow)); CK(cudaMalloc(&ds, N * srow)); CK(cudaMalloc(&db, N * srow));
  int64_t at = 0;
  bool any_bias = false;
  for (auto& p : parts) {
    const kc_tensor_view* w = idx.take(p.prefix + ".weight");
    const kc_tensor_view* s = idx.take(p.prefix + ".scales");
    const kc_tensor_view* b = idx.take(p.prefix + ".biases");
    if (!w || !s || !b) { cudaFree(dw); cudaFree(ds); cudaFree(db); return fail(KC_ERR_INVALID, "missing tensor %s.{weight,scales,biases}", p.prefix.c_str()); }
    if (w->dtype != KC_U32 || s->dtype != KC_BF16 || b->dtype != KC_BF16 || w->ndim != 2 || s->ndim != 2 || b->ndim != 2 ||
        w->shape[1] != (int64_t)K_full * bits / 32 || s->shape[1] != K_full / group || b->shape[1] != K_full / group ||
        w->shape[0] < p.r1 || s->shape[0] != w->shape[0] || b->shape[0] != w->shape[0]) {
      cudaFree(dw); cudaFree(ds); cudaFree(db);
      return fail(KC_ERR_INVALID, "tensor %s: shape/dtype does not match the config (in %d, bits %d, group %d)",
                  p.prefix.c_str(), K_full, bits, group);
    }
    const size_t wfull = (size_t)K_full * bits / 8, sfull = (size_t)(K_full / group) * 2;
    int rc;
    if ((rc = copy_slice(c, w, wfull, p.r0, p.r1, (size_t)k0 * bits / 8, (size_t)k1 * bits / 8, dw + at * wrow)) ||
        (rc = copy_slice(c, s, sfull, p.r0, p.r1, (size_t)(k0 / group) * 2, (size_t)(k1 / group) * 2, ds + at * srow)) ||
        (rc = copy_slice(c, b, sfull, p.r0, p.r1, (size_t)(k0 / group) * 2, (size_t)(k1 / group) * 2, db + at * srow))) {
      cudaFree(dw); cudaFree(ds); cudaFree(db); return rc;
    }
    if (bias_out && idx.m.count(p.prefix + ".bias")) any_bias = true;
    at += p.r1 - p.r0;
  }
  if (bias_out && any_bias) {
    CK(cudaMalloc(&dbias, N * sizeof(bf16)));
    CK(cudaMemsetAsync(dbias, 0, N * sizeof(bf16), c->stream));
    at = 0;
    for (auto& p : parts) {
      const kc_tensor_view* bi = idx.take(p.prefix + ".bias");
      if (bi) {
        if (bi->dtype != KC_BF16 || bi->shape[0] < p.r1) { cudaFree(dw); cudaFree(ds); cudaFree(db); return fail(KC_ERR_INVALID, "tensor %s.bias: bad shape/dtype", p.prefix.c_str()); }
        CK(cudaMemcpyAsync(dbias + at, static_cast<const bf16*>(bi->data) + p.r0, (p.r1 - p.r0) * sizeof(bf16),
                           bi->on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, c->stream));
      }
      at += p.r1 - p.r0;
    }
    *bias_out = dbias;
  }
  cudaError_t e = qweight_build(out, (const uint32_t*)dw, (const bf16*)ds, (const bf16*)db, (int)N, K, bits, group,
                                c->sm_count, c->stream);
  cudaStreamSynchronize(c->stream);
  cudaFree(dw); cudaFree(ds); cudaFree(db);
  if (e != cudaSuccess) return fail(e == cudaErrorMemoryAllocation ? KC_ERR_OOM : KC_ERR_CUDA, "re-tiling %s: %s", parts[0].prefix.c_str(), cudaGetErrorString(e));
  m->weight_bytes += (int64_t)out->mlx_bytes();
  return KC_OK;
}

// Norm weight [H] bf16; Gemma's 1 + w is folded in at load (NormStyle::OnePlus, nn.rs:241-257).
int load_norm(kc_model* m, TensorIndex& idx, const std::string& name, bool one_plus, bf16** out) {
  const kc_tensor_view* t = idx.take(name);
  const int H = m->d.hidden_size;
  if (!t) return fail(KC_ERR_INVALID, "missing tensor %s", name.c_str());
  if (t->dtype != KC_BF16 || t->shape[0] != H) return fail(KC_ERR_INVALID, "tensor %s: expected bf16 [%d]", name.c_str(), H);
  std::vector<uint16_t> host(H);
  CK(cudaMemcpyAsync(host.data(), t->data, H * 2, t->on_device ? cudaMemcpyDeviceToHost : cudaMemcpyHostToHost, m->ctx->stream));
  CK(cudaStreamSynchronize(m->ctx->stream));
  if (one_plus) {
    for (auto& v : host) {
      uint32_t u = (uint32_t)v << 16; float f; memcpy(&f, &u, 4);
      f = 1.0f + f;  // bf16 add of the weak scalar 1
      memcpy(&u, &f, 4);
      const uint32_t lsb = (u >> 16) & 1u;
      u += 0x7fffu + lsb;
      v = (uint16_t)(u >> 16);
    }
  }
  CK(cudaMalloc(out, H * 2));
  CK(cudaMemcpyAsync(*out, host.data(), H * 2, cudaMemcpyHostToDevice, m->ctx->stream));
  CK(cudaStreamSynchronize(m->ctx->stream));
  return KC_OK;
}

// Rope frequency table (crates/kiln-models/src/nn.rs:1409-1477): inv_freq[i] multiplies the position.
std::vector<float> rope_inv_freq(const kc_model_desc& d) {
  const int half = d.head_dim / 2;
  std::vector<float> inv(half);
  for (int i = 0; i < half; ++i) {
    // freqs = base ** (arange(0, dims, 2) / dims) in float32
    const float expo = (float)(2 * i) / (float)d.head_dim;
    float freq = powf(d.rope_theta, expo);
    if (d.rope_scaling == KC_ROPE_LLAMA3) {
      const float wavelen = (float)(2.0 * M_PI) * freq;
      const float low_wl = d.rope_original_max_position / d.rope_low_freq_factor;
      const float high_wl = d.rope_original_max_position / d.rope_high_freq_factor;
      float f = freq;
      if (wavelen > low_wl) f = freq * d.rope_factor;
      const bool medium = wavelen > high_wl && wavelen < low_wl;
      if (medium) {
        const float smooth = (d.rope_original_max_position / wavelen - d.rope_low_freq_factor) /
                             (d.rope_high_freq_factor - d.rope_low_freq_factor);
        f = f / ((1.0f - smooth) / d.rope_factor + smooth);
      }
      freq = f;
    }
    float v = 1.0f / freq;
    if (d.rope_scaling == KC_ROPE_LINEAR && d.rope_factor != 0.f) v *= 1.0f / d.rope_factor;
    inv[i] = v;
  }
  return inv;
}

void free_model(kc_model* m) {
  cudaFree(m->partial_gu); cudaFree(m->argmax_scratch);
  for (auto& L : m->layers) {
    qweight_free(&L.qkv); qweight_free(&L.o); qweight_free(&L.gate_up); qweight_free(&L.down);
    cudaFree(L.qkv_bias); cudaFree(L.input_ln); cudaFree(L.post_attn_ln); cudaFree(L.pre_ffw_ln); cudaFree(L.post_ffw_ln);
  }
  qweight_free(&m->head);
  cudaFree(m->emb_w); cudaFree(m->emb_s); cudaFree(m->emb_b); cudaFree(m->final_norm); cudaFree(m->inv_freq);
  cudaFree(m->h); cudaFree(m->normed); cudaFree(m->qkv); cudaFree(m->q_rot); cudaFree(m->attn); cudaFree(m->proj); cudaFree(m->proj_ranks);
  cudaFree(m->gu); cudaFree(m->act); cudaFree(m->hs); cudaFree(m->logits); cudaFree(m->partial); cudaFree(m->attn_ws);
  cudaFree(m->tp_buf);
  if (m->tp_p2p)
    for (int r = 0; r < m->d.tp_world; ++r) {
      if (r == m->d.tp_rank) continue;
      for (int b = 0; b < 2; ++b) if (m->peer_out[b][r]) cudaIpcCloseMemHandle(m->peer_out[b][r]);
      if (m->peer_flags[r]) cudaIpcCloseMemHandle(m->peer_flags[r]);
    }
  cudaFree(m->tp_out[0]); cudaFree(m->tp_out[1]); cudaFree(m->tp_flags);
  cudaFree(m->meta_dev);
  for (int i = 0; i < kc_model::kStaging; ++i) {
    if (m->meta_host[i]) cudaFreeHost(m->meta_host[i]);
    if (m->meta_ev[i]) cudaEventDestroy(m->meta_ev[i]);
  }
  cudaFree(m->row_tokens); cudaFree(m->n_committed); cudaFree(m->n_accepted); cudaFree(m->committed);
  if (m->result_host) cudaFreeHost(m->result_host);
  for (int i = 0; i < 2; ++i) {
    cudaFree(m->pipe_tokens[i]);
    if (m->pipe_host[i]) cudaFreeHost(m->pipe_host[i]);
    if (m->pipe_ev[i]) cudaEventDestroy(m->pipe_ev[i]);
  }
  delete m;
}

}  // namespace

extern "C" int kc_model_load(kc_ctx_t c, const kc_model_desc* desc, const kc_tensor_view* tensors, size_t n_tensors,
                             kc_model_t* out) {
  if (!c || !desc || !tensors || !out) return fail(KC_ERR_INVALID, "kc_model_load: NULL argument");
  const kc_model_desc& d = *desc;
  if (d.arch != KC_ARCH_LLAMA && d.arch != KC_ARCH_QWEN2 && d.arch != KC_ARCH_GEMMA2)
    return fail(KC_ERR_UNSUPPORTED, "kc_model_load: arch %d", d.arch);
  if (d.hidden_size < 64 || d.num_layers < 1 || d.num_heads < 1 || d.num_kv_heads < 1 || d.vocab_size < 1 ||
      d.intermediate_size < 64 || d.num_heads % d.num_kv_heads)
    return fail(KC_ERR_INVALID, "kc_model_load: bad geometry");
  if (d.head_dim != 64 && d.head_dim != 128 && d.head_dim != 256)
    return fail(KC_ERR_UNSUPPORTED, "kc_model_load: head_dim %d (64, 128 or 256)", d.head_dim);
  const int tp = d.tp_world < 1 ? 1 : d.tp_world;
  if (d.tp_rank < 0 || d.tp_rank >= tp) return fail(KC_ERR_INVALID, "kc_model_load: tp rank %d of %d", d.tp_rank, tp);
  if (d.num_kv_heads % tp || d.intermediate_size % (tp * 64))
    return fail(KC_ERR_UNSUPPORTED, "kc_model_load: kv heads %d / intermediate %d do not split %d ways", d.num_kv_heads,
                d.intermediate_size, tp);
  if (tp > 1 && (c->tp_world != tp || c->tp_rank != d.tp_rank))
    return fail(KC_ERR_INVALID, "kc_model_load: call kc_tp_init(rank %d, world %d) first", d.tp_rank, tp);
  int rc;
  if ((rc = check_quant(d.bits, d.group_size, d.hidden_size, "kc_model_load(hidden)"))) return rc;
  if ((rc = check_quant(d.bits, d.group_size, d.intermediate_size / tp, "kc_model_load(intermediate)"))) return rc;
  if ((rc = check_quant(d.bits, d.group_size, d.num_heads / tp * d.head_dim, "kc_model_load(attention width)"))) return rc;
  if (d.max_step_tokens < 1 || d.max_step_seqs < 1) return fail(KC_ERR_INVALID, "kc_model_load: max_step_tokens/seqs");
  const int gqa = d.num_heads / d.num_kv_heads;
  if (gqa > 64) return fail(KC_ERR_UNSUPPORTED, "kc_model_load: %d query heads per kv head", gqa);
  CK(cudaSetDevice(c->device));

  TensorIndex idx;
  for (size_t i = 0; i < n_tensors; ++i) {
    if (!tensors[i].name || !tensors[i].data) return fail(KC_ERR_INVALID, "kc_model_load: tensor %zu has no name/data", i);
    idx.m[tensors[i].name] = &tensors[i];
  }

  kc_model* m = new kc_model;
  m->ctx = c; m->device = c->device; m->d = d; m->d.tp_world = tp;
  m->Hq = d.num_heads / tp; m->Hkv = d.num_kv_heads / tp; m->F = d.intermediate_size / tp;
  m->n_qkv = (m->Hq + 2 * m->Hkv) * d.head_dim;
  const int H = d.hidden_size, D = d.head_dim, V = d.vocab_size;
  const bool gemma = d.arch == KC_ARCH_GEMMA2;
  m->attn_scale = gemma && d.query_pre_attn_scalar > 0.f ? (float)(1.0 / std::sqrt((double)d.query_pre_attn_scalar))
                                                         : (float)std::pow((double)D, -0.5);
  m->embed_scale = gemma ? (float)std::sqrt((double)H) : 0.f;

#define LOAD_FAIL(rcexpr) do { int r__ = (rcexpr); if (r__) { std::string keep = g_err; free_model(m); g_err = keep; return r__; } } while (0)

  // embedding (mlx layout, gathered) — nn.rs:1092
  {
    const kc_tensor_view* w = idx.take("model.embed_tokens.weight");
    const kc_tensor_view* s = idx.take("model.embed_tokens.scales");
    const kc_tensor_view* b = idx.take("model.embed_tokens.biases");
    if (!w || !s || !b || w->dtype != KC_U32 || w->shape[0] != V || w->shape[1] != (int64_t)H * d.bits / 32 ||
        s->shape[0] != V || s->shape[1] != H / d.group_size)
      LOAD_FAIL(fail(KC_ERR_INVALID, "model.embed_tokens: missing or mis-shaped quantised tensors"));
    LOAD_FAIL(upload(c, w->data, (size_t)V * H * d.bits / 8, w->on_device, (void**)&m->emb_w));
    LOAD_FAIL(upload(c, s->data, (size_t)V * (H / d.group_size) * 2, s->on_device, (void**)&m->emb_s));
    LOAD_FAIL(upload(c, b->data, (size_t)V * (H / d.group_size) * 2, b->on_device, (void**)&m->emb_b));
  }
  m->layers.resize(d.num_layers);
  for (int l = 0; l < d.num_layers; ++l) {
    Layer& L = m->layers[l];
    const std::string p = "model.layers." + std::to_string(l);
    const int64_t q0 = (int64_t)d.tp_rank * m->Hq * D, q1 = q0 + (int64_t)m->Hq * D;
    const int64_t k0 = (int64_t)d.tp_rank * m->Hkv * D, k1 = k0 + (int64_t)m->Hkv * D;
    LOAD_FAIL(build_linear(m, idx, {{p + ".self_attn.q_proj", q0, q1}, {p + ".self_attn.k_proj", k0, k1}, {p + ".self_attn.v_proj", k0, k1}},
                           H, 0, H, &L.qkv, &L.qkv_bias));
    LOAD_FAIL(build_linear(m, idx, {{p + ".self_attn.o_proj", 0, H}}, d.num_heads * D, (int)q0, (int)q1, &L.o, nullptr));
    const int64_t f0 = (int64_t)d.tp_rank * m->F, f1 = f0 + m->F;
    {
      // gate and up rows alternate in blocks of one GEMM tile (128 rows) when the width allows it, so a CTA that owns
      // two neighbouring tiles holds gate and up of the same features
      std::vector<Part> gu_parts;
      m->glu_interleaved = m->F % 128 == 0;
      if (m->glu_interleaved) {
        for (int64_t r = f0; r < f1; r += 128) {
          gu_parts.push_back({p + ".mlp.gate_proj", r, r + 128});
          gu_parts.push_back({p + ".mlp.up_proj", r, r + 128});
        }
      } else {
        gu_parts = {{p + ".mlp.gate_proj", f0, f1}, {p + ".mlp.up_proj", f0, f1}};
      }
      LOAD_FAIL(build_linear(m, idx, gu_parts, H, 0, H, &L.gate_up, nullptr));
    }
    LOAD_FAIL(build_linear(m, idx, {{p + ".mlp.down_proj", 0, H}}, d.intermediate_size, (int)f0, (int)f1, &L.down, nullptr));
    LOAD_FAIL(load_norm(m, idx, p + ".input_layernorm.weight", gemma, &L.input_ln));
    LOAD_FAIL(load_norm(m, idx, p + ".post_attention_layernorm.weight", gemma, &L.post_attn_ln));
    if (gemma) {
      LOAD_FAIL(load_norm(m, idx, p + ".pre_feedforward_layernorm.weight", true, &L.pre_ffw_ln));
      LOAD_FAIL(load_norm(m, idx, p + ".post_feedforward_layernorm.weight", true, &L.post_ffw_ln));
    }
  }
  LOAD_FAIL(load_norm(m, idx, "model.norm.weight", gemma, &m->final_norm));
  const bool tied = gemma || d.tie_word_embeddings;
  if (tied) {
    // mlx-lm sanitize drops a stray lm_head on tied models (nn.rs:1107-1112)
    idx.take("lm_head.weight"); idx.take("lm_head.scales"); idx.take("lm_head.biases");
    idx.used["model.embed_tokens.weight"] = idx.used["model.embed_tokens.scales"] = idx.used["model.embed_tokens.biases"] = true;
    LOAD_FAIL(build_linear(m, idx, {{"model.embed_tokens", 0, V}}, H, 0, H, &m->head, nullptr));
  } else {
    LOAD_FAIL(build_linear(m, idx, {{"lm_head", 0, V}}, H, 0, H, &m->head, nullptr));
    m->weight_bytes += (int64_t)m->head.mlx_bytes();  // the untied embedding table is held as well
  }
  // leftovers fail the load (nn.rs:1118-1128); rotary tables are ignored like mlx-lm's sanitize
  for (auto& kv : idx.m)
    if (!idx.used.count(kv.first) && kv.first.find("self_attn.rotary_emb.inv_freq") == std::string::npos)
      LOAD_FAIL(fail(KC_ERR_INVALID, "unconsumed tensor in checkpoint: %s", kv.first.c_str()));

  // rope table
  {
    std::vector<float> inv = rope_inv_freq(d);
    LOAD_FAIL(upload(c, inv.data(), inv.size() * 4, 0, (void**)&m->inv_freq));
    CK(cudaStreamSynchronize(c->stream));
  }

  // activations
  m->max_rows = (int)align_up(d.max_step_tokens, 64);
  m->max_seqs = d.max_step_seqs;
  m->logit_rows = std::min(m->max_rows, QL_MAX_M);
  const size_t R = m->max_rows;
  auto dalloc = [&](bf16** p, size_t elems) -> int {
    CK(cudaMalloc(p, elems * sizeof(bf16)));
    CK(cudaMemsetAsync(*p, 0, elems * sizeof(bf16), c->stream));
    return KC_OK;
  };
  LOAD_FAIL(dalloc(&m->h, R * H)); LOAD_FAIL(dalloc(&m->normed, R * H)); LOAD_FAIL(dalloc(&m->qkv, R * m->n_qkv));
  LOAD_FAIL(dalloc(&m->q_rot, R * m->Hq * D)); LOAD_FAIL(dalloc(&m->attn, R * m->Hq * D)); LOAD_FAIL(dalloc(&m->proj, R * H));
  if (d.tp_world > 1) LOAD_FAIL(dalloc(&m->proj_ranks, (size_t)d.tp_world * R * H));
  LOAD_FAIL(dalloc(&m->gu, R * 2 * m->F)); LOAD_FAIL(dalloc(&m->act, R * m->F)); LOAD_FAIL(dalloc(&m->hs, (size_t)m->logit_rows * H));
  LOAD_FAIL(dalloc(&m->logits, (size_t)m->logit_rows * V));
  const char* terr = "";
  if (!act_operand_init(&m->op_normed, m->normed, (int)R, H, &terr) || !act_operand_init(&m->op_attn, m->attn, (int)R, m->Hq * D, &terr) ||
      !act_operand_init(&m->op_act, m->act, (int)R, m->F, &terr) || !act_operand_init(&m->op_hs, m->hs, m->logit_rows, H, &terr))
    LOAD_FAIL(fail(KC_ERR_CUDA, "kc_model_load: %s", terr));
  // split-K workspace: the largest splits * N over all weights, for one 512-row slab
  {
    size_t need = 0;
    auto acc = [&](const QWeight& w) {
      if (w.splits > 1) need = std::max(need, (size_t)w.splits * QL_MAX_M * w.N * sizeof(float));
      // the weight-streaming lane's partials, at most 8 rows
      need = std::max(need, (size_t)qlinear_stream_pieces(w) * QL_STREAM_MAX_M * w.N * sizeof(float));
      need = std::max(need, (size_t)qlinear_gemv_pieces(w) * QL_STREAM_MAX_M * w.N * sizeof(float));
    };
    for (auto& L : m->layers) { acc(L.qkv); acc(L.o); acc(L.gate_up); acc(L.down); }
    acc(m->head);
    if (need) { cudaError_t e = cudaMalloc(&m->partial, need); if (e != cudaSuccess) LOAD_FAIL(fail(KC_ERR_OOM, "split-K workspace: %s", cudaGetErrorString(e))); }
    m->partial_bytes = need;
  }
  if (tp > 1) {
    cudaError_t e = cudaMalloc(&m->tp_buf, R * H * sizeof(float));
    m->tp_sum_off = R * H;
    for (int b = 0; b < 2 && e == cudaSuccess; ++b) e = cudaMalloc(&m->tp_out[b], 2 * R * H * sizeof(bf16));
    if (e == cudaSuccess) e = cudaMalloc(&m->tp_flags, 2 * KC_MAX_TP * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemsetAsync(m->tp_flags, 0, 2 * KC_MAX_TP * sizeof(uint32_t), c->stream);
    if (e != cudaSuccess) LOAD_FAIL(fail(KC_ERR_OOM, "tensor-parallel buffers: %s", cudaGetErrorString(e)));
  }
  {
    cudaError_t e = cudaSuccess;
    if (e == cudaSuccess) e = cudaMalloc(&m->row_tokens, R * 4);
    if (e == cudaSuccess) e = cudaMalloc(&m->n_committed, (size_t)m->max_seqs * 4);
    if (e == cudaSuccess) e = cudaMalloc(&m->n_accepted, (size_t)m->max_seqs * 4);
    if (e == cudaSuccess) e = cudaMalloc(&m->committed, R * 4);
    if (e == cudaSuccess) e = cudaMallocHost(&m->result_host, R * 4 + (size_t)m->max_seqs * 8 + 64);
    for (int i = 0; i < kc_model::kStaging && e == cudaSuccess; ++i) e = cudaEventCreateWithFlags(&m->meta_ev[i], cudaEventDisableTiming);
    for (int i = 0; i < 2 && e == cudaSuccess; ++i) {
      e = cudaMalloc(&m->pipe_tokens[i], (size_t)m->max_seqs * 4);
      if (e == cudaSuccess) e = cudaMallocHost(&m->pipe_host[i], ((size_t)m->max_seqs + 1) * 4);
      if (e == cudaSuccess) e = cudaEventCreateWithFlags(&m->pipe_ev[i], cudaEventDisableTiming);
    }
    if (e != cudaSuccess) LOAD_FAIL(fail(KC_ERR_OOM, "kc_model_load: result buffers: %s", cudaGetErrorString(e)));
  }
  CK(cudaStreamSynchronize(c->stream));
#undef LOAD_FAIL
  g_live++;
  *out = m;
  return KC_OK;
}

extern "C" void kc_model_free(kc_model_t m) {
  if (!m) return;
  quiesce(m->ctx, m->device);
  free_model(m);
  g_live--;
}

extern "C" int64_t kc_model_weight_bytes(kc_model_t m) { return m ? m->weight_bytes : 0; }

extern "C" int kc_envelope(kc_model_t m, int32_t* max_gamma, int32_t* max_key_len, int32_t* det_width) {
  if (!m) return fail(KC_ERR_INVALID, "kc_envelope: NULL model");
  // Every kernel is row-invariant, so the envelope is what the attention CTA holds:
  // (gamma + 1) * gqa query rows <= 64, and at most 8 rows per segment.
  const int gqa = m->d.num_heads / m->d.num_kv_heads;
  const int rows = std::min(8, 64 / gqa);
  if (max_gamma) *max_gamma = std::max(0, rows - 1);
  if (max_key_len) *max_key_len = 0;   // unbounded: chunk geometry does not change with key length
  if (det_width) *det_width = 32;      // the cap the reference's calibration can reach (nn.rs:1247)
  return KC_OK;
}

// ---------------------------------------------------------------------------
// step metadata
// ---------------------------------------------------------------------------

constexpr int KC_TP_HANDLES = 3;   // per rank: tp_out[0], tp_out[1], tp_flags

namespace {

struct StepPlan {
  int n = 0, n_seqs = 0, n_sampled = 0, max_blocks = 0, n_work = 0, tokens_per_item = 1, max_chunks = 1;
  int max_len = 1;
  MetaLayout lay{};
};

int validate_step(kc_model* m, kc_kv* kv, const uint32_t* token_ids, int32_t n, const kc_seq_step* seqs, int32_t n_seqs,
                  int32_t pad_rows, StepPlan* plan) {
  if (!m || !kv || !token_ids || !seqs) return fail(KC_ERR_INVALID, "forward_step: NULL argument");
  if (kv->ctx != m->ctx) return fail(KC_ERR_INVALID, "forward_step: model and pools belong to different contexts");
  if (kv->layers != m->d.num_layers || kv->kv_heads != m->Hkv || kv->head_dim != m->d.head_dim)
    return fail(KC_ERR_INVALID, "forward_step: pool geometry [%d layers, %d kv heads, %d] does not match the model", kv->layers,
                kv->kv_heads, kv->head_dim);
  if (pad_rows != 0) return fail(KC_ERR_UNSUPPORTED, "forward_step: %d pad rows (kernel-class padding does not exist on this backend)", pad_rows);
  long long total = 0;
  for (int i = 0; i < n_seqs; ++i) total += seqs[i].len;
  if (n <= 0 || n_seqs <= 0 || total != n)
    return fail(KC_ERR_INVALID, "step batch of %d token(s) for %lld sequence position(s)", n, total);  // nn.rs:1311-1315
  if (n > m->max_rows) return fail(KC_ERR_INVALID, "step of %d tokens exceeds max_step_tokens %d", n, m->d.max_step_tokens);
  if (n_seqs > m->max_seqs) return fail(KC_ERR_INVALID, "step of %d sequences exceeds max_step_seqs %d", n_seqs, m->max_seqs);
  StepPlan p;
  p.n = n; p.n_seqs = n_seqs;
  int max_ctx = 1;
  for (int i = 0; i < n_seqs; ++i) {
    const kc_seq_step& s = seqs[i];
    if (s.len <= 0 || s.offset < 0) return fail(KC_ERR_INVALID, "segment %d: len %d offset %d", i, s.len, s.offset);
    if (s.sample_rows < 0 || s.sample_rows > s.len)
      return fail(KC_ERR_INVALID, "segment samples %d of its %d position(s)", s.sample_rows, s.len);  // nn.rs:1316-1327
    const long long need = ((long long)s.offset + s.len + kv->block_size - 1) / kv->block_size;
    if (!s.blocks || s.n_blocks < need)
      return fail(KC_ERR_INVALID, "segment %d: %d block(s) cannot hold %d token(s)", i, s.n_blocks, s.offset + s.len);
    for (int b = 0; b < s.n_blocks; ++b)
      if (s.blocks[b] >= (uint32_t)kv->num_blocks) return fail(KC_ERR_INVALID, "segment %d: block id %u of %d", i, s.blocks[b], kv->num_blocks);
    p.n_sampled += s.sample_rows;
    p.max_blocks = std::max(p.max_blocks, (int)need);
    p.max_len = std::max(p.max_len, s.len);
    max_ctx = std::max(max_ctx, s.offset + s.len);
  }
  for (int i = 0; i < n; ++i)
    if (token_ids[i] >= (uint32_t)m->d.vocab_size) return fail(KC_ERR_INVALID, "token id %u outside the vocabulary (%d)", token_ids[i], m->d.vocab_size);
  if (p.n_sampled > m->logit_rows) return fail(KC_ERR_INVALID, "step samples %d rows; at most %d", p.n_sampled, m->logit_rows);
  const int gqa = m->d.num_heads / m->d.num_kv_heads;
  p.tokens_per_item = attn_tokens_per_item(gqa, p.max_len);
  for (int i = 0; i < n_seqs; ++i) p.n_work += (seqs[i].len + p.tokens_per_item - 1) / p.tokens_per_item;
  p.max_chunks = (max_ctx + ATT_CHUNK - 1) / ATT_CHUNK;
  MetaLayout& L = p.lay;
  size_t at = 0;
  auto put = [&](size_t bytes) { size_t o = at; at = align_up(at + bytes, 16); return o; };
  L.tokens = put((size_t)n * 4); L.token_pos = put((size_t)n * 4); L.kv_slot = put((size_t)n * 4);
  L.sampled = put((size_t)std::max(1, p.n_sampled) * 4);
  L.tables = put((size_t)n_seqs * p.max_blocks * 4);
  L.work = put((size_t)p.n_work * 16);
  L.v_row_off = put((size_t)n_seqs * 4); L.v_draft_off = put((size_t)n_seqs * 4); L.v_draft_len = put((size_t)n_seqs * 4);
  L.v_draft = put((size_t)n * 4);
  L.feed = put((size_t)n * 4);
  L.total = at;
  *plan = p;
  return KC_OK;
}

// Packs the metadata on the host and queues the single host->device copy.
// `before_copy` (optional) is recorded on the stream after the host-side packing and before the copy is queued: the
// device span of a step starts there, so host packing time is not counted as device time.
int upload_meta(kc_model* m, kc_kv* kv, const uint32_t* token_ids, const kc_seq_step* seqs, const StepPlan& p,
                cudaEvent_t before_copy = nullptr, const int32_t* feed = nullptr) {
  kc_ctx* c = m->ctx;
  const MetaLayout& L = p.lay;
  if (L.total > m->meta_cap) {
    CK(cudaStreamSynchronize(c->stream));
    const size_t cap = align_up(std::max<size_t>(L.total * 2, 1 << 16), 4096);
    cudaFree(m->meta_dev); m->meta_dev = nullptr;
    for (int i = 0; i < kc_model::kStaging; ++i) { if (m->meta_host[i]) cudaFreeHost(m->meta_host[i]); m->meta_host[i] = nullptr; }
    CK(cudaMalloc(&m->meta_dev, cap));
    for (int i = 0; i < kc_model::kStaging; ++i) CK(cudaMallocHost(&m->meta_host[i], cap));
    m->meta_cap = cap;
  }
  const int slot = m->meta_next;
  m->meta_next = (m->meta_next + 1) % kc_model::kStaging;
  CK(cudaEventSynchronize(m->meta_ev[slot]));  // the copy that last used this staging buffer has finished
  uint8_t* hbuf = m->meta_host[slot];
  uint32_t* tokens = reinterpret_cast<uint32_t*>(hbuf + L.tokens);
  int32_t* pos = reinterpret_cast<int32_t*>(hbuf + L.token_pos);
  int32_t* slotv = reinterpret_cast<int32_t*>(hbuf + L.kv_slot);
  int32_t* sampled = reinterpret_cast<int32_t*>(hbuf + L.sampled);
  int32_t* tables = reinterpret_cast<int32_t*>(hbuf + L.tables);
  int32_t* work = reinterpret_cast<int32_t*>(hbuf + L.work);
  int32_t* v_row = reinterpret_cast<int32_t*>(hbuf + L.v_row_off);
  int32_t* v_doff = reinterpret_cast<int32_t*>(hbuf + L.v_draft_off);
  int32_t* v_dlen = reinterpret_cast<int32_t*>(hbuf + L.v_draft_len);
  uint32_t* v_draft = reinterpret_cast<uint32_t*>(hbuf + L.v_draft);
  memcpy(tokens, token_ids, (size_t)p.n * 4);
  if (feed) memcpy(hbuf + L.feed, feed, (size_t)p.n * 4);
  const int BS = kv->block_size;
  int row = 0, srow = 0, w = 0, dat = 0;
  for (int i = 0; i < p.n_seqs; ++i) {
    const kc_seq_step& s = seqs[i];
    for (int b = 0; b < p.max_blocks; ++b) tables[(size_t)i * p.max_blocks + b] = b < s.n_blocks ? (int32_t)s.blocks[b] : 0;
    for (int t = 0; t < s.len; ++t) {
      const int pp = s.offset + t;
      pos[row + t] = pp;
      slotv[row + t] = (int32_t)s.blocks[pp / BS] * BS + pp % BS;   // WriteRun derivation, engine.rs:2757-2769
    }
    for (int t = 0; t < s.len; t += p.tokens_per_item) {
      work[4 * w + 0] = i; work[4 * w + 1] = row + t; work[4 * w + 2] = std::min(p.tokens_per_item, s.len - t);
      work[4 * w + 3] = s.offset + t;
      ++w;
    }
    // trailing sample_rows positions (nn.rs:1367-1372)
    v_row[i] = srow; v_doff[i] = dat; v_dlen[i] = s.sample_rows - 1;   // -1: nothing sampled
    for (int t = s.len - s.sample_rows; t < s.len; ++t) sampled[srow++] = row + t;
    // the proposal a verify segment carries = its sampled inputs after the first
    for (int t = s.len - s.sample_rows + 1; t < s.len; ++t) v_draft[dat++] = token_ids[row + t];
    row += s.len;
  }
  if (before_copy) CK(cudaEventRecord(before_copy, c->stream));
  CK(cudaMemcpyAsync(m->meta_dev, hbuf, L.total, cudaMemcpyHostToDevice, c->stream));
  CK(cudaEventRecord(m->meta_ev[slot], c->stream));
  return KC_OK;
}

int ensure_attn_ws(kc_model* m, const StepPlan& p) {
  const size_t rows = (size_t)p.n * m->Hq * p.max_chunks;
  const size_t need = rows * m->d.head_dim * 4 + rows * 8 + 256;
  if (need > m->attn_ws_bytes) {
    CK(cudaStreamSynchronize(m->ctx->stream));
    cudaFree(m->attn_ws); m->attn_ws = nullptr; m->attn_ws_bytes = 0;
    const size_t cap = align_up(need + need / 4, 1 << 20);
    cudaError_t e = cudaMalloc(&m->attn_ws, cap);
    if (e != cudaSuccess) return fail(KC_ERR_OOM, "attention workspace of %zu bytes: %s", cap, cudaGetErrorString(e));
    m->attn_ws_bytes = cap;
  }
  return KC_OK;
}

AttnParams attn_params(kc_model* m, kc_kv* kv, const StepPlan& p, int layer, const bf16* q, bf16* out, float scale,
                       float softcap, int window, int Hq) {
  AttnParams a{};
  const size_t rows = (size_t)p.n * Hq * p.max_chunks;
  a.q = q; a.out = out;
  a.part_o = m->attn_ws;
  a.part_ml = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(m->attn_ws) + align_up(rows * m->d.head_dim * 4, 256));
  a.block_tables = reinterpret_cast<const int32_t*>(m->meta_dev + p.lay.tables);
  a.work = reinterpret_cast<const int4*>(m->meta_dev + p.lay.work);
  a.token_pos = reinterpret_cast<const int32_t*>(m->meta_dev + p.lay.token_pos);
  a.status = m->ctx->status;
  a.max_blocks = p.max_blocks;
  a.Hq = Hq; a.Hkv = kv->kv_heads; a.gqa = Hq / kv->kv_heads;
  a.layer = layer; a.NB = kv->num_blocks; a.BS = kv->block_size;
  a.max_chunks = p.max_chunks; a.chunk_lo_grid = 0;
  a.single_chunk = p.max_chunks == 1 ? 1 : 0;
  a.scale = scale; a.softcap = softcap; a.window = window;
  a.pool = kv->pool;
  a.kv4d = kv->map4d ? 1 : 0;
  return a;
}

// Brings every tensor-parallel rank's bf16 [n, H] sublayer output to every rank: out[r] = rank r's rows. The SUM is
// left to the consumer kernel, which adds the ranks in rank order in fp32 and rounds once. An all-gather only moves
// bytes, so a row's bits cannot depend on which algorithm the library picks for a message size — a reduction inside
// the collective did depend on it (speculation on and off disagreed on 6 of 64 sequences of the 70B configuration
// when the all-reduce's choice differed between 64-row and 320-row messages).
int tp_allgather(kc_model* m, const bf16* local, bf16* out, int n) {
  ncclResult_t r = ncclAllGather(local, out, (size_t)n * m->d.hidden_size, ncclBfloat16, m->ctx->comm, m->ctx->stream);
  if (r != ncclSuccess) return fail(KC_ERR_CUDA, "ncclAllGather: %s", ncclGetErrorString(r));
  return KC_OK;
}

// The exchange after o_proj / down_proj. With peer memory attached (kc_tp_attach) nothing is copied: the GEMM has
// written this rank's rows to tp_out[e & 1], a one-warp kernel publishes `e` into every rank's flag array, and the
// consumer kernel reads every rank's rows where they lie, in rank order. Buffer e & 1 is written again at exchange
// e + 2, which this rank's GEMM reaches only after its consumer of e + 1 has seen every peer's flag e + 1, i.e. after
// every peer has finished reading e. Otherwise: NCCL all-gather into proj_ranks.
int tp_exchange(kc_model* m, int n, SublayerOut* so) {
  kc_ctx* c = m->ctx;
  const int H = m->d.hidden_size;
  if (m->tp_p2p) {
    const uint32_t e = m->tp_epoch;   // set by tp_out_buffer for this exchange
    const int W = m->d.tp_world, me = m->d.tp_rank;
    LAUNCH(c, KC_PROF_ROWWISE, 1, launch_tp_signal(m->peer_flags, W, me, e, c->stream));
    if (!m->tp_two_phase) {
      *so = SublayerOut::of_peers(m->peer_out[e & 1], W, H, m->tp_flags, e, c->status);
      return KC_OK;
    }
    // Two phases, the shape of a reduce-scatter followed by an all-gather: this rank sums ITS column slice of every
    // rank's rows (pulling (W - 1) / W of a [rows, H] buffer instead of W - 1 whole ones), publishes it, and the
    // consumer gathers the W summed slices. Same rank-ordered fp32 sum, same single rounding: the same bits.
    const int sw = H / W;
    const bf16* slices[KC_MAX_TP] = {};
    uint32_t* flags2[KC_MAX_TP] = {};
    for (int r = 0; r < W; ++r) { slices[r] = m->peer_out[e & 1][r] + m->tp_sum_off; flags2[r] = m->peer_flags[r] + KC_MAX_TP; }
    LAUNCH(c, KC_PROF_ROWWISE, 1, launch_tp_reduce_slice(m->peer_out[e & 1], W, me, n, H, sw, m->tp_flags, e, c->status,
                                                        m->tp_out[e & 1] + m->tp_sum_off, c->stream));
    LAUNCH(c, KC_PROF_ROWWISE, 1, launch_tp_signal(flags2, W, me, e, c->stream));
    *so = SublayerOut::of_peer_slices(slices, W, H, sw, m->tp_flags + KC_MAX_TP, e, c->status);
    return KC_OK;
  }
  int rc = tp_allgather(m, m->proj, m->proj_ranks, n);
  if (rc) return rc;
  *so = SublayerOut::of_ranks(m->proj_ranks, m->d.tp_world, (size_t)n, H);
  return KC_OK;
}
// Where the GEMM of the next exchange writes this rank's rows.
bf16* tp_out_buffer(kc_model* m) {
  if (!m->tp_p2p) return m->proj;
  m->tp_epoch += 1;
  return m->tp_out[m->tp_epoch & 1];
}

// The forward proper. tokens_dev: n u32 on the device (normally the metadata arena's copy).
// greedy_out (optional, device): where a single sampled row's raw arg-max goes when the head's reduction can produce
// it itself (*greedy_done = true then; otherwise the caller samples from the logits as usual).
int run_forward(kc_model* m, kc_kv* kv, const uint32_t* tokens_dev, const StepPlan& p, bool want_logits, uint32_t* greedy_out = nullptr,
                bool* greedy_done = nullptr) {
  kc_ctx* c = m->ctx;
  const kc_model_desc& d = m->d;
  const int n = p.n, H = d.hidden_size, D = d.head_dim;
  const bool gemma = d.arch == KC_ARCH_GEMMA2;
  const int32_t* token_pos = reinterpret_cast<const int32_t*>(m->meta_dev + p.lay.token_pos);
  const int32_t* kv_slot = reinterpret_cast<const int32_t*>(m->meta_dev + p.lay.kv_slot);
  int rc;
  if ((rc = ensure_attn_ws(m, p))) return rc;
  const bool stream = m->stream_lane && n <= QL_STREAM_MAX_M && d.tp_world <= 1;
  // Per weight: the streaming kernel pays for itself from about 24 MB of records on (8B-class layers, every head); below
  // that the launch is latency-bound either way and the consumer would only have more partial pieces to sum. A
  // function of the weight's size alone, so a model takes the same kernels for every small step.
  auto streams = [&](const QWeight& w) { return stream && w.bytes() >= m->stream_min_bytes; };
  // ... and the smaller ones the small-weight lane of the same arithmetic (one CTA per tile and run of k-blocks, all
  // records requested at once), where their shape fits it
  auto small = [&](const QWeight& w) { return stream && !streams(w) && qlinear_gemv_pieces(w) > 0; };
  LAUNCH(c, KC_PROF_ROWWISE, 1, launch_embed(m->emb_w, m->emb_s, m->emb_b, tokens_dev, n, H, d.bits, d.group_size, m->embed_scale, d.vocab_size, m->h, c->stream));
  LAUNCH(c, KC_PROF_ROWWISE, 1, launch_add_rmsnorm(m->h, SublayerOut::none(), nullptr, m->layers[0].input_ln, nullptr, n, H, d.rms_norm_eps, nullptr, m->normed, c->stream));
  for (int l = 0; l < d.num_layers; ++l) {
    Layer& L = m->layers[l];
    SublayerOut so;
    if (streams(L.qkv)) RC(run_stream(c, L.qkv, m->normed, n, m->qkv, m->n_qkv, m->partial, &so));
    else if (small(L.qkv)) RC(run_gemv(c, L.qkv, m->normed, n, m->qkv, m->n_qkv, m->partial, &so));
    else RC(run_qlinear(c, L.qkv, m->op_normed, n, m->qkv, m->n_qkv, m->partial, &so));
    LAUNCH(c, KC_PROF_ROWWISE, 1, launch_rope_kv_write(so, L.qkv_bias, m->inv_freq, token_pos, kv_slot, n, m->Hq, m->Hkv, D, d.rope_traditional, l,
                            kv->num_blocks, kv->block_size, kv->pool, m->q_rot, c->stream));
    const int window = (d.sliding_window > 0 && (l % 2 == 0)) ? d.sliding_window : 0;
    AttnParams a = attn_params(m, kv, p, l, m->q_rot, m->attn, m->attn_scale, gemma ? d.attn_logit_softcapping : 0.f, window, m->Hq);
    LAUNCH(c, KC_PROF_ATTN, a.single_chunk ? 1 : 2, paged_attention(kv->map, a, D, p.tokens_per_item, p.n_work, p.max_chunks, n, c->stream));
    if (streams(L.o)) RC(run_stream(c, L.o, m->attn, n, m->proj, H, m->partial, &so));
    else if (small(L.o)) RC(run_gemv(c, L.o, m->attn, n, m->proj, H, m->partial, &so));
    else RC(run_qlinear(c, L.o, m->op_attn, n, d.tp_world > 1 ? tp_out_buffer(m) : m->proj, H, m->partial, d.tp_world > 1 ? nullptr : &so));
    if (d.tp_world > 1 && (rc = tp_exchange(m, n, &so))) return rc;
    if (gemma) LAUNCH(c, KC_PROF_ROWWISE, 1, launch_add_rmsnorm(m->h, so, L.post_attn_ln, L.pre_ffw_ln, nullptr, n, H, d.rms_norm_eps, m->h, m->normed, c->stream));
    else LAUNCH(c, KC_PROF_ROWWISE, 1, launch_add_rmsnorm(m->h, so, nullptr, L.post_attn_ln, nullptr, n, H, d.rms_norm_eps, m->h, m->normed, c->stream));
    // a down projection on the small-weight lane applies the activation itself while it stages its input, straight
    // from gate_up's fp32 partials (kept in a workspace of their own: down writes its partials meanwhile)
    bool gated_down = false;
    SublayerOut gu;
    if (streams(L.gate_up) || small(L.gate_up)) {
      gated_down = small(L.down) && m->partial_gu && (m->F % 128) == 0;
      float* ws = gated_down ? m->partial_gu : m->partial;
      if (streams(L.gate_up)) RC(run_stream(c, L.gate_up, m->normed, n, m->gu, 2 * m->F, ws, &gu));
      else RC(run_gemv(c, L.gate_up, m->normed, n, m->gu, 2 * m->F, ws, &gu));
      if (!gated_down) LAUNCH(c, KC_PROF_ROWWISE, 1, launch_glu_from(gu, n, m->F, gemma ? 1 : 0, m->glu_interleaved ? 1 : 0, m->act, c->stream));
    } else {
      RC(run_gated(c, L.gate_up, m->op_normed, n, m->gu, m->F, gemma ? 1 : 0, m->glu_interleaved, m->act, m->partial));
    }
    if (streams(L.down)) RC(run_stream(c, L.down, m->act, n, m->proj, H, m->partial, &so));
    else if (gated_down) {
      const QvGatedInput in{gu.part, gu.splits, gemma, m->glu_interleaved};
      LAUNCH(c, KC_PROF_GEMM, 1, qlinear_gemv(L.down, nullptr, 0, n, m->partial, c->status, c->stream, &in));
      so = SublayerOut::partials(m->partial, qlinear_gemv_pieces(L.down), (size_t)n, H);
    }
    else if (small(L.down)) RC(run_gemv(c, L.down, m->act, n, m->proj, H, m->partial, &so));
    else RC(run_qlinear(c, L.down, m->op_act, n, d.tp_world > 1 ? tp_out_buffer(m) : m->proj, H, m->partial, d.tp_world > 1 ? nullptr : &so));
    if (d.tp_world > 1 && (rc = tp_exchange(m, n, &so))) return rc;
    const bf16* next_ln = l + 1 < d.num_layers ? m->layers[l + 1].input_ln : nullptr;
    LAUNCH(c, KC_PROF_ROWWISE, 1, launch_add_rmsnorm(m->h, so, gemma ? L.post_ffw_ln : nullptr, next_ln, nullptr, n, H, d.rms_norm_eps, m->h, m->normed, c->stream));
  }
  if (want_logits && p.n_sampled > 0) {
    const int32_t* sampled = reinterpret_cast<const int32_t*>(m->meta_dev + p.lay.sampled);
    LAUNCH(c, KC_PROF_ROWWISE, 1, launch_add_rmsnorm(m->h, SublayerOut::none(), nullptr, m->final_norm, sampled, p.n_sampled, H, d.rms_norm_eps, nullptr, m->hs, c->stream));
    if (streams(m->head) && greedy_out && p.n_sampled == 1 && m->argmax_scratch && !(gemma && d.final_logit_softcapping > 0.f)) {
      LAUNCH(c, KC_PROF_GEMM, 1, qlinear_stream(m->head, m->hs, m->head.K, 1, m->partial, c->status, c->stream));
      LAUNCH(c, KC_PROF_SAMPLE, 1, qlinear_reduce_argmax(m->partial, qlinear_stream_pieces(m->head), d.vocab_size, m->logits, m->argmax_scratch,
                                                         greedy_out, c->stream));
      if (greedy_done) *greedy_done = true;
    }
    else if (streams(m->head)) RC(run_stream(c, m->head, m->hs, p.n_sampled, m->logits, d.vocab_size, m->partial, nullptr));
    else if (small(m->head) && p.n_sampled <= QL_STREAM_MAX_M) RC(run_gemv(c, m->head, m->hs, p.n_sampled, m->logits, d.vocab_size, m->partial, nullptr));
    else RC(run_qlinear(c, m->head, m->op_hs, p.n_sampled, m->logits, d.vocab_size, m->partial));
    if (gemma && d.final_logit_softcapping > 0.f)
      LAUNCH(c, KC_PROF_ROWWISE, 1, launch_softcap(m->logits, (long long)p.n_sampled * d.vocab_size, d.final_logit_softcapping, c->stream));
  }
  return KC_OK;
}

}  // namespace

extern "C" int kc_tp_export(kc_model_t m, void* handles_out) {
  if (!m || !handles_out) return fail(KC_ERR_INVALID, "kc_tp_export: NULL argument");
  if (m->d.tp_world < 2) return fail(KC_ERR_INVALID, "kc_tp_export: the model is not a tensor-parallel slice");
  CK(cudaSetDevice(m->ctx->device));
  cudaIpcMemHandle_t* h = reinterpret_cast<cudaIpcMemHandle_t*>(handles_out);
  CK(cudaIpcGetMemHandle(&h[0], m->tp_out[0]));
  CK(cudaIpcGetMemHandle(&h[1], m->tp_out[1]));
  CK(cudaIpcGetMemHandle(&h[2], m->tp_flags));
  return KC_OK;
}

extern "C" int kc_tp_attach(kc_model_t m, const void* handles_all) {
  if (!m || !handles_all) return fail(KC_ERR_INVALID, "kc_tp_attach: NULL argument");
  const int W = m->d.tp_world, me = m->d.tp_rank;
  if (W < 2 || W > KC_MAX_TP) return fail(KC_ERR_INVALID, "kc_tp_attach: world %d (2..%d)", W, KC_MAX_TP);
  if (m->tp_p2p) return fail(KC_ERR_INVALID, "kc_tp_attach: peers are already attached");
  CK(cudaSetDevice(m->ctx->device));
  CK(cudaStreamSynchronize(m->ctx->stream));
  const cudaIpcMemHandle_t* h = reinterpret_cast<const cudaIpcMemHandle_t*>(handles_all);
  for (int r = 0; r < W; ++r) {
    if (r == me) {
      m->peer_out[0][r] = m->tp_out[0]; m->peer_out[1][r] = m->tp_out[1]; m->peer_flags[r] = m->tp_flags;
      continue;
    }
    void* p[3] = {nullptr, nullptr, nullptr};
    for (int k = 0; k < 3; ++k) {
      cudaError_t e = cudaIpcOpenMemHandle(&p[k], h[r * KC_TP_HANDLES + k], cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) {
        for (int j = 0; j < k; ++j) cudaIpcCloseMemHandle(p[j]);
        for (int q = 0; q < r; ++q) {
          if (q == me) continue;
          cudaIpcCloseMemHandle(m->peer_out[0][q]); cudaIpcCloseMemHandle(m->peer_out[1][q]); cudaIpcCloseMemHandle(m->peer_flags[q]);
          m->peer_out[0][q] = m->peer_out[1][q] = nullptr; m->peer_flags[q] = nullptr;
        }
        cudaGetLastError();
        return fail(KC_ERR_CUDA, "kc_tp_attach: cannot map rank %d's buffer %d: %s", r, k, cudaGetErrorString(e));
      }
    }
    m->peer_out[0][r] = (bf16*)p[0]; m->peer_out[1][r] = (bf16*)p[1]; m->peer_flags[r] = (uint32_t*)p[2];
  }
  m->tp_p2p = true;
  m->tp_epoch = 0;
  // the two-phase form pays from 4 ranks on (at 2 ranks both forms move the same bytes and it only adds launches)
  m->tp_two_phase = W >= 4 && m->d.hidden_size % (8 * W) == 0;
  if (const char* env = getenv("KILN_TP_TWO_PHASE")) m->tp_two_phase = atoi(env) != 0 && m->d.hidden_size % (8 * W) == 0;
  return KC_OK;
}

extern "C" int kc_model_set_stream_lane(kc_model_t m, int32_t on) {
  if (!m) return fail(KC_ERR_INVALID, "kc_model_set_stream_lane: model is NULL");
  if (on && m->d.tp_world > 1) return fail(KC_ERR_UNSUPPORTED, "kc_model_set_stream_lane: not available on a tensor-parallel slice");
  m->stream_lane = on != 0;
  m->stream_min_bytes = on == 2 ? 0 : QL_STREAM_MIN_BYTES;
  if (on && !m->argmax_scratch) {
    const size_t bytes = (size_t)(2 * qlinear_reduce_argmax_ctas(m->d.vocab_size) + 4) * sizeof(float);
    CK(cudaSetDevice(m->ctx->device));
    CK(cudaMalloc(&m->argmax_scratch, bytes));
    CK(cudaMemsetAsync(m->argmax_scratch, 0, bytes, m->ctx->stream));
  }
  if (on && !m->partial_gu && !m->layers.empty()) {
    const QWeight& gu = m->layers[0].gate_up;
    const size_t pieces = (size_t)std::max(qlinear_stream_pieces(gu), qlinear_gemv_pieces(gu));
    CK(cudaSetDevice(m->ctx->device));
    CK(cudaMalloc(&m->partial_gu, pieces * QL_STREAM_MAX_M * gu.N * sizeof(float)));
  }
  return KC_OK;
}

extern "C" int kc_forward_step(kc_model_t m, kc_kv_t kv, const uint32_t* token_ids, int32_t n, const kc_seq_step* seqs,
                               int32_t n_seqs, int32_t pad_rows, void** logits_dev, int32_t* n_sampled) {
  StepPlan p;
  int rc = validate_step(m, kv, token_ids, n, seqs, n_seqs, pad_rows, &p);
  if (rc) return rc;
  CK(cudaSetDevice(m->ctx->device));
  if ((rc = upload_meta(m, kv, token_ids, seqs, p))) return rc;
  if ((rc = run_forward(m, kv, reinterpret_cast<const uint32_t*>(m->meta_dev + p.lay.tokens), p, true))) return rc;
  if (logits_dev) *logits_dev = p.n_sampled ? (void*)m->logits : nullptr;
  if (n_sampled) *n_sampled = p.n_sampled;
  return KC_OK;
}

extern "C" int kc_greedy_rows(kc_ctx_t c, const void* logits_dev, int32_t rows, int32_t vocab, int32_t normalize,
                              uint32_t* tokens_out_dev) {
  if (!c || !logits_dev || !tokens_out_dev) return fail(KC_ERR_INVALID, "kc_greedy_rows: NULL argument");
  if (rows < 1 || vocab < 1) return fail(KC_ERR_INVALID, "kc_greedy_rows: [%d, %d]", rows, vocab);
  CK(cudaSetDevice(c->device));
  LAUNCH(c, KC_PROF_SAMPLE, 1, launch_greedy_rows((const bf16*)logits_dev, rows, vocab, normalize, tokens_out_dev, c->stream));
  return KC_OK;
}

extern "C" int kc_verify_accept(kc_ctx_t c, const uint32_t* row_tokens_dev, const int32_t* seq_row_offsets_dev,
                                const uint32_t* draft_dev, const int32_t* draft_offsets_dev, const int32_t* draft_len_dev,
                                int32_t n_seqs, int32_t max_commit, uint32_t* committed_out_dev,
                                int32_t* n_committed_out_dev, int32_t* n_accepted_out_dev) {
  if (!c || !row_tokens_dev || !seq_row_offsets_dev || !draft_dev || !draft_offsets_dev || !draft_len_dev ||
      !committed_out_dev || !n_committed_out_dev || !n_accepted_out_dev)
    return fail(KC_ERR_INVALID, "kc_verify_accept: NULL argument");
  if (n_seqs < 1 || max_commit < 1) return fail(KC_ERR_INVALID, "kc_verify_accept: n_seqs %d max_commit %d", n_seqs, max_commit);
  CK(cudaSetDevice(c->device));
  LAUNCH(c, KC_PROF_SAMPLE, 1, launch_verify_accept(row_tokens_dev, seq_row_offsets_dev, draft_dev, draft_offsets_dev, draft_len_dev, n_seqs,
                          max_commit, committed_out_dev, n_committed_out_dev, n_accepted_out_dev, c->stream));
  return KC_OK;
}

extern "C" int kc_verify_step(kc_model_t m, kc_kv_t kv, const uint32_t* token_ids, int32_t n, const kc_seq_step* seqs,
                              int32_t n_seqs, uint32_t* row_tokens_out, int32_t* n_committed_out, int32_t* n_accepted_out) {
  StepPlan p;
  int rc = validate_step(m, kv, token_ids, n, seqs, n_seqs, 0, &p);
  if (rc) return rc;
  kc_ctx* c = m->ctx;
  CK(cudaSetDevice(c->device));
  if ((rc = upload_meta(m, kv, token_ids, seqs, p, c->step_a))) return rc;
  if ((rc = run_forward(m, kv, reinterpret_cast<const uint32_t*>(m->meta_dev + p.lay.tokens), p, true))) return rc;
  if (p.n_sampled > 0) {
    LAUNCH(c, KC_PROF_SAMPLE, 1, launch_greedy_rows(m->logits, p.n_sampled, m->d.vocab_size, 1, m->row_tokens, c->stream));
    // max_commit = 0: the committed list is row_tokens[row_off .. row_off + n_committed), no second copy needed
    LAUNCH(c, KC_PROF_SAMPLE, 1, launch_verify_accept(m->row_tokens, reinterpret_cast<const int32_t*>(m->meta_dev + p.lay.v_row_off),
                            reinterpret_cast<const uint32_t*>(m->meta_dev + p.lay.v_draft),
                            reinterpret_cast<const int32_t*>(m->meta_dev + p.lay.v_draft_off),
                            reinterpret_cast<const int32_t*>(m->meta_dev + p.lay.v_draft_len), n_seqs, 0, m->committed,
                            m->n_committed, m->n_accepted, c->stream));
    uint8_t* hb = m->result_host;
    const size_t o1 = align_up((size_t)p.n_sampled * 4, 16), o2 = o1 + align_up((size_t)n_seqs * 4, 16);
    CK(cudaMemcpyAsync(hb, m->row_tokens, (size_t)p.n_sampled * 4, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaMemcpyAsync(hb + o1, m->n_committed, (size_t)n_seqs * 4, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaMemcpyAsync(hb + o2, m->n_accepted, (size_t)n_seqs * 4, cudaMemcpyDeviceToHost, c->stream));
    CK(status_fetch(c));
    CK(cudaEventRecord(c->step_b, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    cudaEventElapsedTime(&c->last_step_ms, c->step_a, c->step_b);
    RC(status_verdict(c, "kc_verify_step"));
    if (row_tokens_out) memcpy(row_tokens_out, hb, (size_t)p.n_sampled * 4);
    if (n_committed_out) memcpy(n_committed_out, hb + o1, (size_t)n_seqs * 4);
    if (n_accepted_out) memcpy(n_accepted_out, hb + o2, (size_t)n_seqs * 4);
  } else {
    CK(status_fetch(c));
    CK(cudaEventRecord(c->step_b, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    cudaEventElapsedTime(&c->last_step_ms, c->step_a, c->step_b);
    RC(status_verdict(c, "kc_verify_step"));
    if (n_committed_out) memset(n_committed_out, 0, (size_t)n_seqs * 4);
    if (n_accepted_out) memset(n_accepted_out, 0, (size_t)n_seqs * 4);
  }
  return KC_OK;
}

extern "C" int kc_draft_chain(kc_model_t m, kc_kv_t kv, uint32_t first_token, int32_t offset, const uint32_t* blocks,
                              int32_t n_blocks, int32_t gamma, uint32_t* proposal_out) {
  if (!m || !kv || !blocks || !proposal_out) return fail(KC_ERR_INVALID, "kc_draft_chain: NULL argument");
  if (gamma < 1 || gamma > 64) return fail(KC_ERR_INVALID, "kc_draft_chain: gamma %d", gamma);
  kc_ctx* c = m->ctx;
  CK(cudaSetDevice(c->device));
  const auto t_begin = std::chrono::steady_clock::now();
  // Step j feeds one token at position offset + j; its input is the previous step's raw argmax,
  // read on the device (row_tokens[j-1]) — the lazy feed of draft.rs:382-386.
  for (int j = 0; j < gamma; ++j) {
    kc_seq_step s{1, offset + j, 1, n_blocks, blocks};
    StepPlan p;
    uint32_t tok = j == 0 ? first_token : 0;  // placeholder id for validation when j > 0
    int rc = validate_step(m, kv, &tok, 1, &s, 1, 0, &p);
    if (rc) return rc;
    if ((rc = upload_meta(m, kv, &tok, &s, p))) return rc;
    const uint32_t* tokens_dev = j == 0 ? reinterpret_cast<const uint32_t*>(m->meta_dev + p.lay.tokens) : m->row_tokens + (j - 1);
    bool sampled = false;
    if ((rc = run_forward(m, kv, tokens_dev, p, true, m->row_tokens + j, &sampled))) return rc;
    if (!sampled) LAUNCH(c, KC_PROF_SAMPLE, 1, launch_greedy_rows(m->logits, 1, m->d.vocab_size, 0, m->row_tokens + j, c->stream));
  }
  CK(cudaMemcpyAsync(m->result_host, m->row_tokens, (size_t)gamma * 4, cudaMemcpyDeviceToHost, c->stream));
  CK(status_fetch(c));
  CK(cudaStreamSynchronize(c->stream));
  RC(status_verdict(c, "kc_draft_chain"));
  memcpy(proposal_out, m->result_host, (size_t)gamma * 4);
  c->draft_ms += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t_begin).count();
  c->draft_tokens += gamma; c->draft_calls += 1;
  return KC_OK;
}

// Pipelined plain decode (crates/kiln-engine/src/engine.rs:1428-1455, 1656-1744). The reference builds step N + 1 from
// step N's still-lazy sampled tokens and reads step N back afterwards (async_eval); here step N + 1 is queued on the
// stream with a kernel that takes its input ids from step N's token buffer, and step N's tokens reach the host through
// a pinned slot and an event, so the host never waits between the two launches.
extern "C" int kc_decode_launch(kc_model_t m, kc_kv_t kv, const uint32_t* token_ids, const int32_t* feed,
                                const kc_seq_step* seqs, int32_t n_seqs, uint64_t* ticket_out) {
  if (!m || !kv || !token_ids || !feed || !seqs || !ticket_out) return fail(KC_ERR_INVALID, "kc_decode_launch: NULL argument");
  if (n_seqs < 1 || n_seqs > m->max_seqs) return fail(KC_ERR_INVALID, "kc_decode_launch: %d sequences (at most %d)", n_seqs, m->max_seqs);
  const int prev = (int)(m->pipe_ticket % 2);
  bool any_feed = false;
  std::vector<uint32_t> ids(n_seqs);
  for (int i = 0; i < n_seqs; ++i) {
    if (seqs[i].len != 1 || seqs[i].sample_rows != 1)
      return fail(KC_ERR_INVALID, "kc_decode_launch: segment %d has len %d, samples %d (a decode step feeds and samples one row)", i,
                  seqs[i].len, seqs[i].sample_rows);
    if (feed[i] >= 0) {
      if (m->pipe_ticket == 0 || feed[i] >= m->pipe_n[prev])
        return fail(KC_ERR_INVALID, "kc_decode_launch: feed row %d of a previous launch with %d rows", feed[i],
                    m->pipe_ticket ? m->pipe_n[prev] : 0);
      any_feed = true;
      ids[i] = 0;  // replaced on the device
    } else {
      ids[i] = token_ids[i];
    }
  }
  StepPlan p;
  int rc = validate_step(m, kv, ids.data(), n_seqs, seqs, n_seqs, 0, &p);
  if (rc) return rc;
  kc_ctx* c = m->ctx;
  CK(cudaSetDevice(c->device));
  if ((rc = upload_meta(m, kv, ids.data(), seqs, p, nullptr, feed))) return rc;
  uint32_t* tokens_dev = reinterpret_cast<uint32_t*>(m->meta_dev + p.lay.tokens);
  if (any_feed)
    LAUNCH(c, KC_PROF_SAMPLE, 1, launch_feed_tokens(tokens_dev, reinterpret_cast<const int32_t*>(m->meta_dev + p.lay.feed),
                                                   m->pipe_tokens[prev], n_seqs, m->pipe_n[prev], c->stream));
  if ((rc = run_forward(m, kv, tokens_dev, p, true))) return rc;
  const uint64_t ticket = m->pipe_ticket + 1;
  const int slot = (int)(ticket % 2);
  LAUNCH(c, KC_PROF_SAMPLE, 1, launch_greedy_rows(m->logits, n_seqs, m->d.vocab_size, 1, m->pipe_tokens[slot], c->stream));
  CK(cudaMemcpyAsync(m->pipe_host[slot], m->pipe_tokens[slot], (size_t)n_seqs * 4, cudaMemcpyDeviceToHost, c->stream));
  CK(cudaMemcpyAsync(m->pipe_host[slot] + m->max_seqs, c->status, sizeof(uint32_t), cudaMemcpyDeviceToHost, c->stream));
  CK(cudaEventRecord(m->pipe_ev[slot], c->stream));
  m->pipe_ticket = ticket;
  m->pipe_n[slot] = n_seqs;
  *ticket_out = ticket;
  return KC_OK;
}

extern "C" int kc_decode_collect(kc_model_t m, uint64_t ticket, uint32_t* row_tokens_out, int32_t n) {
  if (!m || !row_tokens_out) return fail(KC_ERR_INVALID, "kc_decode_collect: NULL argument");
  if (ticket == 0 || ticket > m->pipe_ticket || ticket + 1 < m->pipe_ticket)
    return fail(KC_ERR_INVALID, "kc_decode_collect: ticket %llu is not one of the two most recent launches (latest %llu)",
                (unsigned long long)ticket, (unsigned long long)m->pipe_ticket);
  const int slot = (int)(ticket % 2);
  if (n != m->pipe_n[slot]) return fail(KC_ERR_INVALID, "kc_decode_collect: %d rows asked of a launch of %d", n, m->pipe_n[slot]);
  kc_ctx* c = m->ctx;
  CK(cudaSetDevice(c->device));
  CK(cudaEventSynchronize(m->pipe_ev[slot]));
  const uint32_t st = m->pipe_host[slot][m->max_seqs];
  if (st) {
    cudaMemsetAsync(c->status, 0, sizeof(uint32_t), c->stream);
    return fail(KC_ERR_TIMEOUT, "kc_decode_collect: device status 0x%x: a bounded wait gave up (kernel 0x%x, wait %u); the tokens of "
                "this launch and of any launch fed from it are not valid", st, st & 0xff00u, st & 0xffu);
  }
  memcpy(row_tokens_out, m->pipe_host[slot], (size_t)n * 4);
  return KC_OK;
}

// ---------------------------------------------------------------------------
// single ops over a caller-described step
// ---------------------------------------------------------------------------

// A throw-away model shell that owns only step metadata and the attention workspace,
// so the single-op entry points share upload_meta / attn_params with the forward.
static int op_shell(kc_ctx* c, kc_kv* kv, int num_heads, int n, int n_seqs, kc_model** out) {
  kc_model* m = new kc_model;
  m->ctx = c;
  m->d.num_layers = kv->layers; m->d.head_dim = kv->head_dim; m->d.num_heads = num_heads; m->d.num_kv_heads = kv->kv_heads;
  m->d.vocab_size = 0x7fffffff; m->d.hidden_size = 0; m->d.max_step_tokens = n; m->d.tp_world = 1;
  m->Hq = num_heads; m->Hkv = kv->kv_heads;
  m->max_rows = n; m->max_seqs = n_seqs; m->logit_rows = n;
  for (int i = 0; i < kc_model::kStaging; ++i)
    if (cudaEventCreateWithFlags(&m->meta_ev[i], cudaEventDisableTiming) != cudaSuccess) { free_model(m); return fail(KC_ERR_CUDA, "event"); }
  *out = m;
  return KC_OK;
}

extern "C" int kc_paged_attention(kc_ctx_t c, kc_kv_t kv, int32_t layer, const void* q_dev, int32_t n, int32_t num_heads,
                                  const kc_seq_step* seqs, int32_t n_seqs, float scale, float softcap, int32_t window,
                                  void* out_dev) {
  if (!c || !kv || !q_dev || !seqs || !out_dev) return fail(KC_ERR_INVALID, "kc_paged_attention: NULL argument");
  if (layer < 0 || layer >= kv->layers) return fail(KC_ERR_INVALID, "kc_paged_attention: layer %d of %d", layer, kv->layers);
  if (num_heads < kv->kv_heads || num_heads % kv->kv_heads || num_heads / kv->kv_heads > 64)
    return fail(KC_ERR_INVALID, "kc_paged_attention: %d heads over %d kv heads", num_heads, kv->kv_heads);
  CK(cudaSetDevice(c->device));
  kc_model* m = nullptr;
  int rc = op_shell(c, kv, num_heads, n, n_seqs, &m);
  if (rc) return rc;
  std::vector<uint32_t> ids(std::max(n, 1), 0);
  StepPlan p;
  rc = validate_step(m, kv, ids.data(), n, seqs, n_seqs, 0, &p);
  if (!rc) rc = upload_meta(m, kv, ids.data(), seqs, p);
  if (!rc) rc = ensure_attn_ws(m, p);
  if (!rc) {
    AttnParams a = attn_params(m, kv, p, layer, (const bf16*)q_dev, (bf16*)out_dev, scale, softcap, window, num_heads);
    rc = [&]() -> int {
      LAUNCH(c, KC_PROF_ATTN, a.single_chunk ? 1 : 2, paged_attention(kv->map, a, kv->head_dim, p.tokens_per_item, p.n_work, p.max_chunks, n, c->stream));
      return KC_OK;
    }();
  }
  cudaStreamSynchronize(c->stream);
  std::string keep = g_err;
  free_model(m);
  g_err = keep;
  return rc;
}

extern "C" int kc_rope_kv_write(kc_ctx_t c, kc_kv_t kv, int32_t layer, const void* qkv_dev, const void* qkv_bias_dev,
                                const float* inv_freq_dev, int32_t n, int32_t num_heads, int32_t traditional,
                                const kc_seq_step* seqs, int32_t n_seqs, void* q_out_dev) {
  if (!c || !kv || !qkv_dev || !inv_freq_dev || !seqs || !q_out_dev) return fail(KC_ERR_INVALID, "kc_rope_kv_write: NULL argument");
  if (layer < 0 || layer >= kv->layers) return fail(KC_ERR_INVALID, "kc_rope_kv_write: layer %d of %d", layer, kv->layers);
  CK(cudaSetDevice(c->device));
  kc_model* m = nullptr;
  int rc = op_shell(c, kv, num_heads, n, n_seqs, &m);
  if (rc) return rc;
  std::vector<uint32_t> ids(std::max(n, 1), 0);
  StepPlan p;
  rc = validate_step(m, kv, ids.data(), n, seqs, n_seqs, 0, &p);
  if (!rc) rc = upload_meta(m, kv, ids.data(), seqs, p);
  if (!rc) {
    cudaError_t e = launch_rope_kv_write(SublayerOut::dense((const bf16*)qkv_dev, (num_heads + 2 * kv->kv_heads) * kv->head_dim), (const bf16*)qkv_bias_dev, inv_freq_dev,
                                         reinterpret_cast<const int32_t*>(m->meta_dev + p.lay.token_pos),
                                         reinterpret_cast<const int32_t*>(m->meta_dev + p.lay.kv_slot), n, num_heads,
                                         kv->kv_heads, kv->head_dim, traditional, layer, kv->num_blocks, kv->block_size,
                                         kv->pool, (bf16*)q_out_dev, c->stream);
    if (e != cudaSuccess) rc = fail(KC_ERR_CUDA, "kc_rope_kv_write: %s", cudaGetErrorString(e));
  }
  cudaStreamSynchronize(c->stream);
  std::string keep = g_err;
  free_model(m);
  g_err = keep;
  return rc;
}
