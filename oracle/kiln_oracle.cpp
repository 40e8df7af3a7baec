// CPU ORACLE — test infrastructure, not product code.
//
// A plain C++ (OpenMP) restatement of the floating-point side of kiln's
// speculative-decoding verify path. Only tests/, __graft_entry__.smoke() and
// bench.py's cpu_baseline / --impl reference legs may load this library; the
// product (kiln_b200/, libkiln_cuda.so) never does.
//
// PARITY UNPINNED for floating point: the reference's arithmetic lives in MLX
// v0.31.1 (through mlx-c v0.6.0, pinned by docs/decisions/0001-mlx-c-pin.md:16-21),
// whose sources are absent from the reference tree and which cannot be installed
// here. No in-tree reference test fixes a floating-point result for this path
// without the (absent) Hugging Face checkpoints. This file therefore restates
// the op graph the reference builds, op by op and rounding point by rounding
// point, with MLX's published algorithms for the fused ops:
//
//   forward            crates/kiln-models/src/nn.rs:1303-1388   CausalLm::forward_step
//   embedding          crates/kiln-models/src/nn.rs:159-176, 1143-1154
//   quantised linear   crates/kiln-models/src/nn.rs:79-102; crates/kiln-mlx/src/ops.rs:362-388
//                      (mlx affine: w = q*scale + bias; fp32 accumulation, one rounding)
//   block              crates/kiln-models/src/nn.rs:969-1019
//   attention step     crates/kiln-models/src/nn.rs:715-845; crates/kiln-engine/src/paged.rs:147-225
//   SDPA algebra       crates/kiln-engine/src/paged_attn.rs:59-155 (fp32 scores on scale*q,
//                      softmax in fp32, o / sum cast to T); causal predicate bottom-right aligned
//   gemma-2 attention  crates/kiln-models/src/nn.rs:497-580
//   mlp / gelu         crates/kiln-models/src/nn.rs:221-235, 284-294
//   logit softcap      crates/kiln-models/src/nn.rs:1158-1169
//   rope               crates/kiln-models/src/nn.rs:1409-1477, 1555-1579
//   greedy sampling    crates/kiln-engine/src/engine.rs:879-901; crates/kiln-engine/src/sampler.rs:100-104;
//                      crates/kiln-models/src/draft.rs:379-381
//
// Integer-side behaviour (block tables, acceptance walk, rollback) is restated in
// oracle/bookkeeping.py and IS pinned by the reference's in-tree unit tests.
#include <algorithm>
#include <cmath>
#include <omp.h>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../include/kiln_cuda.h"

#define KO_API extern "C" __attribute__((visibility("default")))

namespace {

typedef uint16_t bf16_t;

inline float b2f(bf16_t v) { uint32_t u = (uint32_t)v << 16; float f; memcpy(&f, &u, 4); return f; }
inline bf16_t f2b(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (bf16_t)((u >> 16) | 0x40);  // NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return (bf16_t)(u >> 16);
}
inline float rb(float f) { return b2f(f2b(f)); }  // round to bf16, keep as float

struct QLinear {
  std::vector<uint32_t> w; std::vector<bf16_t> s, b, bias;
  int N = 0, K = 0, bits = 4, group = 64;
};

// MLX evaluates quantized_matmul in two arithmetic classes, chosen by the row count of x:
//   0  row-vector class (qmv): y = sum_g scale_g * (sum_k x_k q_k) + bias_g * (sum_k x_k), all fp32 —
//      what the reference's per-sequence verify forwards (M <= 8) run;
//   1  tile class (qmm): every weight is first dequantised to the activation dtype,
//      w = bf16(q * scale + bias), then multiplied with fp32 accumulation — what MLX runs for wide
//      batches, and the class of this build's tensor-core kernel.
// Both round the result once. Which class a launch lands in is MLX dispatch, not kiln code.
int g_weight_class = 0;

// mlx affine layout: element j of a row sits in bits [bits*(j % (32/bits)), +bits) of word j / (32/bits).
inline uint32_t qval(const uint32_t* row, int j, int bits) {
  const int per = 32 / bits;
  return (row[j / per] >> (bits * (j % per))) & ((1u << bits) - 1u);
}

// y[m, n] = bf16(sum_g scale_g * (sum_k x_k q_k) + bias_g * (sum_k x_k)) [+ bias in bf16]
void qmatmul(const QLinear& L, const float* x, int M, float* y /* [M, N], bf16-valued */) {
  const int N = L.N, K = L.K, G = L.group, bits = L.bits;
  const int ng = K / G, wpr = K * bits / 32;
  std::vector<float> xs((size_t)M * ng);
  for (int m = 0; m < M; ++m)
    for (int g = 0; g < ng; ++g) {
      float s = 0.f;
      for (int k = 0; k < G; ++k) s += x[(size_t)m * K + g * G + k];
      xs[(size_t)m * ng + g] = s;
    }
#pragma omp parallel
  {
    std::vector<float> q(K);
#pragma omp for schedule(static)
    for (int n = 0; n < N; ++n) {
      const uint32_t* row = &L.w[(size_t)n * wpr];
      for (int k = 0; k < K; ++k) q[k] = (float)qval(row, k, bits);
      if (g_weight_class == 1)
        for (int k = 0; k < K; ++k) q[k] = rb(std::fma(q[k], b2f(L.s[(size_t)n * ng + k / G]), b2f(L.b[(size_t)n * ng + k / G])));
      for (int m = 0; m < M; ++m) {
        const float* xr = x + (size_t)m * K;
        float acc = 0.f;
        for (int g = 0; g < ng; ++g) {
          float a = 0.f;
          const float* qq = &q[g * G]; const float* xx = xr + g * G;
          for (int k = 0; k < G; ++k) a += xx[k] * qq[k];
          if (g_weight_class == 1) acc += a;
          else acc += b2f(L.s[(size_t)n * ng + g]) * a + b2f(L.b[(size_t)n * ng + g]) * xs[(size_t)m * ng + g];
        }
        float v = rb(acc);
        if (!L.bias.empty()) v = rb(v + b2f(L.bias[n]));  // separate bf16 add, nn.rs:98-101
        y[(size_t)m * N + n] = v;
      }
    }
  }
}

void rms_norm(const float* x, const bf16_t* w, int rows, int H, float eps, float* y) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (size_t)r * H;
    float ss = 0.f;
    for (int i = 0; i < H; ++i) ss += xr[i] * xr[i];
    const float inv = 1.0f / std::sqrt(ss / (float)H + eps);
    for (int i = 0; i < H; ++i) y[(size_t)r * H + i] = rb(b2f(w[i]) * (xr[i] * inv));
  }
}

struct Layer {
  QLinear q, k, v, o, gate, up, down;
  std::vector<bf16_t> input_ln, post_attn_ln, pre_ffw_ln, post_ffw_ln;
};

}  // namespace

struct ko_model {
  kc_model_desc d;
  QLinear embed, head; bool tied = false;
  std::vector<Layer> layers;
  std::vector<bf16_t> norm;
  std::vector<float> inv_freq;
  float scale = 0.f;
  int layer_limit = 0;  // >0: run only the first layer_limit layers (bounded timing samples)
};

struct ko_kv {
  int layers, kv_heads, head_dim, num_blocks, block_size;
  std::vector<bf16_t> pool;  // [layers][2][num_blocks][kv_heads][block_size][head_dim]
  size_t idx(int layer, int kvsel, int block, int head, int row) const {
    return ((((size_t)layer * 2 + kvsel) * num_blocks + block) * kv_heads + head) * block_size * (size_t)head_dim +
           (size_t)row * head_dim;
  }
};

static thread_local std::string g_err;
KO_API const char* ko_last_error() { return g_err.c_str(); }
KO_API void ko_set_weight_class(int cls) { g_weight_class = cls; }

namespace {

bool load_q(const std::map<std::string, const kc_tensor_view*>& idx, const std::string& p, int N, int K, int bits, int group,
            QLinear* out) {
  auto w = idx.find(p + ".weight"), s = idx.find(p + ".scales"), b = idx.find(p + ".biases");
  if (w == idx.end() || s == idx.end() || b == idx.end()) { g_err = "missing tensor " + p; return false; }
  out->N = N; out->K = K; out->bits = bits; out->group = group;
  const size_t nw = (size_t)N * K * bits / 32, ns = (size_t)N * (K / group);
  out->w.assign((const uint32_t*)w->second->data, (const uint32_t*)w->second->data + nw);
  out->s.assign((const bf16_t*)s->second->data, (const bf16_t*)s->second->data + ns);
  out->b.assign((const bf16_t*)b->second->data, (const bf16_t*)b->second->data + ns);
  auto bi = idx.find(p + ".bias");
  if (bi != idx.end()) out->bias.assign((const bf16_t*)bi->second->data, (const bf16_t*)bi->second->data + N);
  return true;
}

bool load_norm(const std::map<std::string, const kc_tensor_view*>& idx, const std::string& name, int H, bool one_plus,
               std::vector<bf16_t>* out) {
  auto t = idx.find(name);
  if (t == idx.end()) { g_err = "missing tensor " + name; return false; }
  out->assign((const bf16_t*)t->second->data, (const bf16_t*)t->second->data + H);
  if (one_plus) for (auto& v : *out) v = f2b(1.0f + b2f(v));  // NormStyle::OnePlus, nn.rs:246-256
  return true;
}

}  // namespace

KO_API int ko_model_load(const kc_model_desc* desc, const kc_tensor_view* tensors, size_t n, ko_model** out) {
  const kc_model_desc& d = *desc;
  std::map<std::string, const kc_tensor_view*> idx;
  for (size_t i = 0; i < n; ++i) idx[tensors[i].name] = &tensors[i];
  ko_model* m = new ko_model;
  m->d = d;
  const int H = d.hidden_size, D = d.head_dim, F = d.intermediate_size, V = d.vocab_size;
  const bool gemma = d.arch == KC_ARCH_GEMMA2;
  bool ok = load_q(idx, "model.embed_tokens", V, H, d.bits, d.group_size, &m->embed);
  m->layers.resize(d.num_layers);
  for (int l = 0; ok && l < d.num_layers; ++l) {
    Layer& L = m->layers[l];
    const std::string p = "model.layers." + std::to_string(l);
    ok = load_q(idx, p + ".self_attn.q_proj", d.num_heads * D, H, d.bits, d.group_size, &L.q) &&
         load_q(idx, p + ".self_attn.k_proj", d.num_kv_heads * D, H, d.bits, d.group_size, &L.k) &&
         load_q(idx, p + ".self_attn.v_proj", d.num_kv_heads * D, H, d.bits, d.group_size, &L.v) &&
         load_q(idx, p + ".self_attn.o_proj", H, d.num_heads * D, d.bits, d.group_size, &L.o) &&
         load_q(idx, p + ".mlp.gate_proj", F, H, d.bits, d.group_size, &L.gate) &&
         load_q(idx, p + ".mlp.up_proj", F, H, d.bits, d.group_size, &L.up) &&
         load_q(idx, p + ".mlp.down_proj", H, F, d.bits, d.group_size, &L.down) &&
         load_norm(idx, p + ".input_layernorm.weight", H, gemma, &L.input_ln) &&
         load_norm(idx, p + ".post_attention_layernorm.weight", H, gemma, &L.post_attn_ln);
    if (ok && gemma)
      ok = load_norm(idx, p + ".pre_feedforward_layernorm.weight", H, true, &L.pre_ffw_ln) &&
           load_norm(idx, p + ".post_feedforward_layernorm.weight", H, true, &L.post_ffw_ln);
  }
  ok = ok && load_norm(idx, "model.norm.weight", H, gemma, &m->norm);
  m->tied = gemma || d.tie_word_embeddings;
  if (ok && !m->tied) ok = load_q(idx, "lm_head", V, H, d.bits, d.group_size, &m->head);
  if (!ok) { delete m; return 1; }
  // Attention scale: head_dim ** -0.5 in f64 narrowed to f32 (nn.rs:438-440); gemma 1/sqrt(query_pre_attn_scalar).
  m->scale = gemma && d.query_pre_attn_scalar > 0.f ? (float)(1.0 / std::sqrt((double)d.query_pre_attn_scalar))
                                                    : (float)std::pow((double)D, -0.5);
  // Rope frequencies (nn.rs:1409-1477), float32 like the MLX graph; the rotation uses position / freq.
  m->inv_freq.resize(D / 2);
  for (int i = 0; i < D / 2; ++i) {
    float freq = std::pow(d.rope_theta, (float)(2 * i) / (float)D);
    if (d.rope_scaling == KC_ROPE_LLAMA3) {
      const float wavelen = (float)(2.0 * M_PI) * freq;
      const float low_wl = d.rope_original_max_position / d.rope_low_freq_factor;
      const float high_wl = d.rope_original_max_position / d.rope_high_freq_factor;
      float f = wavelen > low_wl ? freq * d.rope_factor : freq;
      if (wavelen > high_wl && wavelen < low_wl) {
        const float smooth = (d.rope_original_max_position / wavelen - d.rope_low_freq_factor) /
                             (d.rope_high_freq_factor - d.rope_low_freq_factor);
        f = f / ((1.0f - smooth) / d.rope_factor + smooth);
      }
      freq = f;
    }
    float inv = 1.0f / freq;
    if (d.rope_scaling == KC_ROPE_LINEAR && d.rope_factor != 0.f) inv *= 1.0f / d.rope_factor;
    m->inv_freq[i] = inv;
  }
  *out = m;
  return 0;
}
KO_API void ko_model_free(ko_model* m) { delete m; }
KO_API void ko_model_set_layer_limit(ko_model* m, int layers) { m->layer_limit = layers; }

KO_API int ko_kv_create(int layers, int kv_heads, int head_dim, int num_blocks, int block_size, ko_kv** out) {
  ko_kv* kv = new ko_kv{layers, kv_heads, head_dim, num_blocks, block_size, {}};
  kv->pool.assign((size_t)layers * 2 * num_blocks * kv_heads * block_size * head_dim, 0);
  *out = kv;
  return 0;
}
KO_API void ko_kv_free(ko_kv* kv) { delete kv; }
KO_API void* ko_kv_data(ko_kv* kv) { return kv->pool.data(); }
KO_API void ko_kv_copy_block(ko_kv* kv, uint32_t src, uint32_t dst) {  // paged.rs:230-250
  const size_t be = (size_t)kv->kv_heads * kv->block_size * kv->head_dim;
  for (int p = 0; p < kv->layers * 2; ++p)
    memcpy(&kv->pool[((size_t)p * kv->num_blocks + dst) * be], &kv->pool[((size_t)p * kv->num_blocks + src) * be], be * 2);
}

namespace {

// fused SDPA over this sequence's history for query rows at positions offset..offset+len-1
// (nn.rs:800-817 + paged_attn.rs:83-153 algebra): q pre-scaled in fp32, fp32 softmax, o / sum -> bf16.
void sdpa_plain(const ko_model& m, const ko_kv& kv, int layer, const kc_seq_step& s, const float* q /* [len, Hq, D] */,
                float* out /* [len, Hq*D] */, int window = 0) {
  const int Hq = m.d.num_heads, Hkv = m.d.num_kv_heads, D = m.d.head_dim, gqa = Hq / Hkv, BS = kv.block_size;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int t = 0; t < s.len; ++t)
    for (int h = 0; h < Hq; ++h) {
      const int nkeys = s.offset + t + 1;  // causal, bottom-right aligned
      const int kh = h / gqa;
      std::vector<float> qs(D), sc(nkeys), o(D, 0.f);
      for (int d = 0; d < D; ++d) qs[d] = m.scale * q[((size_t)t * Hq + h) * D + d];
      float mx = -INFINITY;
      const int first = window > 0 ? std::max(0, nkeys - window) : 0;  // this build's window: the last `window` keys
      for (int i = first; i < nkeys; ++i) {
        const bf16_t* kr = &kv.pool[kv.idx(layer, 0, s.blocks[i / BS], kh, i % BS)];
        float a = 0.f;
        for (int d = 0; d < D; ++d) a += qs[d] * b2f(kr[d]);
        sc[i] = a; mx = std::max(mx, a);
      }
      float sum = 0.f;
      for (int i = first; i < nkeys; ++i) {
        const float e = std::exp(sc[i] - mx);
        sum += e;
        const bf16_t* vr = &kv.pool[kv.idx(layer, 1, s.blocks[i / BS], kh, i % BS)];
        for (int d = 0; d < D; ++d) o[d] += e * b2f(vr[d]);
      }
      for (int d = 0; d < D; ++d) out[(size_t)t * Hq * D + h * D + d] = rb(sum == 0.f ? o[d] : o[d] / sum);
    }
}

// Gemma-2 manual attention (nn.rs:497-580), every composed op rounded to bf16; softmax precise.
// window > 0 (this build's own definition; the reference has none): key j visible iff p - window < j <= p.
void sdpa_softcap(const ko_model& m, const ko_kv& kv, int layer, const kc_seq_step& s, const float* q, float cap, int window,
                  float* out) {
  const int Hq = m.d.num_heads, Hkv = m.d.num_kv_heads, D = m.d.head_dim, gqa = Hq / Hkv, BS = kv.block_size;
  const float scale_b = rb(m.scale), cap_b = rb(cap);
  const float neg_min = -(2.0f - 1.0f / 128.0f) * std::pow(2.0f, 127.0f);  // finfo(bf16).min
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int t = 0; t < s.len; ++t)
    for (int h = 0; h < Hq; ++h) {
      const int S = s.offset + s.len, p = s.offset + t;
      const int kh = h / gqa;
      std::vector<float> qs(D), sc(S), o(D, 0.f);
      for (int d = 0; d < D; ++d) qs[d] = rb(q[((size_t)t * Hq + h) * D + d] * scale_b);
      float mx = -INFINITY;
      for (int i = 0; i < S; ++i) {
        const bf16_t* kr = &kv.pool[kv.idx(layer, 0, s.blocks[i / BS], kh, i % BS)];
        float a = 0.f;
        for (int d = 0; d < D; ++d) a += qs[d] * b2f(kr[d]);
        a = rb(a);
        a = rb(rb(std::tanh(rb(a / cap_b))) * cap_b);
        const bool keep = i <= p && (window <= 0 || i > p - window);
        if (!keep) a = neg_min;
        sc[i] = a; mx = std::max(mx, a);
      }
      float sum = 0.f;
      for (int i = 0; i < S; ++i) { sc[i] = std::exp(sc[i] - mx); sum += sc[i]; }
      for (int i = 0; i < S; ++i) {
        const float pr = rb(sc[i] / sum);
        if (pr == 0.f) continue;
        const bf16_t* vr = &kv.pool[kv.idx(layer, 1, s.blocks[i / BS], kh, i % BS)];
        for (int d = 0; d < D; ++d) o[d] += pr * b2f(vr[d]);
      }
      for (int d = 0; d < D; ++d) out[(size_t)t * Hq * D + h * D + d] = rb(o[d]);
    }
}

inline float silu_mul(float g, float u) {  // nn.rs:289-293: three bf16 ops
  const float sg = rb(1.0f / (1.0f + std::exp(-g)));
  return rb(rb(g * sg) * u);
}
inline float gelu_mul(float g, float u) {  // nn.rs:221-235 op for op, weak scalars cast to bf16
  const float cube = rb(g * g * g);
  const float inner = rb(g + rb(rb(0.044715f) * cube));
  const float scaled = rb(rb(0.7978845608028654f) * inner);
  const float gate = rb(1.0f + rb(std::tanh(scaled)));
  return rb(rb(rb(0.5f * g) * gate) * u);
}

// rope (fast::rope, fp32 inside, one rounding) on [heads, D] of one token at position pos
void rope_row(const ko_model& m, float* x, int heads, float pos) {
  const int D = m.d.head_dim, half = D / 2;
  for (int h = 0; h < heads; ++h)
    for (int j = 0; j < half; ++j) {
      const int i0 = m.d.rope_traditional ? 2 * j : j, i1 = m.d.rope_traditional ? 2 * j + 1 : j + half;
      const float th = pos * m.inv_freq[j], c = std::cos(th), sn = std::sin(th);
      const float a = x[h * D + i0], b = x[h * D + i1];
      x[h * D + i0] = rb(a * c - b * sn);
      x[h * D + i1] = rb(a * sn + b * c);
    }
}

}  // namespace

// CausalLm::forward_step. logits_out: bf16 [n_sampled, vocab] (may be NULL to skip the head).
KO_API int ko_forward_step(ko_model* mp, ko_kv* kv, const uint32_t* token_ids, int32_t n, const kc_seq_step* seqs,
                           int32_t n_seqs, uint16_t* logits_out, int32_t* n_sampled_out) {
  const ko_model& m = *mp;
  const kc_model_desc& d = m.d;
  const int H = d.hidden_size, D = d.head_dim, Hq = d.num_heads, Hkv = d.num_kv_heads, F = d.intermediate_size, V = d.vocab_size;
  const bool gemma = d.arch == KC_ARCH_GEMMA2;
  long long total = 0;
  for (int i = 0; i < n_seqs; ++i) total += seqs[i].len;
  if (n <= 0 || total != n) { g_err = "step batch size mismatch"; return 1; }
  // embed (+ gemma scale, a bf16 multiply by bf16(sqrt(H)))
  std::vector<float> h((size_t)n * H), normed((size_t)n * H), tmp((size_t)n * H);
  const float es = gemma ? rb((float)std::sqrt((double)H)) : 0.f;
  {
    const int ng = H / d.group_size, wpr = H * d.bits / 32;
    for (int t = 0; t < n; ++t) {
      const uint32_t id = token_ids[t];
      if (id >= (uint32_t)V) { g_err = "token id outside vocabulary"; return 1; }
      const uint32_t* row = &m.embed.w[(size_t)id * wpr];
      for (int j = 0; j < H; ++j) {
        float v = rb((float)qval(row, j, d.bits) * b2f(m.embed.s[(size_t)id * ng + j / d.group_size]) +
                     b2f(m.embed.b[(size_t)id * ng + j / d.group_size]));
        if (gemma) v = rb(v * es);
        h[(size_t)t * H + j] = v;
      }
    }
  }
  std::vector<float> q((size_t)n * Hq * D), k((size_t)n * Hkv * D), v((size_t)n * Hkv * D), att((size_t)n * Hq * D),
      proj((size_t)n * H), gate((size_t)n * F), up((size_t)n * F);
  const int nl = m.layer_limit > 0 ? std::min(m.layer_limit, d.num_layers) : d.num_layers;
  for (int l = 0; l < nl; ++l) {
    const Layer& L = m.layers[l];
    rms_norm(h.data(), L.input_ln.data(), n, H, d.rms_norm_eps, normed.data());
    qmatmul(L.q, normed.data(), n, q.data());
    qmatmul(L.k, normed.data(), n, k.data());
    qmatmul(L.v, normed.data(), n, v.data());
    // per sequence: rope at its own offset, write K/V rows into the pools (paged.rs:147-187)
    int row = 0;
    for (int si = 0; si < n_seqs; ++si) {
      const kc_seq_step& s = seqs[si];
      for (int t = 0; t < s.len; ++t) {
        const int pos = s.offset + t;
        rope_row(m, &q[(size_t)(row + t) * Hq * D], Hq, (float)pos);
        rope_row(m, &k[(size_t)(row + t) * Hkv * D], Hkv, (float)pos);
        for (int kh = 0; kh < Hkv; ++kh)
          for (int dd = 0; dd < D; ++dd) {
            kv->pool[kv->idx(l, 0, s.blocks[pos / kv->block_size], kh, pos % kv->block_size) + dd] = f2b(k[((size_t)(row + t) * Hkv + kh) * D + dd]);
            kv->pool[kv->idx(l, 1, s.blocks[pos / kv->block_size], kh, pos % kv->block_size) + dd] = f2b(v[((size_t)(row + t) * Hkv + kh) * D + dd]);
          }
      }
      row += s.len;
    }
    row = 0;
    for (int si = 0; si < n_seqs; ++si) {
      const kc_seq_step& s = seqs[si];
      if (gemma) {
        const int window = (d.sliding_window > 0 && l % 2 == 0) ? d.sliding_window : 0;
        sdpa_softcap(m, *kv, l, s, &q[(size_t)row * Hq * D], d.attn_logit_softcapping, window, &att[(size_t)row * Hq * D]);
      } else {
        sdpa_plain(m, *kv, l, s, &q[(size_t)row * Hq * D], &att[(size_t)row * Hq * D]);
      }
      row += s.len;
    }
    qmatmul(L.o, att.data(), n, proj.data());
    if (gemma) {  // sandwich block, nn.rs:974-982
      rms_norm(proj.data(), L.post_attn_ln.data(), n, H, d.rms_norm_eps, tmp.data());
      for (size_t i = 0; i < h.size(); ++i) h[i] = rb(h[i] + tmp[i]);
      rms_norm(h.data(), L.pre_ffw_ln.data(), n, H, d.rms_norm_eps, normed.data());
    } else {      // pre-norm block, nn.rs:983-988
      for (size_t i = 0; i < h.size(); ++i) h[i] = rb(h[i] + proj[i]);
      rms_norm(h.data(), L.post_attn_ln.data(), n, H, d.rms_norm_eps, normed.data());
    }
    qmatmul(L.gate, normed.data(), n, gate.data());
    qmatmul(L.up, normed.data(), n, up.data());
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n * F; ++i) gate[i] = gemma ? gelu_mul(gate[i], up[i]) : silu_mul(gate[i], up[i]);
    qmatmul(L.down, gate.data(), n, proj.data());
    if (gemma) {
      rms_norm(proj.data(), L.post_ffw_ln.data(), n, H, d.rms_norm_eps, tmp.data());
      for (size_t i = 0; i < h.size(); ++i) h[i] = rb(h[i] + tmp[i]);
    } else {
      for (size_t i = 0; i < h.size(); ++i) h[i] = rb(h[i] + proj[i]);
    }
  }
  // sampled rows: trailing sample_rows of each sequence (nn.rs:1367-1381)
  std::vector<int> sampled;
  int pos = 0;
  for (int si = 0; si < n_seqs; ++si) { pos += seqs[si].len; for (int r = pos - seqs[si].sample_rows; r < pos; ++r) sampled.push_back(r); }
  if (n_sampled_out) *n_sampled_out = (int)sampled.size();
  if (sampled.empty() || !logits_out) return 0;
  const int ns = (int)sampled.size();
  std::vector<float> hs((size_t)ns * H), hn((size_t)ns * H), lg((size_t)ns * V);
  for (int i = 0; i < ns; ++i) memcpy(&hs[(size_t)i * H], &h[(size_t)sampled[i] * H], H * sizeof(float));
  rms_norm(hs.data(), m.norm.data(), ns, H, d.rms_norm_eps, hn.data());
  qmatmul(m.tied ? m.embed : m.head, hn.data(), ns, lg.data());
  if (gemma && d.final_logit_softcapping > 0.f) {
    const float cap = rb(d.final_logit_softcapping);
    for (auto& x : lg) x = rb(rb(std::tanh(rb(x / cap))) * cap);
  }
  for (size_t i = 0; i < lg.size(); ++i) logits_out[i] = f2b(lg[i]);
  return 0;
}

// Worker threads of the OpenMP regions in this file: the timed CPU baseline sets them explicitly, because launchers
// such as torchrun export OMP_NUM_THREADS=1 to every rank. Returns the count now in force.
KO_API int ko_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
}

// Greedy token per row (engine.rs:899-900 + sampler.rs:102-104 when normalize, draft.rs:379-381 otherwise).
KO_API void ko_greedy_rows(const uint16_t* logits, int rows, int vocab, int normalize, uint32_t* out) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const uint16_t* row = logits + (size_t)r * vocab;
    float lse = 0.f;
    if (normalize) {
      float mx = -INFINITY;
      for (int i = 0; i < vocab; ++i) mx = std::max(mx, b2f(row[i]));
      double s = 0.0;
      for (int i = 0; i < vocab; ++i) s += std::exp((double)(b2f(row[i]) - mx));
      lse = rb(mx + (float)std::log(s));
    }
    float best = -INFINITY; int bi = 0;
    for (int i = 0; i < vocab; ++i) {
      float x = b2f(row[i]);
      if (normalize) x = rb(x - lse);
      if (x > best) { best = x; bi = i; }  // strict: the lowest index wins ties
    }
    out[r] = (uint32_t)bi;
  }
}

// Stand-alone ops for kernel-level parity tests. All tensors bf16 unless noted.
KO_API void ko_quantized_matmul(const uint16_t* x, const uint32_t* w, const uint16_t* scales, const uint16_t* biases, int M,
                                int N, int K, int bits, int group, uint16_t* y) {
  QLinear L;
  L.N = N; L.K = K; L.bits = bits; L.group = group;
  L.w.assign(w, w + (size_t)N * K * bits / 32);
  L.s.assign(scales, scales + (size_t)N * (K / group));
  L.b.assign(biases, biases + (size_t)N * (K / group));
  std::vector<float> xf((size_t)M * K), yf((size_t)M * N);
  for (size_t i = 0; i < xf.size(); ++i) xf[i] = b2f(x[i]);
  qmatmul(L, xf.data(), M, yf.data());
  for (size_t i = 0; i < yf.size(); ++i) y[i] = f2b(yf[i]);
}

KO_API void ko_rms_norm(const uint16_t* x, const uint16_t* w, int rows, int H, float eps, uint16_t* y) {
  std::vector<float> xf((size_t)rows * H), yf((size_t)rows * H);
  for (size_t i = 0; i < xf.size(); ++i) xf[i] = b2f(x[i]);
  rms_norm(xf.data(), w, rows, H, eps, yf.data());
  for (size_t i = 0; i < yf.size(); ++i) y[i] = f2b(yf[i]);
}

// Attention over pools that already hold this step's K/V. q: bf16 [n, Hq, D]; out: bf16 [n, Hq*D].
KO_API void ko_paged_attention(ko_kv* kv, int layer, const uint16_t* q, int n, int num_heads, const kc_seq_step* seqs,
                               int n_seqs, float scale, float softcap, int window, uint16_t* out) {
  ko_model m;
  memset(&m.d, 0, sizeof m.d);
  m.d.num_heads = num_heads; m.d.num_kv_heads = kv->kv_heads; m.d.head_dim = kv->head_dim;
  m.scale = scale;
  const int D = kv->head_dim;
  std::vector<float> qf((size_t)n * num_heads * D), of((size_t)n * num_heads * D);
  for (size_t i = 0; i < qf.size(); ++i) qf[i] = b2f(q[i]);
  int row = 0;
  for (int si = 0; si < n_seqs; ++si) {
    if (softcap > 0.f) sdpa_softcap(m, *kv, layer, seqs[si], &qf[(size_t)row * num_heads * D], softcap, window, &of[(size_t)row * num_heads * D]);
    else sdpa_plain(m, *kv, layer, seqs[si], &qf[(size_t)row * num_heads * D], &of[(size_t)row * num_heads * D], window);
    row += seqs[si].len;
  }
  for (size_t i = 0; i < of.size(); ++i) out[i] = f2b(of[i]);
}
