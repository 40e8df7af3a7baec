// Greedy sampling and the verify settle walk on the device.
#include "kc_fused.cuh"

namespace kc {

namespace {

struct ArgMax { float v; int i; };
__device__ __forceinline__ void load8_bf16(const bf16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf162(u.x), b = unpack_bf162(u.y), c = unpack_bf162(u.z), d = unpack_bf162(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  // larger value wins; on equal values the lower index wins (MLX argmax tie-break as
  // observed in docs/decisions/0004-golden-parity-device-scope-and-dtype-aware-delta.md:53-56)
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

// sample_from_row + Sampler::sample, greedy lane (crates/kiln-engine/src/engine.rs:879-901,
// crates/kiln-engine/src/sampler.rs:100-104): logprobs = logits - logsumexp(logits) in the
// logits dtype, then argmax. The logsumexp accumulates in double and is rounded to bf16 before
// the subtraction; the subtraction result is rounded to bf16, which can merge neighbouring
// logits into ties — hence the explicit lowest-index rule.
// normalize == 0: argmax of the raw row (crates/kiln-models/src/draft.rs:379-381).
__global__ void __launch_bounds__(1024)
greedy_rows_kernel(const bf16* __restrict__ logits, int vocab, int normalize, uint32_t* __restrict__ tokens) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red_m[32];
  __shared__ double red_s[32];
  __shared__ ArgMax red_a[32];
  __shared__ float s_lse;
  const bf16* row = logits + (size_t)blockIdx.x * vocab;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const bool vec = (vocab & 7) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0;   // rows start on 16-byte boundaries
  if (normalize) {
    // Pass 1: the row maximum (exact). Pass 2: sum of exp(x - max), every term from the full-precision expf, the
    // running sums in double, so that the logsumexp — max + float(log(sum)), then one rounding to bf16 — lands on
    // the same bf16 value as a double-precision evaluation unless it sits within about 1e-6 of a rounding boundary.
    float m = -INFINITY;
    if (vec) {
      for (int i = threadIdx.x * 8; i < vocab; i += blockDim.x * 8) {
        float x[8];
        load8_bf16(row + i, x);
#pragma unroll
        for (int k = 0; k < 8; ++k) m = fmaxf(m, x[k]);
      }
    } else {
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) m = fmaxf(m, __bfloat162float(row[i]));
    }
    m = warp_max(m);
    if (lane == 0) red_m[warp] = m;
    __syncthreads();
    m = lane < nw ? red_m[lane] : -INFINITY;
    m = warp_max(m);                       // every thread now holds the row maximum
    double sum = 0.0;
    if (vec) {
      for (int i = threadIdx.x * 8; i < vocab; i += blockDim.x * 8) {
        float x[8];
        load8_bf16(row + i, x);
        float part = 0.f;                  // eight terms in fp32 (each at most 1), then into the double sum
#pragma unroll
        for (int k = 0; k < 8; ++k) part += expf(x[k] - m);
        sum += (double)part;
      }
    } else {
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) sum += (double)expf(__bfloat162float(row[i]) - m);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) red_s[warp] = sum;
    __syncthreads();
    if (warp == 0) {
      sum = lane < nw ? red_s[lane] : 0.0;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane == 0) s_lse = bf16_round(m + (float)log(sum));
    }
    __syncthreads();
  }
  const float lse = normalize ? s_lse : 0.f;
  ArgMax best{-INFINITY, 0x7fffffff};
  if (vec) {
    for (int i = threadIdx.x * 8; i < vocab; i += blockDim.x * 8) {
      float x[8];
      load8_bf16(row + i, x);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float v = normalize ? bf16_round(x[k] - lse) : x[k];
        if (v > best.v) best = ArgMax{v, i + k};   // indices rise within a thread: strict > keeps the lowest
      }
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      float x = __bfloat162float(row[i]);
      if (normalize) x = bf16_round(x - lse);
      best = better(best, ArgMax{x, i});
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b2{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, b2);
  }
  if (lane == 0) red_a[warp] = best;
  __syncthreads();
  if (warp == 0) {
    best = lane < nw ? red_a[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax b2{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = better(best, b2);
    }
    if (lane == 0) tokens[blockIdx.x] = (uint32_t)(best.i == 0x7fffffff ? 0 : best.i);
  }
}

// The settle walk (engine.rs:2336-2366): walk rows j = 0..|draft|; row j's token is committed;
// it "agrees" when j < |draft| and equals draft[j]; the walk stops after the first row that
// does not agree. n_committed = rows walked, n_accepted = agreeing rows.
__global__ void verify_accept_kernel(const uint32_t* __restrict__ row_tokens, const int32_t* __restrict__ seq_row_offsets,
                                     const uint32_t* __restrict__ draft, const int32_t* __restrict__ draft_offsets,
                                     const int32_t* __restrict__ draft_len, int n_seqs, int max_commit,
                                     uint32_t* __restrict__ committed, int32_t* __restrict__ n_committed,
                                     int32_t* __restrict__ n_accepted) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_seqs) return;
  const int dl = draft_len[i];
  if (dl < 0) { n_committed[i] = 0; n_accepted[i] = 0; return; }  // segment samples nothing
  const uint32_t* rows = row_tokens + seq_row_offsets[i];
  const uint32_t* d = draft + draft_offsets[i];
  int acc = 0, com = 0;
  for (int j = 0; j <= dl; ++j) {
    const uint32_t tok = rows[j];
    const bool agrees = j < dl && tok == d[j];
    if (agrees) ++acc;
    if (com < max_commit) committed[(size_t)i * max_commit + com] = tok;
    ++com;
    if (!agrees) break;
  }
  n_committed[i] = com;
  n_accepted[i] = acc;
}

// Device-side token feedback of the pipelined decode (StepInput::Lazy, crates/kiln-engine/src/step.rs:45-56;
// engine.rs:1711-1713): row i of the step takes the token that row feed[i] of the previous step sampled.
__global__ void feed_tokens_kernel(uint32_t* __restrict__ tokens, const int32_t* __restrict__ feed,
                                   const uint32_t* __restrict__ prev, int n, int prev_n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int f = feed[i];
  if (f >= 0 && f < prev_n) tokens[i] = prev[f];
}

}  // namespace

cudaError_t launch_feed_tokens(uint32_t* tokens, const int32_t* feed, const uint32_t* prev, int n, int prev_n, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  return launch_k(feed_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, s, tokens, feed, prev, n, prev_n);
}

cudaError_t launch_greedy_rows(const bf16* logits, int rows, int vocab, int normalize, uint32_t* tokens,
                               cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  return launch_k(greedy_rows_kernel, dim3(rows), dim3(1024), 0, s, logits, vocab, normalize, tokens);
}

cudaError_t launch_verify_accept(const uint32_t* row_tokens, const int32_t* seq_row_offsets, const uint32_t* draft,
                                 const int32_t* draft_offsets, const int32_t* draft_len, int n_seqs, int max_commit,
                                 uint32_t* committed, int32_t* n_committed, int32_t* n_accepted, cudaStream_t s) {
  if (n_seqs <= 0) return cudaSuccess;
  return launch_k(verify_accept_kernel, dim3((n_seqs + 127) / 128), dim3(128), 0, s, row_tokens, seq_row_offsets, draft,
                  draft_offsets, draft_len, n_seqs, max_commit, committed, n_committed, n_accepted);
}

}  // namespace kc
