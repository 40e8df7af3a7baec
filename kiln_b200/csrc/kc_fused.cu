// Element-wise and row-wise ops of the trunk, with the reference's rounding
// points: every MLX op returns its result rounded to the activation dtype
// (bf16); fused mlx.fast ops compute in fp32 and round once.
#include "kc_fused.cuh"

#include <algorithm>

namespace kc {

namespace {

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// ---------------------------------------------------------------------------
// Embedding::lookup (crates/kiln-models/src/nn.rs:159-176): gather the packed
// row, dequantise to bf16(q*scale + bias); Gemma then multiplies by
// bf16(sqrt(hidden)) in bf16 (nn.rs:1143-1154).
// ---------------------------------------------------------------------------
__global__ void embed_kernel(const uint32_t* __restrict__ w, const bf16* __restrict__ scales,
                             const bf16* __restrict__ biases, const uint32_t* __restrict__ ids, int H, int bits,
                             int group, float embed_scale, int vocab, bf16* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int tok = blockIdx.x;
  uint32_t id = ids[tok];
  if (id >= (uint32_t)vocab) id = 0;  // ids are validated on the host; never index out of the table
  const int per_word = 32 / bits;
  const int words = H / per_word;
  const uint32_t* wr = w + (size_t)id * words;
  const bf16* sr = scales + (size_t)id * (H / group);
  const bf16* br = biases + (size_t)id * (H / group);
  const uint32_t mask = (1u << bits) - 1u;
  const float es = embed_scale != 0.f ? bf16_round(embed_scale) : 0.f;
  for (int wi = threadIdx.x; wi < words; wi += blockDim.x) {
    const uint32_t u = wr[wi];
    const int j0 = wi * per_word;
    const float s = __bfloat162float(sr[j0 / group]), b = __bfloat162float(br[j0 / group]);
    for (int e = 0; e < per_word; ++e) {
      float v = bf16_round(fmaf((float)((u >> (bits * e)) & mask), s, b));
      if (es != 0.f) v = bf16_round(v * es);
      out[(size_t)tok * H + j0 + e] = __float2bfloat16_rn(v);
    }
  }
}

// A sublayer output as its consumer reads it: either bf16 [rows, N], or the fp32 split-K partials
// [splits][rows][N] of the GEMM that produced it, summed in split order and rounded to bf16 once here
// (the rounding the GEMM's own output would have had).
struct RowSource {
  const bf16* y;        // bf16 form, or null
  const float* part;    // partial form, or null
  int splits;
  size_t split_stride;  // rows * N
  int ld;               // row pitch in elements (N)
  const bf16* rank_y;   // per-rank bf16 form [ranks][rows][ld], or null
  int ranks;
  size_t rank_stride;
  const bf16* peer_y[KC_MAX_TP];   // per-rank bf16 [rows][ld] in each rank's own memory (peer loads), peers > 0
  int peers;
  const uint32_t* flags;           // this rank's flag array: flags[r] >= epoch once rank r's output is complete
  uint32_t epoch;
  uint32_t* status;
  int slice_w;                     // > 0: peer_y[s] holds the summed columns s * slice_w .. as [rows][slice_w]
};

// Waits until every tensor-parallel rank has published the output of exchange `epoch`. The flags live in this GPU's
// own memory (the peers store into them), so the poll is local. Bounded: after the limit the status word gets
// KC_DEV_TP | 1 and the kernel goes on (its result is then not valid; the host sees the status at its next
// synchronisation). Every thread of the CTA must call it.
__device__ __forceinline__ void tp_wait(const RowSource& s) {
  if ((int)threadIdx.x < s.peers) {
    const uint32_t* f = s.flags + threadIdx.x;
    auto ready = [&]() {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      return (int32_t)(v - s.epoch) >= 0;
    };
    if (!ready()) {
      const unsigned long long t0 = globaltimer_ns();
      uint32_t spins = 0;
      while (!ready()) {
        if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > KC_SPIN_LIMIT_NS) {
          if (s.status) atomicOr(s.status, KC_DEV_TP | 1u);
          break;
        }
      }
    }
  }
  __syncthreads();
}
__device__ __forceinline__ void load8(const RowSource& s, size_t row, int col, float (&v)[8]) {
  if (s.part) {
    const float* p0 = s.part + row * s.ld + col;
    float4 a = *reinterpret_cast<const float4*>(p0), b = *reinterpret_cast<const float4*>(p0 + 4);
    // the additions run in piece order; the loads of four pieces are issued together so that their latencies overlap
    int k = 1;
    for (; k + 4 <= s.splits; k += 4) {
      float4 c[4], d[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        c[j] = *reinterpret_cast<const float4*>(p0 + (k + j) * s.split_stride);
        d[j] = *reinterpret_cast<const float4*>(p0 + (k + j) * s.split_stride + 4);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        a.x += c[j].x; a.y += c[j].y; a.z += c[j].z; a.w += c[j].w; b.x += d[j].x; b.y += d[j].y; b.z += d[j].z; b.w += d[j].w;
      }
    }
    for (; k < s.splits; ++k) {
      const float4 c = *reinterpret_cast<const float4*>(p0 + k * s.split_stride);
      const float4 d = *reinterpret_cast<const float4*>(p0 + k * s.split_stride + 4);
      a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w; b.x += d.x; b.y += d.y; b.z += d.z; b.w += d.w;
    }
    v[0] = bf16_round(a.x); v[1] = bf16_round(a.y); v[2] = bf16_round(a.z); v[3] = bf16_round(a.w);
    v[4] = bf16_round(b.x); v[5] = bf16_round(b.y); v[6] = bf16_round(b.z); v[7] = bf16_round(b.w);
  } else if (s.peers && s.slice_w) {
    // already summed and rounded by the slice's owner: gather
    const int owner = col / s.slice_w;
    const uint4 u = __ldcv(reinterpret_cast<const uint4*>(s.peer_y[owner] + row * s.slice_w + (col - owner * s.slice_w)));
    const float2 a = unpack_bf162(u.x), b = unpack_bf162(u.y), c = unpack_bf162(u.z), d = unpack_bf162(u.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  } else if (s.peers) {
    // rank order, fp32, one rounding; the peers' rows are read where they were written (NVLink loads, not cached here)
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    uint4 u[KC_MAX_TP];
#pragma unroll
    for (int r = 0; r < KC_MAX_TP; ++r)
      if (r < s.peers) u[r] = __ldcv(reinterpret_cast<const uint4*>(s.peer_y[r] + row * s.ld + col));
#pragma unroll
    for (int r = 0; r < KC_MAX_TP; ++r) {
      if (r < s.peers) {
        const float2 a = unpack_bf162(u[r].x), b = unpack_bf162(u[r].y), c = unpack_bf162(u[r].z), d = unpack_bf162(u[r].w);
        acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = bf16_round(acc[k]);
  } else if (s.rank_y) {
    // rank order, fp32, one rounding: the same bits whatever collective moved the per-rank outputs here
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < s.ranks; ++r) {
      const uint4 u = *reinterpret_cast<const uint4*>(s.rank_y + r * s.rank_stride + row * s.ld + col);
      const float2 a = unpack_bf162(u.x), b = unpack_bf162(u.y), c = unpack_bf162(u.z), d = unpack_bf162(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = bf16_round(acc[k]);
  } else {
    const uint4 u = *reinterpret_cast<const uint4*>(s.y + row * s.ld + col);
    const float2 a = unpack_bf162(u.x), b = unpack_bf162(u.y), c = unpack_bf162(u.z), d = unpack_bf162(u.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
}
__device__ __forceinline__ void load8_bf16(const bf16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf162(u.x), b = unpack_bf162(u.y), c = unpack_bf162(u.z), d = unpack_bf162(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
__device__ __forceinline__ void store8_bf16(bf16* p, const float (&v)[8]) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack_bf162(v[0], v[1]), pack_bf162(v[2], v[3]), pack_bf162(v[4], v[5]), pack_bf162(v[6], v[7]));
}

// ---------------------------------------------------------------------------
// Residual add + RMSNorm (Block::forward_step / Block::finish, nn.rs:969-1019;
// fast::rms_norm, crates/kiln-mlx/src/fast.rs:36-41).
//   t = w_pre ? rms_norm(y, w_pre) : y            (gemma sandwich norm)
//   h = y ? bf16(x + t) : x                       (plain bf16 add, nn.rs:984, 987)
//   normed = w_out ? rms_norm(h, w_out) : (none)
// row_map (optional) selects input rows (the sampled-row `take`, nn.rs:1376-1381).
// One CTA per row, 8 elements per thread per pass; the row lives in shared memory between passes.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(const bf16* __restrict__ x, RowSource y, const bf16* __restrict__ w_pre,
                   const bf16* __restrict__ w_out, const int32_t* __restrict__ row_map, int H, float eps,
                   bf16* __restrict__ h_out, bf16* __restrict__ normed) {
  // with peer inputs the kernels after this one are released only once the peers' data is here: nothing of the next
  // kernel sits resident, counting down its own bounded waits, while this one waits for another GPU
  if (!y.peers) pdl_launch_dependents();
  pdl_wait();
  if (y.peers) { tp_wait(y); pdl_launch_dependents(); }
  extern __shared__ float srow[];   // H floats
  __shared__ float red[32];
  const int row = blockIdx.x;
  const size_t src = row_map ? row_map[row] : row;
  const bf16* xr = x + src * H;
  const bool has_y = y.y || y.part || y.rank_y || y.peers;
  float ss = 0.f;
  if (has_y && w_pre) {
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float v[8];
      load8(y, src, i, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) { srow[i + k] = v[k]; ss += v[k] * v[k]; }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    ss = 0.f;
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float xv[8], wv[8];
      load8_bf16(xr + i, xv);
      load8_bf16(w_pre + i, wv);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float t = bf16_round(wv[k] * (srow[i + k] * inv));
        const float h = bf16_round(xv[k] + t);
        srow[i + k] = h;
        ss += h * h;
      }
    }
  } else {
    for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
      float xv[8];
      load8_bf16(xr + i, xv);
      if (has_y) {
        float v[8];
        load8(y, src, i, v);
#pragma unroll
        for (int k = 0; k < 8; ++k) xv[k] = bf16_round(xv[k] + v[k]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) { srow[i + k] = xv[k]; ss += xv[k] * xv[k]; }
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float h[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) h[k] = srow[i + k];
    if (h_out) store8_bf16(h_out + (size_t)row * H + i, h);
    if (w_out) {
      float wv[8];
      load8_bf16(w_out + i, wv);
#pragma unroll
      for (int k = 0; k < 8; ++k) h[k] = wv[k] * (h[k] * inv);
      store8_bf16(normed + (size_t)row * H + i, h);
    }
  }
}

// The same operation for the common case (no sandwich norm, H = 2048 * CPT): the row stays in registers and all
// loads of a thread are issued before the first use, so a row costs one round trip to L2 instead of one per chunk.
// Element for element the arithmetic (and its order) is that of add_rmsnorm_kernel.
template <int CPT>
__global__ void __launch_bounds__(256)
add_rmsnorm_reg_kernel(const bf16* __restrict__ x, RowSource y, const bf16* __restrict__ w_out,
                       const int32_t* __restrict__ row_map, float eps, bf16* __restrict__ h_out,
                       bf16* __restrict__ normed) {
  if (!y.peers) pdl_launch_dependents();
  pdl_wait();
  if (y.peers) { tp_wait(y); pdl_launch_dependents(); }
  constexpr int H = 2048 * CPT;
  __shared__ float red[32];
  const int row = blockIdx.x;
  const size_t src = row_map ? row_map[row] : row;
  const bf16* xr = x + src * H;
  const bool has_y = y.y || y.part || y.rank_y || y.peers;
  float v[CPT][8];
  uint4 xraw[CPT];
#pragma unroll
  for (int c = 0; c < CPT; ++c) xraw[c] = *reinterpret_cast<const uint4*>(xr + (c * 256 + threadIdx.x) * 8);
  if (has_y) {
    if (y.part) {
      float4 a[CPT], b[CPT];
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        const float* p0 = y.part + src * y.ld + (c * 256 + threadIdx.x) * 8;
        a[c] = *reinterpret_cast<const float4*>(p0);
        b[c] = *reinterpret_cast<const float4*>(p0 + 4);
      }
#pragma unroll 4
      for (int k = 1; k < y.splits; ++k) {
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
          const float* p0 = y.part + k * y.split_stride + src * y.ld + (c * 256 + threadIdx.x) * 8;
          const float4 e = *reinterpret_cast<const float4*>(p0), f = *reinterpret_cast<const float4*>(p0 + 4);
          a[c].x += e.x; a[c].y += e.y; a[c].z += e.z; a[c].w += e.w;
          b[c].x += f.x; b[c].y += f.y; b[c].z += f.z; b[c].w += f.w;
        }
      }
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        v[c][0] = bf16_round(a[c].x); v[c][1] = bf16_round(a[c].y); v[c][2] = bf16_round(a[c].z); v[c][3] = bf16_round(a[c].w);
        v[c][4] = bf16_round(b[c].x); v[c][5] = bf16_round(b[c].y); v[c][6] = bf16_round(b[c].z); v[c][7] = bf16_round(b[c].w);
      }
    } else {
#pragma unroll
      for (int c = 0; c < CPT; ++c) load8(y, src, (c * 256 + threadIdx.x) * 8, v[c]);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    const float2 p0 = unpack_bf162(xraw[c].x), p1 = unpack_bf162(xraw[c].y), p2 = unpack_bf162(xraw[c].z), p3 = unpack_bf162(xraw[c].w);
    const float xv[8] = {p0.x, p0.y, p1.x, p1.y, p2.x, p2.y, p3.x, p3.y};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      v[c][k] = has_y ? bf16_round(xv[k] + v[c][k]) : xv[k];
      ss += v[c][k] * v[c][k];
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    const int i = (c * 256 + threadIdx.x) * 8;
    if (h_out) store8_bf16(h_out + (size_t)row * H + i, v[c]);
    if (w_out) {
      float wv[8], o[8];
      load8_bf16(w_out + i, wv);
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = wv[k] * (v[c][k] * inv);
      store8_bf16(normed + (size_t)row * H + i, o);
    }
  }
}

// ---------------------------------------------------------------------------
// (bias +) RoPE + PagedKv::write (nn.rs:724-726, 760-769; paged.rs:147-187;
// fast::rope, crates/kiln-mlx/src/fast.rs:45-104). One CTA per token; K is
// rotated, V copied, both land in the pool rows of the token's slot.
// ---------------------------------------------------------------------------
// sin/cos of the token's angles are computed once per CTA and shared by all heads; every thread then moves
// 8 consecutive features of each half with 16-byte loads and stores.
__global__ void __launch_bounds__(256)
rope_kv_write_kernel(RowSource qkv, const bf16* __restrict__ bias, const float* __restrict__ inv_freq,
                     const int32_t* __restrict__ token_pos, const int32_t* __restrict__ kv_slot, int Hq, int Hkv,
                     int D, int traditional, int layer, int NB, int BS, bf16* __restrict__ pool,
                     bf16* __restrict__ q_out) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float s_cs[128], s_sn[128];   // head_dim <= 256
  const int tok = blockIdx.x;
  const int heads = Hq + 2 * Hkv;
  const int half = D / 2;
  const float pos = (float)token_pos[tok];
  const int slot = kv_slot[tok];
  const int blk = slot / BS, r = slot % BS;
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &s_sn[j], &s_cs[j]);
  __syncthreads();
  const int per_head = D / 16;             // work items per head: 8 features of each half, or 16 interleaved ones
  for (int it = threadIdx.x; it < heads * per_head; it += blockDim.x) {
    const int h = it / per_head, c = it - h * per_head;
    // features [e0, e0 + 8) and [e1, e1 + 8) of head h; the rotation pairs are (e0 + k, e1 + k) for split
    // halves and (e0 + 2k, e0 + 2k + 1), (e1 + 2k, e1 + 2k + 1) for the interleaved convention
    const int e0 = traditional ? 16 * c : 8 * c;
    const int e1 = traditional ? 16 * c + 8 : half + 8 * c;
    float a[8], b[8];
    load8(qkv, tok, h * D + e0, a);
    load8(qkv, tok, h * D + e1, b);
    if (bias) {
      float ba[8], bb[8];
      load8_bf16(bias + h * D + e0, ba);
      load8_bf16(bias + h * D + e1, bb);
#pragma unroll
      for (int k = 0; k < 8; ++k) { a[k] = bf16_round(a[k] + ba[k]); b[k] = bf16_round(b[k] + bb[k]); }
    }
    bf16* dst;
    if (h < Hq) {
      dst = q_out + ((size_t)tok * Hq + h) * D;
    } else {
      const int kvsel = (h - Hq) / Hkv, kh = (h - Hq) % Hkv;
      dst = pool + (((((size_t)layer * 2 + kvsel) * NB + blk) * Hkv + kh) * BS + r) * D;
    }
    if (h < Hq + Hkv) {
      if (!traditional) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float cs = s_cs[8 * c + k], sn = s_sn[8 * c + k];
          const float ra = a[k] * cs - b[k] * sn, rb = a[k] * sn + b[k] * cs;
          a[k] = ra; b[k] = rb;
        }
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float cs = s_cs[8 * c + k], sn = s_sn[8 * c + k];
          float ra = a[2 * k] * cs - a[2 * k + 1] * sn, rb = a[2 * k] * sn + a[2 * k + 1] * cs;
          a[2 * k] = ra; a[2 * k + 1] = rb;
          cs = s_cs[8 * c + 4 + k]; sn = s_sn[8 * c + 4 + k];
          ra = b[2 * k] * cs - b[2 * k + 1] * sn; rb = b[2 * k] * sn + b[2 * k + 1] * cs;
          b[2 * k] = ra; b[2 * k + 1] = rb;
        }
      }
    }
    store8_bf16(dst + e0, a);
    store8_bf16(dst + e1, b);
  }
}

// ---------------------------------------------------------------------------
// Mlp::forward activation (nn.rs:284-294): silu(gate) * up with the three bf16
// roundings of the composed ops, or gelu_approx(gate) * up op for op (nn.rs:221-235).
// gu: [n, 2F] (gate | up)
// ---------------------------------------------------------------------------
// interleaved: gate and up features alternate in blocks of 128 columns (gate block j at columns 256 j, up block j at
// 256 j + 128) instead of all gate columns followed by all up columns.
__global__ void __launch_bounds__(256) glu_kernel(const bf16* __restrict__ gu, int n, int F, int gelu, int interleaved, bf16* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = F / 8;
  const int total = n * per_row;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int row = i / per_row, col = (i - row * per_row) * 8;
    const int gcol = interleaved ? (col >> 7) * 256 + (col & 127) : col;
    const int ucol = interleaved ? gcol + 128 : F + col;
    float g[8], u[8];
    load8_bf16(gu + (size_t)row * 2 * F + gcol, g);
    load8_bf16(gu + (size_t)row * 2 * F + ucol, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] = gelu ? act_gelu_mul(g[k], u[k]) : act_silu_mul(g[k], u[k]);
    store8_bf16(out + (size_t)row * F + col, g);
  }
}

// The same activation over a GEMM output still in its consumer form (bf16, or fp32 k-split partials summed here).
__global__ void __launch_bounds__(256) glu_from_kernel(const RowSource gu, int n, int F, int gelu, int interleaved, bf16* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = F / 8;
  const int total = n * per_row;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int row = i / per_row, col = (i - row * per_row) * 8;
    const int gcol = interleaved ? (col >> 7) * 256 + (col & 127) : col;
    const int ucol = interleaved ? gcol + 128 : F + col;
    float g[8], u[8];
    load8(gu, (size_t)row, gcol, g);
    load8(gu, (size_t)row, ucol, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] = gelu ? act_gelu_mul(g[k], u[k]) : act_silu_mul(g[k], u[k]);
    store8_bf16(out + (size_t)row * F + col, g);
  }
}

// Publishes "this rank's output of exchange `epoch` is complete" to every rank (its own flag array included). The
// kernel follows the producing GEMM on the stream; the GEMM's stores are in this GPU's L2, where the peers' loads
// are served, once it has finished.
struct TpFlagPtrs { uint32_t* p[KC_MAX_TP]; };
__global__ void tp_signal_kernel(TpFlagPtrs flags, int world, int rank, uint32_t epoch) {
  pdl_launch_dependents();
  pdl_wait();
  if ((int)threadIdx.x < world) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.p[threadIdx.x] + rank), "r"(epoch) : "memory");
  }
}

// First phase of the two-phase tensor-parallel exchange (a reduce-scatter over peer memory): this rank sums its
// column slice of every rank's partial output. One CTA per row.
__global__ void __launch_bounds__(128) tp_reduce_slice_kernel(RowSource src, int rank, int H, int slice_w, bf16* __restrict__ out) {
  pdl_wait();
  tp_wait(src);
  pdl_launch_dependents();
  const size_t row = blockIdx.x;
  for (int c = threadIdx.x * 8; c < slice_w; c += blockDim.x * 8) {
    float v[8];
    load8(src, row, rank * slice_w + c, v);   // src.slice_w == 0: the rank-ordered sum
    store8_bf16(out + row * slice_w + c, v);
  }
}

// CausalLm::softcap_logits (nn.rs:1158-1169): tanh(l / cap) * cap, each op rounded to bf16.
__global__ void softcap_kernel(bf16* __restrict__ x, long long total, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  const float capb = bf16_round(cap);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = __bfloat162float(x[i]);
    const float t = bf16_round(tanhf(bf16_round(v / capb)));
    x[i] = __float2bfloat16_rn(t * capb);
  }
}

// PagedKv::copy_block (paged.rs:230-250): rows of `src` into `dst` in every layer, K and V.
__global__ void copy_block_kernel(bf16* __restrict__ pool, int planes, int NB, size_t block_elems, uint32_t src,
                                  uint32_t dst) {
  pdl_launch_dependents();
  pdl_wait();
  const int plane = blockIdx.y;  // layer * 2 + kv
  if (plane >= planes) return;
  uint4* base = reinterpret_cast<uint4*>(pool + ((size_t)plane * NB) * block_elems);
  const size_t n16 = block_elems / 8;
  const uint4* s = base + (size_t)src * n16;
  uint4* d = base + (size_t)dst * n16;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) d[i] = s[i];
}

}  // namespace

cudaError_t launch_embed(const uint32_t* w, const bf16* scales, const bf16* biases, const uint32_t* ids, int n, int H,
                         int bits, int group, float embed_scale, int vocab, bf16* out, cudaStream_t s) {
  // The first kernel of a step follows the copy of the step's metadata: it is launched with plain stream order so
  // that its dependency on that copy is the ordinary one; the kernels after it chain from it.
  embed_kernel<<<n, 256, 0, s>>>(w, scales, biases, ids, H, bits, group, embed_scale, vocab, out);
  return cudaGetLastError();
}

static RowSource row_source(const SublayerOut& y) {
  RowSource r;
  r.y = y.y; r.part = y.part; r.splits = y.splits; r.split_stride = y.split_stride; r.ld = y.ld;
  r.rank_y = y.rank_y; r.ranks = y.ranks; r.rank_stride = y.rank_stride;
  for (int i = 0; i < KC_MAX_TP; ++i) r.peer_y[i] = y.peer_y[i];
  r.peers = y.peers; r.flags = y.flags; r.epoch = y.epoch; r.status = y.status; r.slice_w = y.slice_w;
  return r;
}

cudaError_t launch_add_rmsnorm(const bf16* x, const SublayerOut& y, const bf16* w_pre, const bf16* w_out,
                               const int32_t* row_map, int rows, int H, float eps, bf16* h_out, bf16* normed,
                               cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  if (H % 8) return cudaErrorInvalidValue;
  const bool aligned = !y.part || ((reinterpret_cast<uintptr_t>(y.part) & 15) == 0 && (y.ld & 3) == 0 && (y.split_stride & 3) == 0);
  const bool early = y.rank_y == nullptr;   // per-rank inputs arrive from a collective: see launch_k_opt
  if (!w_pre && aligned) {
    if (H == 2048) return launch_k_opt(early, add_rmsnorm_reg_kernel<1>, dim3(rows), dim3(256), 0, s, x, row_source(y), w_out, row_map, eps, h_out, normed);
    if (H == 4096) return launch_k_opt(early, add_rmsnorm_reg_kernel<2>, dim3(rows), dim3(256), 0, s, x, row_source(y), w_out, row_map, eps, h_out, normed);
    if (H == 8192) return launch_k_opt(early, add_rmsnorm_reg_kernel<4>, dim3(rows), dim3(256), 0, s, x, row_source(y), w_out, row_map, eps, h_out, normed);
  }
  return launch_k_opt(early, add_rmsnorm_kernel, dim3(rows), dim3(256), H * sizeof(float), s, x, row_source(y), w_pre, w_out, row_map, H, eps, h_out, normed);
}

cudaError_t launch_rope_kv_write(const SublayerOut& qkv, const bf16* bias, const float* inv_freq, const int32_t* token_pos,
                                 const int32_t* kv_slot, int n, int Hq, int Hkv, int D, int traditional, int layer,
                                 int NB, int BS, bf16* pool, bf16* q_out, cudaStream_t s) {
  if (D % 16 || D > 256) return cudaErrorInvalidValue;
  return launch_k(rope_kv_write_kernel, dim3(n), dim3(256), 0, s, row_source(qkv), bias, inv_freq, token_pos, kv_slot, Hq, Hkv, D,
                  traditional, layer, NB, BS, pool, q_out);
}

cudaError_t launch_glu(const bf16* gu, int n, int F, int gelu, int interleaved, bf16* out, cudaStream_t s) {
  if (F % 8 || (interleaved && F % 128)) return cudaErrorInvalidValue;
  const long long total = (long long)n * (F / 8);
  const int blocks = (int)std::min<long long>((total + 255) / 256, 148LL * 8);
  return launch_k(glu_kernel, dim3(blocks), dim3(256), 0, s, gu, n, F, gelu, interleaved, out);
}

cudaError_t launch_tp_signal(uint32_t* const* peer_flags, int world, int rank, uint32_t epoch, cudaStream_t s) {
  if (world < 1 || world > KC_MAX_TP) return cudaErrorInvalidValue;
  TpFlagPtrs f{};
  for (int r = 0; r < world; ++r) f.p[r] = peer_flags[r];
  return launch_k(tp_signal_kernel, dim3(1), dim3(32), 0, s, f, world, rank, epoch);
}

cudaError_t launch_tp_reduce_slice(const bf16* const* peer_y, int world, int rank, int rows, int H, int slice_w, const uint32_t* flags,
                                   uint32_t epoch, uint32_t* status, bf16* out, cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  if (world < 2 || world > KC_MAX_TP || slice_w % 8 || slice_w * world != H) return cudaErrorInvalidValue;
  return launch_k(tp_reduce_slice_kernel, dim3(rows), dim3(128), 0, s,
                  row_source(SublayerOut::of_peers(peer_y, world, H, flags, epoch, status)), rank, H, slice_w, out);
}

cudaError_t launch_glu_from(const SublayerOut& gu, int n, int F, int gelu, int interleaved, bf16* out, cudaStream_t s) {
  if (n <= 0) return cudaSuccess;
  if (F % 8 || (interleaved && F % 128) || gu.ld != 2 * F) return cudaErrorInvalidValue;
  const int total = n * (F / 8);
  const int blocks = std::max(1, std::min((total + 255) / 256, 148 * 8));
  return launch_k(glu_from_kernel, dim3(blocks), dim3(256), 0, s, row_source(gu), n, F, gelu, interleaved, out);
}

cudaError_t launch_softcap(bf16* x, long long total, float cap, cudaStream_t s) {
  const int blocks = (int)std::min<long long>((total + 255) / 256, 148LL * 8);
  return launch_k(softcap_kernel, dim3(blocks), dim3(256), 0, s, x, total, cap);
}

cudaError_t launch_copy_block(bf16* pool, int layers, int NB, size_t block_elems, uint32_t src, uint32_t dst,
                              cudaStream_t s) {
  dim3 grid((unsigned)std::max<size_t>(1, std::min<size_t>(block_elems / 8 / 256, 16)), layers * 2);
  return launch_k(copy_block_kernel, grid, dim3(256), 0, s, pool, layers * 2, NB, block_elems, src, dst);
}

}  // namespace kc
