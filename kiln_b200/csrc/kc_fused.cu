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

// ---------------------------------------------------------------------------
// Residual add + RMSNorm (Block::forward_step / Block::finish, nn.rs:969-1019;
// fast::rms_norm, crates/kiln-mlx/src/fast.rs:36-41).
//   t = w_pre ? rms_norm(y, w_pre) : y            (gemma sandwich norm)
//   h = y ? bf16(x + t) : x                       (plain bf16 add, nn.rs:984, 987)
//   normed = w_out ? rms_norm(h, w_out) : (none)
// row_map (optional) selects input rows (the sampled-row `take`, nn.rs:1376-1381).
// ---------------------------------------------------------------------------
template <int VEC>
__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ y, const bf16* __restrict__ w_pre,
                   const bf16* __restrict__ w_out, const int32_t* __restrict__ row_map, int H, float eps,
                   bf16* __restrict__ h_out, bf16* __restrict__ normed) {
  extern __shared__ float srow[];   // H floats
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int src = row_map ? row_map[row] : row;
  const bf16* xr = x + (size_t)src * H;
  const bf16* yr = y ? y + (size_t)src * H : nullptr;
  float ss = 0.f;
  if (yr && w_pre) {
    for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
      const float2 v = __bfloat1622float2(*reinterpret_cast<const bf162*>(yr + i));
      ss += v.x * v.x + v.y * v.y;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    ss = 0.f;
    for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
      const float2 v = __bfloat1622float2(*reinterpret_cast<const bf162*>(yr + i));
      const float2 wv = __bfloat1622float2(*reinterpret_cast<const bf162*>(w_pre + i));
      const float2 xv = __bfloat1622float2(*reinterpret_cast<const bf162*>(xr + i));
      const float t0 = bf16_round(wv.x * (v.x * inv)), t1 = bf16_round(wv.y * (v.y * inv));
      const float h0 = bf16_round(xv.x + t0), h1 = bf16_round(xv.y + t1);
      srow[i] = h0; srow[i + 1] = h1;
      ss += h0 * h0 + h1 * h1;
    }
  } else {
    for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
      const float2 xv = __bfloat1622float2(*reinterpret_cast<const bf162*>(xr + i));
      float h0 = xv.x, h1 = xv.y;
      if (yr) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const bf162*>(yr + i));
        h0 = bf16_round(h0 + v.x); h1 = bf16_round(h1 + v.y);
      }
      srow[i] = h0; srow[i + 1] = h1;
      ss += h0 * h0 + h1 * h1;
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x * 2; i < H; i += blockDim.x * 2) {
    const float h0 = srow[i], h1 = srow[i + 1];
    if (h_out) *reinterpret_cast<bf162*>(h_out + (size_t)row * H + i) = __floats2bfloat162_rn(h0, h1);
    if (w_out) {
      const float2 wv = __bfloat1622float2(*reinterpret_cast<const bf162*>(w_out + i));
      *reinterpret_cast<bf162*>(normed + (size_t)row * H + i) = __floats2bfloat162_rn(wv.x * (h0 * inv), wv.y * (h1 * inv));
    }
  }
}

// ---------------------------------------------------------------------------
// (bias +) RoPE + PagedKv::write (nn.rs:724-726, 760-769; paged.rs:147-187;
// fast::rope, crates/kiln-mlx/src/fast.rs:45-104). One CTA per token; K is
// rotated, V copied, both land in the pool rows of the token's slot.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rope_kv_write_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ bias, const float* __restrict__ inv_freq,
                     const int32_t* __restrict__ token_pos, const int32_t* __restrict__ kv_slot, int Hq, int Hkv,
                     int D, int traditional, int layer, int NB, int BS, bf16* __restrict__ pool,
                     bf16* __restrict__ q_out) {
  const int tok = blockIdx.x;
  const int heads = Hq + 2 * Hkv;
  const int half = D / 2;
  const float pos = (float)token_pos[tok];
  const int slot = kv_slot[tok];
  const int blk = slot / BS, r = slot % BS;
  const bf16* src = qkv + (size_t)tok * heads * D;
  for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
    const int h = i / half, j = i % half;
    const int i0 = traditional ? 2 * j : j, i1 = traditional ? 2 * j + 1 : j + half;
    float a = __bfloat162float(src[h * D + i0]), b = __bfloat162float(src[h * D + i1]);
    if (bias) {
      a = bf16_round(a + __bfloat162float(bias[h * D + i0]));
      b = bf16_round(b + __bfloat162float(bias[h * D + i1]));
    }
    bf16* dst;
    if (h < Hq) {
      dst = q_out + ((size_t)tok * Hq + h) * D;
    } else {
      const int kvsel = (h - Hq) / Hkv, kh = (h - Hq) % Hkv;
      dst = pool + (((((size_t)layer * 2 + kvsel) * NB + blk) * Hkv + kh) * BS + r) * D;
    }
    if (h < Hq + Hkv) {
      float sn, cs;
      sincosf(pos * inv_freq[j], &sn, &cs);
      const float ra = a * cs - b * sn, rb = a * sn + b * cs;
      a = ra; b = rb;
    }
    dst[i0] = __float2bfloat16_rn(a);
    dst[i1] = __float2bfloat16_rn(b);
  }
}

// ---------------------------------------------------------------------------
// Mlp::forward activation (nn.rs:284-294): silu(gate) * up with the three bf16
// roundings of the composed ops, or gelu_approx(gate) * up op for op (nn.rs:221-235).
// gu: [n, 2F] (gate | up)
// ---------------------------------------------------------------------------
__device__ __forceinline__ float act_silu_mul(float g, float u) {
  const float s = bf16_round(1.f / (1.f + __expf(-g)));
  const float t = bf16_round(g * s);
  return bf16_round(t * u);
}
__device__ __forceinline__ float act_gelu_mul(float g, float u) {
  const float cube = bf16_round(g * g * g);  // power(x, 3) in fp32, rounded once
  const float inner = bf16_round(g + bf16_round(bf16_round(0.044715f) * cube));
  const float scaled = bf16_round(bf16_round(0.7978845608028654f) * inner);
  const float gate = bf16_round(1.f + bf16_round(tanhf(scaled)));
  const float act = bf16_round(bf16_round(0.5f * g) * gate);
  return bf16_round(act * u);
}

__global__ void glu_kernel(const bf16* __restrict__ gu, int n, int F, int gelu, bf16* __restrict__ out) {
  const long long total = (long long)n * F / 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long e = i * 2;
    const int row = (int)(e / F), col = (int)(e % F);
    const float2 g = __bfloat1622float2(*reinterpret_cast<const bf162*>(gu + (size_t)row * 2 * F + col));
    const float2 u = __bfloat1622float2(*reinterpret_cast<const bf162*>(gu + (size_t)row * 2 * F + F + col));
    float2 r;
    if (gelu) { r.x = act_gelu_mul(g.x, u.x); r.y = act_gelu_mul(g.y, u.y); }
    else { r.x = act_silu_mul(g.x, u.x); r.y = act_silu_mul(g.y, u.y); }
    *reinterpret_cast<bf162*>(out + (size_t)row * F + col) = __floats2bfloat162_rn(r.x, r.y);
  }
}

// CausalLm::softcap_logits (nn.rs:1158-1169): tanh(l / cap) * cap, each op rounded to bf16.
__global__ void softcap_kernel(bf16* __restrict__ x, long long total, float cap) {
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
  embed_kernel<<<n, 256, 0, s>>>(w, scales, biases, ids, H, bits, group, embed_scale, vocab, out);
  return cudaGetLastError();
}

cudaError_t launch_add_rmsnorm(const bf16* x, const bf16* y, const bf16* w_pre, const bf16* w_out,
                               const int32_t* row_map, int rows, int H, float eps, bf16* h_out, bf16* normed,
                               cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  add_rmsnorm_kernel<2><<<rows, 256, H * sizeof(float), s>>>(x, y, w_pre, w_out, row_map, H, eps, h_out, normed);
  return cudaGetLastError();
}

cudaError_t launch_rope_kv_write(const bf16* qkv, const bf16* bias, const float* inv_freq, const int32_t* token_pos,
                                 const int32_t* kv_slot, int n, int Hq, int Hkv, int D, int traditional, int layer,
                                 int NB, int BS, bf16* pool, bf16* q_out, cudaStream_t s) {
  rope_kv_write_kernel<<<n, 256, 0, s>>>(qkv, bias, inv_freq, token_pos, kv_slot, Hq, Hkv, D, traditional, layer, NB,
                                         BS, pool, q_out);
  return cudaGetLastError();
}

cudaError_t launch_glu(const bf16* gu, int n, int F, int gelu, bf16* out, cudaStream_t s) {
  const long long total = (long long)n * F / 2;
  const int blocks = (int)std::min<long long>((total + 255) / 256, 148LL * 8);
  glu_kernel<<<blocks, 256, 0, s>>>(gu, n, F, gelu, out);
  return cudaGetLastError();
}

cudaError_t launch_softcap(bf16* x, long long total, float cap, cudaStream_t s) {
  const int blocks = (int)std::min<long long>((total + 255) / 256, 148LL * 8);
  softcap_kernel<<<blocks, 256, 0, s>>>(x, total, cap);
  return cudaGetLastError();
}

cudaError_t launch_copy_block(bf16* pool, int layers, int NB, size_t block_elems, uint32_t src, uint32_t dst,
                              cudaStream_t s) {
  dim3 grid((unsigned)std::max<size_t>(1, std::min<size_t>(block_elems / 8 / 256, 16)), layers * 2);
  copy_block_kernel<<<grid, 256, 0, s>>>(pool, layers * 2, NB, block_elems, src, dst);
  return cudaGetLastError();
}

}  // namespace kc
