// Paged multi-query attention over block tables (sm_100a).
//
// Replaces, for every query length, the reference's gather + fused SDPA
// (crates/kiln-engine/src/paged.rs:191-225; crates/kiln-models/src/nn.rs:800-817)
// and its decode-only Metal kernels (crates/kiln-engine/src/paged_attn.rs:59-303):
// token i of kv-head h is read at pool[tbl[i / BS], h, i % BS, :] (paged_attn.rs:95-99),
// never copied. Scores use the reference's algebra — fp32 scores, fp32 online
// softmax with exp(max - new_max) rescaling, output o / sum (paged_attn.rs:106-153);
// the causal predicate is bottom-right aligned: query at absolute position p
// sees keys 0..p. Gemma-2's softcap (nn.rs:527-534) and a sliding window are
// optional.
//
// Partition geometry is a function of absolute key position only: keys are cut
// into chunks of ATT_CHUNK, a chunk into 16-key tiles, tile t of a chunk belongs
// to key-split t % KS, splits and chunks are merged in index order. A query
// row's result therefore does not depend on how many other rows (of its own
// sequence or of others) share the launch.
//
// One CTA = (chunk, kv head, work item); a work item is up to MT*16/gqa
// consecutive tokens of one sequence, so the CTA's MT*16 query rows (token x
// head-in-group) all read the same K/V tiles: K/V bytes cross HBM once per
// (sequence, kv head). K/V tiles arrive by TMA (cp.async.bulk.tensor, 128-byte
// swizzle) through an mbarrier ring; QK^T and PV run on mma.sync m16n8k16.
#include "kc_attn.cuh"

#include <algorithm>

namespace kc {

namespace {

// A multiple of every key-split count, so one ring slot is always drained by the same
// consumer warps and each warp meets a slot's barrier phases strictly in order.
constexpr int ATT_STAGES = 8;
constexpr int ATT_MINB = 3;   // CTAs per SM the compiler must leave room for (head_dim <= 128, at most 32 query rows)

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Key-splits per chunk. A constant (never a function of how many query rows the CTA
// holds): the split a key tile belongs to, and so the merge order a row sees, must be the
// same in a one-token decode launch and in a verify launch.
template <int MT> struct KeySplit { static constexpr int value = 2; };
static_assert(KeySplit<1>::value > 1, "the partial kernel finishes single-chunk rows in its key-split merge");

// Shared memory: [stages][K tile | V tile] (1024-aligned, swizzled by TMA),
// then the Q rows (padded), then barriers. The K/V ring is reused for the
// cross-split merge after the main loop.
template <int D, int MT>
struct AttnSmem {
  static constexpr int KS = KeySplit<MT>::value;
  static constexpr int CW = MT * KS;                 // consumer warps
  static constexpr int TILE_BYTES = 16 * D * 2;      // one K (or V) tile
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int Q_LD = D * 2 + 16;            // bytes per Q row incl. pad
  static constexpr int Q_BYTES = MT * 16 * Q_LD;
  static constexpr int RING = ATT_STAGES * STAGE_BYTES;
  static constexpr int MERGE = KS > 1 ? KS * MT * 16 * (D + 4) * 4 : 0;
  static constexpr int RING_BYTES = RING > MERGE ? RING : MERGE;
  static constexpr int TOTAL = 1024 + RING_BYTES + Q_BYTES + 2 * ATT_STAGES * 8 + 64;
};

template <int D, int MT>
__global__ void __launch_bounds__((MT * KeySplit<MT>::value + 1) * 32, (D <= 128 && MT <= 2) ? ATT_MINB : 1)
attn_partial_kernel(const __grid_constant__ CUtensorMap kvmap, const AttnParams p) {
  using S = AttnSmem<D, MT>;
  constexpr int KS = S::KS;
  constexpr int CW = S::CW;
  constexpr int NT_D = D / 8;   // PV n-tiles
  constexpr int KSTEPS = D / 16;

  pdl_launch_dependents();
  pdl_wait();   // everything below reads step data (work items, q, block tables, this layer's K/V rows)
  const int chunk = p.chunk_lo_grid + blockIdx.x;
  const int kvh = blockIdx.y;
  const int4 wk = p.work[blockIdx.z];   // {seq, first token row in the step, tokens, position of first token}
  const int seq = wk.x, tok0 = wk.y, qlen = wk.z, pos0 = wk.w;
  const int pos_max = pos0 + qlen - 1;
  const int c_hi = pos_max / ATT_CHUNK;
  int c_lo = 0;
  if (p.window > 0) c_lo = max(0, pos0 - p.window + 1) / ATT_CHUNK;
  if (chunk > c_hi || chunk < c_lo) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  uint8_t* sQ = ring + S::RING_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(sQ + S::Q_BYTES);
  uint64_t* empty = full + ATT_STAGES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gqa = p.gqa;
  const int rows = qlen * gqa;                 // live query rows of this CTA
  const int key_base = chunk * ATT_CHUNK;
  const int keys_here = min(ATT_CHUNK, pos_max + 1 - key_base);
  const int ntiles = (keys_here + 15) >> 4;

  if (threadIdx.x == 0) {
    for (int i = 0; i < ATT_STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], MT); }
    mbar_fence_init();
  }
  __syncthreads();
  // The producer starts on the K/V tiles at once; the consumer warps stage Q meanwhile (its load latency then hides
  // under that of the first tiles). Row r = token (r / gqa), head-in-group (r % gqa); dead rows are zero.
  if (warp < CW) {
    const int chunks_per_row = D / 8;
    for (int i = threadIdx.x; i < MT * 16 * chunks_per_row; i += CW * 32) {
      const int r = i / chunks_per_row, ch = i % chunks_per_row;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < rows) {
        const int t = r / gqa, hg = r % gqa;
        v = *reinterpret_cast<const uint4*>(p.q + ((size_t)(tok0 + t) * p.Hq + kvh * gqa + hg) * D + ch * 8);
      }
      *reinterpret_cast<uint4*>(sQ + r * S::Q_LD + ch * 16) = v;
    }
    named_bar_sync(1, CW * 32);
  }

  if (warp == CW) {
    // ---- producer: one TMA per K+V tile pair (4-D map), or one per 64-feature slab of a K or V tile (2-D map). The chunk's block-table entries (at most
    //      ATT_CHUNK / 16 = 32) are fetched once, one per lane, so the per-tile loop has no global load in it ----
    if (lane == 0) tma_prefetch_desc(&kvmap);
    const int32_t* tbl = p.block_tables + (size_t)seq * p.max_blocks;
    const int blk0 = key_base / p.BS;
    const int nblk = (keys_here + p.BS - 1) / p.BS;
    const int my_blk = lane < nblk ? tbl[blk0 + lane] : 0;   // block_size is a power of two >= 16: chunks start on block edges
    bool alive = true;                                        // lane 0 only: false after a bounded wait gave up
    for (int t = 0; t < ntiles; ++t) {
      const int st = t & (ATT_STAGES - 1); const uint32_t ph = (t / ATT_STAGES) & 1;   // ATT_STAGES is a power of two
      const int koff = t * 16;
      const int blk = __shfl_sync(0xffffffffu, my_blk, koff / p.BS);
      if (lane == 0 && alive) {
        alive = mbar_wait(&empty[st], ph ^ 1, p.status, KC_DEV_ATTN | 1);
        if (!alive) continue;
        const int in_blk = (key_base + koff) % p.BS;
        const long long rowK = ((((long long)p.layer * 2 + 0) * p.NB + blk) * p.Hkv + kvh) * p.BS + in_blk;
        const long long rowV = ((((long long)p.layer * 2 + 1) * p.NB + blk) * p.Hkv + kvh) * p.BS + in_blk;
        mbar_arrive_expect_tx(&full[st], S::STAGE_BYTES);
        uint8_t* dst = ring + (size_t)st * S::STAGE_BYTES;
        if (p.kv4d) {
          // one operation: K slabs then V slabs, the layout of the loads below
          tma_load_4d(dst, &kvmap, 0, (blk * p.Hkv + kvh) * p.BS + in_blk, 0, p.layer * 2, &full[st]);
        } else {
#pragma unroll
          for (int h = 0; h < D / 64; ++h) {
            tma_load_2d(dst + h * 2048, &kvmap, h * 64, (int)rowK, &full[st]);
            tma_load_2d(dst + S::TILE_BYTES + h * 2048, &kvmap, h * 64, (int)rowV, &full[st]);
          }
        }
      }
    }
    __syncwarp();
  } else {
    // ---- consumers: warp (mt, ks) owns query rows 16*mt.. and tiles t % KS == ks ----
    const int mt = warp / KS, ks = warp % KS;
    const int g = lane >> 2, tq = lane & 3;
    const int r_lo = mt * 16 + g, r_hi = r_lo + 8;
    // Absolute position of each of this thread's two rows; -1 = dead row.
    const int p_lo = r_lo < rows ? pos0 + r_lo / gqa : -1;
    const int p_hi = r_hi < rows ? pos0 + r_hi / gqa : -1;
    const int w_lo = (p.window > 0 && p_lo >= 0) ? p_lo - p.window : -1;  // keys <= w are outside the window
    const int w_hi = (p.window > 0 && p_hi >= 0) ? p_hi - p.window : -1;

    float o[NT_D][4];
#pragma unroll
    for (int i = 0; i < NT_D; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

    const uint32_t q_base = smem_u32(sQ) + (mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * S::Q_LD + (lane >> 4) * 16;
    bool ok = true;
    for (int t = ks; t < ntiles; t += KS) {
      const int st = t & (ATT_STAGES - 1); const uint32_t ph = (t / ATT_STAGES) & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&full[st], ph, p.status, KC_DEV_ATTN | 2));
      if (!ok) break;
      const uint32_t kt = smem_u32(ring + (size_t)st * S::STAGE_BYTES);
      const uint32_t vt = kt + S::TILE_BYTES;

      // S = Q K^T for 16 rows x 16 keys
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        uint32_t a[4], b[4];
        ldsm_x4(a, q_base + kk * 32);
        {
          const int mi = lane >> 3;
          const int key = (mi >> 1) * 8 + (lane & 7);
          const int c = (kk & 3) * 2 + (mi & 1);
          ldsm_x4(b, kt + (kk >> 2) * 2048 + key * 128 + ((c ^ (key & 7)) << 4));
        }
        mma16816(s[0], a, b[0], b[1]);
        mma16816(s[1], a, b[2], b[3]);
      }

      // scale, softcap, mask -> log2-domain scores
      const int key0 = key_base + t * 16;
      float tmax_lo = -INFINITY, tmax_hi = -INFINITY;
      bool v[2][4];
      // Every key of the tile is visible to every live row (the rows' positions start at pos0), no window, no softcap:
      // the same arithmetic without the per-element predicates. Dead rows then carry finite garbage nobody stores.
      if (p.window == 0 && p.softcap == 0.f && key0 + 15 <= pos0) {
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float x = s[nt][j] * p.scale;
            x *= 1.4426950408889634f;
            v[nt][j] = true;
            s[nt][j] = x;
            if (j >= 2) tmax_hi = fmaxf(tmax_hi, x); else tmax_lo = fmaxf(tmax_lo, x);
          }
        }
      } else
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int key = key0 + nt * 8 + 2 * tq + (j & 1);
          const bool hi = j >= 2;
          const int lim = hi ? p_hi : p_lo;
          const int wlim = hi ? w_hi : w_lo;
          float x = s[nt][j] * p.scale;
          if (p.softcap > 0.f) x = p.softcap * tanhf(x / p.softcap);
          x *= 1.4426950408889634f;
          const bool valid = key <= lim && key > wlim;
          v[nt][j] = valid;
          s[nt][j] = x;
          if (valid) { if (hi) tmax_hi = fmaxf(tmax_hi, x); else tmax_lo = fmaxf(tmax_lo, x); }
        }
      }
      tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 1));
      tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 2));
      tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 1));
      tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 2));
      const float mn_lo = fmaxf(m_lo, tmax_lo), mn_hi = fmaxf(m_hi, tmax_hi);
      const float al_lo = (mn_lo == -INFINITY) ? 1.f : exp2f(m_lo - mn_lo);
      const float al_hi = (mn_hi == -INFINITY) ? 1.f : exp2f(m_hi - mn_hi);
      m_lo = mn_lo; m_hi = mn_hi;
      float ps_lo = 0.f, ps_hi = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const bool hi = j >= 2;
          const float pv = v[nt][j] ? exp2f(s[nt][j] - (hi ? mn_hi : mn_lo)) : 0.f;
          s[nt][j] = pv;
          if (hi) ps_hi += pv; else ps_lo += pv;
        }
      }
      l_lo = l_lo * al_lo + ps_lo;
      l_hi = l_hi * al_hi + ps_hi;
      uint32_t pa[4];
      pa[0] = pack_bf162(s[0][0], s[0][1]);
      pa[1] = pack_bf162(s[0][2], s[0][3]);
      pa[2] = pack_bf162(s[1][0], s[1][1]);
      pa[3] = pack_bf162(s[1][2], s[1][3]);

      // O = O * alpha + P V. Multiplying by exactly 1 changes no bit, so the rescale is skipped when no row of
      // the warp moved its maximum (the common case once the running maximum has settled).
      if (!__all_sync(0xffffffffu, al_lo == 1.f && al_hi == 1.f)) {
#pragma unroll
        for (int dn = 0; dn < NT_D; ++dn) { o[dn][0] *= al_lo; o[dn][1] *= al_lo; o[dn][2] *= al_hi; o[dn][3] *= al_hi; }
      }
#pragma unroll
      for (int dn = 0; dn < NT_D; dn += 2) {
        uint32_t b[4];
        const int mi = lane >> 3;
        const int key = (mi & 1) * 8 + (lane & 7);
        const int cg = dn + (mi >> 1);         // 8-feature chunk index over D
        const int c = cg & 7;
        ldsm_x4_t(b, vt + (cg >> 3) * 2048 + key * 128 + ((c ^ (key & 7)) << 4));
        mma16816(o[dn], pa, b[0], b[1]);
        mma16816(o[dn + 1], pa, b[2], b[3]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);
    }

    // Row sums live spread over the quad.
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

    if (KS > 1) {
      // Merge the key-splits of each row group in split order through shared memory.
      named_bar_sync(1, CW * 32);   // every consumer is done with the K/V ring
      float* mg = reinterpret_cast<float*>(ring);
      constexpr int RS = D + 4;     // floats per row record: o[D], m, l, pad (keeps rows 16-byte aligned)
      float* rec_lo = mg + ((size_t)(ks * MT * 16) + r_lo) * RS;
      float* rec_hi = mg + ((size_t)(ks * MT * 16) + r_hi) * RS;
#pragma unroll
      for (int dn = 0; dn < NT_D; ++dn) {
        *reinterpret_cast<float2*>(rec_lo + dn * 8 + 2 * tq) = make_float2(o[dn][0], o[dn][1]);
        *reinterpret_cast<float2*>(rec_hi + dn * 8 + 2 * tq) = make_float2(o[dn][2], o[dn][3]);
      }
      if (tq == 0) { rec_lo[D] = m_lo; rec_lo[D + 1] = l_lo; rec_hi[D] = m_hi; rec_hi[D + 1] = l_hi; }
      named_bar_sync(1, CW * 32);
      if (ks == 0 && ok) {
        // warp (mt, 0) merges rows 16*mt..16*mt+15: two lanes per row, half of D each.
        const int r = mt * 16 + (lane >> 1);
        if (r < rows) {
          float mmax = -INFINITY;
          for (int k = 0; k < KS; ++k) mmax = fmaxf(mmax, mg[((size_t)(k * MT * 16) + r) * RS + D]);
          float wgt[KS]; float lsum = 0.f;
          for (int k = 0; k < KS; ++k) {
            const float mk = mg[((size_t)(k * MT * 16) + r) * RS + D];
            wgt[k] = (mk == -INFINITY) ? 0.f : exp2f(mk - mmax);
            lsum += wgt[k] * mg[((size_t)(k * MT * 16) + r) * RS + D + 1];
          }
          const int t = r / gqa, hg = r % gqa;
          const size_t prow = ((size_t)(tok0 + t) * p.Hq + kvh * gqa + hg) * p.max_chunks + chunk;
          float* po = p.part_o + prow * D;
          // When no sequence of the step reaches past the first chunk, the chunk merge is the identity (weight
          // exp2(m - m) = 1) followed by the division: the row is finished here, with the arithmetic the combine
          // kernel would have applied to it, and that launch is skipped.
          bf16* fo = p.out + prow * D;   // max_chunks == 1 and chunk == 0 then: prow is the output row
          const int d0 = (lane & 1) * (D / 2);
          for (int d = d0; d < d0 + D / 2; d += 4) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < KS; ++k) {
              const float4 x = *reinterpret_cast<const float4*>(mg + ((size_t)(k * MT * 16) + r) * RS + d);
              acc.x += wgt[k] * x.x; acc.y += wgt[k] * x.y; acc.z += wgt[k] * x.z; acc.w += wgt[k] * x.w;
            }
            if (p.single_chunk) {
              // 0 + x: what the combine kernel's accumulation from zero yields (a -0 becomes +0 there too)
              acc.x = 0.f + acc.x; acc.y = 0.f + acc.y; acc.z = 0.f + acc.z; acc.w = 0.f + acc.w;
              if (lsum != 0.f) { acc.x = acc.x / lsum; acc.y = acc.y / lsum; acc.z = acc.z / lsum; acc.w = acc.w / lsum; }
              *reinterpret_cast<uint2*>(fo + d) = make_uint2(pack_bf162(acc.x, acc.y), pack_bf162(acc.z, acc.w));
            } else {
              *reinterpret_cast<float4*>(po + d) = acc;
            }
          }
          if ((lane & 1) == 0 && !p.single_chunk) p.part_ml[prow] = make_float2(mmax, lsum);
        }
      }
    } else if (ok) {
      const int rr[2] = {r_lo, r_hi};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = rr[h];
        if (r < rows) {
          const int t = r / gqa, hg = r % gqa;
          const size_t prow = ((size_t)(tok0 + t) * p.Hq + kvh * gqa + hg) * p.max_chunks + chunk;
          float* po = p.part_o + prow * D;
#pragma unroll
          for (int dn = 0; dn < NT_D; ++dn)
            *reinterpret_cast<float2*>(po + dn * 8 + 2 * tq) = make_float2(o[dn][2 * h], o[dn][2 * h + 1]);
          if (tq == 0) p.part_ml[prow] = make_float2(h ? m_hi : m_lo, h ? l_hi : l_lo);
        }
      }
    }
  }
}

// out[token, head, :] = sum_c w_c o_c / sum_c w_c l_c over the row's own chunks, in chunk order.
template <int D>
__global__ void attn_combine_kernel(const AttnParams p, int n_rows) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const int tok = row / p.Hq;
  const int pos = p.token_pos[tok];
  const int c_hi = pos / ATT_CHUNK;
  const int c_lo = p.window > 0 ? max(0, pos - p.window + 1) / ATT_CHUNK : 0;
  const float2* ml = p.part_ml + (size_t)row * p.max_chunks;
  // Chunks are taken eight at a time with all of a batch's loads issued before the first use: the arithmetic and its
  // order are those of a chunk-by-chunk loop, the kernel's duration is two round trips to L2 instead of two per chunk.
  constexpr int CB = 8;
  float mmax = -INFINITY;
  for (int c0 = c_lo; c0 <= c_hi; c0 += CB) {
    float2 v[CB];
#pragma unroll
    for (int j = 0; j < CB; ++j) v[j] = c0 + j <= c_hi ? ml[c0 + j] : make_float2(-INFINITY, 0.f);
#pragma unroll
    for (int j = 0; j < CB; ++j) mmax = fmaxf(mmax, v[j].x);
  }
  constexpr int PER = D / 32;
  float acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) acc[i] = 0.f;
  float lsum = 0.f;
  for (int c0 = c_lo; c0 <= c_hi; c0 += CB) {
    float2 v[CB];
    float po[CB][PER];
#pragma unroll
    for (int j = 0; j < CB; ++j) {
      const bool on = c0 + j <= c_hi;
      v[j] = on ? ml[c0 + j] : make_float2(-INFINITY, 0.f);
      const float* src = p.part_o + ((size_t)row * p.max_chunks + (on ? c0 + j : c_lo)) * D + lane * PER;
      if (PER % 4 == 0) {
#pragma unroll
        for (int i = 0; i < PER; i += 4) {
          const float4 q = on ? *reinterpret_cast<const float4*>(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
          po[j][i] = q.x; po[j][i + 1] = q.y; po[j][i + 2] = q.z; po[j][i + 3] = q.w;
        }
      } else {
        const float2 q = on ? *reinterpret_cast<const float2*>(src) : make_float2(0.f, 0.f);
        po[j][0] = q.x; po[j][PER - 1] = q.y;
      }
    }
#pragma unroll
    for (int j = 0; j < CB; ++j) {
      if (c0 + j <= c_hi) {
        const float w = (v[j].x == -INFINITY) ? 0.f : exp2f(v[j].x - mmax);
        lsum += w * v[j].y;
#pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] += w * po[j][i];
      }
    }
  }
  bf16* out = p.out + (size_t)row * D + lane * PER;
#pragma unroll
  for (int i = 0; i < PER; ++i) out[i] = __float2bfloat16_rn(lsum == 0.f ? acc[i] : acc[i] / lsum);
}

template <int D, int MT>
cudaError_t launch_partial(const CUtensorMap& map, const AttnParams& p, int n_work, int grid_chunks, cudaStream_t s) {
  using S = AttnSmem<D, MT>;
  static DeviceOnce configured;   // the attribute belongs to the device's copy of the kernel
  if (configured.first_on_current_device()) {
    cudaError_t e = cudaFuncSetAttribute(attn_partial_kernel<D, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) { configured.forget_current_device(); return e; }
  }
  dim3 grid(grid_chunks, p.Hkv, n_work);
  return launch_k(attn_partial_kernel<D, MT>, grid, dim3((S::CW + 1) * 32), S::TOTAL, s, map, p);
}

template <int D>
cudaError_t launch_d(const CUtensorMap& map, const AttnParams& p, int mt, int n_work, int grid_chunks, int n_tokens,
                     cudaStream_t s) {
  cudaError_t e;
  switch (mt) {
    case 1: e = launch_partial<D, 1>(map, p, n_work, grid_chunks, s); break;
    case 2: e = launch_partial<D, 2>(map, p, n_work, grid_chunks, s); break;
    case 3: e = launch_partial<D, 3>(map, p, n_work, grid_chunks, s); break;
    default: e = launch_partial<D, 4>(map, p, n_work, grid_chunks, s); break;
  }
  if (e != cudaSuccess || p.single_chunk) return e;
  const int n_rows = n_tokens * p.Hq;
  return launch_k(attn_combine_kernel<D>, dim3((n_rows + 7) / 8), dim3(256), 0, s, p, n_rows);
}

}  // namespace

int attn_tokens_per_item(int gqa, int max_len) {
  // Largest token count whose rows fit 64 (MT <= 4); capped by the longest segment.
  int t = std::max(1, 64 / gqa);
  return std::min(t, std::max(1, max_len));
}

cudaError_t paged_attention(const CUtensorMap& kvmap, const AttnParams& p, int head_dim, int tokens_per_item,
                            int n_work, int grid_chunks, int n_tokens, cudaStream_t s) {
  const int rows = tokens_per_item * p.gqa;
  const int mt = (rows + 15) / 16;
  if (mt < 1 || mt > 4) return cudaErrorInvalidValue;
  switch (head_dim) {
    case 64: return launch_d<64>(kvmap, p, mt, n_work, grid_chunks, n_tokens, s);
    case 128: return launch_d<128>(kvmap, p, mt, n_work, grid_chunks, n_tokens, s);
    case 256: return launch_d<256>(kvmap, p, mt, n_work, grid_chunks, n_tokens, s);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace kc
