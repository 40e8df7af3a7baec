// Affine-dequant GEMM for sm_100a. See kc_qlinear.cuh for the data layout.
//
// qlinear_umma_ta_kernel — one CTA per (one or two 128-row weight tiles, k-split), 20 warps:
//   warp 0      bulk-copies the weight records (cp.async.bulk, mbarrier tx)
//   warp 1      TMA-loads the activation k-blocks (cp.async.bulk.tensor, 128B swizzle)
//   warps 2-3   allocate TMEM, issue tcgen05.mma (weights = A/M side from TENSOR MEMORY, activations = B/N side
//               from shared memory); the two issuing threads take alternate pipeline stages and pass the issue order
//               to each other through an mbarrier
//   warps 4-19  unpack the 4/8-bit words, apply scale/bias in registers and write the bf16 A operand into tensor
//               memory with tcgen05.st; afterwards drain the accumulators (tcgen05.ld) into y, the split-K
//               partials or the gated activation.
// The accumulator D[n, m] lives in TMEM: lane = weight row n, column = activation row m.
// Every output element depends only on its own activation row and on a k order
// fixed by (N, K), which is what lets verify rows share a step with other rows
// and still reproduce the bits of a one-row decode. Launches of more rows than one accumulator set holds are cut
// into row chunks, each its own launch over the same weights: rows are independent, so no bit changes.
#include "kc_qlinear.cuh"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <cstdlib>

namespace kc {

// ---------------------------------------------------------------------------
// Re-tiling
// ---------------------------------------------------------------------------

__global__ void qweight_retile_kernel(uint8_t* __restrict__ records, const uint32_t* __restrict__ w,
                                      const bf16* __restrict__ scales, const bf16* __restrict__ biases,
                                      int N, int K, int bits, int group, int n_tiles, int kblocks,
                                      int gpk, uint32_t packed_bytes, uint32_t record_bytes) {
  const int words_per_row_kb = QL_KB * bits / 32;  // 8 (w4) or 16 (w8)
  const int words_per_rec = QL_TILE_N * words_per_row_kb;
  const int sb_per_rec = QL_TILE_N * gpk;
  const long long per_rec = words_per_rec + sb_per_rec;
  const long long total = (long long)((n_tiles + QL_TILE_GROUP - 1) / QL_TILE_GROUP) * QL_TILE_GROUP * kblocks * per_rec;
  const int src_words_per_row = K * bits / 32;
  const int groups_per_row = K / group;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long rec = i / per_rec;
    const int e = (int)(i % per_rec);
    // record order: [tile group][k-block][tile in group], so the records of 1, 2 or 4 neighbouring tiles for
    // one k-block are contiguous and one bulk copy fetches them
    const int tig = (int)(rec % QL_TILE_GROUP);
    const long long gk = rec / QL_TILE_GROUP;
    const int kb = (int)(gk % kblocks);
    const int tile = (int)(gk / kblocks) * QL_TILE_GROUP + tig;
    uint8_t* base = records + rec * (long long)record_bytes;
    if (e < words_per_rec) {
      const int r = e / words_per_row_kb, c = e % words_per_row_kb;
      const int n = tile * QL_TILE_N + r;
      uint32_t v = 0;
      if (n < N) v = w[(long long)n * src_words_per_row + kb * words_per_row_kb + c];
      if (bits == 4) {
        uint32_t o = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          o |= ((v >> (8 * j)) & 0xFu) << (4 * j);
          o |= ((v >> (8 * j + 4)) & 0xFu) << (16 + 4 * j);
        }
        v = o;
      }
      reinterpret_cast<uint32_t*>(base)[e] = v;
    } else {
      const int e2 = e - words_per_rec;
      const int r = e2 / gpk, gi = e2 % gpk;
      const int n = tile * QL_TILE_N + r;
      bf162 sb = __floats2bfloat162_rn(0.f, 0.f);
      if (n < N) {
        const int g = (kb * QL_KB + gi * group) / group;
        sb.x = scales[(long long)n * groups_per_row + g];
        sb.y = biases[(long long)n * groups_per_row + g];
      }
      reinterpret_cast<bf162*>(base + packed_bytes)[e2] = sb;
    }
  }
}

int qlinear_plan_splits(int n_tiles, int kblocks, int sm_count) {
  // As many k-splits as fill the SMs with one-tile CTAs, each keeping at least 8 k-blocks; none when two-tile CTAs
  // already fill them. Splits need not divide the k-blocks evenly (the kernel cuts [K s / S, K (s + 1) / S)).
  if (n_tiles * 2 >= sm_count) return 1;
  int s = sm_count / n_tiles;
  s = std::min(s, std::min(16, kblocks / 8));
  return std::max(s, 1);
}

cudaError_t qweight_build(QWeight* out, const uint32_t* w, const bf16* scales, const bf16* biases,
                          int N, int K, int bits, int group, int sm_count, cudaStream_t s) {
  QWeight q;
  q.N = N; q.K = K; q.bits = bits; q.group = group;
  q.n_tiles = (N + QL_TILE_N - 1) / QL_TILE_N;
  q.kblocks = K / QL_KB;
  q.gpk = std::max(1, QL_KB / group);
  q.packed_bytes = QL_TILE_N * (QL_KB * bits / 8);
  q.record_bytes = q.packed_bytes + QL_TILE_N * q.gpk * 4;
  q.splits = qlinear_plan_splits(q.n_tiles, q.kblocks, sm_count);
  q.sm_count = sm_count;
  cudaError_t e = cudaMalloc(&q.records, q.bytes());
  if (e != cudaSuccess) return e;
  const long long total = (long long)(q.bytes() / 4);
  const int threads = 256;
  const int blocks = (int)std::min<long long>((total + threads - 1) / threads, 148LL * 16);
  qweight_retile_kernel<<<blocks, threads, 0, s>>>(q.records, w, scales, biases, N, K, bits, group,
                                                   q.n_tiles, q.kblocks, q.gpk, q.packed_bytes,
                                                   q.record_bytes);
  e = cudaGetLastError();
  if (e != cudaSuccess) { cudaFree(q.records); return e; }
  *out = q;
  return cudaSuccess;
}

void qweight_free(QWeight* w) {
  if (w && w->records) { cudaFree(w->records); w->records = nullptr; }
}

// ---------------------------------------------------------------------------
// Tensor maps for the activation operand
// ---------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

bool make_tmap_bf16_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer,
                       uint32_t box_inner, uint32_t box_outer, const char** err) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) { *err = "cuTensorMapEncodeTiled entry point unavailable"; return false; }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {inner * sizeof(bf16)};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { *err = "cuTensorMapEncodeTiled rejected the tensor geometry"; return false; }
  return true;
}

// K/V pools [planes = layers * 2][plane_rows = NB * Hkv * BS][head_dim] bf16 as a 4-D tensor
// {64 features, plane_rows, head_dim / 64 slabs, planes} with box {64, 16, head_dim / 64, 2}: ONE operation brings the
// 16-key K tile and the V tile of a layer (plane 2 * layer and the next), each as head_dim / 64 slabs of [16][128 B]
// with the 128-byte swizzle — the shared-memory image of 2 * head_dim / 64 separate 2-D loads. The slab stride
// (128 B) is smaller than the row stride, which the encoder may refuse: the caller then keeps the 2-D map.
bool make_tmap_kv_4d(CUtensorMap* map, const void* pool, uint32_t head_dim, uint64_t plane_rows, uint64_t planes,
                     const char** err) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) { *err = "cuTensorMapEncodeTiled entry point unavailable"; return false; }
  cuuint64_t dims[4] = {64, plane_rows, head_dim / 64, planes};
  cuuint64_t strides[3] = {head_dim * sizeof(bf16), 128, plane_rows * head_dim * sizeof(bf16)};
  cuuint32_t box[4] = {64, 16, head_dim / 64, 2};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(pool), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);   // head_dim >= 128: a key's row is 256 B or more, both slabs of it in one L2 fill
  if (r != CUDA_SUCCESS) { *err = "cuTensorMapEncodeTiled rejected the 4-D K/V geometry"; return false; }
  return true;
}

// The map whose box covers `m_pad` rows (<= 256), so that one TMA operation brings a whole activation k-block.
// Re-encoded only when the row count changes (a host-side encode, no device work).
static const CUtensorMap* act_operand_rows_map(const ActOperand* op, int m_pad) {
  if (op->rows_map_n != m_pad) {
    const char* err = "";
    if (!make_tmap_bf16_2d(&op->rows_map, op->ptr, op->K, op->rows, QL_KB, m_pad, &err)) return nullptr;
    op->rows_map_n = m_pad;
  }
  return &op->rows_map;
}

bool act_operand_init(ActOperand* op, const bf16* ptr, int rows, int K, const char** err) {
  op->ptr = ptr; op->rows = rows; op->K = K; op->rows_map_n = 0;
  if (K % QL_KB) { *err = "activation width must be a multiple of 64"; return false; }
  if (!make_tmap_bf16_2d(&op->map16, ptr, K, rows, QL_KB, 16, err)) return false;
  if (!make_tmap_bf16_2d(&op->map64, ptr, K, rows, QL_KB, 64, err)) return false;
  return true;
}

// ---------------------------------------------------------------------------
// Dequantisation of one 8-element chunk -> 8 bf16 (16 bytes)
// ---------------------------------------------------------------------------

__device__ __forceinline__ uint4 dequant8_w4(uint32_t u, bf162 sb) {
  const bf162 s2 = __bfloat162bfloat162(sb.x);
  const bf162 b2 = __bfloat162bfloat162(sb.y);
  const bf162 c128 = __floats2bfloat162_rn(128.f, 128.f);
  // The record's nibble order puts element 2j at bits 4j and element 2j + 1 at bits 16 + 4j. Two masks split the word
  // into bytes (even nibbles: elements 0, 4, 1, 5; odd nibbles: 2, 6, 3, 7) and a byte permute sets each under 0x43:
  // 0x4300 | q is the bf16 value 128 + q (exact for q < 128); subtracting 128 is exact.
  const uint32_t lo = u & 0x0F0F0F0Fu, hi = (u >> 4) & 0x0F0F0F0Fu;
  uint32_t t[4];
  t[0] = __byte_perm(lo, 0x43434343u, 0x4240u);   // elements 0, 1
  t[1] = __byte_perm(hi, 0x43434343u, 0x4240u);   // elements 2, 3
  t[2] = __byte_perm(lo, 0x43434343u, 0x4341u);   // elements 4, 5
  t[3] = __byte_perm(hi, 0x43434343u, 0x4341u);   // elements 6, 7
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    bf162 q = __hsub2(*reinterpret_cast<bf162*>(&t[j]), c128);
    bf162 wv = __hfma2(q, s2, b2);  // one rounding: bf16(q*s + b)
    o[j] = *reinterpret_cast<uint32_t*>(&wv);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

__device__ __forceinline__ uint4 dequant8_w8(uint32_t u0, uint32_t u1, bf162 sb) {
  const float s = __bfloat162float(sb.x), b = __bfloat162float(sb.y);
  float f[8];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    // byte k under the exponent of 2^23: the float 8388608 + q, minus 2^23 = q exactly.
    f[k] = __uint_as_float(__byte_perm(u0, 0x4B000000u, 0x7540u | k)) - 8388608.f;
    f[4 + k] = __uint_as_float(__byte_perm(u1, 0x4B000000u, 0x7540u | k)) - 8388608.f;
  }
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) o[j] = pack_bf162(fmaf(f[2 * j], s, b), fmaf(f[2 * j + 1], s, b));
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// ---------------------------------------------------------------------------
// tcgen05 helpers
// ---------------------------------------------------------------------------

__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t smem_addr) {
  // K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);       // start address
  d |= (uint64_t)1 << 16;                           // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                           // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                           // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ uint32_t umma_idesc_bf16(int m, int n) {
  // kind::f16 takes A and B of the SAME 16-bit type: an f16 A against a bf16 B is an illegal instruction.
  uint32_t d = 0;
  d |= 1u << 4;                    // D format f32
  d |= 1u << 7;                    // A format bf16
  d |= 1u << 10;                   // B format bf16
  // a_major (bit 15) = b_major (bit 16) = 0: both K-major
  d |= (uint32_t)(n >> 3) << 17;   // N
  d |= (uint32_t)(m >> 4) << 24;   // M
  return d;
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------

constexpr int QL_DQ_WARP0 = 4;         // first dequant/epilogue warp
constexpr int QL_DQ_GROUPS = 2;        // dequant groups; group g converts k-blocks g, g + G, g + 2G, ...
constexpr int QL_DQ_GROUP_WARPS = 8;
constexpr int QL_DQ_GROUP_THREADS = QL_DQ_GROUP_WARPS * 32;
constexpr int QL_DQ_WARPS = QL_DQ_GROUPS * QL_DQ_GROUP_WARPS;
constexpr int QL_THREADS = (QL_DQ_WARP0 + QL_DQ_WARPS) * 32;   // 20 warps
constexpr int QL_A_BYTES = QL_TILE_N * 128;  // one 128-row A tile of one stage
constexpr int QL_EPI_STAGE_BYTES = 32 * 32 * 4;   // per-warp transpose buffer of the epilogue

struct QlKernelParams {
  const uint8_t* records;
  uint32_t record_bytes;
  int N, n_tiles, kblocks;
  int M, m_pad;          // live rows, rows rounded up to 16
  int row0;              // first activation row
  int splits;
  int a_stages, r_stages, b_stages;   // b_stages: activation ring of the kernel that keeps its A ring in TMEM
  uint32_t raw_stride;   // distance between the records of neighbouring tiles in a raw stage (= record_bytes)
  int b_single;          // 1: the first tensor map's box spans all m_pad rows (one TMA operation per k-block)
  int glu;               // 0, or 1 (silu) / 2 (gelu_approx): the epilogue writes act = activation(gate tile) * up tile
  bf16* act; int ld_act;
  uint32_t tmem_cols;    // power of two >= max(32, NT * m_pad)
  bf16* y; int ldy;
  float* partial;        // [splits][part_M][N]; this launch writes rows part_row0 .. part_row0 + M
  int part_M, part_row0;
  uint32_t* status;
};

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The epilogue shared by the GEMM kernels: every epilogue warp drains its TMEM lane quarter, 32 columns (rows of the
// step) at a time, transposes through a private 4 KB shared buffer and stores row-contiguous vectors: bf16 y, fp32
// split-K partials, or — when the CTA owns (gate, up) tile pairs — the gated activation.
template <int NT>
__device__ __forceinline__ void ql_epilogue(const QlKernelParams& p, uint8_t* smem, int warp, int lane, uint32_t tmem_base,
                                            int tile0, int nt_live, int split) {
  tc_fence_after();
  // every MMA has completed and every copy into the rings has been consumed: the ring memory is free
  float* stage = reinterpret_cast<float*>(smem + (size_t)(warp - QL_DQ_WARP0) * QL_EPI_STAGE_BYTES);
  const int q = warp & 3;                        // TMEM lane quarter this warp may read
  const int eg = (warp - QL_DQ_WARP0) >> 2;      // warps of one quarter split the 32-column chunks
  const int chunks = (p.m_pad + 31) >> 5;
  const int col_stride = (p.m_pad + 31) & ~31;
  const bool vec_ok = p.splits == 1 ? ((p.ldy & 3) == 0 && (reinterpret_cast<uintptr_t>(p.y) & 7) == 0)
                                    : ((p.N & 3) == 0 && (reinterpret_cast<uintptr_t>(p.partial) & 15) == 0);
  const int nl = 4 * (lane & 7), mr0 = lane >> 3;
  if (NT >= 2 && p.glu) {
    // tiles (2 pr, 2 pr + 1) of this CTA are the gate and up halves of features 128 * (tile0 / 2 + pr) ..:
    // both accumulators' values of a (feature, row) sit in the same thread, 16 rows at a time
    const int chunks16 = p.m_pad >> 4;
    for (int item = eg; item < (nt_live >> 1) * chunks16; item += QL_DQ_WARPS / 4) {
      const int pr = item / chunks16, ch = item - pr * chunks16;
      uint32_t g[16], u[16];
      tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (2 * pr) * col_stride + ch * 16, g);
      tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (2 * pr + 1) * col_stride + ch * 16, u);
      __syncwarp();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float gv = bf16_round(__uint_as_float(g[j])), uv = bf16_round(__uint_as_float(u[j]));
        stage[j * 32 + lane] = p.glu == 2 ? act_gelu_mul(gv, uv) : act_silu_mul(gv, uv);
      }
      __syncwarp();
      const int f = ((tile0 >> 1) + pr) * QL_TILE_N + q * 32 + nl;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int mr = 4 * k + mr0;
        const int m = ch * 16 + mr;
        if (m >= p.M) continue;
        const float4 v4 = *reinterpret_cast<const float4*>(stage + mr * 32 + nl);
        *reinterpret_cast<uint2*>(p.act + (size_t)(p.row0 + m) * p.ld_act + f) =
            make_uint2(pack_bf162(v4.x, v4.y), pack_bf162(v4.z, v4.w));
      }
    }
  } else
  for (int item = eg; item < nt_live * chunks; item += QL_DQ_WARPS / 4) {
    const int t = item / chunks, ch = item - t * chunks;
    const int col = (NT == 1 ? 0 : t * col_stride) + ch * 32;   // NT == 1: columns are m directly (incl. the 256+ accumulator)
    uint32_t v[32];
    tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + col, v);
    __syncwarp();                                // the previous item's reads of the buffer are done
#pragma unroll
    for (int j = 0; j < 32; ++j) stage[j * 32 + lane] = __uint_as_float(v[j]);   // stage[m][n]
    __syncwarp();
    const int n = (tile0 + t) * QL_TILE_N + q * 32 + nl;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int mr = 4 * k + mr0;
      const int m = ch * 32 + mr;
      if (m >= p.M || n >= p.N) continue;
      const float4 f = *reinterpret_cast<const float4*>(stage + mr * 32 + nl);
      if (p.splits == 1) {
        bf16* dst = p.y + (size_t)(p.row0 + m) * p.ldy + n;
        if (vec_ok && n + 3 < p.N) {
          *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf162(f.x, f.y), pack_bf162(f.z, f.w));
        } else {
          const float e[4] = {f.x, f.y, f.z, f.w};
          for (int c = 0; c < 4 && n + c < p.N; ++c) dst[c] = __float2bfloat16_rn(e[c]);
        }
      } else {
        float* dst = p.partial + ((size_t)split * p.part_M + p.part_row0 + m) * p.N + n;
        if (vec_ok && n + 3 < p.N) {
          *reinterpret_cast<float4*>(dst) = f;
        } else {
          const float e[4] = {f.x, f.y, f.z, f.w};
          for (int c = 0; c < 4 && n + c < p.N; ++c) dst[c] = e[c];
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// The kernel. The dequantised weights reach the tensor core through TENSOR MEMORY (tcgen05.mma with the A operand in
// TMEM), not through shared memory. Measured reason: an M = 128, N = 192 MMA needs 97 cycles when run alone, but a
// kernel that staged the bf16 weights in shared memory took about 1140 cycles per k-block of eight of them — its 154 KB
// of shared-memory traffic per k-block (32 KB of bf16 weights written, 32 KB read back by the MMAs, the activation
// k-block read once per tile, the copies) is what the 128 B/clk shared memory can move in that time. Here a
// dequantiser thread owns one weight row (= one TMEM lane) of one unit, expands its 64 weights in registers and writes
// them with one tcgen05.st (column c = weights 2c and 2c + 1), so the MMAs read only the activation k-block from shared
// memory and the A ring costs no shared memory at all. Units per stage are fixed at two: two tiles of one k-block
// (NT == 2), or two k-blocks of one tile (NT == 1; a split with an odd number of k-blocks ends with a one-unit
// stage). NT is free to depend on the row count: it changes which CTA computes an output element, never the order in
// which that element's k-blocks are accumulated.
//
// TMEM columns: [NT accumulators of round32(m_pad)] [a_stages x 2 units x 32 columns of bf16 pairs].
// ---------------------------------------------------------------------------
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t d_hi, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(d_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

template <int BITS, int GPK, int NT>
__global__ void __launch_bounds__(QL_THREADS, 1)
qlinear_umma_ta_kernel(const __grid_constant__ CUtensorMap map_rows, const QlKernelParams p) {
  constexpr int KC = NT == 1 ? 2 : 1;
  constexpr int UNITS = 2;
  static_assert(NT * KC == UNITS, "two units per stage");
  constexpr uint32_t PACKED = QL_TILE_N * (QL_KB * BITS / 8);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int SA = p.a_stages, SB = p.b_stages, RS = p.r_stages;
  const uint32_t bk_bytes = (uint32_t)p.m_pad * 128u;   // one activation k-block
  const uint32_t b_stage = KC * bk_bytes;
  const uint32_t r_stage = UNITS * p.raw_stride;
  uint8_t* sB = smem;
  uint8_t* sR = sB + (size_t)SB * b_stage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sR + (size_t)RS * r_stage);
  uint64_t* raw_full = bars;
  uint64_t* raw_empty = raw_full + RS;
  uint64_t* b_full = raw_empty + RS;
  uint64_t* b_empty = b_full + SB;
  uint64_t* a_ready = b_empty + SB;
  uint64_t* a_empty = a_ready + SA;
  uint64_t* acc_full = a_empty + SA;
  uint64_t* turn = acc_full + 1;                        // the two MMA issuers hand the issue order to each other through it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(turn + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile0 = blockIdx.x * NT, split = blockIdx.y;
  const int nt_live = min(NT, p.n_tiles - tile0);
  // splits may be uneven: split s takes k-blocks [K s / S, K (s + 1) / S) — a fixed function of the weight's shape
  const int kb0 = (int)((long long)p.kblocks * split / p.splits);
  const int nkb = (int)((long long)p.kblocks * (split + 1) / p.splits) - kb0;
  const int nst = (nkb + KC - 1) / KC;                  // pipeline stages of this CTA
  const int tail_kc = nkb - (nst - 1) * KC;             // k-blocks of the last stage (1 or KC)
  const int n_issuers = 1;   // a stage's MMAs are all issued (and its slots released) by one thread
  const uint32_t col_stride = (uint32_t)(p.m_pad + 31) & ~31u;
  const uint32_t a_col0 = NT * col_stride;              // first column of the A ring

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int i = 0; i < RS; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], QL_DQ_GROUP_WARPS); }
    for (int i = 0; i < SB; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], n_issuers); }
    for (int i = 0; i < SA; ++i) { mbar_init(&a_ready[i], QL_DQ_GROUP_WARPS); mbar_init(&a_empty[i], n_issuers); }
    mbar_init(acc_full, 2);   // both issuing threads commit to it after their last stage
    mbar_init(turn, 1);
    mbar_fence_init();
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp == 1 && lane == 0) tma_prefetch_desc(&map_rows);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp == 0) {
    // ---- weight record producer ----
    if (lane == 0) {
      RingPos rp;
      for (int i = 0; i < nst; ++i, rp.advance(RS)) {
        if (!mbar_wait(&raw_empty[rp.stage], rp.phase ^ 1, p.status, KC_DEV_QLINEAR | 1)) { ok = false; break; }
        const int kcs = i == nst - 1 ? tail_kc : KC;
        mbar_arrive_expect_tx(&raw_full[rp.stage], p.record_bytes * nt_live * kcs);
#pragma unroll
        for (int kc = 0; kc < KC; ++kc)
          if (kc < kcs)
          bulk_g2s(sR + (size_t)rp.stage * r_stage + (size_t)kc * NT * p.raw_stride,
                   p.records + (((size_t)(tile0 / QL_TILE_GROUP) * p.kblocks + kb0 + i * KC + kc) * QL_TILE_GROUP + tile0 % QL_TILE_GROUP) * p.record_bytes,
                   p.record_bytes * nt_live, &raw_full[rp.stage]);
      }
    }
  } else if (warp == 1) {
    // ---- activation producer: the first access of this kernel to memory written by earlier kernels ----
    if (lane == 0) {
      pdl_wait();
      RingPos bp;
      for (int i = 0; i < nst; ++i, bp.advance(SB)) {
        if (!mbar_wait(&b_empty[bp.stage], bp.phase ^ 1, p.status, KC_DEV_QLINEAR | 2)) { ok = false; break; }
        const int kcs = i == nst - 1 ? tail_kc : KC;
        mbar_arrive_expect_tx(&b_full[bp.stage], kcs * bk_bytes);
#pragma unroll
        for (int kc = 0; kc < KC; ++kc)
          if (kc < kcs)
          tma_load_2d(sB + (size_t)bp.stage * b_stage + (size_t)kc * bk_bytes, &map_rows, (kb0 + i * KC + kc) * QL_KB, p.row0,
                      &b_full[bp.stage]);
      }
    }
  } else if (warp == 2 || warp == 3) {
    // ---- MMA issuers: warp 2 takes the even stages, warp 3 the odd ones ----
    // Two issuing threads take alternate stages (all MMAs of a stage, both tiles): while one issues, the other is
    // already through the waits, the fence and the descriptor arithmetic of the next stage. The order in which the
    // MMAs enter the tensor pipe is handed over through `turn`: the issuer of stage i arrives on it after its last
    // MMA instruction, the issuer of stage i + 1 waits for that before its first.
    if (lane == 0) {
      pdl_wait();
      const int me = warp - 2;
      const uint32_t idesc = umma_idesc_bf16(QL_TILE_N, p.m_pad);
      const uint64_t proto = umma_smem_desc_sw128(0);
      const uint32_t d_hi = (uint32_t)(proto >> 32), d_lo = (uint32_t)proto;
      const uint32_t b_lo0 = d_lo | ((smem_u32(sB) >> 4) & 0x3FFF);
      const uint32_t b_step = b_stage >> 4;
      RingPos ap, bp;
      for (int i = 0; i < nst; ++i, ap.advance(SA), bp.advance(SB)) {
        if ((i & 1) != me) continue;
        if (!mbar_wait(&a_ready[ap.stage], ap.phase, p.status, KC_DEV_QLINEAR | 3)) { ok = false; break; }
        if (!mbar_wait(&b_full[bp.stage], bp.phase, p.status, KC_DEV_QLINEAR | 4)) { ok = false; break; }
        tc_fence_after();   // the A operand was written with tcgen05.st by other threads
        const uint32_t b_lo = b_lo0 + bp.stage * b_step;
        const uint32_t a_t = tmem_base + a_col0 + ap.stage * (UNITS * 32);
        const uint32_t acc = i > 0 ? 1u : 0u;
        if (i > 0 && !mbar_wait(turn, (uint32_t)(i - 1) & 1u, p.status, KC_DEV_QLINEAR | 8)) { ok = false; break; }
#pragma unroll
        for (int u = 0; u < UNITS; ++u) {
          if ((NT == 2 ? u < nt_live : true) && (NT == 2 || u == 0 || i < nst - 1 || tail_kc == KC)) {
            const int t = NT == 2 ? u : 0, kc = NT == 2 ? 0 : u;
            const uint32_t b_u = b_lo + kc * (bk_bytes >> 4);
#pragma unroll
            for (int ks = 0; ks < QL_KB / 16; ++ks)
              umma_bf16_ts(tmem_base + t * col_stride, a_t + u * 32 + 8 * ks, b_u + 2 * ks, d_hi, idesc,
                           (NT == 1 && u == 1) ? 1u : (ks == 0 ? acc : 1u));
          }
        }
        mbar_arrive(turn);
        umma_commit(&a_empty[ap.stage]);
        umma_commit(&b_empty[bp.stage]);
      }
      umma_commit(acc_full);
    }
  } else {
    // ---- dequantisers: thread = one weight row (TMEM lane 32 * (warp % 4) + lane) of one unit ----
    const int td = threadIdx.x - QL_DQ_WARP0 * 32;  // 0..511
    const int grp = td / QL_DQ_GROUP_THREADS;
    const int wj = (warp - QL_DQ_WARP0) & 7;        // warp inside the group; (wj & 3) == (warp & 3): the lane quarter
    const int unit = wj >> 2;
    const int row = (wj & 3) * 32 + lane;
    const bool live = NT == 1 || unit < nt_live;
    const uint32_t raw_off = (uint32_t)unit * p.raw_stride + row * (QL_KB * BITS / 8);
    const uint32_t sb_off = (uint32_t)unit * p.raw_stride + PACKED + row * GPK * 4;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    RingPos rp, ap;
    for (int g = 0; g < grp; ++g) { rp.advance(RS); ap.advance(SA); }
    bool released = false;
    for (int i = grp; i < nst && ok; i += QL_DQ_GROUPS) {
      // the first SA stages are dequantised under the tail of the previous kernel; a slot that is being reused is freed
      // by an MMA, which needs activations, which need the previous kernel: the bounded wait for it counts from there
      if (!released && i >= SA) { pdl_wait(); released = true; }
      ok = __all_sync(0xffffffffu, mbar_wait(&raw_full[rp.stage], rp.phase, p.status, KC_DEV_QLINEAR | 5));
      if (!ok) break;
      uint32_t v[32];
      const bool unit_live = live && (NT == 2 || unit == 0 || i < nst - 1 || tail_kc == KC);
      if (unit_live) {
        const uint8_t* rec = sR + (size_t)rp.stage * r_stage;
        bf162 sb[GPK];
#pragma unroll
        for (int g = 0; g < GPK; ++g) sb[g] = *reinterpret_cast<const bf162*>(rec + sb_off + g * 4);
        if (BITS == 4) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint4 q = *reinterpret_cast<const uint4*>(rec + raw_off + h * 16);
            const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const uint4 o = dequant8_w4(w4[c], sb[GPK == 2 ? h : 0]);
              v[(h * 4 + c) * 4 + 0] = o.x; v[(h * 4 + c) * 4 + 1] = o.y; v[(h * 4 + c) * 4 + 2] = o.z; v[(h * 4 + c) * 4 + 3] = o.w;
            }
          }
        } else {
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const uint4 q = *reinterpret_cast<const uint4*>(rec + raw_off + h * 16);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const uint4 o = dequant8_w8(c ? q.z : q.x, c ? q.w : q.y, sb[GPK == 2 ? (h >> 1) : 0]);
              v[(h * 2 + c) * 4 + 0] = o.x; v[(h * 2 + c) * 4 + 1] = o.y; v[(h * 2 + c) * 4 + 2] = o.z; v[(h * 2 + c) * 4 + 3] = o.w;
            }
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0u;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&raw_empty[rp.stage]);   // the record is in registers: its slot can refill
      ok = __all_sync(0xffffffffu, mbar_wait(&a_empty[ap.stage], ap.phase ^ 1, p.status, KC_DEV_QLINEAR | 6));
      if (!ok) break;
      tc_fence_after();
      tmem_st32(tmem_base + lane_addr + a_col0 + ap.stage * (UNITS * 32) + unit * 32, v);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_ready[ap.stage]);
#pragma unroll
      for (int g = 0; g < QL_DQ_GROUPS; ++g) { rp.advance(RS); ap.advance(SA); }
    }
    // ---- epilogue ----
    pdl_wait();   // the stores below may overwrite what an earlier kernel still reads
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(acc_full, 0, p.status, KC_DEV_QLINEAR | 7));
    if (ok) ql_epilogue<NT>(p, smem, warp, lane, tmem_base, tile0, nt_live, split);
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols)
                 : "memory");
  }
}

// Ring depths and shared memory of one launch geometry; ok == false when it does not fit tensor or shared memory.
struct TaPlan { bool ok; int sa, sb, rs; uint32_t tmem_cols; size_t smem; };
static TaPlan plan_ta(int nt, int m_pad, uint32_t raw_stride) {
  TaPlan t{};
  const int kc = nt == 1 ? 2 : 1;
  const int col_stride = (m_pad + 31) & ~31;
  const int acc_cols = nt * col_stride;
  int sa = (512 - acc_cols) / 64;            // two units of 32 columns per stage
  if (sa > 4) sa = 4;
  if (sa < 2 || m_pad > 256) return t;
  uint32_t cols = 32;
  while ((int)cols < acc_cols + sa * 64) cols <<= 1;
  const size_t budget = (size_t)212 * 1024;
  const size_t b_stage = (size_t)kc * m_pad * 128;
  const size_t rstage = (size_t)2 * raw_stride;
  if (budget < 6 * rstage + 2 * b_stage) return t;
  const int sb = (int)std::min<size_t>(4, (budget - 6 * rstage) / b_stage);
  int rs = (int)std::min<size_t>(24, (budget - (size_t)sb * b_stage) / rstage);
  if (sb < 2 || rs < 3) return t;
  // the epilogue's per-warp transpose buffers reuse the ring memory from its start
  while ((size_t)sb * b_stage + (size_t)rs * rstage < (size_t)QL_DQ_WARPS * QL_EPI_STAGE_BYTES) ++rs;
  const size_t smem = 1024 + (size_t)sb * b_stage + (size_t)rs * rstage + (2 * rs + 2 * sb + 2 * sa + 2) * 8 + 16;
  if (smem > 227 * 1024) return t;
  t.ok = true; t.sa = sa; t.sb = sb; t.rs = rs; t.tmem_cols = cols; t.smem = smem;
  return t;
}

template <int BITS, int GPK, int NT>
static cudaError_t launch_umma_ta(const QLinearLaunch& l, QlKernelParams& p, cudaStream_t s) {
  const QWeight& w = *l.w;
  const TaPlan t = plan_ta(NT, p.m_pad, p.raw_stride);
  if (!t.ok) return cudaErrorInvalidValue;   // the caller sized the row chunk with plan_ta
  p.tmem_cols = t.tmem_cols;
  p.a_stages = t.sa; p.b_stages = t.sb; p.r_stages = t.rs;
  static DeviceOnce configured;   // the attribute belongs to the device's copy of the kernel
  if (configured.first_on_current_device()) {
    cudaError_t e = cudaFuncSetAttribute(qlinear_umma_ta_kernel<BITS, GPK, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) { configured.forget_current_device(); return e; }
  }
  const CUtensorMap* rows = act_operand_rows_map(l.x, p.m_pad);
  if (!rows) return cudaErrorInvalidValue;
  p.b_single = 1;
  dim3 grid((w.n_tiles + NT - 1) / NT, w.splits);
  return launch_k(qlinear_umma_ta_kernel<BITS, GPK, NT>, grid, dim3(QL_THREADS), t.smem, s, *rows, p);
}

template <int BITS, int GPK>
static cudaError_t launch_umma_nt(const QLinearLaunch& l, QlKernelParams& p, int nt, cudaStream_t s) {
  return nt == 2 ? launch_umma_ta<BITS, GPK, 2>(l, p, s) : launch_umma_ta<BITS, GPK, 1>(l, p, s);
}

// Weight tiles per CTA: two when the grid then still has about 0.7 CTAs per SM (measured: 112 CTAs of two tiles beat
// 224 CTAs of one on 148 SMs — the activation k-block is read from L2 once per CTA), else one.
static int plan_tiles_per_cta(const QWeight& w, int sm_count) {
  return ((w.n_tiles + 1) / 2) * w.splits * 10 >= sm_count * 7 ? 2 : 1;
}

// The most rows one launch of this weight takes: what the accumulators (two tiles: 192 columns each, one tile: 256)
// and the rings of the weight's record size leave room for.
static int plan_row_cap(int nt, uint32_t raw_stride) {
  static const int caps[] = {256, 192, 128, 64, 32, 16};
  for (int c : caps)
    if (plan_ta(nt, c, raw_stride).ok) return c;
  return 0;
}

cudaError_t qlinear_umma(const QLinearLaunch& l, cudaStream_t s) {
  const QWeight& w = *l.w;
  if (l.M < 1 || l.M > QL_MAX_M) return cudaErrorInvalidValue;
  if (l.row0 % 16 || l.row0 + ((l.M + 15) & ~15) > l.x->rows) return cudaErrorInvalidValue;
  const int nt = plan_tiles_per_cta(w, w.sm_count);
  const int cap = plan_row_cap(nt, w.record_bytes);
  if (cap == 0) return cudaErrorInvalidValue;
  // the gated activation is fused when a CTA owns whole (gate, up) tile pairs and writes final values
  const bool glu = l.glu && nt == 2 && w.splits == 1 && (w.n_tiles & 1) == 0 && (w.N % (2 * QL_TILE_N)) == 0 && l.act &&
                   (l.ld_act & 3) == 0 && (reinterpret_cast<uintptr_t>(l.act) & 7) == 0;
  if (l.glu_done) *l.glu_done = glu ? 1 : 0;
  // equal row chunks (multiples of 16 rows): fewer accumulator columns per chunk leave more A stages
  const int chunks = (l.M + cap - 1) / cap;
  const int per = (((l.M + chunks - 1) / chunks) + 15) & ~15;
  for (int r0 = 0; r0 < l.M; r0 += per) {
    QlKernelParams p;
    p.records = w.records; p.record_bytes = w.record_bytes;
    p.N = w.N; p.n_tiles = w.n_tiles; p.kblocks = w.kblocks;
    p.M = std::min(per, l.M - r0); p.m_pad = (p.M + 15) & ~15; p.row0 = l.row0 + r0;
    p.splits = w.splits;
    p.raw_stride = w.record_bytes;
    p.y = l.y; p.ldy = l.ldy; p.partial = l.partial; p.part_M = l.M; p.part_row0 = r0; p.status = l.status;
    p.glu = glu ? l.glu : 0; p.act = l.act; p.ld_act = l.ld_act;
    cudaError_t e;
    if (w.bits == 4) e = w.gpk == 2 ? launch_umma_nt<4, 2>(l, p, nt, s) : launch_umma_nt<4, 1>(l, p, nt, s);
    else e = w.gpk == 2 ? launch_umma_nt<8, 2>(l, p, nt, s) : launch_umma_nt<8, 1>(l, p, nt, s);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

int qlinear_launches(const QWeight& w, int M) {
  const int nt = plan_tiles_per_cta(w, w.sm_count);
  const int cap = plan_row_cap(nt, w.record_bytes);
  return cap ? (M + cap - 1) / cap : 0;
}

// ---------------------------------------------------------------------------
// The weight-streaming lane: at most 8 activation rows (the draft model's chained decode forwards,
// crates/kiln-models/src/draft.rs:354-388). Such a launch is bound by the weight bytes alone, and the tensor-core
// kernel above spends most of its time setting up its pipelines. Here the weight is one flat list of units (one
// k-block of one group of four neighbouring tiles: contiguous in memory) that a grid of persistent CTAs cuts into equal
// contiguous runs; a producer warp bulk-copies a CTA's units through a shared-memory ring, and eight consumer warps,
// 16 rows of each of the four tiles apiece, multiply them with mma.sync.m16n8k16, the activation rows riding as the 8
// columns of the B operand (one activation fragment serves the four tiles).
//
// Arithmetic: MLX's row-vector class (its qmv kernels, which serve small batches there too): per quantisation group
// y += scale * sum_k(x_k q_k) + bias * sum_k(x_k) in fp32. The MMA runs on the raw integers (a 4-bit q enters as the
// bf16 value 128 + q, which one OR builds; the 128 is folded into the bias term), so nothing is dequantised per
// element. The 16 k positions of an MMA are assigned to the lanes so that lane (g, t) owns input features
// 32 h + 8 t .. + 7 of each 32-feature half h of the k-block — 4 contiguous bytes of a 4-bit row — and the activation
// fragment is gathered with the same assignment, so the sum runs over the same products.
//
// A run that crosses a group boundary flushes one partial per group it touches. The partials are fp32
// [pieces][M][N]; which CTA writes which piece of which group is a function of the weight's shape and the SM count
// only, and the consumer kernel sums the pieces in index order, so the result does not depend on timing or on M.
// ---------------------------------------------------------------------------

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int QG_CONSUMER_WARPS = 8;                       // x 16 weight rows = the 128 rows of a tile
constexpr int QG_THREADS = 32 * (QG_CONSUMER_WARPS + 1);   // + the producer warp
#ifndef QG_CTAS
#define QG_CTAS 2
#endif
constexpr int QG_CTAS_PER_SM = QG_CTAS;
constexpr int QG_MAX_PIECES = 40;                          // fp32 partials per output element, at most
constexpr int QG_MIN_UNITS = 4;                            // a CTA's run is at least this long (about 72 KB of 4-bit records)
constexpr int QG_MAX_STAGES = QG_CTAS == 3 ? 3 : 4;
constexpr size_t QG_RING_BYTES = QG_CTAS == 3 ? 60 * 1024 : 80 * 1024;

// One unit of work = the records of one k-block of a whole tile group (QL_TILE_GROUP neighbouring tiles, contiguous in
// memory): one bulk copy, one barrier round, one activation fragment for 4 x 128 weight rows.
struct QgParams {
  const uint8_t* records;
  uint32_t record_bytes;
  int N, n_groups, kblocks, pieces, stages;
  const bf16* x;   // [M, ldx]
  int ldx, M;
  float* partial;  // [pieces][M][N]
  uint32_t* status;
};

// The persistent CTA that owns unit r of T when G CTAs cut the list into runs [T c / G, T (c + 1) / G).
__host__ __device__ inline long long qg_owner(long long r, long long T, long long G) { return ((r + 1) * G + T - 1) / T - 1; }

// Elements (2p, 2p + 1), p = 0..3, of the lane's 8 features as bf16 pairs holding the raw integers.
template <int BITS>
__device__ __forceinline__ void qg_raw_pairs(const uint32_t* u, uint32_t (&e)[4]) {
  if (BITS == 4) {
    // The record's nibble order puts element 2p at bits 4p and element 2p + 1 at bits 16 + 4p. Two masks split the
    // word into bytes (even nibbles: elements 0, 4, 1, 5; odd nibbles: 2, 6, 3, 7), and a byte permute sets each
    // under 0x43: the bf16 value 128 + q, exact.
    const uint32_t lo = u[0] & 0x0F0F0F0Fu, hi = (u[0] >> 4) & 0x0F0F0F0Fu;
    e[0] = __byte_perm(lo, 0x43434343u, 0x4240u);   // elements 0, 1
    e[1] = __byte_perm(hi, 0x43434343u, 0x4240u);   // elements 2, 3
    e[2] = __byte_perm(lo, 0x43434343u, 0x4341u);   // elements 4, 5
    e[3] = __byte_perm(hi, 0x43434343u, 0x4341u);   // elements 6, 7
  } else {
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const uint32_t w = u[p >> 1];
      const int k = (p & 1) * 2;
      // byte k under the exponent of 2^23: the float 8388608 + q, minus 2^23 = q exactly; q < 256 is exact in bf16
      const float lo = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u | k)) - 8388608.f;
      const float hi = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u | (k + 1))) - 8388608.f;
      e[p] = pack_bf162(lo, hi);
    }
  }
}

template <int BITS, int GPK>
__global__ void __launch_bounds__(QG_THREADS, QG_CTAS_PER_SM) qlinear_stream_kernel(const QgParams p) {
  constexpr int ROW_BYTES = QL_KB * BITS / 8;          // bytes of one weight row in one k-block: 32 or 64
  constexpr int PACKED = QL_TILE_N * ROW_BYTES;
  constexpr int HALF_BYTES = ROW_BYTES / 2;            // one 32-feature half of a row
  constexpr int LANE_WORDS = BITS / 4;                 // 32-bit words holding the lane's 8 features of a half
  constexpr int NT = QL_TILE_GROUP;
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = p.stages;
  const uint32_t unit_bytes = NT * p.record_bytes;
  uint8_t* ring = smem;
  float* xs = reinterpret_cast<float*>(smem + (size_t)S * unit_bytes);               // [kblocks][GPK][8]
  uint64_t* full = reinterpret_cast<uint64_t*>(xs + (size_t)p.kblocks * GPK * 8);
  uint64_t* empty = full + S;
  const long long T = (long long)p.n_groups * p.kblocks, G = gridDim.x;
  const long long R0 = T * blockIdx.x / G, R1 = T * (blockIdx.x + 1) / G;
  const int n_units = (int)(R1 - R0);
  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], QG_CONSUMER_WARPS); }
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == QG_CONSUMER_WARPS) {
    // ---- producer: the weights do not depend on the kernels before this one, so it never waits for them ----
    if (lane == 0) {
      RingPos rp;
      int issued = 0;
      bool ok = true;
      const uint8_t* src = p.records + (size_t)R0 * unit_bytes;   // units are contiguous: [group][k-block][tile in group]
      for (int i = 0; i < n_units; ++i, rp.advance(S), src += unit_bytes) {
        if (!mbar_wait(&empty[rp.stage], rp.phase ^ 1, p.status, KC_DEV_QLINEAR | 0x11)) { ok = false; break; }
        mbar_arrive_expect_tx(&full[rp.stage], unit_bytes);
        bulk_g2s(ring + (size_t)rp.stage * unit_bytes, src, unit_bytes, &full[rp.stage]);
        ++issued;
      }
      if (!ok) {
        // gave up: the copies already issued still land in this CTA's shared memory; wait for them (bounded) before leaving
        RingPos dp;
        for (int i = 0; i < issued; ++i, dp.advance(S))
          if (i >= issued - S) mbar_wait(&full[dp.stage], dp.phase, p.status, KC_DEV_QLINEAR | 0x12);
      }
    }
  } else {
    // ---- consumers ----
    const int g = lane >> 2, t = lane & 3;
    const int r0 = warp * 16 + g;                      // this lane's weight rows in each tile: r0 and r0 + 8
    const bool x_live = g < p.M;
    const bf16* xr = p.x + (size_t)(x_live ? g : 0) * p.ldx + 8 * t;
    pdl_wait();   // x comes from the kernel before; the partials below may still be read by it
    // sum_k x_k per (k-block, group half, activation row) for the k-blocks of this CTA's run
    {
      const int n_kb = n_units < p.kblocks ? n_units : p.kblocks;
      for (int i = warp; i < n_kb; i += QG_CONSUMER_WARPS) {
        const int kb = (int)((R0 + i) % p.kblocks);
        float sh[2] = {0.f, 0.f};
        if (x_live) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint4 v = *reinterpret_cast<const uint4*>(xr + (size_t)kb * QL_KB + 32 * h);
            const float2 a = unpack_bf162(v.x), b = unpack_bf162(v.y), c = unpack_bf162(v.z), d = unpack_bf162(v.w);
            sh[h] = ((a.x + a.y) + (b.x + b.y)) + ((c.x + c.y) + (d.x + d.y));
          }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          sh[h] += __shfl_xor_sync(0xffffffffu, sh[h], 1);
          sh[h] += __shfl_xor_sync(0xffffffffu, sh[h], 2);
        }
        if (t == 0) {
          if (GPK == 2) { xs[((size_t)kb * 2 + 0) * 8 + g] = sh[0]; xs[((size_t)kb * 2 + 1) * 8 + g] = sh[1]; }
          else xs[(size_t)kb * 8 + g] = sh[0] + sh[1];
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(QG_CONSUMER_WARPS * 32) : "memory");
    }
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    int grp = (int)(R0 / p.kblocks), kb = (int)(R0 % p.kblocks);
    long long seg0 = R0;   // first unit of the current group's segment
    bool ok = true;
    RingPos rp;
    auto flush = [&](long long seg_end) {
      // acc[j][0], [1] = weight row r0 of tile j against activation rows 2t, 2t + 1; [2], [3] = row r0 + 8
      const long long t_first = (long long)grp * p.kblocks, t_last = t_first + p.kblocks - 1;
      const int c_first = (int)qg_owner(t_first, T, G);
      const int piece = (int)blockIdx.x - c_first;
      const int n_pieces = (int)qg_owner(t_last, T, G) - c_first + 1;
      const bool closes = seg_end == t_last + 1;       // the CTA holding a group's last unit also clears its unused slots
#pragma unroll
      for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int n = (grp * NT + j) * QL_TILE_N + r0 + 8 * h;
          if (n < p.N) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int m = 2 * t + e;
              if (m < p.M) {
                p.partial[((size_t)piece * p.M + m) * p.N + n] = acc[j][2 * h + e];
                if (closes)
                  for (int q = n_pieces; q < p.pieces; ++q) p.partial[((size_t)q * p.M + m) * p.N + n] = 0.f;
              }
            }
          }
        }
        acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
      }
    };
    const uint32_t lane_off = (uint32_t)r0 * ROW_BYTES + t * (4 * LANE_WORDS);
    const uint32_t sb_off = PACKED + (uint32_t)r0 * GPK * 4;
    // the activation fragment and the row sums of a unit are fetched one unit ahead
    uint4 xa[2], xa_next[2];
    float2 xsum[GPK], xsum_next[GPK];
    auto fetch_x = [&](int kbn, uint4 (&xv)[2], float2 (&sv)[GPK]) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        xv[h] = make_uint4(0, 0, 0, 0);
        if (x_live) xv[h] = *reinterpret_cast<const uint4*>(xr + (size_t)kbn * QL_KB + 32 * h);
      }
#pragma unroll
      for (int q = 0; q < GPK; ++q) sv[q] = *reinterpret_cast<const float2*>(xs + ((size_t)kbn * GPK + q) * 8 + 2 * t);
    };
    fetch_x(kb, xa_next, xsum_next);
    for (int i = 0; i < n_units; ++i, rp.advance(S)) {
      xa[0] = xa_next[0]; xa[1] = xa_next[1];
#pragma unroll
      for (int q = 0; q < GPK; ++q) xsum[q] = xsum_next[q];
      if (i + 1 < n_units) fetch_x(kb + 1 == p.kblocks ? 0 : kb + 1, xa_next, xsum_next);
      ok = __all_sync(0xffffffffu, mbar_wait(&full[rp.stage], rp.phase, p.status, KC_DEV_QLINEAR | 0x13));
      if (!ok) break;
      const uint8_t* unit = ring + (size_t)rp.stage * unit_bytes;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const uint8_t* rec = unit + (size_t)j * p.record_bytes;
        uint32_t u[2][2][LANE_WORDS];   // [half][row r0 / r0 + 8][words]
        uint32_t sbw[2][GPK];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const uint8_t* src = rec + lane_off + r * 8 * ROW_BYTES + h * HALF_BYTES;
            if (LANE_WORDS == 1) u[h][r][0] = *reinterpret_cast<const uint32_t*>(src);
            else { const uint2 v = *reinterpret_cast<const uint2*>(src); u[h][r][0] = v.x; u[h][r][LANE_WORDS - 1] = v.y; }
          }
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int q = 0; q < GPK; ++q) sbw[r][q] = *reinterpret_cast<const uint32_t*>(rec + sb_off + r * 8 * GPK * 4 + q * 4);
        float raw[2][4];   // one accumulator per 32-feature half: the two MMA chains are independent
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          raw[h][0] = raw[h][1] = raw[h][2] = raw[h][3] = 0.f;
          uint32_t e0[4], e1[4];
          qg_raw_pairs<BITS>(u[h][0], e0);
          qg_raw_pairs<BITS>(u[h][1], e1);
          mma_bf16_16816(raw[h], e0[0], e1[0], e0[2], e1[2], xa[h].x, xa[h].z);
          mma_bf16_16816(raw[h], e0[1], e1[1], e0[3], e1[3], xa[h].y, xa[h].w);
        }
        if (GPK == 1) {
#pragma unroll
          for (int c = 0; c < 4; ++c) raw[0][c] += raw[1][c];
        }
#pragma unroll
        for (int q = 0; q < GPK; ++q) {
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const float sc = __uint_as_float(sbw[r][q] << 16), bi = __uint_as_float(sbw[r][q] & 0xFFFF0000u);
            const float bc = BITS == 4 ? fmaf(-128.f, sc, bi) : bi;   // the 128 every 4-bit q carries
            acc[j][2 * r + 0] = fmaf(sc, raw[q][2 * r + 0], fmaf(bc, xsum[q].x, acc[j][2 * r + 0]));
            acc[j][2 * r + 1] = fmaf(sc, raw[q][2 * r + 1], fmaf(bc, xsum[q].y, acc[j][2 * r + 1]));
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[rp.stage]);   // the unit has been read: its slot can refill
      if (++kb == p.kblocks) {
        flush(R0 + i + 1);
        kb = 0; ++grp; seg0 = R0 + i + 1;
      }
    }
    if (ok && seg0 < R1) flush(R1);
  }
}

static int qg_groups(const QWeight& w) { return (w.n_tiles + QL_TILE_GROUP - 1) / QL_TILE_GROUP; }

// Persistent CTAs of the weight-streaming lane: a function of the weight's shape and the SM count only.
static int qg_ctas(const QWeight& w) {
  const long long T = (long long)qg_groups(w) * w.kblocks;
  // a run is at least QG_MIN_UNITS units, and long enough that a group's k-blocks spread over at most QG_MAX_PIECES
  // runs (each piece is one more fp32 partial the consumer kernel has to read)
  const long long run = std::max<long long>(QG_MIN_UNITS, (w.kblocks + QG_MAX_PIECES - 2) / (QG_MAX_PIECES - 1));
  return (int)std::max<long long>(1, std::min<long long>(T / run, (long long)QG_CTAS_PER_SM * w.sm_count));
}

int qlinear_stream_pieces(const QWeight& w) {
  const long long T = (long long)qg_groups(w) * w.kblocks, G = qg_ctas(w);
  int most = 1;
  for (int grp = 0; grp < qg_groups(w); ++grp) {
    const long long first = (long long)grp * w.kblocks;
    most = std::max(most, (int)(qg_owner(first + w.kblocks - 1, T, G) - qg_owner(first, T, G)) + 1);
  }
  return most;
}

template <int BITS, int GPK>
static cudaError_t launch_stream(const QgParams& p, int ctas, size_t smem, cudaStream_t s) {
  static DeviceOnce configured;
  if (configured.first_on_current_device()) {
    cudaError_t e = cudaFuncSetAttribute(qlinear_stream_kernel<BITS, GPK>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
    if (e != cudaSuccess) { configured.forget_current_device(); return e; }
  }
  return launch_k(qlinear_stream_kernel<BITS, GPK>, dim3(ctas), dim3(QG_THREADS), smem, s, p);
}

cudaError_t qlinear_stream(const QWeight& w, const bf16* x, int ldx, int M, float* partial, uint32_t* status, cudaStream_t s) {
  if (M < 1 || M > QL_STREAM_MAX_M || !partial) return cudaErrorInvalidValue;
  if ((ldx & 7) || (reinterpret_cast<uintptr_t>(x) & 15)) return cudaErrorInvalidValue;   // 16-byte activation loads
  QgParams p;
  p.records = w.records; p.record_bytes = w.record_bytes;
  p.N = w.N; p.n_groups = qg_groups(w); p.kblocks = w.kblocks; p.pieces = qlinear_stream_pieces(w);
  const size_t unit_bytes = (size_t)QL_TILE_GROUP * w.record_bytes;
  p.stages = (int)std::max<size_t>(2, std::min<size_t>(QG_MAX_STAGES, QG_RING_BYTES / unit_bytes));
  p.x = x; p.ldx = ldx; p.M = M; p.partial = partial; p.status = status;
  const size_t smem = (size_t)p.stages * unit_bytes + (size_t)w.kblocks * w.gpk * 8 * sizeof(float) + 2 * p.stages * sizeof(uint64_t);
  if (smem > 110 * 1024) return cudaErrorInvalidValue;
  const int ctas = qg_ctas(w);
  if (w.bits == 4) return w.gpk == 2 ? launch_stream<4, 2>(p, ctas, smem, s) : launch_stream<4, 1>(p, ctas, smem, s);
  return w.gpk == 2 ? launch_stream<8, 2>(p, ctas, smem, s) : launch_stream<8, 1>(p, ctas, smem, s);
}

// ---------------------------------------------------------------------------
// The small-weight lane of the same arithmetic: at most 8 rows against a weight of a few MB (the layers of a 1B-class
// draft model), where a launch is a chain of latencies and not a stream. One CTA = (tile, run of k-blocks); thread 0
// asks for ALL of the CTA's records with bulk copies onto one barrier before the kernel waits for its predecessor
// (weights depend on nothing), the activation slice of the run is staged once, and the eight warps (16 weight rows
// of the tile each) then work through records that are all resident, four at a time, with no ring and no hand-over.
// The k-blocks of a tile are cut into at most QV_MAX_PIECES runs — a function of the weight's shape and the SM count
// only — and leave fp32 partials [pieces][M][N] like the streaming kernel's, for the consumer kernel to sum in order.
// ---------------------------------------------------------------------------
constexpr int QV_WARPS = 8;
constexpr int QV_THREADS = QV_WARPS * 32;
constexpr int QV_MAX_PIECES = 8;
constexpr size_t QV_SMEM_BUDGET = 96 * 1024;   // two CTAs per SM

struct QvParams {
  const uint8_t* records;
  uint32_t record_bytes;
  int N, n_tiles, kblocks, c_used, kbper;
  const bf16* x;   // [M, ldx]
  int ldx, M;
  float* partial;  // [c_used][M][N]
  uint32_t* status;
  // Optional gated-activation operand: x is then not read; the activations are silu(gate) * up (gelu_approx for
  // glu == 2) of a gate_up output still in its fp32 partial form [gu_pieces][M][2 K] (K = this weight's input width).
  const float* gu;
  int gu_pieces, glu, gu_interleaved;
};

template <int BITS, int GPK>
__global__ void __launch_bounds__(QV_THREADS) qlinear_gemv_kernel(const QvParams p) {
  constexpr int ROW_BYTES = QL_KB * BITS / 8;
  constexpr int PACKED = QL_TILE_N * ROW_BYTES;
  constexpr int HALF_BYTES = ROW_BYTES / 2;
  constexpr int LANE_WORDS = BITS / 4;
  constexpr int RB = BITS == 4 ? 4 : 2;               // records whose loads and MMA chains overlap
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x / p.c_used, part = blockIdx.x - tile * p.c_used;
  const int kb0 = part * p.kbper, kb1 = min(p.kblocks, kb0 + p.kbper), nkb = kb1 - kb0;
  uint8_t* recs = smem;                                                     // [nkb][record_bytes]
  bf16* xs = reinterpret_cast<bf16*>(recs + (size_t)p.kbper * p.record_bytes);      // [8][kbper * 64]
  float* xsum = reinterpret_cast<float*>(xs + (size_t)8 * p.kbper * QL_KB);         // [kbper][GPK][8]
  uint64_t* bar = reinterpret_cast<uint64_t*>(xsum + (size_t)p.kbper * GPK * 8);   // one per batch of RB records
  const int n_batches = (nkb + RB - 1) / RB;
  if (threadIdx.x == 0) {
    for (int b = 0; b < n_batches; ++b) mbar_init(&bar[b], 1);
    mbar_fence_init();
    const uint8_t* src = p.records + ((size_t)(tile >> 2) * p.kblocks + kb0) * QL_TILE_GROUP * p.record_bytes + (size_t)(tile & 3) * p.record_bytes;
    for (int b = 0; b < n_batches; ++b) {
      const int in_batch = min(RB, nkb - b * RB);
      mbar_arrive_expect_tx(&bar[b], (uint32_t)in_batch * p.record_bytes);
      for (int i = b * RB; i < b * RB + in_batch; ++i, src += (size_t)QL_TILE_GROUP * p.record_bytes)
        bulk_g2s(recs + (size_t)i * p.record_bytes, src, p.record_bytes, &bar[b]);
    }
  }
  __syncthreads();
  pdl_wait();   // x comes from the kernel before; the partials below may still be read by it
  // the activation slice of this run, rows past M as zeros
  const int row_elems = p.kbper * QL_KB;
  for (int i = threadIdx.x; i < 8 * nkb * 8; i += QV_THREADS) {
    const int m = i / (nkb * 8), c8 = i - m * (nkb * 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (m < p.M) {
      if (!p.gu) {
        v = *reinterpret_cast<const uint4*>(p.x + (size_t)m * p.ldx + (size_t)kb0 * QL_KB + c8 * 8);
      } else {
        // Mlp::forward's activation (nn.rs:284-294) on the way in: the arithmetic of glu_from_kernel
        const int F = p.kblocks * QL_KB, col = kb0 * QL_KB + c8 * 8;
        const int gcol = p.gu_interleaved ? (col >> 7) * 256 + (col & 127) : col;
        const int ucol = p.gu_interleaved ? gcol + 128 : F + col;
        const float* base = p.gu + (size_t)m * 2 * F;
        float4 g0 = *reinterpret_cast<const float4*>(base + gcol), g1 = *reinterpret_cast<const float4*>(base + gcol + 4);
        float4 u0 = *reinterpret_cast<const float4*>(base + ucol), u1 = *reinterpret_cast<const float4*>(base + ucol + 4);
        for (int k = 1; k < p.gu_pieces; ++k) {
          const float* pk = base + (size_t)k * p.M * 2 * F;
          const float4 a = *reinterpret_cast<const float4*>(pk + gcol), b = *reinterpret_cast<const float4*>(pk + gcol + 4);
          const float4 c = *reinterpret_cast<const float4*>(pk + ucol), d = *reinterpret_cast<const float4*>(pk + ucol + 4);
          g0.x += a.x; g0.y += a.y; g0.z += a.z; g0.w += a.w; g1.x += b.x; g1.y += b.y; g1.z += b.z; g1.w += b.w;
          u0.x += c.x; u0.y += c.y; u0.z += c.z; u0.w += c.w; u1.x += d.x; u1.y += d.y; u1.z += d.z; u1.w += d.w;
        }
        const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w}, uv[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
        float a[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
          a[k] = p.glu == 2 ? act_gelu_mul(bf16_round(gv[k]), bf16_round(uv[k])) : act_silu_mul(bf16_round(gv[k]), bf16_round(uv[k]));
        v = make_uint4(pack_bf162(a[0], a[1]), pack_bf162(a[2], a[3]), pack_bf162(a[4], a[5]), pack_bf162(a[6], a[7]));
      }
    }
    *reinterpret_cast<uint4*>(xs + (size_t)m * row_elems + c8 * 8) = v;
    // the sum of x per (k-block, scale group, row) in the same pass: the 64 / GPK features of a group are the chunks of
    // 8 / GPK neighbouring threads (the loop's trip count is a multiple of 64, so a warp is in it whole or not at all)
    const float2 e0 = unpack_bf162(v.x), e1 = unpack_bf162(v.y), e2 = unpack_bf162(v.z), e3 = unpack_bf162(v.w);
    float sx = ((e0.x + e0.y) + (e1.x + e1.y)) + ((e2.x + e2.y) + (e3.x + e3.y));
    sx += __shfl_xor_sync(0xffffffffu, sx, 1);
    sx += __shfl_xor_sync(0xffffffffu, sx, 2);
    if (GPK == 1) sx += __shfl_xor_sync(0xffffffffu, sx, 4);
    if ((c8 & (8 / GPK - 1)) == 0) xsum[(size_t)((c8 >> 3) * GPK + ((c8 & 7) >> (GPK == 1 ? 3 : 2))) * 8 + m] = sx;
  }
  __syncthreads();
  const int g = lane >> 2, t = lane & 3;
  const int r0 = warp * 16 + g;
  const uint32_t lane_off = (uint32_t)r0 * ROW_BYTES + t * (4 * LANE_WORDS);
  const uint32_t sb_off = PACKED + (uint32_t)r0 * GPK * 4;
  const bf16* xrow = xs + (size_t)g * row_elems + 8 * t;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int kbl = 0; kbl < nkb; kbl += RB) {
    const int nb = nkb - kbl < RB ? nkb - kbl : RB;
    // the batch's records have landed (the later batches are still on their way: copy and arithmetic overlap)
    if (!__all_sync(0xffffffffu, mbar_wait(&bar[kbl / RB], 0, p.status, KC_DEV_QLINEAR | 0x21))) {
      // gave up: the copies may still land in this CTA's shared memory; one more bounded wait for each of them
      for (int b = kbl / RB; b < n_batches; ++b) mbar_wait(&bar[b], 0, nullptr, 0);
      return;
    }
    uint4 xa[RB][2];
    float2 xsv[RB][GPK];
    uint32_t u[RB][2][2][LANE_WORDS];
    uint32_t sbw[RB][2][GPK];
#pragma unroll
    for (int i = 0; i < RB; ++i) {
      const int kk = kbl + (i < nb ? i : 0);
      const uint8_t* rc = recs + (size_t)kk * p.record_bytes;
#pragma unroll
      for (int h = 0; h < 2; ++h) xa[i][h] = *reinterpret_cast<const uint4*>(xrow + kk * QL_KB + 32 * h);
#pragma unroll
      for (int q = 0; q < GPK; ++q) xsv[i][q] = *reinterpret_cast<const float2*>(xsum + (size_t)(kk * GPK + q) * 8 + 2 * t);
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const uint8_t* src = rc + lane_off + r * 8 * ROW_BYTES + h * HALF_BYTES;
          if (LANE_WORDS == 1) u[i][h][r][0] = *reinterpret_cast<const uint32_t*>(src);
          else { const uint2 v = *reinterpret_cast<const uint2*>(src); u[i][h][r][0] = v.x; u[i][h][r][LANE_WORDS - 1] = v.y; }
        }
#pragma unroll
      for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int q = 0; q < GPK; ++q) sbw[i][r][q] = *reinterpret_cast<const uint32_t*>(rc + sb_off + r * 8 * GPK * 4 + q * 4);
    }
    float raw[RB][2][4];
#pragma unroll
    for (int i = 0; i < RB; ++i) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        raw[i][h][0] = raw[i][h][1] = raw[i][h][2] = raw[i][h][3] = 0.f;
        uint32_t e0[4], e1[4];
        qg_raw_pairs<BITS>(u[i][h][0], e0);
        qg_raw_pairs<BITS>(u[i][h][1], e1);
        mma_bf16_16816(raw[i][h], e0[0], e1[0], e0[2], e1[2], xa[i][h].x, xa[i][h].z);
        mma_bf16_16816(raw[i][h], e0[1], e1[1], e0[3], e1[3], xa[i][h].y, xa[i][h].w);
      }
    }
    // the sums join the accumulator in k-block order: the result does not depend on RB
#pragma unroll
    for (int i = 0; i < RB; ++i) {
      if (i < nb) {
        if (GPK == 1) {
#pragma unroll
          for (int k = 0; k < 4; ++k) raw[i][0][k] += raw[i][1][k];
        }
#pragma unroll
        for (int q = 0; q < GPK; ++q) {
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const float sc = __uint_as_float(sbw[i][r][q] << 16), bi = __uint_as_float(sbw[i][r][q] & 0xFFFF0000u);
            const float bc = BITS == 4 ? fmaf(-128.f, sc, bi) : bi;   // the 128 every 4-bit q carries
            acc[2 * r + 0] = fmaf(sc, raw[i][q][2 * r + 0], fmaf(bc, xsv[i][q].x, acc[2 * r + 0]));
            acc[2 * r + 1] = fmaf(sc, raw[i][q][2 * r + 1], fmaf(bc, xsv[i][q].y, acc[2 * r + 1]));
          }
        }
      }
    }
  }
  // acc[0], [1] = weight row r0 against activation rows 2t, 2t + 1; [2], [3] = row r0 + 8
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int n = tile * QL_TILE_N + r0 + 8 * r;
    if (n < p.N) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int m = 2 * t + e;
        if (m < p.M) p.partial[((size_t)part * p.M + m) * p.N + n] = acc[2 * r + e];
      }
    }
  }
}

// The cut of a weight for the small-weight lane: runs of kbper k-blocks, c_used of them per tile.
struct QvPlan { bool ok; int c_used, kbper; size_t smem; };
static QvPlan qv_plan(const QWeight& w) {
  QvPlan q{false, 0, 0, 0};
  if (w.n_tiles < 1 || w.kblocks < 1) return q;
  const size_t per_kb = (size_t)w.record_bytes + 8 * QL_KB * sizeof(bf16) + (size_t)w.gpk * 8 * sizeof(float) + 8;   // + a barrier
  const int cap_kb = (int)((QV_SMEM_BUDGET - 64) / per_kb);
  if (cap_kb < 1) return q;
  // runs of about 8 k-blocks (a few microseconds of copy and arithmetic), fewer runs where the tiles alone fill the
  // SMs: every run is one more fp32 partial for the consumer kernel to read
  int c = std::max(1, std::min(QV_MAX_PIECES, w.kblocks / 8));
  c = std::min(c, std::max(1, 2 * w.sm_count / w.n_tiles));
  int kbper = std::min((w.kblocks + c - 1) / c, cap_kb);
  q.kbper = kbper;
  q.c_used = (w.kblocks + kbper - 1) / kbper;
  q.smem = (size_t)kbper * per_kb + 64;
  q.ok = q.c_used <= QV_MAX_PIECES;
  return q;
}

int qlinear_gemv_pieces(const QWeight& w) {
  const QvPlan q = qv_plan(w);
  return q.ok ? q.c_used : 0;
}

template <int BITS, int GPK>
static cudaError_t launch_gemv(const QvParams& p, int ctas, size_t smem, cudaStream_t s) {
  static DeviceOnce configured;
  if (configured.first_on_current_device()) {
    cudaError_t e = cudaFuncSetAttribute(qlinear_gemv_kernel<BITS, GPK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)QV_SMEM_BUDGET);
    if (e != cudaSuccess) { configured.forget_current_device(); return e; }
  }
  return launch_k(qlinear_gemv_kernel<BITS, GPK>, dim3(ctas), dim3(QV_THREADS), smem, s, p);
}

cudaError_t qlinear_gemv(const QWeight& w, const bf16* x, int ldx, int M, float* partial, uint32_t* status, cudaStream_t s,
                         const QvGatedInput* gated) {
  const QvPlan q = qv_plan(w);
  if (!q.ok || M < 1 || M > QL_STREAM_MAX_M || !partial) return cudaErrorInvalidValue;
  if (!gated && ((ldx & 7) || (reinterpret_cast<uintptr_t>(x) & 15))) return cudaErrorInvalidValue;   // 16-byte activation loads
  if (gated && (!gated->partial || gated->pieces < 1 || (reinterpret_cast<uintptr_t>(gated->partial) & 15) || (w.K & 127)))
    return cudaErrorInvalidValue;
  QvParams p;
  p.gu = gated ? gated->partial : nullptr; p.gu_pieces = gated ? gated->pieces : 0;
  p.glu = gated ? (gated->gelu ? 2 : 1) : 0; p.gu_interleaved = gated && gated->interleaved ? 1 : 0;
  p.records = w.records; p.record_bytes = w.record_bytes;
  p.N = w.N; p.n_tiles = w.n_tiles; p.kblocks = w.kblocks; p.c_used = q.c_used; p.kbper = q.kbper;
  p.x = x; p.ldx = ldx; p.M = M; p.partial = partial; p.status = status;
  const int ctas = w.n_tiles * q.c_used;
  if (w.bits == 4) return w.gpk == 2 ? launch_gemv<4, 2>(p, ctas, q.smem, s) : launch_gemv<4, 1>(p, ctas, q.smem, s);
  return w.gpk == 2 ? launch_gemv<8, 2>(p, ctas, q.smem, s) : launch_gemv<8, 1>(p, ctas, q.smem, s);
}

// ---------------------------------------------------------------------------
// Split-K reduction
// ---------------------------------------------------------------------------

// Pairs of neighbouring features go through 8-byte loads when every row of the partials and of y starts on the
// matching boundary (N, ldy even, bases aligned); otherwise one element per thread. The additions of an element are
// the same on both paths.
__global__ void qlinear_reduce_kernel(const float* __restrict__ partial, int splits, int M, int N,
                                      bf16* __restrict__ y, int ldy, int vec) {
  pdl_launch_dependents();
  pdl_wait();
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long first = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const size_t split_stride = (size_t)M * N;
  if (vec) {
    const long long total = (long long)M * N / 2;
    for (long long i = first; i < total; i += stride) {
      const long long e = i * 2;
      const int m = (int)(e / N), n = (int)(e % N);
      float2 acc = *reinterpret_cast<const float2*>(partial + e);
      for (int s = 1; s < splits; ++s) {
        const float2 v = *reinterpret_cast<const float2*>(partial + s * split_stride + e);
        acc.x += v.x; acc.y += v.y;
      }
      *reinterpret_cast<bf162*>(y + (size_t)m * ldy + n) = __floats2bfloat162_rn(acc.x, acc.y);
    }
  } else {
    const long long total = (long long)M * N;
    for (long long e = first; e < total; e += stride) {
      const int m = (int)(e / N), n = (int)(e % N);
      float acc = partial[e];
      for (int s = 1; s < splits; ++s) acc += partial[s * split_stride + e];
      y[(size_t)m * ldy + n] = __float2bfloat16_rn(acc);
    }
  }
}

// The reduction of ONE row fused with its raw arg-max (the head of a draft model's chained step, draft.rs:379-381:
// argmax of the logits row, lowest index on ties): every CTA sums its slice of the pieces in index order, rounds to
// bf16 (the head's output, also stored to y), keeps the best of its slice, and the CTA that finishes last — counted
// with one atomic per CTA, nobody waits — takes the best over the CTAs and stores the token. scratch: 2 floats per
// CTA followed by one counter word that is zero between launches (the last CTA resets it).
__global__ void __launch_bounds__(256) qlinear_reduce_argmax_kernel(const float* __restrict__ partial, int splits, int N,
                                                                    bf16* __restrict__ y, float* __restrict__ scratch,
                                                                    uint32_t* __restrict__ token) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float s_v[8];
  __shared__ int s_i[8];
  __shared__ bool s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  auto better = [](float av, int ai, float bv, int bi) { return bv > av || (bv == av && bi < ai); };
  float best_v = -INFINITY;
  int best_i = 0x7fffffff;
  for (int n = blockIdx.x * blockDim.x + threadIdx.x; n < N; n += gridDim.x * blockDim.x) {
    float acc = partial[n];
    for (int k = 1; k < splits; ++k) acc += partial[(size_t)k * N + n];
    const bf16 r = __float2bfloat16_rn(acc);
    y[n] = r;
    const float v = __bfloat162float(r);
    if (better(best_v, best_i, v, n)) { best_v = v; best_i = n; }
  }
  auto reduce_block = [&]() {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (better(best_v, best_i, ov, oi)) { best_v = ov; best_i = oi; }
    }
    if (lane == 0) { s_v[warp] = best_v; s_i[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
        if (better(best_v, best_i, s_v[w], s_i[w])) { best_v = s_v[w]; best_i = s_i[w]; }
    }
  };
  reduce_block();
  uint32_t* counter = reinterpret_cast<uint32_t*>(scratch + 2 * gridDim.x);
  if (threadIdx.x == 0) {
    scratch[2 * blockIdx.x] = best_v;
    scratch[2 * blockIdx.x + 1] = __int_as_float(best_i);
    __threadfence();
    s_last = atomicAdd(counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  best_v = -INFINITY; best_i = 0x7fffffff;
  for (int b = threadIdx.x; b < (int)gridDim.x; b += blockDim.x) {
    const float v = __ldcg(scratch + 2 * b);
    const int i = __float_as_int(__ldcg(scratch + 2 * b + 1));
    if (better(best_v, best_i, v, i)) { best_v = v; best_i = i; }
  }
  __syncthreads();   // s_v / s_i are reused
  reduce_block();
  if (threadIdx.x == 0) {
    *token = (uint32_t)best_i < (uint32_t)N ? (uint32_t)best_i : 0u;   // a row of NaNs has no maximum
    *counter = 0u;
  }
}

int qlinear_reduce_argmax_ctas(int N) { return std::max(1, std::min((N + 511) / 512, 296)); }

cudaError_t qlinear_reduce_argmax(const float* partial, int splits, int N, bf16* y, float* scratch, uint32_t* token, cudaStream_t s) {
  if (!partial || !y || !scratch || !token || splits < 1 || N < 1) return cudaErrorInvalidValue;
  return launch_k(qlinear_reduce_argmax_kernel, dim3(qlinear_reduce_argmax_ctas(N)), dim3(256), 0, s, partial, splits, N, y, scratch, token);
}

cudaError_t qlinear_reduce_splits(const float* partial, int splits, int M, int N, bf16* y, int ldy,
                                  cudaStream_t s) {
  const int vec = (N % 2 == 0 && ldy % 2 == 0 && (reinterpret_cast<uintptr_t>(partial) & 7) == 0 &&
                   (reinterpret_cast<uintptr_t>(y) & 3) == 0) ? 1 : 0;
  const long long total = vec ? (long long)M * N / 2 : (long long)M * N;
  const int threads = 256;
  const int blocks = (int)std::max<long long>(1, std::min<long long>((total + threads - 1) / threads, 148LL * 8));
  return launch_k(qlinear_reduce_kernel, dim3(blocks), dim3(threads), 0, s, partial, splits, M, N, y, ldy, vec);
}

}  // namespace kc

