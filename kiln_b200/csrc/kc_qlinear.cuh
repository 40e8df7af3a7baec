// Affine-quantised linear layer: y[M, N] = x[M, K] · dequant(W)ᵀ.
//
// Replaces mlx_quantized_matmul(x, w, scales, biases, transpose=true, group,
// bits, "affine") as kiln calls it (crates/kiln-mlx/src/ops.rs:362-388;
// crates/kiln-models/src/nn.rs:79-102, 179-193).
//
// Device layout ("records"). At load the mlx tensors (u32 [N, K*bits/32],
// bf16 scales/biases [N, K/group]) are re-tiled so that everything one CTA
// needs for one k-block is ONE contiguous, 16-byte aligned run that a single
// bulk copy brings into shared memory:
//
//   record(tile t, kblock kb) = packed[128 rows][64*bits/8 bytes]   (stored in the order [t / 4][kb][t % 4])
//                             ++ sb[128 rows][gpk] as bf162 (scale, bias)
//
// with 128 output rows per tile, 64 input features per k-block and gpk =
// max(1, 64/group) groups per k-block (group 128: the pair is repeated for both
// k-blocks of the group). Rows past N are zero (scale = bias = 0 ⇒ w = 0).
// 4-bit words are nibble-permuted so that (u >> 4j) & 0x000F000F yields the
// element pair (2j, 2j+1) in bf162 order; 8-bit words keep mlx's byte order.
// Weights are dequantised to bf16 (w = bf16(q*scale + bias), one rounding) before
// the tensor core sees them — the arithmetic class of MLX's own dequantise-then-
// MMA kernels for wide batches, not of its fp32 row-vector kernels.
#pragma once

#include "kc_common.cuh"

namespace kc {

constexpr int QL_TILE_N = 128;  // output features per tile = UMMA M
constexpr int QL_KB = 64;       // input features per k-block = one 128-byte swizzle row of bf16
constexpr int QL_MAX_M = 512;   // activation rows per qlinear_umma call (one slab of the split-K workspace)
constexpr size_t QL_STREAM_MIN_BYTES = (size_t)24 << 20;  // records of a weight from which a model's small steps stream it
constexpr int QL_STREAM_MAX_M = 8;  // activation rows the weight-streaming lane takes (the 8 columns of one mma.sync)
constexpr int QL_TILE_GROUP = 4;  // tiles whose records are interleaved per k-block (the most one CTA owns)

struct QWeight {
  uint8_t* records = nullptr;  // [n_tiles][kblocks][record_bytes]
  int N = 0, K = 0, bits = 0, group = 0;
  int n_tiles = 0, kblocks = 0, gpk = 0;
  uint32_t packed_bytes = 0;   // per record
  uint32_t record_bytes = 0;
  int splits = 1;              // fixed function of (N, K): never of M
  int sm_count = 148;
  size_t bytes() const { return (size_t)((n_tiles + QL_TILE_GROUP - 1) / QL_TILE_GROUP) * QL_TILE_GROUP * kblocks * record_bytes; }
  // Algorithmic bytes of the mlx tensors this weight was built from.
  size_t mlx_bytes() const { return (size_t)N * K * bits / 8 + (size_t)2 * N * (K / group) * 2; }
};

// Activation operand: a bf16 [rows, K] row-major device buffer plus the two
// tensor maps (16-row and 64-row boxes of 64 features, 128-byte swizzle) the
// TMA loads use.
struct ActOperand {
  const bf16* ptr = nullptr;
  int rows = 0;  // allocated rows (multiple of 16)
  int K = 0;
  CUtensorMap map16;
  CUtensorMap map64;
  mutable CUtensorMap rows_map;   // box of rows_map_n rows: one TMA operation per k-block while the row count is stable
  mutable int rows_map_n = 0;
};

struct QLinearLaunch {
  const QWeight* w;
  const ActOperand* x;
  int row0;         // first activation row of this launch (x, y and partial are indexed from it)
  int M;            // live activation rows, 1..QL_MAX_M
  bf16* y;          // [M, ldy] bf16 when the weight has splits == 1 (else unused)
  int ldy;
  float* partial;   // [splits][M][N] fp32 workspace when splits > 1 (rows relative to row0)
  uint32_t* status; // device status word
  // Optional fused gated activation for a weight whose 128-row tiles alternate gate / up (tile 2j = gate features
  // 128 j.., tile 2j + 1 = the matching up features): glu = 1 (silu) or 2 (gelu_approx) asks the epilogue to write
  // act[M, N / 2] = activation(gate) * up instead of y. Honoured only when one CTA owns whole gate/up tile pairs and
  // K is not split; *glu_done then is set to 1, otherwise y is written as usual and *glu_done is 0.
  int glu = 0;
  bf16* act = nullptr;
  int ld_act = 0;
  int* glu_done = nullptr;
};

// Fixed split-K plan: a function of the weight's shape only, so a row's
// accumulation order never depends on how many rows ride the step.
int qlinear_plan_splits(int n_tiles, int kblocks, int sm_count);

// Re-tile on the device. w/scales/biases are device pointers in mlx layout.
cudaError_t qweight_build(QWeight* out, const uint32_t* w, const bf16* scales, const bf16* biases,
                          int N, int K, int bits, int group, int sm_count, cudaStream_t s);
void qweight_free(QWeight* w);

// Creates the tensor maps of an activation buffer. Returns false (and sets
// *err) if the driver entry point is unavailable or rejects the geometry.
bool act_operand_init(ActOperand* op, const bf16* ptr, int rows, int K, const char** err);

// The GEMM (tcgen05 + TMEM + TMA). Returns a CUDA error. A launch of more rows than the accumulators hold (192 with
// two weight tiles per CTA, 256 with one) is issued as several kernels over equal row chunks.
cudaError_t qlinear_umma(const QLinearLaunch& l, cudaStream_t s);
// Kernels qlinear_umma issues for M rows of this weight.
int qlinear_launches(const QWeight& w, int M);

// The weight-streaming lane for at most QL_STREAM_MAX_M rows: x bf16 [M, ldx] against dequant(W)^T, left as fp32
// partials [qlinear_stream_pieces(w)][M][N] that the caller's consumer kernel (or qlinear_reduce_splits) sums in index
// order. MLX's row-vector arithmetic class: scale and bias are applied per group to fp32 sums of x q and of x.
int qlinear_stream_pieces(const QWeight& w);
cudaError_t qlinear_stream(const QWeight& w, const bf16* x, int ldx, int M, float* partial, uint32_t* status, cudaStream_t s);

// The same arithmetic for a weight of a few MB (a draft model's layers): one CTA per (tile, run of k-blocks), all of
// its records requested at once. Partials [qlinear_gemv_pieces(w)][M][N]; 0 pieces = the weight's shape does not fit
// the lane (the caller keeps another one).
int qlinear_gemv_pieces(const QWeight& w);
// gated (optional): the activations are not read from x but computed on the way in as silu(gate) * up (gelu_approx
// with gelu) from a gate_up output in its fp32 partial form [pieces][M][2 K] — the down projection of an MLP whose
// gate_up went through one of the fp32-partial lanes, without a separate activation kernel.
struct QvGatedInput { const float* partial; int pieces; bool gelu, interleaved; };
cudaError_t qlinear_gemv(const QWeight& w, const bf16* x, int ldx, int M, float* partial, uint32_t* status, cudaStream_t s,
                         const QvGatedInput* gated = nullptr);

// One row: y[n] = bf16(sum over pieces of partial[k][n]) and *token = arg-max of that row (lowest index on ties), in
// one launch. scratch: 2 * qlinear_reduce_argmax_ctas(N) floats followed by one zeroed 32-bit counter (left zero).
int qlinear_reduce_argmax_ctas(int N);
cudaError_t qlinear_reduce_argmax(const float* partial, int splits, int N, bf16* y, float* scratch, uint32_t* token, cudaStream_t s);

// out[m, n] = bf16(sum over splits of partial[s][m][n]) in split order.
cudaError_t qlinear_reduce_splits(const float* partial, int splits, int M, int N, bf16* y, int ldy,
                                  cudaStream_t s);

}  // namespace kc
