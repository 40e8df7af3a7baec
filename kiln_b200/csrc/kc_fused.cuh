// Row-wise / element-wise trunk ops and the sampling kernels. See kc_fused.cu, kc_sample.cu.
#pragma once

#include "kc_common.cuh"

namespace kc {

cudaError_t launch_embed(const uint32_t* w, const bf16* scales, const bf16* biases, const uint32_t* ids, int n, int H,
                         int bits, int group, float embed_scale, int vocab, bf16* out, cudaStream_t s);

// A GEMM output as its consumer reads it: bf16 [rows, ld], or the GEMM's fp32 split-K partials
// [splits][rows][ld] (summed in split order and rounded to bf16 by the consumer), or the bf16 outputs of the
// tensor-parallel ranks [ranks][rows][ld] (summed in rank order in fp32 and rounded once by the consumer), or nothing.
constexpr int KC_MAX_TP = 8;

struct SublayerOut {
  const bf16* y = nullptr;
  const float* part = nullptr;
  int splits = 0;
  size_t split_stride = 0;
  int ld = 0;
  const bf16* rank_y = nullptr;
  int ranks = 0;
  size_t rank_stride = 0;
  // Tensor-parallel peers: every rank's bf16 [rows, ld] output where it was written (this rank's own buffer and the
  // peers' buffers mapped into this process), read in place once flags[r] >= epoch for every rank r.
  const bf16* peer_y[KC_MAX_TP] = {};
  int peers = 0;
  const uint32_t* flags = nullptr;
  uint32_t epoch = 0;
  uint32_t* status = nullptr;
  // slice_w > 0: the peers' buffers hold ALREADY SUMMED column slices, [rows][slice_w] each, rank s owning columns
  // s * slice_w .. (the second phase of the two-phase exchange): the row is gathered, nothing is added.
  int slice_w = 0;
  static SublayerOut of_peer_slices(const bf16* const* peer_y, int peers, int ld, int slice_w, const uint32_t* flags, uint32_t epoch,
                                    uint32_t* status) {
    SublayerOut s = of_peers(peer_y, peers, ld, flags, epoch, status);
    s.slice_w = slice_w;
    return s;
  }
  static SublayerOut of_peers(const bf16* const* peer_y, int peers, int ld, const uint32_t* flags, uint32_t epoch, uint32_t* status) {
    SublayerOut s; s.peers = peers; s.ld = ld; s.flags = flags; s.epoch = epoch; s.status = status;
    for (int r = 0; r < peers; ++r) s.peer_y[r] = peer_y[r];
    return s;
  }
  static SublayerOut of_ranks(const bf16* rank_y, int ranks, size_t rows, int ld) {
    SublayerOut s; s.rank_y = rank_y; s.ranks = ranks; s.rank_stride = rows * (size_t)ld; s.ld = ld; return s;
  }
  static SublayerOut none() { return SublayerOut{}; }
  static SublayerOut dense(const bf16* y, int ld) { SublayerOut s; s.y = y; s.ld = ld; return s; }
  static SublayerOut partials(const float* part, int splits, size_t rows, int ld) {
    SublayerOut s; s.part = part; s.splits = splits; s.split_stride = rows * (size_t)ld; s.ld = ld; return s;
  }
};

// h = y ? bf16(x + (w_pre ? rms_norm(y, w_pre) : y)) : x ; normed = w_out ? rms_norm(h, w_out) : unused.
// row_map (optional) picks the input rows. h_out / normed may be null when not wanted.
cudaError_t launch_add_rmsnorm(const bf16* x, const SublayerOut& y, const bf16* w_pre, const bf16* w_out,
                               const int32_t* row_map, int rows, int H, float eps, bf16* h_out, bf16* normed,
                               cudaStream_t s);

cudaError_t launch_rope_kv_write(const SublayerOut& qkv, const bf16* bias, const float* inv_freq, const int32_t* token_pos,
                                 const int32_t* kv_slot, int n, int Hq, int Hkv, int D, int traditional, int layer,
                                 int NB, int BS, bf16* pool, bf16* q_out, cudaStream_t s);

// After the kernels before it on the stream have finished, stores `epoch` into slot `rank` of every rank's flag array
// (peer_flags[r] = rank r's array as mapped into this process): "this rank's output of exchange `epoch` is complete".
cudaError_t launch_tp_signal(uint32_t* const* peer_flags, int world, int rank, uint32_t epoch, cudaStream_t s);
// First phase of the two-phase exchange: once flags[r] >= epoch for every rank, sums column slice `rank` (slice_w
// columns from rank * slice_w) of every rank's bf16 [rows, H] output in rank order in fp32, rounds once and writes
// out[rows][slice_w].
cudaError_t launch_tp_reduce_slice(const bf16* const* peer_y, int world, int rank, int rows, int H, int slice_w, const uint32_t* flags,
                                   uint32_t epoch, uint32_t* status, bf16* out, cudaStream_t s);

cudaError_t launch_glu(const bf16* gu, int n, int F, int gelu, int interleaved, bf16* out, cudaStream_t s);
// The same over a GEMM output in its consumer form (gu.ld must be 2 F).
cudaError_t launch_glu_from(const SublayerOut& gu, int n, int F, int gelu, int interleaved, bf16* out, cudaStream_t s);
cudaError_t launch_softcap(bf16* x, long long total, float cap, cudaStream_t s);
cudaError_t launch_copy_block(bf16* pool, int layers, int NB, size_t block_elems, uint32_t src, uint32_t dst,
                              cudaStream_t s);

// Greedy token per logits row; see kc_greedy_rows in kiln_cuda.h.
cudaError_t launch_greedy_rows(const bf16* logits, int rows, int vocab, int normalize, uint32_t* tokens,
                               cudaStream_t s);
// tokens[i] = prev[feed[i]] where feed[i] >= 0: the device-side token feedback of kc_decode_launch.
cudaError_t launch_feed_tokens(uint32_t* tokens, const int32_t* feed, const uint32_t* prev, int n, int prev_n, cudaStream_t s);
// The settle walk per verify segment; see kc_verify_accept in kiln_cuda.h.
cudaError_t launch_verify_accept(const uint32_t* row_tokens, const int32_t* seq_row_offsets, const uint32_t* draft,
                                 const int32_t* draft_offsets, const int32_t* draft_len, int n_seqs, int max_commit,
                                 uint32_t* committed, int32_t* n_committed, int32_t* n_accepted, cudaStream_t s);

}  // namespace kc
