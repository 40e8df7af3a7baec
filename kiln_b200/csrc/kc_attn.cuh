// Paged multi-query attention: launch parameters. See kc_attn.cu.
#pragma once

#include "kc_common.cuh"

namespace kc {

// Keys per chunk. Chunks are cut at absolute key positions, so the partition a
// query row sees depends only on its own position.
#ifndef ATT_CHUNK_KEYS
#define ATT_CHUNK_KEYS 512
#endif
constexpr int ATT_CHUNK = ATT_CHUNK_KEYS;

struct AttnParams {
  const bf16* q;               // [n_tokens, Hq, D] post-RoPE
  bf16* out;                   // [n_tokens, Hq * D]
  float* part_o;               // [n_tokens * Hq][max_chunks][D]  un-normalised partial outputs
  float2* part_ml;             // [n_tokens * Hq][max_chunks]     (running max in log2 units, sum)
  const int32_t* block_tables; // [n_seqs][max_blocks]
  const int4* work;            // [n_work] {seq, first token row, tokens, absolute position of first token}
  const int32_t* token_pos;    // [n_tokens] absolute position of each token row
  uint32_t* status;
  int max_blocks;
  int Hq, Hkv, gqa;
  int layer, NB, BS;
  int max_chunks;
  int single_chunk;            // 1: max_chunks == 1, the partial kernel writes `out` itself and no combine kernel follows
  int chunk_lo_grid;           // chunk index of blockIdx.x == 0
  float scale;                 // softmax scale (applied to fp32 scores)
  float softcap;               // 0 = off
  int window;                  // 0 = global
  const bf16* pool;            // K/V pools: [layers][2][NB][Hkv][BS][head_dim]
  int kv4d;                    // kvmap is the 4-D map (one operation per K+V tile pair) instead of the 2-D one
};

// Tokens of one sequence that share a CTA (their rows x gqa must fit 64 rows).
int attn_tokens_per_item(int gqa, int max_len);

// kvmap: 2-D tensor map over all pool rows ([layers*2*NB*Hkv*BS, D] bf16, box {64, 16}, 128-byte swizzle), or, with
// p.kv4d, the 4-D map of make_tmap_kv_4d. n_work CTAs in z, grid_chunks in x.
cudaError_t paged_attention(const CUtensorMap& kvmap, const AttnParams& p, int head_dim, int tokens_per_item,
                            int n_work, int grid_chunks, int n_tokens, cudaStream_t s);

}  // namespace kc
