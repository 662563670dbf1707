// Plain-old-data parameter blocks passed by value to the kernels.
#pragma once
#include <stdint.h>

namespace dsa {

// Sparse MLA forward.  All tensors contiguous row-major.
//   q        [B, S, H, D]            bf16 / fp16
//   kv       [B, S_kv, 1, D]         (or [num_blocks, block_size, 1, D] when block_table != null)
//   indices  [B, S, 1, topk] int32   (-1, >= kv_len, or beyond the causal limit = not taking part)
//   out      [B, S, H, DV]           same dtype as q
//   lse      [B, S, H] fp32          (nullable)
struct FwdParams {
  const void* q;
  const void* kv;
  const int32_t* indices;
  void* out;
  float* lse;
  int B, S, S_kv, H, topk, D, DV;
  int q_start;                 // absolute position of query 0 (used when q_start_b == null)
  int causal;                  // 1: key idx takes part only if idx <= q_start + t
  const int32_t* q_start_b;    // [B] per-sequence start position (act_kv - act_q), nullable
  const int32_t* kv_len_b;     // [B] per-sequence key count, nullable (default S_kv)
  const int32_t* q_len_b;      // [B] per-sequence query count, nullable (default S)
  const int32_t* block_table;  // [B, max_blocks] paged KV, nullable
  int block_size, max_blocks;
  float scale_log2;            // sm_scale * log2(e)
  int* status;                 // device status word (0 = ok)
  // Split-KV (tensor-core kernel only): with nsplit > 1 every (query, head block) is handled by nsplit work units, each
  // taking a contiguous share of the query's key tiles and writing a normalised partial result; a second kernel
  // combines them.  part_out [nsplit, B*S, H, DV] fp32, part_lse [nsplit, B*S, H] fp32 (natural log, -inf = no key).
  int nsplit;
  float* part_out;
  float* part_lse;
  // With nsplit > 1 and 0 < split_queries < B * S only the FIRST split_queries of the B * S queries (in memory order: the
  // ones a persistent kernel reaches last) are split; part_out / part_lse then hold nsplit x split_queries x H rows.  0 = all.
  int split_queries;
  // Key rows in two parts (SM-pair kernel, D = 576 / DV = 512 only): when kv_rope is set, kv holds rows of DV values (the
  // latent part) and kv_rope rows of D - DV values (the rope part), both addressed by the same row number -- the layout of
  // the dense MLA decode kernels' KV / K_pe tensors, which are then used in place instead of being concatenated first.
  const void* kv_rope;
#ifdef DSA_TRACE
  long long* trace;            // development builds only: clock samples of cluster 0, [2 CTAs][16 events][64 tiles]
#endif
};

// Sparse MLA backward: the forward's fields (out / lse hold the forward results) plus gradients.
struct BwdParams {
  FwdParams f;
  const void* d_out;  // [B, S, H, DV]
  void* d_q;          // [B, S, H, D]
  float* d_kv;        // fp32, same shape as kv, accumulated into
  float sm_scale;
};

// Lightning-indexer scores.  All tensors contiguous row-major.
//   q       [B, S1, N1, D]  bf16 / fp16
//   k       [B, S2, 1, D]
//   w       [B, S1, N1]     fp32
//   scores  [B, S1, S2]     fp32; entries at or beyond the row's limit are -inf
struct IndexerParams {
  const void* q;
  const void* k;
  const float* w;
  float* scores;
  int B, S1, S2, N1, D;
  int sparse_mode;            // 3: causal limit k < ak - aq + s1 + 1 (all keys if that is <= 0); 0: k < ak
  const int32_t* q_len_b;     // [B] actual query counts (nullable: S1)
  const int32_t* k_len_b;     // [B] actual key counts (nullable: S2)
  int32_t* limits;            // [B, S1] out, nullable: number of leading keys that are candidates per row
  int fill_masked;            // 1: also write -inf into tiles that lie entirely beyond the limit
  int* status;
  // paged keys (nullable): k is the cache [num_blocks, block_size, 1, D]; logical key j of batch b is row
  // block_table[b * max_blocks + j / block_size] * block_size + j % block_size; S2 is the largest logical length
  const int32_t* block_table;
  int block_size, max_blocks, num_blocks;
  int box_rows;               // set by the launcher: rows per TMA box of a paged cache
};

// Block-sparse indexer logits (HISA).
struct BlockSparseLogitsParams {
  const void* q;            // [S, H, D]
  const void* k;            // [S_kv, D]
  const int32_t* blocks;    // [S, topk]
  const void* w;            // [S, H], dtype w_dtype
  const int32_t* ks;        // [S]
  const int32_t* ke;        // [S]
  float* logits;            // [S, topk, block]
  int S, S_kv, H, D, block, topk;
  int w_dtype;              // 0 bf16, 1 fp16, 2 fp32
  // paged keys (nullable): k is [num_phys_blocks, block, 1, D]; logical block j of the sequence of query s sits at
  // block_table[(s / tokens_per_seq) * max_blocks + j]
  const int32_t* block_table;
  int max_blocks, tokens_per_seq;
  int* status;              // device status word (0 = ok)
};

}  // namespace dsa
