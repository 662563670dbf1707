// Block-sparse indexer logits (HISA): for every query, the lightning-indexer score of the keys of its selected KV blocks,
//   logits[q, j, b] = sum_h w[q, h] * relu(q[q, h, :] . k[blk[q, j] * block + b, :]),
// -inf for positions outside the key tensor or outside the query's [ks, ke) range.  Semantics follow
// ref_block_sparse_mqa_attn (examples/HISA/block_sparse_mqa_attn_expert_test.py:548-587) and the kernel
// block_sparse_mqa_attn_return_logits (:24-545).
//
// CUDA-core fp32 kernel: one CTA per (query, group of 4 selected blocks); the query's heads sit in shared memory as fp32,
// a lane owns one key (its row is read once, 8 dims at a time) and keeps one accumulator per head in registers, so the
// head sum needs no cross-lane traffic and a warp writes 32 consecutive logits.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "params.h"

namespace dsa {

namespace bsl {
constexpr int kMaxH = 64, kMaxD = 256, kBlocksPerCta = 4, kThreads = 256;
}

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = static_cast<float>(e[i]);
}

template <typename T>
__global__ void __launch_bounds__(bsl::kThreads) block_sparse_logits_kernel(const BlockSparseLogitsParams p) {
  using namespace bsl;
  extern __shared__ __align__(16) float smem_f[];
  float* sq = smem_f;                 // [H][D]
  float* sw = smem_f + p.H * p.D;     // [H]
  const int qi = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const T* qrow = reinterpret_cast<const T*>(p.q) + static_cast<int64_t>(qi) * p.H * p.D;
  for (int i = tid; i < p.H * p.D; i += kThreads) sq[i] = static_cast<float>(qrow[i]);
  for (int h = tid; h < p.H; h += kThreads) {
    const int64_t wi = static_cast<int64_t>(qi) * p.H + h;
    sw[h] = p.w_dtype == 2 ? reinterpret_cast<const float*>(p.w)[wi]
            : p.w_dtype == 0 ? static_cast<float>(reinterpret_cast<const __nv_bfloat16*>(p.w)[wi])
                             : static_cast<float>(reinterpret_cast<const __half*>(p.w)[wi]);
  }
  __syncthreads();
  const int lo = p.ks[qi], hi = p.ke[qi];
  const int chunks = (p.block + 31) / 32;
  const int j0 = blockIdx.y * kBlocksPerCta;
  for (int item = warp; item < kBlocksPerCta * chunks; item += kThreads / 32) {
    const int j = j0 + item / chunks, c = item % chunks;
    if (j >= p.topk) break;
    const int off = c * 32 + lane;
    const int blk = p.blocks[static_cast<int64_t>(qi) * p.topk + j];
    const int64_t pos = static_cast<int64_t>(blk) * p.block + off;   // logical position
    const bool in_block = off < p.block;
    bool valid = in_block && blk >= 0 && (p.block_table ? blk < p.max_blocks : pos < p.S_kv) && pos >= lo && pos < hi;
    int64_t row = pos;
    if (valid && p.block_table) {
      // the table is read only for positions that take part (entries past a sequence's context are padding), and a
      // physical block outside the cache is not dereferenced
      const int phys = p.block_table[static_cast<int64_t>(qi / p.tokens_per_seq) * p.max_blocks + blk];
      valid = phys >= 0 && (static_cast<int64_t>(phys) + 1) * p.block <= p.S_kv;
      row = static_cast<int64_t>(phys) * p.block + off;
    }
    if (!valid) row = 0;
    float acc[kMaxH];
#pragma unroll
    for (int h = 0; h < kMaxH; ++h) acc[h] = 0.f;
    if (valid) {
      const uint4* krow = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.k) + row * p.D);
      for (int d0 = 0; d0 < p.D; d0 += 8) {
        float kf[8];
        unpack8<T>(__ldg(krow + (d0 >> 3)), kf);
#pragma unroll
        for (int h = 0; h < kMaxH; ++h) {
          if (h < p.H) {
            const float4 a = *reinterpret_cast<const float4*>(sq + h * p.D + d0);
            const float4 b = *reinterpret_cast<const float4*>(sq + h * p.D + d0 + 4);
            acc[h] += a.x * kf[0] + a.y * kf[1] + a.z * kf[2] + a.w * kf[3] + b.x * kf[4] + b.y * kf[5] + b.z * kf[6] + b.w * kf[7];
          }
        }
      }
    }
    float total = 0.f;
#pragma unroll
    for (int h = 0; h < kMaxH; ++h)
      if (h < p.H) total += sw[h] * fmaxf(acc[h], 0.f);
    if (in_block) p.logits[(static_cast<int64_t>(qi) * p.topk + j) * p.block + off] = valid ? total : -INFINITY;
  }
}

bool block_sparse_logits_supported(const BlockSparseLogitsParams& p) {
  return p.H >= 1 && p.H <= bsl::kMaxH && p.D >= 8 && p.D <= bsl::kMaxD && p.D % 8 == 0;
}

int launch_block_sparse_logits(const BlockSparseLogitsParams& p, bool bf16, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(p.H) * p.D * 4 + static_cast<size_t>(p.H) * 4;
  dim3 grid(static_cast<unsigned>(p.S), static_cast<unsigned>((p.topk + bsl::kBlocksPerCta - 1) / bsl::kBlocksPerCta));
  cudaError_t e;
  if (bf16) {
    e = cudaFuncSetAttribute(block_sparse_logits_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    block_sparse_logits_kernel<__nv_bfloat16><<<grid, bsl::kThreads, smem, stream>>>(p);
  } else {
    e = cudaFuncSetAttribute(block_sparse_logits_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    block_sparse_logits_kernel<__half><<<grid, bsl::kThreads, smem, stream>>>(p);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace dsa

// -------------------------------------------------------------------------------------------------
// tcgen05 kernel: blocks of 128 keys, index_dim 128, up to 64 heads
// -------------------------------------------------------------------------------------------------
// One CTA per query (two resident per SM).  A selected block is one UMMA tile: A = its 128 keys x 128 dims (two
// K-major chunks of 64 dims in the 128-byte swizzle, fetched with two TMA tile loads per block -- a selected block is 128
// consecutive rows of k -- into a 2-stage ring; row by row with cp.async when no tensor map can be made), B = the
// query's heads x 128 dims (loaded once, rows beyond the head count are zero), D = 128 keys x 64 heads fp32 in one of two
// tensor-memory buffers.  The epilogue thread of a key reads its 64 head scores, applies ReLU and the head weights and
// writes one logit; a warp writes 32 consecutive logits.
#include <stdlib.h>
#include <string.h>

#include "ptx.cuh"
#include "tensor_map.h"

namespace dsa {
namespace bsltc {
constexpr int kKeys = 128, kDim = 128, kHeads = 64, kStages = 2, kThreads = 288;
constexpr uint32_t kChunk = kKeys * 128;                  // 128 keys x 64 dims
constexpr uint32_t kStageBytes = 2 * kChunk;              // 32 KB
constexpr uint32_t kOffQ = kStages * kStageBytes;         // B operand: two chunks of [64 heads x 128 B]
constexpr uint32_t kOffBar = kOffQ + 2 * kHeads * 128;
constexpr uint32_t kOffW = kOffBar + 128;
constexpr uint32_t kSmemBytes = kOffW + kHeads * 4 + 1024;
static_assert(2 * kSmemBytes <= 232448 - 2048, "two CTAs per SM");
}  // namespace bsltc

template <bool kBF16>
__global__ void __launch_bounds__(bsltc::kThreads, 2)
    block_sparse_logits_tc_kernel(const __grid_constant__ BlockSparseLogitsParams p, const __grid_constant__ CUtensorMap kmap, const int use_tma) {
  using namespace bsltc;
  using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sBase = smem_u32(smem), sQ = sBase + kOffQ;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
  uint64_t* full = bars;          // [2] count 128: the block's rows landed (and were made visible to the tensor core's proxy)
  uint64_t* empty = bars + 3;     // [2] count 1: commit after the MMAs of the stage
  uint64_t* d_full = bars + 6;    // [2] count 1: commit after the MMAs of a block
  uint64_t* d_free = bars + 8;    // [2] count 4: the epilogue warps have read the buffer
  uint64_t* q_ready = bars + 10;  // count 128
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  float* sw = reinterpret_cast<float*>(smem + kOffW);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, qi = blockIdx.x;
  // a failed wait records its status in the device status word and ends the CTA's loops; launches that find the word set exit
  __shared__ int s_start_status;
  if (tid == 0) s_start_status = *reinterpret_cast<volatile int*>(p.status);
  __syncthreads();
  if (s_start_status != kStatusOk) return;
  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) { mbar_init(&full[i], use_tma ? 1 : 128); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&d_full[i], 1); mbar_init(&d_free[i], 4); }
    mbar_init(q_ready, 128);
    mbar_init_fence();
  }
  for (int h = tid; h < kHeads; h += kThreads) {
    float v = 0.f;
    if (h < p.H) {
      const int64_t wi = static_cast<int64_t>(qi) * p.H + h;
      v = p.w_dtype == 2 ? reinterpret_cast<const float*>(p.w)[wi]
          : p.w_dtype == 0 ? static_cast<float>(reinterpret_cast<const __nv_bfloat16*>(p.w)[wi])
                           : static_cast<float>(reinterpret_cast<const __half*>(p.w)[wi]);
    }
    sw[h] = v;
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tD = *tmem_slot;
  const int32_t* blocks = p.blocks + static_cast<int64_t>(qi) * p.topk;
  bool ok = true;

  if (warp >= 4 && warp < 8) {
    // ================================ loaders: thread = key row of every block ======================
    const int r = tid - 128;
    const int lo = p.ks[qi], hi = p.ke[qi];
    {  // the query's heads: thread r < 64 copies head r (256 bytes), rows without a head are zero-filled
      if (r < kHeads) {
        const uint8_t* qrow = reinterpret_cast<const uint8_t*>(p.q) + (static_cast<int64_t>(qi) * p.H + (r < p.H ? r : 0)) * (kDim * 2);
#pragma unroll
        for (int u = 0; u < 16; ++u) cp_async16(sQ + (u >> 3) * (kHeads * 128) + sw128_offset(r, u & 7), qrow + u * 16, r < p.H ? 16u : 0u);
      }
      cp_async_commit();
      cp_async_wait<0>();
      fence_proxy_async_smem();
      mbar_arrive(q_ready);
    }
    if (use_tma) {
      // One thread: a block of which at least one logit is kept is fetched whole with two tile loads (rows outside [ks, ke)
      // or beyond the key tensor -- which read as zeros -- only produce logits that the epilogue replaces by -inf); a block
      // of which nothing is kept is not fetched at all (its stage holds stale data, all its logits are -inf).
      if (r == 0) {
        prefetch_tensormap(&kmap);
        for (int j = 0; j < p.topk; ++j) {
          const int s = j % kStages;
          const int blk = blocks[j];
          const int64_t first = static_cast<int64_t>(blk) * kKeys;
          bool fetch = blk >= 0 && (p.block_table ? blk < p.max_blocks : first < p.S_kv) && first + kKeys > lo && first < hi;
          int64_t row0 = first;
          if (fetch && p.block_table) {
            const int phys = p.block_table[static_cast<int64_t>(qi / p.tokens_per_seq) * p.max_blocks + blk];
            fetch = phys >= 0 && (static_cast<int64_t>(phys) + 1) * kKeys <= p.S_kv;
            row0 = static_cast<int64_t>(phys) * kKeys;
          }
          if (j >= kStages && !mbar_wait(&empty[s], ((j / kStages) + 1) & 1, p.status)) { ok = false; break; }
          if (fetch) {
            const uint32_t stage = sBase + s * kStageBytes, fb = smem_u32(&full[s]);
            mbar_arrive_expect_tx(&full[s], kStageBytes);
            tma_load_2d(stage, &kmap, fb, 0, static_cast<int>(row0));
            tma_load_2d(stage + kChunk, &kmap, fb, 64, static_cast<int>(row0));
          } else {
            mbar_arrive(&full[s]);
          }
        }
      }
    } else {
    for (int j = 0; j < p.topk && ok; ++j) {
      const int s = j % kStages;
      const int blk = blocks[j];
      const int64_t pos = static_cast<int64_t>(blk) * kKeys + r;
      // a row is fetched only if its logit is kept: inside the key tensor / block table AND inside [ks, ke).  Table entries of
      // blocks past a sequence's context are padding and are not read; a physical block outside the cache is not dereferenced.
      bool in_range = blk >= 0 && (p.block_table ? blk < p.max_blocks : pos < p.S_kv) && pos >= lo && pos < hi;
      int64_t row = pos;
      if (in_range && p.block_table) {
        const int phys = p.block_table[static_cast<int64_t>(qi / p.tokens_per_seq) * p.max_blocks + blk];
        in_range = phys >= 0 && (static_cast<int64_t>(phys) + 1) * kKeys <= p.S_kv;
        row = static_cast<int64_t>(phys) * kKeys + r;
      }
      if (!in_range) row = 0;
      const uint8_t* krow = reinterpret_cast<const uint8_t*>(p.k) + row * (kDim * 2);
      if (j >= kStages && !mbar_wait<true>(&empty[s], ((j / kStages) + 1) & 1, p.status)) { ok = false; break; }
      const uint32_t stage = sBase + s * kStageBytes;
#pragma unroll
      for (int u = 0; u < 16; ++u) cp_async16(stage + (u >> 3) * kChunk + sw128_offset(r, u & 7), krow + u * 16, in_range ? 16u : 0u);
      cp_async_commit();
      // the previous block's rows have landed once only this block's group is outstanding
      if (j >= 1) {
        cp_async_wait<1>();
        fence_proxy_async_smem();
        mbar_arrive(&full[(j - 1) % kStages]);
      }
    }
    cp_async_wait<0>();
    if (ok && p.topk >= 1) {
      fence_proxy_async_smem();
      mbar_arrive(&full[(p.topk - 1) % kStages]);
    }
    }
  } else if (warp == 8) {
    // ================================ MMA issuer ====================================================
    // the whole warp walks the loop and waits, converged; one elected lane issues through predicated instructions
    {
      // UMMA N = the head count rounded up to 16 (rows of the B image beyond the head count are zero)
      const uint32_t idesc = make_idesc_f16(kBF16, kKeys, static_cast<uint32_t>((p.H + 15) & ~15), 0, 0);
      const uint32_t go = elect_one_lane();
      ok = __all_sync(0xffffffffu, mbar_wait(q_ready, 0, p.status));
      const uint64_t db0 = make_smem_desc(sQ, 16, 1024, kSwizzle128B);
      for (int j = 0; j < p.topk && ok; ++j) {
        const int s = j % kStages, db = j & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(&full[s], (j / kStages) & 1, p.status))) { ok = false; break; }
        if (j >= 2 && !__all_sync(0xffffffffu, mbar_wait(&d_free[db], ((j >> 1) + 1) & 1, p.status))) { ok = false; break; }
        tc_fence_after();
        const uint64_t da0 = make_smem_desc(sBase + s * kStageBytes, 16, 1024, kSwizzle128B);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int kq = 0; kq < 4; ++kq)
            umma_ss_if(go, tD + db * kHeads, da0 + ((c * kChunk + kq * 32) >> 4), db0 + ((c * (kHeads * 128) + kq * 32) >> 4), idesc, (c | kq) != 0);
        }
        umma_commit_if(go, &d_full[db]);
        umma_commit_if(go, &empty[s]);
      }
    }
  } else {
    // ================================ epilogue: thread = key ========================================
    const int r = warp * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int lo = p.ks[qi], hi = p.ke[qi];
    for (int j = 0; j < p.topk && ok; ++j) {
      const int db = j & 1;
      const int blk = blocks[j];
      const int64_t pos = static_cast<int64_t>(blk) * kKeys + r;
      bool valid = blk >= 0 && (p.block_table ? blk < p.max_blocks : pos < p.S_kv) && pos >= lo && pos < hi;
      if (valid && p.block_table) {  // same rule as the loader: a row that was not fetched has no logit
        const int phys = p.block_table[static_cast<int64_t>(qi / p.tokens_per_seq) * p.max_blocks + blk];
        valid = phys >= 0 && (static_cast<int64_t>(phys) + 1) * kKeys <= p.S_kv;
      }
      if (!__all_sync(0xffffffffu, mbar_wait(&d_full[db], (j >> 1) & 1, p.status))) { ok = false; break; }
      tc_fence_after();
      uint32_t v[64];
      tmem_ld32(tD + db * kHeads + lane_base, v);
      if (p.H > 32) tmem_ld32(tD + db * kHeads + 32 + lane_base, v + 32);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&d_free[db]);
      float total = 0.f;
      const float4* sw4 = reinterpret_cast<const float4*>(sw);   // four weights per (broadcast) load
#pragma unroll
      for (int h4 = 0; h4 < kHeads / 4; ++h4) {   // columns at or beyond the head count hold stale tensor memory (or were not loaded): skipped
        if (4 * h4 < p.H) {
          const float4 wv = sw4[h4];
          total += wv.x * fmaxf(__uint_as_float(v[4 * h4]), 0.f);
          if (4 * h4 + 1 < p.H) total += wv.y * fmaxf(__uint_as_float(v[4 * h4 + 1]), 0.f);
          if (4 * h4 + 2 < p.H) total += wv.z * fmaxf(__uint_as_float(v[4 * h4 + 2]), 0.f);
          if (4 * h4 + 3 < p.H) total += wv.w * fmaxf(__uint_as_float(v[4 * h4 + 3]), 0.f);
        }
      }
      p.logits[(static_cast<int64_t>(qi) * p.topk + j) * kKeys + r] = valid ? total : -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tD, 128);
}

bool block_sparse_logits_tc_supported(const BlockSparseLogitsParams& p) {
  return p.block == bsltc::kKeys && p.D == bsltc::kDim && p.H >= 1 && p.H <= bsltc::kHeads && (reinterpret_cast<uintptr_t>(p.k) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(p.q) & 15u) == 0;
}

int launch_block_sparse_logits_tc(const BlockSparseLogitsParams& p, bool bf16, cudaStream_t stream) {
  auto kern = bf16 ? block_sparse_logits_tc_kernel<true> : block_sparse_logits_tc_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bsltc::kSmemBytes));
  if (e != cudaSuccess) return static_cast<int>(e);
  // k as a tensor map with a box of one block half (64 dims x 128 keys); DSA_HISA_NO_TMA=1 in the environment forces the
  // cp.async loaders (used by the tests to cover that path)
  alignas(64) CUtensorMap kmap;
  memset(&kmap, 0, sizeof(kmap));
  const char* no_tma = getenv("DSA_HISA_NO_TMA");
  const int use_tma = (!(no_tma && no_tma[0] == '1') && encode_rows_map(p.k, p.S_kv, bsltc::kDim, bf16, bsltc::kKeys, &kmap)) ? 1 : 0;
  kern<<<static_cast<unsigned>(p.S), bsltc::kThreads, bsltc::kSmemBytes, stream>>>(p, kmap, use_tma);
  return static_cast<int>(cudaGetLastError());
}
}  // namespace dsa
