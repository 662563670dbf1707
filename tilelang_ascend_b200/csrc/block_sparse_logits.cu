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
    const int64_t pos = static_cast<int64_t>(p.blocks[static_cast<int64_t>(qi) * p.topk + j]) * p.block + off;
    const bool in_block = off < p.block;
    const bool valid = in_block && pos >= 0 && pos < p.S_kv && pos >= lo && pos < hi;
    float acc[kMaxH];
#pragma unroll
    for (int h = 0; h < kMaxH; ++h) acc[h] = 0.f;
    if (valid) {
      const uint4* krow = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.k) + pos * p.D);
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
