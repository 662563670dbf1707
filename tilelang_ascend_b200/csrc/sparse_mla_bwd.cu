// Sparse MLA backward (correctness-first CUDA-core kernel).
//
// Given q, kv, indices, the forward's out / lse and the output gradient dO it produces
//   dQ  [B, S, H, D]      (input dtype)
//   dKV [B, S_kv, 1, D]   fp32, scatter-accumulated with atomics (the caller zeroes it)
// with   P = exp(s - lse),  delta = sum_d dO*O,  dS = P * (dO.V^T - delta) * sm_scale,
//        dQ = dS.K,  dKV[idx] += dS^T.Q (all D dims)  and  dKV[idx][:DV] += P^T.dO.
// The reference has no sparse-MLA backward; the decomposition (delta preprocess, P recomputed from
// the saved LSE, fp32 atomic accumulation of the key gradient) is the one its dense backward uses
// (examples_experiment/example_gqa_bwd/example_gqa_bwd.py:189-223, 312-556).
//
// One CTA per (query, group of 8 heads), one warp per head; a tile of 32 gathered KV rows sits in
// shared memory next to an fp32 tile that collects the 8 heads' key gradients before they go to
// global memory as one atomic add per element.
#include "params.h"
#include "ptx.cuh"

namespace dsa {

namespace bwd {
constexpr int kBK = 32, kHeadsPerCta = 8, kMaxD = 640, kMaxDV = 512;
}

__device__ __forceinline__ bool bwd_index_valid(int idx, int kv_len, int pos_limit) { return idx >= 0 && idx < kv_len && idx <= pos_limit; }

template <typename T>
__global__ void __launch_bounds__(256) sparse_mla_bwd_kernel(const BwdParams bp) {
  using namespace bwd;
  const FwdParams& p = bp.f;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int D = p.D, DV = p.DV;
  T* tile = reinterpret_cast<T*>(smem_raw);                                                  // [kBK][D]
  float* dkv_tile = reinterpret_cast<float*>(smem_raw + static_cast<size_t>(kBK) * D * sizeof(T));  // [kBK][D]
  __shared__ int s_idx[kBK];
  __shared__ long long s_row[kBK];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bt = blockIdx.y;
  const int b = bt / p.S, t = bt - b * p.S;
  const int h = blockIdx.x * kHeadsPerCta + warp;
  const bool head_ok = h < p.H;
  if (p.q_len_b && t >= p.q_len_b[b]) return;
  const int qs = p.q_start_b ? p.q_start_b[b] : p.q_start;
  const int kv_len = p.kv_len_b ? p.kv_len_b[b] : p.S_kv;
  const int pos_limit = p.causal ? qs + t : 0x7fffffff;
  const int32_t* idx_row = p.indices + static_cast<int64_t>(bt) * p.topk;

  float qreg[kMaxD / 32], dq[kMaxD / 32], doreg[kMaxDV / 32];
  const int64_t hrow = static_cast<int64_t>(bt) * p.H + (head_ok ? h : 0);
  const T* qrow = reinterpret_cast<const T*>(p.q) + hrow * D;
  const T* dorow = reinterpret_cast<const T*>(bp.d_out) + hrow * DV;
  const T* orow = reinterpret_cast<const T*>(p.out) + hrow * DV;
  float delta = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxD / 32; ++i) {
    const int d = lane + 32 * i;
    qreg[i] = (head_ok && d < D) ? static_cast<float>(qrow[d]) : 0.f;
    dq[i] = 0.f;
  }
#pragma unroll
  for (int i = 0; i < kMaxDV / 32; ++i) {
    const int d = lane + 32 * i;
    doreg[i] = (head_ok && d < DV) ? static_cast<float>(dorow[d]) : 0.f;
    if (head_ok && d < DV) delta += doreg[i] * static_cast<float>(orow[d]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) delta += __shfl_xor_sync(0xffffffffu, delta, o);
  const float lse = head_ok ? p.lse[hrow] : 0.f;
  const float lse2 = lse * 1.4426950408889634f;  // log2 domain

  const int ntiles = (p.topk + kBK - 1) / kBK;
  for (int tile_i = 0; tile_i < ntiles; ++tile_i) {
    __syncthreads();
    if (tid < kBK) {
      const int slot = tile_i * kBK + tid;
      const int idx = slot < p.topk ? idx_row[slot] : -1;
      const bool v = bwd_index_valid(idx, kv_len, pos_limit);
      s_idx[tid] = v ? idx : -1;
      long long row = 0;
      if (v) {
        if (p.block_table) {
          const int blk = p.block_table[static_cast<int64_t>(b) * p.max_blocks + idx / p.block_size];
          row = static_cast<long long>(blk) * p.block_size + idx % p.block_size;
        } else {
          row = static_cast<long long>(b) * p.S_kv + idx;
        }
      }
      s_row[tid] = row;
    }
    __syncthreads();
    const int units = D / 8;
    for (int u = tid; u < kBK * units; u += blockDim.x) {
      const int key = u / units, unit = u - key * units;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (s_idx[key] >= 0) val = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.kv) + s_row[key] * D + unit * 8);
      *reinterpret_cast<uint4*>(tile + key * D + unit * 8) = val;
    }
    for (int i = tid; i < kBK * D; i += blockDim.x) dkv_tile[i] = 0.f;
    __syncthreads();
    if (head_ok) {
      for (int j = 0; j < kBK; ++j) {
        if (s_idx[j] < 0) continue;
        const T* krow = tile + j * D;
        float dot = 0.f, dp = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxD / 32; ++i) {
          const int d = lane + 32 * i;
          if (d < D) dot += qreg[i] * static_cast<float>(krow[d]);
        }
#pragma unroll
        for (int i = 0; i < kMaxDV / 32; ++i) {
          const int d = lane + 32 * i;
          if (d < DV) dp += doreg[i] * static_cast<float>(krow[d]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          dot += __shfl_xor_sync(0xffffffffu, dot, o);
          dp += __shfl_xor_sync(0xffffffffu, dp, o);
        }
        const float prob = exp2f(dot * p.scale_log2 - lse2);
        const float ds = prob * (dp - delta) * bp.sm_scale;
        float* gk = dkv_tile + j * D;
#pragma unroll
        for (int i = 0; i < kMaxD / 32; ++i) {
          const int d = lane + 32 * i;
          if (d < D) {
            dq[i] += ds * static_cast<float>(krow[d]);
            float g = ds * qreg[i];
            if (d < DV) g += prob * doreg[i < kMaxDV / 32 ? i : 0];
            atomicAdd(gk + d, g);
          }
        }
      }
    }
    __syncthreads();
    for (int i = tid; i < kBK * D; i += blockDim.x) {
      const int key = i / D;
      if (s_idx[key] >= 0) {
        const float g = dkv_tile[i];
        if (g != 0.f) atomicAdd(bp.d_kv + s_row[key] * D + (i - key * D), g);
      }
    }
  }
  if (head_ok) {
    T* dqrow = reinterpret_cast<T*>(bp.d_q) + hrow * D;
#pragma unroll
    for (int i = 0; i < kMaxD / 32; ++i) {
      const int d = lane + 32 * i;
      if (d < D) dqrow[d] = static_cast<T>(dq[i]);
    }
  }
}

int launch_sparse_mla_bwd(const BwdParams& bp, bool bf16, cudaStream_t stream) {
  const FwdParams& p = bp.f;
  const size_t smem = static_cast<size_t>(bwd::kBK) * p.D * (2 + 4);
  dim3 grid((p.H + bwd::kHeadsPerCta - 1) / bwd::kHeadsPerCta, p.B * p.S);
  cudaError_t e;
  if (bf16) {
    e = cudaFuncSetAttribute(sparse_mla_bwd_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    sparse_mla_bwd_kernel<__nv_bfloat16><<<grid, 256, smem, stream>>>(bp);
  } else {
    e = cudaFuncSetAttribute(sparse_mla_bwd_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    sparse_mla_bwd_kernel<__half><<<grid, 256, smem, stream>>>(bp);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace dsa
