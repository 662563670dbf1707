// Sparse MLA backward (CUDA-core kernels).
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
// Two kernels.  Generic (any D <= 640, DV <= 512): one CTA per (query, group of 8 heads), one warp per head; a tile of
// 32 gathered KV rows sits in shared memory next to an fp32 tile that collects the 8 heads' key gradients before
// they go to global memory as one atomic add per element.  D = 576 / DV = 512: see sparse_mla_bwd_mla_kernel below.
#include <type_traits>

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

// -------------------------------------------------------------------------------------------------
// D = 576 / DV = 512: one CTA per (query, group of 32 heads), 256 threads
// -------------------------------------------------------------------------------------------------
// Per tile of 32 gathered KV rows:
//   phase A (8 warps, 4 heads each): per (head, key) the two dot products q.k and dO.v over the lanes, P and dS from
//            them, dQ += dS * k in registers; P and dS of the 32 x 32 (head, key) pairs go to shared memory;
//   phase B (all threads, 288 slots of 4 dims x 16 keys): the tile's key gradient  dKV[j, :] = sum_h dS[h, j] q[h, :] + P[h, j] dO[h, :]  as a small
//            register-tiled matrix product (thread = 4 dims x 16 keys, loop over the 32 heads), then ONE vector atomic
//            per (key, 4 dims) to global memory -- a quarter of the atomics of the generic kernel and none in shared memory.
namespace bwd2 {
constexpr int kBK = 32, kHG = 32, kThreads = 256, kD = 576, kDV = 512;  // 8 warps: two per scheduler, up to 255 registers
constexpr size_t kOffK = 0;                                   // [32][576] T
constexpr size_t kOffQ = kOffK + kBK * kD * 2;                // [32][576] T
constexpr size_t kOffDO = kOffQ + kHG * kD * 2;               // [32][512] T
constexpr size_t kOffDS = kOffDO + kHG * kDV * 2;             // [32 heads][32 keys] fp32
constexpr size_t kOffP = kOffDS + kHG * kBK * 4;              // [32 heads][32 keys] fp32
constexpr size_t kSmemBytes = kOffP + kHG * kBK * 4;          // 114688
}  // namespace bwd2

template <typename T>
__device__ __forceinline__ float2 pair_to_float2(uint32_t u) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
  } else {
    const __half2 h = *reinterpret_cast<const __half2*>(&u);
    return __half22float2(h);
  }
}

template <typename T>
__global__ void __launch_bounds__(bwd2::kThreads, 1) sparse_mla_bwd_mla_kernel(const BwdParams bp) {
  using namespace bwd2;
  const FwdParams& p = bp.f;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  T* Ks = reinterpret_cast<T*>(smem_raw + kOffK);
  T* Qs = reinterpret_cast<T*>(smem_raw + kOffQ);
  T* dOs = reinterpret_cast<T*>(smem_raw + kOffDO);
  float* DSs = reinterpret_cast<float*>(smem_raw + kOffDS);
  float* Ps = reinterpret_cast<float*>(smem_raw + kOffP);
  __shared__ int s_valid[kBK];
  __shared__ long long s_row[kBK];
  __shared__ float s_delta[kHG], s_lse2[kHG];
  __shared__ int s_any;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bt = blockIdx.y;
  const int b = bt / p.S, t = bt - b * p.S;
  const int h0 = blockIdx.x * kHG;
  if (p.q_len_b && t >= p.q_len_b[b]) return;
  const int qs = p.q_start_b ? p.q_start_b[b] : p.q_start;
  const int kv_len = p.kv_len_b ? p.kv_len_b[b] : p.S_kv;
  const int pos_limit = p.causal ? qs + t : 0x7fffffff;
  const int32_t* idx_row = p.indices + static_cast<int64_t>(bt) * p.topk;

  // ---- Q and dO of the 32 heads to shared memory (zeros for heads that do not exist), delta and lse per head ----
  for (int u = tid; u < kHG * (kD / 8); u += kThreads) {
    const int hh = u / (kD / 8), unit = u - hh * (kD / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (h0 + hh < p.H) v = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.q) + (static_cast<int64_t>(bt) * p.H + h0 + hh) * kD + unit * 8);
    *reinterpret_cast<uint4*>(Qs + hh * kD + unit * 8) = v;
  }
  for (int u = tid; u < kHG * (kDV / 8); u += kThreads) {
    const int hh = u / (kDV / 8), unit = u - hh * (kDV / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (h0 + hh < p.H) v = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(bp.d_out) + (static_cast<int64_t>(bt) * p.H + h0 + hh) * kDV + unit * 8);
    *reinterpret_cast<uint4*>(dOs + hh * kDV + unit * 8) = v;
  }
  __syncthreads();
  if (warp < 8) {
#pragma unroll
    for (int hq = 0; hq < 4; ++hq) {
      const int hh = warp * 4 + hq;
      float d = 0.f;
      if (h0 + hh < p.H) {
        const uint32_t* orow = reinterpret_cast<const uint32_t*>(reinterpret_cast<const T*>(p.out) + (static_cast<int64_t>(bt) * p.H + h0 + hh) * kDV);
        const uint32_t* drow = reinterpret_cast<const uint32_t*>(dOs + hh * kDV);
#pragma unroll
        for (int i = 0; i < kDV / 64; ++i) {
          const float2 o = pair_to_float2<T>(orow[i * 32 + lane]), g = pair_to_float2<T>(drow[i * 32 + lane]);
          d += o.x * g.x + o.y * g.y;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (lane == 0) {
        s_delta[hh] = d;
        s_lse2[hh] = (h0 + hh < p.H) ? p.lse[static_cast<int64_t>(bt) * p.H + h0 + hh] * 1.4426950408889634f : 0.f;
      }
    }
  }
  float dq[4][18];
#pragma unroll
  for (int hq = 0; hq < 4; ++hq)
#pragma unroll
    for (int i = 0; i < 18; ++i) dq[hq][i] = 0.f;

  const int ntiles = (p.topk + kBK - 1) / kBK;
  for (int tile_i = 0; tile_i < ntiles; ++tile_i) {
    __syncthreads();  // previous tile's phase B is done with Ks / DSs / Ps / s_row
    if (tid < kBK) {
      const int slot = tile_i * kBK + tid;
      const int idx = slot < p.topk ? idx_row[slot] : -1;
      const bool v = bwd_index_valid(idx, kv_len, pos_limit);
      long long row = 0;
      if (v) {
        if (p.block_table) {
          const int blk = p.block_table[static_cast<int64_t>(b) * p.max_blocks + idx / p.block_size];
          row = static_cast<long long>(blk) * p.block_size + idx % p.block_size;
        } else {
          row = static_cast<long long>(b) * p.S_kv + idx;
        }
      }
      s_valid[tid] = v ? 1 : 0;
      s_row[tid] = row;
      const unsigned any = __ballot_sync(0xffffffffu, v);
      if (tid == 0) s_any = any != 0u;
    }
    __syncthreads();
    if (!s_any) continue;  // no key of this tile takes part (uniform over the CTA)
    for (int u = tid; u < kBK * (kD / 8); u += kThreads) {
      const int key = u / (kD / 8), unit = u - key * (kD / 8);
      uint4 val = make_uint4(0, 0, 0, 0);
      if (s_valid[key]) val = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.kv) + s_row[key] * kD + unit * 8);
      *reinterpret_cast<uint4*>(Ks + key * kD + unit * 8) = val;
    }
    __syncthreads();
    // ---- phase A ----
    {
#pragma unroll
      for (int hq = 0; hq < 4; ++hq) {
        const int hh = warp * 4 + hq;
        float2 q2[9], g2[8];
        const uint32_t* qrow = reinterpret_cast<const uint32_t*>(Qs + hh * kD);
        const uint32_t* grow = reinterpret_cast<const uint32_t*>(dOs + hh * kDV);
#pragma unroll
        for (int i = 0; i < 9; ++i) q2[i] = pair_to_float2<T>(qrow[i * 32 + lane]);
#pragma unroll
        for (int i = 0; i < 8; ++i) g2[i] = pair_to_float2<T>(grow[i * 32 + lane]);
        const float delta = s_delta[hh], lse2 = s_lse2[hh];
        // four keys at a time: their dot products, reductions and dQ updates are independent chains that overlap
#pragma unroll 1
        for (int j0 = 0; j0 < kBK; j0 += 4) {
          float2 k2[4][9];
          float dot[4], dp[4];
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const uint32_t* krow = reinterpret_cast<const uint32_t*>(Ks + (j0 + jj) * kD);
#pragma unroll
            for (int i = 0; i < 9; ++i) k2[jj][i] = pair_to_float2<T>(krow[i * 32 + lane]);
          }
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
            for (int i = 0; i < 9; ++i) { a0 = fmaf(q2[i].x, k2[jj][i].x, a0); a1 = fmaf(q2[i].y, k2[jj][i].y, a1); }
#pragma unroll
            for (int i = 0; i < 8; ++i) { b0 = fmaf(g2[i].x, k2[jj][i].x, b0); b1 = fmaf(g2[i].y, k2[jj][i].y, b1); }
            dot[jj] = a0 + a1;
            dp[jj] = b0 + b1;
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              dot[jj] += __shfl_xor_sync(0xffffffffu, dot[jj], o);
              dp[jj] += __shfl_xor_sync(0xffffffffu, dp[jj], o);
            }
          }
          float prob[4], ds[4];
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            // a key that does not take part was gathered as zeros: its probability must still be forced to zero
            prob[jj] = s_valid[j0 + jj] ? exp2f(dot[jj] * p.scale_log2 - lse2) : 0.f;
            ds[jj] = prob[jj] * (dp[jj] - delta) * bp.sm_scale;
          }
#pragma unroll
          for (int i = 0; i < 9; ++i) {
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              dq[hq][2 * i] = fmaf(ds[jj], k2[jj][i].x, dq[hq][2 * i]);
              dq[hq][2 * i + 1] = fmaf(ds[jj], k2[jj][i].y, dq[hq][2 * i + 1]);
            }
          }
          if (lane < 4) {
            const float dsl = lane == 0 ? ds[0] : lane == 1 ? ds[1] : lane == 2 ? ds[2] : ds[3];
            const float pl = lane == 0 ? prob[0] : lane == 1 ? prob[1] : lane == 2 ? prob[2] : prob[3];
            DSs[hh * kBK + j0 + lane] = dsl;
            Ps[hh * kBK + j0 + lane] = pl;
          }
        }
      }
    }
    __syncthreads();
    // ---- phase B: slot = (4 dims, 16 keys); 288 slots over 256 threads ----
    for (int slot = tid; slot < 288; slot += kThreads) {
      const int dg = slot % 144, kh = slot / 144;
      float acc[16][4];
#pragma unroll
      for (int j = 0; j < 16; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;
      const bool has_v = dg < kDV / 4;
#pragma unroll 2
      for (int hh = 0; hh < kHG; ++hh) {
        const uint2 qraw = *reinterpret_cast<const uint2*>(Qs + hh * kD + dg * 4);
        const float2 qa = pair_to_float2<T>(qraw.x), qb = pair_to_float2<T>(qraw.y);
        const float qv[4] = {qa.x, qa.y, qb.x, qb.y};
        float gv[4] = {0.f, 0.f, 0.f, 0.f};
        if (has_v) {
          const uint2 graw = *reinterpret_cast<const uint2*>(dOs + hh * kDV + dg * 4);
          const float2 ga = pair_to_float2<T>(graw.x), gb = pair_to_float2<T>(graw.y);
          gv[0] = ga.x; gv[1] = ga.y; gv[2] = gb.x; gv[3] = gb.y;
        }
        const float4* dsr = reinterpret_cast<const float4*>(DSs + hh * kBK + kh * 16);
        const float4* pr = reinterpret_cast<const float4*>(Ps + hh * kBK + kh * 16);
#pragma unroll
        for (int jq = 0; jq < 4; ++jq) {
          const float4 d4 = dsr[jq], p4 = pr[jq];
          const float dsv[4] = {d4.x, d4.y, d4.z, d4.w}, pv[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[jq * 4 + jj][c] = fmaf(dsv[jj], qv[c], fmaf(pv[jj], gv[c], acc[jq * 4 + jj][c]));
        }
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int key = kh * 16 + j;
        if (s_valid[key]) {
          float4* dst = reinterpret_cast<float4*>(bp.d_kv + s_row[key] * kD + dg * 4);
          atomicAdd(dst, make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]));
        }
      }
    }
  }
  // ---- dQ ----
  if (warp < 8) {
#pragma unroll
    for (int hq = 0; hq < 4; ++hq) {
      const int hh = warp * 4 + hq;
      if (h0 + hh < p.H) {
        T* dqrow = reinterpret_cast<T*>(bp.d_q) + (static_cast<int64_t>(bt) * p.H + h0 + hh) * kD;
#pragma unroll
        for (int i = 0; i < 9; ++i) {
          dqrow[i * 64 + 2 * lane] = static_cast<T>(dq[hq][2 * i]);
          dqrow[i * 64 + 2 * lane + 1] = static_cast<T>(dq[hq][2 * i + 1]);
        }
      }
    }
  }
}

int launch_sparse_mla_bwd(const BwdParams& bp, bool bf16, cudaStream_t stream) {
  const FwdParams& p = bp.f;
  cudaError_t e;
  // the vector atomics of the MLA kernel need 16-byte aligned dKV rows (576 floats per row: the base decides)
  if (p.D == bwd2::kD && p.DV == bwd2::kDV && (reinterpret_cast<uintptr_t>(bp.d_kv) & 15u) == 0 && (reinterpret_cast<uintptr_t>(p.kv) & 15u) == 0 &&
      (reinterpret_cast<uintptr_t>(p.q) & 15u) == 0 && (reinterpret_cast<uintptr_t>(bp.d_out) & 15u) == 0) {
    dim3 grid((p.H + bwd2::kHG - 1) / bwd2::kHG, p.B * p.S);
    if (bf16) {
      e = cudaFuncSetAttribute(sparse_mla_bwd_mla_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bwd2::kSmemBytes));
      if (e != cudaSuccess) return static_cast<int>(e);
      sparse_mla_bwd_mla_kernel<__nv_bfloat16><<<grid, bwd2::kThreads, bwd2::kSmemBytes, stream>>>(bp);
    } else {
      e = cudaFuncSetAttribute(sparse_mla_bwd_mla_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bwd2::kSmemBytes));
      if (e != cudaSuccess) return static_cast<int>(e);
      sparse_mla_bwd_mla_kernel<__half><<<grid, bwd2::kThreads, bwd2::kSmemBytes, stream>>>(bp);
    }
    return static_cast<int>(cudaGetLastError());
  }
  const size_t smem = static_cast<size_t>(bwd::kBK) * p.D * (2 + 4);
  dim3 grid((p.H + bwd::kHeadsPerCta - 1) / bwd::kHeadsPerCta, p.B * p.S);
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
