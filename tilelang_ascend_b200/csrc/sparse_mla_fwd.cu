// Sparse MLA forward for sm_100a.
//
// For every query token the kernel gathers the latent KV rows its index list names, computes
// S = sm_scale * Q K^T over all D dims for all heads, an online softmax over the gathered keys, and
// O = P V over the first DV dims, and writes O (input dtype) and the natural-log LSE (fp32).
// Semantics follow ref_sparse_attention_fwd_interface
// (examples/sparse_flash_attention/example_sparse_flash_attn.py:255-292) and the -1 / length rules
// of the paged variant (example_sparse_flash_attn_mask_pa.py:221-238).
//
// Two kernels:
//  * sparse_mla_fwd_tc_kernel  -- D = 576, DV = 512: tcgen05 tensor-core MMAs with TMEM accumulators.
//    One CTA per (query, half of the DV columns, block of 128 heads).  TMEM cannot hold a
//    128 x 512 fp32 output tile and a score tile at once, so the output columns are split across
//    two CTAs; each computes the full score tile.
//  * sparse_mla_fwd_generic_kernel -- any D <= 640 / DV <= 512 (e.g. the GQA example with dim 128):
//    CUDA-core fp32, one warp per head.
#include <type_traits>

#include "params.h"
#include "ptx.cuh"

namespace dsa {

// -------------------------------------------------------------------------------------------------
// shared helpers
// -------------------------------------------------------------------------------------------------
struct RowCtx {
  int b, t;         // batch, query inside the batch
  int pos_limit;    // largest key index allowed by the causal rule (INT_MAX when not causal)
  int kv_len;       // number of keys of this sequence
  const int32_t* idx_row;
  bool active;      // query exists (t < q_len)
};

__device__ __forceinline__ RowCtx make_row_ctx(const FwdParams& p, int bt) {
  RowCtx c;
  c.b = bt / p.S;
  c.t = bt - c.b * p.S;
  const int qs = p.q_start_b ? p.q_start_b[c.b] : p.q_start;
  c.kv_len = p.kv_len_b ? p.kv_len_b[c.b] : p.S_kv;
  c.pos_limit = p.causal ? qs + c.t : 0x7fffffff;
  c.idx_row = p.indices + static_cast<int64_t>(bt) * p.topk;
  c.active = p.q_len_b ? (c.t < p.q_len_b[c.b]) : true;
  return c;
}

__device__ __forceinline__ bool index_valid(const RowCtx& c, int idx) {
  return idx >= 0 && idx < c.kv_len && idx <= c.pos_limit;
}

// Row number of key `idx` of batch b inside the kv tensor.
__device__ __forceinline__ int64_t kv_row(const FwdParams& p, int b, int idx) {
  if (p.block_table) {
    const int blk = p.block_table[static_cast<int64_t>(b) * p.max_blocks + idx / p.block_size];
    return static_cast<int64_t>(blk) * p.block_size + idx % p.block_size;
  }
  return static_cast<int64_t>(b) * p.S_kv + idx;
}

template <bool kBF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (kBF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// -------------------------------------------------------------------------------------------------
// tcgen05 kernel
// -------------------------------------------------------------------------------------------------
namespace tc {
constexpr int kD = 576, kDV = 512, kChunks = 9;     // 9 chunks of 64 dims (128 B of bf16)
constexpr int kM = 128;                             // heads per CTA = UMMA M
constexpr int kBK = 32;                             // keys per tile
constexpr int kStages = 2;
constexpr int kHalfDV = 256;                        // output columns per CTA
constexpr int kMaxTiles = 256;                      // topk <= 8192
constexpr uint32_t kQBytes = kChunks * kM * 128;    // 147456
constexpr uint32_t kKVChunkBytes = kBK * 128;       // 4096
constexpr uint32_t kKVStageBytes = kChunks * kKVChunkBytes;  // 36864
constexpr uint32_t kPBytes = kM * kBK * 2;          // 8192
constexpr uint32_t kOffKV = kQBytes;
constexpr uint32_t kOffP = kOffKV + kStages * kKVStageBytes;  // 221184
constexpr uint32_t kOffBar = kOffP + kPBytes;                 // 229376
constexpr uint32_t kOffMask = kOffBar + 128;
constexpr uint32_t kOffList = kOffMask + kMaxTiles * 4;
constexpr uint32_t kSmemBytes = kOffList + kMaxTiles * 2 + 1024;  // + slack to align the base to 1024 B
constexpr int kThreads = 288;                       // 4 softmax warps, 1 MMA warp, 4 gather warps
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 0, kColS = 256;
constexpr float kRescaleThreshold = 8.0f;           // log2 units: P stays below 2^8
}  // namespace tc

template <bool kBF16>
__global__ void __launch_bounds__(tc::kThreads, 1) sparse_mla_fwd_tc_kernel(const FwdParams p) {
  using namespace tc;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sKV = sQ + kOffKV;
  const uint32_t sP = sQ + kOffP;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
  uint64_t* kv_full = bars;        // [2] count 128: gather threads
  uint64_t* kv_empty = bars + 2;   // [2] count 1: tcgen05.commit after the PV MMAs of the stage
  uint64_t* s_full = bars + 4;     // count 1: commit after the QK MMAs
  uint64_t* p_full = bars + 5;     // count 128: softmax threads wrote P
  uint64_t* o_full = bars + 6;     // count 1: commit after the last PV
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  int* n_valid_tiles = reinterpret_cast<int*>(bars + 9);
  int* start_status = reinterpret_cast<int*>(bars + 10);
  uint32_t* masks = reinterpret_cast<uint32_t*>(smem + kOffMask);
  uint16_t* tile_list = reinterpret_cast<uint16_t*>(smem + kOffList);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int half = blockIdx.x;           // which 256 output columns
  const int bt = blockIdx.y;             // flat (batch, query)
  const int h0 = blockIdx.z * kM;        // first head of this CTA
  const RowCtx ctx = make_row_ctx(p, bt);
  const int ntiles = (p.topk + kBK - 1) / kBK;
  using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;

  if (tid == 0) *start_status = *reinterpret_cast<volatile int*>(p.status);
  __syncthreads();
  if (*start_status != kStatusOk || !ctx.active) return;  // an earlier CTA failed, or padding row

  // ---- setup: barriers, TMEM, per-tile validity masks, Q -----------------------------------------
  if (tid == 0) {
    mbar_init(&kv_full[0], 128);
    mbar_init(&kv_full[1], 128);
    mbar_init(&kv_empty[0], 1);
    mbar_init(&kv_empty[1], 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 128);
    mbar_init(o_full, 1);
    mbar_init_fence();
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  for (int tile = warp; tile < ntiles; tile += kThreads / 32) {
    const int slot = tile * kBK + lane;
    const int idx = slot < p.topk ? ctx.idx_row[slot] : -1;
    const uint32_t m = __ballot_sync(0xffffffffu, index_valid(ctx, idx));
    if (lane == 0) masks[tile] = m;
  }
  {  // Q tile: rows = heads, 9 chunks of [128 x 128 B], 128-byte swizzle; missing heads are zero
    const T* qrow = reinterpret_cast<const T*>(p.q) + (static_cast<int64_t>(bt) * p.H + h0) * kD;
    for (int u = tid; u < kM * (kD / 8); u += kThreads) {
      const int r = u / (kD / 8), unit = u - r * (kD / 8);
      const bool ok = h0 + r < p.H;
      const T* src = ok ? qrow + static_cast<int64_t>(r) * kD + unit * 8 : reinterpret_cast<const T*>(p.q);
      cp_async16(sQ + (unit >> 3) * (kM * 128) + sw128_offset(r, unit & 7), src, ok ? 16u : 0u);
    }
    cp_async_commit();
    cp_async_wait<0>();
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (tid == 0) {  // compact list of tiles with at least one key taking part
    int n = 0;
    for (int tile = 0; tile < ntiles; ++tile)
      if (masks[tile] != 0) tile_list[n++] = static_cast<uint16_t>(tile);
    *n_valid_tiles = n;
  }
  __syncthreads();
  const int nvt = *n_valid_tiles;
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tO = tmem_base + kColO, tS = tmem_base + kColS;
  bool ok = true;

  if (warp >= 5) {
    // ================================ gather producers =============================================
    const int pt = tid - 160;  // 0..127
    const uint8_t* kv_bytes = reinterpret_cast<const uint8_t*>(p.kv);
    for (int it = 0; it < nvt; ++it) {
      const int tile = tile_list[it], s = it & 1;
      if (it >= kStages && !mbar_wait(&kv_empty[s], ((it >> 1) + 1) & 1, p.status)) { ok = false; break; }
      const uint32_t stage = sKV + s * kKVStageBytes;
#pragma unroll 6
      for (int j = 0; j < (kBK * 72) / 128; ++j) {
        const int u = pt + 128 * j;
        const int key = u / 72, unit = u - key * 72;
        const int slot = tile * kBK + key;
        const int idx = slot < p.topk ? __ldg(ctx.idx_row + slot) : -1;
        const bool v = index_valid(ctx, idx);
        const uint8_t* src = v ? kv_bytes + kv_row(p, ctx.b, idx) * (kD * 2) + unit * 16 : kv_bytes;
        cp_async16(stage + (unit >> 3) * kKVChunkBytes + sw128_offset(key, unit & 7), src, v ? 16u : 0u);
      }
      cp_async_commit();
      if (it >= 1) {
        cp_async_wait<1>();
        fence_proxy_async_smem();
        mbar_arrive(&kv_full[(it - 1) & 1]);
      }
    }
    cp_async_wait<0>();
    if (ok && nvt > 0) {
      fence_proxy_async_smem();
      mbar_arrive(&kv_full[(nvt - 1) & 1]);
    }
  } else if (warp == 4) {
    // ================================ MMA issuer ====================================================
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(kBF16, kM, kBK, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_f16(kBF16, kM, kHalfDV, 0, 1);
      for (int it = 0; it < nvt; ++it) {
        const int s = it & 1;
        const uint32_t stage = sKV + s * kKVStageBytes;
        if (!mbar_wait(&kv_full[s], (it >> 1) & 1, p.status)) { ok = false; break; }
        tc_fence_after();
        // S[128 x 32] = Q[128 x 576] . K^T : both operands K-major, 36 steps of 16 dims
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t da = make_smem_desc(sQ + c * (kM * 128) + k * 32, 16, 1024, kSwizzle128B);
            const uint64_t db = make_smem_desc(stage + c * kKVChunkBytes + k * 32, 16, 1024, kSwizzle128B);
            umma_ss(tS, da, db, idesc_qk, (c | k) != 0);
          }
        }
        umma_commit(s_full);
        if (!mbar_wait(p_full, it & 1, p.status)) { ok = false; break; }
        tc_fence_after();
        // O[128 x 256] += P[128 x 32] . V[32 x 256] : P K-major (no swizzle), V MN-major (dims contiguous)
#pragma unroll
        for (int ks = 0; ks < kBK / 16; ++ks) {
          const uint64_t da = make_smem_desc(sP + ks * 256, 128, 512, kSwizzleNone);
          const uint64_t db = make_smem_desc(stage + (4 * half) * kKVChunkBytes + ks * 2048, kKVChunkBytes, 1024, kSwizzle128B);
          umma_ss(tO, da, db, idesc_pv, (it | ks) != 0);
        }
        umma_commit(&kv_empty[s]);
      }
      if (ok) umma_commit(o_full);
    }
  } else {
    // ================================ softmax + epilogue ============================================
    const int r = tid;  // TMEM lane = head row
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    uint32_t v[32];
    for (int it = 0; it < nvt; ++it) {
      const uint32_t mask = masks[tile_list[it]];
      if (!mbar_wait(s_full, it & 1, p.status)) { ok = false; break; }
      tc_fence_after();
      tmem_ld32(tS + lane_base, v);
      tmem_wait_ld();
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float x = __uint_as_float(v[j]) * p.scale_log2;
        v[j] = __float_as_uint(x);
        if ((mask >> j) & 1u) mx = fmaxf(mx, x);
      }
      // lazy rescale: keep the old reference maximum unless the new one is far above it
      float factor = 1.f;
      if (mx > m_used + kRescaleThreshold || m_used == -INFINITY) {
        factor = (m_used == -INFINITY) ? 0.f : exp2f(m_used - mx);
        m_used = mx;
      }
      if (it > 0 && __any_sync(0xffffffffu, factor != 1.f)) {
        uint32_t o[32];
#pragma unroll 1
        for (int cc = 0; cc < kHalfDV / 32; ++cc) {
          tmem_ld32(tO + lane_base + cc * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * factor);
          tmem_st32(tO + lane_base + cc * 32, o);
        }
        tmem_wait_st();
      }
      l *= factor;
      float sum = 0.f;
      uint32_t pk[16];
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float p0 = ((mask >> j) & 1u) ? exp2f(__uint_as_float(v[j]) - m_used) : 0.f;
        const float p1 = ((mask >> (j + 1)) & 1u) ? exp2f(__uint_as_float(v[j + 1]) - m_used) : 0.f;
        sum += p0 + p1;
        pk[j >> 1] = pack2<kBF16>(p0, p1);
      }
      l += sum;
      // P[128 x 32], K-major without swizzle: 8x16-byte core matrices, 128 B apart along K, 512 B apart along M
      uint8_t* prow = smem + kOffP + (r >> 3) * 512 + (r & 7) * 16;
#pragma unroll
      for (int g = 0; g < 4; ++g)
        *reinterpret_cast<uint4*>(prow + g * 128) = make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    // ---- epilogue ----
    const int h = h0 + r;
    T* orow = reinterpret_cast<T*>(p.out) + (static_cast<int64_t>(bt) * p.H + h) * kDV + half * kHalfDV;
    if (nvt == 0) {
      if (h < p.H) {
        for (int j = 0; j < kHalfDV / 8; ++j) reinterpret_cast<uint4*>(orow)[j] = make_uint4(0, 0, 0, 0);
        if (half == 0 && p.lse) p.lse[static_cast<int64_t>(bt) * p.H + h] = -INFINITY;
      }
    } else if (ok && mbar_wait(o_full, 0, p.status)) {
      tc_fence_after();
      const float inv_l = 1.f / l;
#pragma unroll 1
      for (int cc = 0; cc < kHalfDV / 32; ++cc) {
        tmem_ld32(tO + lane_base + cc * 32, v);
        tmem_wait_ld();
        if (h < p.H) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack2<kBF16>(__uint_as_float(v[8 * g + 0]) * inv_l, __uint_as_float(v[8 * g + 1]) * inv_l);
            w.y = pack2<kBF16>(__uint_as_float(v[8 * g + 2]) * inv_l, __uint_as_float(v[8 * g + 3]) * inv_l);
            w.z = pack2<kBF16>(__uint_as_float(v[8 * g + 4]) * inv_l, __uint_as_float(v[8 * g + 5]) * inv_l);
            w.w = pack2<kBF16>(__uint_as_float(v[8 * g + 6]) * inv_l, __uint_as_float(v[8 * g + 7]) * inv_l);
            reinterpret_cast<uint4*>(orow + cc * 32)[g] = w;
          }
        }
      }
      if (half == 0 && p.lse && h < p.H)
        p.lse[static_cast<int64_t>(bt) * p.H + h] = m_used * 0.6931471805599453f + logf(l);
    }
  }

  // ---- teardown: every role comes here, also after a failed wait ------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, kTmemCols);
}

// -------------------------------------------------------------------------------------------------
// generic CUDA-core kernel: one warp per head, fp32 arithmetic
// -------------------------------------------------------------------------------------------------
namespace gen {
constexpr int kBK = 32, kHeadsPerCta = 8, kMaxD = 640, kMaxDV = 512;
}

template <typename T>
__global__ void __launch_bounds__(256) sparse_mla_fwd_generic_kernel(const FwdParams p) {
  using namespace gen;
  extern __shared__ uint8_t smem_raw[];
  T* tile = reinterpret_cast<T*>(smem_raw);  // [kBK][D]
  __shared__ int s_idx[kBK];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bt = blockIdx.y;
  const int h = blockIdx.x * kHeadsPerCta + warp;
  const RowCtx ctx = make_row_ctx(p, bt);
  if (!ctx.active) return;
  const int D = p.D, DV = p.DV;
  const bool head_ok = h < p.H;

  float qreg[kMaxD / 32];
  float acc[kMaxDV / 32];
  const T* qrow = reinterpret_cast<const T*>(p.q) + (static_cast<int64_t>(bt) * p.H + (head_ok ? h : 0)) * D;
#pragma unroll
  for (int i = 0; i < kMaxD / 32; ++i) {
    const int d = lane + 32 * i;
    qreg[i] = (head_ok && d < D) ? static_cast<float>(qrow[d]) : 0.f;
  }
#pragma unroll
  for (int i = 0; i < kMaxDV / 32; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  const int ntiles = (p.topk + kBK - 1) / kBK;
  for (int tile_i = 0; tile_i < ntiles; ++tile_i) {
    __syncthreads();
    if (tid < kBK) {
      const int slot = tile_i * kBK + tid;
      const int idx = slot < p.topk ? ctx.idx_row[slot] : -1;
      s_idx[tid] = index_valid(ctx, idx) ? idx : -1;
    }
    __syncthreads();
    const int units = D / 8;  // 16-byte units per row (D % 8 == 0 is checked on the host)
    for (int u = tid; u < kBK * units; u += blockDim.x) {
      const int key = u / units, unit = u - key * units;
      const int idx = s_idx[key];
      uint4 val = make_uint4(0, 0, 0, 0);
      if (idx >= 0)
        val = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.kv) + kv_row(p, ctx.b, idx) * D + unit * 8);
      *reinterpret_cast<uint4*>(tile + key * D + unit * 8) = val;
    }
    __syncthreads();
    for (int j = 0; j < kBK; ++j) {
      if (s_idx[j] < 0) continue;  // uniform across the CTA
      const T* krow = tile + j * D;
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) dot += qreg[i] * static_cast<float>(krow[d]);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float x = dot * p.scale_log2;
      const float m_new = fmaxf(m, x);
      const float f = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
      const float pj = exp2f(x - m_new);
      l = l * f + pj;
      m = m_new;
#pragma unroll
      for (int i = 0; i < kMaxDV / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < DV) acc[i] = acc[i] * f + pj * static_cast<float>(krow[d]);
      }
    }
  }
  if (!head_ok) return;
  T* orow = reinterpret_cast<T*>(p.out) + (static_cast<int64_t>(bt) * p.H + h) * DV;
  const float inv_l = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < kMaxDV / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < DV) orow[d] = static_cast<T>(acc[i] * inv_l);
  }
  if (lane == 0 && p.lse) p.lse[static_cast<int64_t>(bt) * p.H + h] = l > 0.f ? m * 0.6931471805599453f + logf(l) : -INFINITY;
}

// -------------------------------------------------------------------------------------------------
// host launchers (return a cudaError_t as int; 0 = launched)
// -------------------------------------------------------------------------------------------------
bool sparse_mla_fwd_tc_supported(const FwdParams& p) {
  return p.D == tc::kD && p.DV == tc::kDV && p.topk <= tc::kMaxTiles * tc::kBK;
}

int launch_sparse_mla_fwd_tc(const FwdParams& p, bool bf16, cudaStream_t stream) {
  auto kern = bf16 ? sparse_mla_fwd_tc_kernel<true> : sparse_mla_fwd_tc_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(tc::kSmemBytes));
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid(2, p.B * p.S, (p.H + tc::kM - 1) / tc::kM);
  kern<<<grid, tc::kThreads, tc::kSmemBytes, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

int launch_sparse_mla_fwd_generic(const FwdParams& p, bool bf16, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(gen::kBK) * p.D * 2;
  dim3 grid((p.H + gen::kHeadsPerCta - 1) / gen::kHeadsPerCta, p.B * p.S);
  if (bf16)
    sparse_mla_fwd_generic_kernel<__nv_bfloat16><<<grid, 256, smem, stream>>>(p);
  else
    sparse_mla_fwd_generic_kernel<__half><<<grid, 256, smem, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace dsa
