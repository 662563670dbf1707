// Lightning-indexer score kernel for sm_100a.
//
//   score[b, s1, s2] = sum_h w[b, s1, h] * relu( q[b, s1, h, :] . k[b, s2, 0, :] )        (fp32)
//
// with keys at or beyond the row's limit set to -inf (causal rule of sparse_mode 3).  Semantics
// follow cpu_lightning_indexer, examples/deepseek_v4/lightning_indexer.py:303-314.
//
// Tensor-core kernel (D = 128): the MMA is issued transposed -- A = a tile of 128 keys x 128 dims
// (UMMA M = keys), B = (QB queries x N1 heads = 256 rows) x 128 dims -- so the TMEM accumulator has
// one key per lane and all heads of a query in consecutive columns.  The ReLU, the per-head weight
// and the sum over heads are then a per-thread reduction over columns, and a warp writes 32
// consecutive keys of one query row (coalesced).  Two accumulators (2 x 256 TMEM columns) let the
// reduction of tile i overlap the MMAs of tile i+1.  Key tiles are dense (128 consecutive keys x 128 dims): one thread
// fetches each with two TMA tile loads (64 dims x 128 keys, 128-byte swizzle) into a 3-stage ring; when no tensor
// map could be made for k (unaligned pointer) four warps fetch the tiles with cp.async instead.
//
// Generic kernel (any D, any N1): CUDA-core fp32.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>
#include <type_traits>

#include "launch_util.h"
#include "params.h"
#include "ptx.cuh"
#include "tensor_map.h"

namespace dsa {

__device__ __forceinline__ int indexer_limit(const IndexerParams& p, int b, int s1, int* ak_out) {
  const int aq = p.q_len_b ? p.q_len_b[b] : p.S1;
  const int ak = p.k_len_b ? p.k_len_b[b] : p.S2;
  *ak_out = ak;
  if (s1 >= aq || ak <= 0) return 0;
  if (p.sparse_mode == 3) {
    const int cl = ak - aq + s1 + 1;
    return cl > 0 ? (cl < ak ? cl : ak) : ak;
  }
  return ak;
}

namespace itc {
constexpr int kD = 128;
constexpr int kKeys = 128;                         // keys per tile = UMMA M
constexpr int kN = 256;                            // (queries x heads) per CTA = UMMA N
constexpr int kStages = 3;
constexpr uint32_t kQBytes = 2 * kN * 128;         // 65536: 2 chunks of [256 rows x 128 B]
constexpr uint32_t kKStageBytes = 2 * kKeys * 128; // 32768
constexpr uint32_t kOffK = kQBytes;
constexpr uint32_t kOffW = kOffK + kStages * kKStageBytes;  // 163840
constexpr uint32_t kOffBar = kOffW + kN * 4;
constexpr uint32_t kSmemBytes = kOffBar + 256 + 1024;
constexpr int kEpilogueWarps = 8;                  // warp w: keys 32 (w & 3) .. +31 of a tile, half (w >> 2) of the CTA's queries
constexpr int kMmaWarp = 8;
constexpr int kThreads = 416;                      // 8 reduce warps, the MMA warp, 4 producer warps
constexpr uint32_t kTmemCols = 512;
}  // namespace itc

template <bool kBF16, int N1>
__global__ void __launch_bounds__(itc::kThreads, 1)
    indexer_scores_tc_kernel(const __grid_constant__ IndexerParams p, const __grid_constant__ CUtensorMap kmap, const int use_tma) {
  using namespace itc;
  constexpr int QB = kN / N1;  // queries per CTA
  using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + kOffK;
  float* sW = reinterpret_cast<float*>(smem + kOffW);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
  uint64_t* k_full = bars;          // [3] count 1 + 32768 transaction bytes (TMA) or count 128 (cp.async producers)
  uint64_t* k_empty = bars + 3;     // [3] count 1 (commit)
  uint64_t* acc_full = bars + 6;    // [2] count 1 (commit)
  uint64_t* acc_empty = bars + 8;   // [2] count 256
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  int* start_status = reinterpret_cast<int*>(bars + 11);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nqb = (p.S1 + QB - 1) / QB;
  const int b = blockIdx.x / nqb;
  const int qb = nqb - 1 - (blockIdx.x - b * nqb);  // late (long) query blocks first
  const int q0 = qb * QB;

  if (tid == 0) *start_status = *reinterpret_cast<volatile int*>(p.status);
  __syncthreads();
  if (*start_status != kStatusOk) return;

  // key range this CTA has to score: up to the largest limit among its queries
  int ak = 0, max_lim = 0;
  for (int i = 0; i < QB; ++i) {
    const int s1 = q0 + i;
    if (s1 < p.S1) { const int l = indexer_limit(p, b, s1, &ak); max_lim = l > max_lim ? l : max_lim; }
  }
  const int ntiles_mma = (max_lim + kKeys - 1) / kKeys;
  const int ntiles_all = p.fill_masked ? (p.S2 + kKeys - 1) / kKeys : ntiles_mma;

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) { mbar_init(&k_full[i], use_tma ? 1 : 128); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], kEpilogueWarps * 32); }
    mbar_init_fence();
  }
  if (warp == kMmaWarp) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
  {  // Q rows (query, head) -> B operand rows; weights
    const T* qbase = reinterpret_cast<const T*>(p.q) + (static_cast<int64_t>(b) * p.S1 + q0) * N1 * kD;
    for (int u = tid; u < kN * 16; u += kThreads) {
      const int r = u >> 4, unit = u & 15;
      const bool ok = q0 + r / N1 < p.S1;
      const T* src = ok ? qbase + static_cast<int64_t>(r) * kD + unit * 8 : reinterpret_cast<const T*>(p.q);
      cp_async16(sQ + (unit >> 3) * (kN * 128) + sw128_offset(r, unit & 7), src, ok ? 16u : 0u);
    }
    cp_async_commit();
    for (int r = tid; r < kN; r += kThreads)
      sW[r] = (q0 + r / N1 < p.S1) ? p.w[(static_cast<int64_t>(b) * p.S1 + q0) * N1 + r] : 0.f;
    cp_async_wait<0>();
    fence_proxy_async_smem();
  }
  if (p.limits && tid < QB && q0 + tid < p.S1) {
    int dummy;
    p.limits[static_cast<int64_t>(b) * p.S1 + q0 + tid] = indexer_limit(p, b, q0 + tid, &dummy);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp > kMmaWarp) {
    // ================================ key-tile producers ============================================
    const int pt = tid - (kMmaWarp + 1) * 32;
    const T* kbase = reinterpret_cast<const T*>(p.k) + (p.block_table ? 0 : static_cast<int64_t>(b) * p.S2 * kD);
    if (use_tma) {
      // one thread: k as a 2-D tensor [B * S2 keys, 128 dims]; keys past the row's limit (or past the batch entry: they
      // belong to the next one) only produce scores that the reduce warps replace by -inf
      if (pt == 0) {
        prefetch_tensormap(&kmap);
        for (int it = 0; it < ntiles_mma; ++it) {
          const int s = it % kStages;
          if (it >= kStages && !mbar_wait(&k_empty[s], ((it / kStages) + 1) & 1, p.status)) { ok = false; break; }
          const uint32_t stage = sK + s * kKStageBytes, full = smem_u32(&k_full[s]);
          mbar_arrive_expect_tx(&k_full[s], kKStageBytes);
          if (p.block_table) {
            // paged cache: the tile is 128 / box_rows boxes, each inside one block (box_rows divides the block size);
            // a table entry that is padding (< 0) or beyond the pool gives a row coordinate outside the tensor: zeros
            const int R = p.box_rows;
            for (int j = 0; j < kKeys / R; ++j) {
              const int key0 = it * kKeys + j * R, lb = key0 / p.block_size;
              const int phys = lb < p.max_blocks ? __ldg(p.block_table + static_cast<int64_t>(b) * p.max_blocks + lb) : -1;
              const int y = (phys >= 0 && phys < p.num_blocks) ? phys * p.block_size + key0 % p.block_size : -R;
              tma_load_2d(stage + j * R * 128, &kmap, full, 0, y);
              tma_load_2d(stage + kKeys * 128 + j * R * 128, &kmap, full, 64, y);
            }
          } else {
            tma_load_2d(stage, &kmap, full, 0, b * p.S2 + it * kKeys);
            tma_load_2d(stage + kKeys * 128, &kmap, full, 64, b * p.S2 + it * kKeys);
          }
        }
      }
    } else
    for (int it = 0; it < ntiles_mma; ++it) {
      const int s = it % kStages;
      if (it >= kStages && !mbar_wait(&k_empty[s], ((it / kStages) + 1) & 1, p.status)) { ok = false; break; }
      const uint32_t stage = sK + s * kKStageBytes;
#pragma unroll 4
      for (int j = 0; j < 16; ++j) {
        const int u = pt + 128 * j;
        const int r = u >> 4, unit = u & 15;
        const int key = it * kKeys + r;
        bool v = key < ak;
        int64_t row = key;
        if (p.block_table) {  // logical key -> row of the paged cache; padding entries of the table are not read
          const int lb = key / p.block_size;
          const int phys = (v && lb < p.max_blocks) ? __ldg(p.block_table + static_cast<int64_t>(b) * p.max_blocks + lb) : -1;
          v = phys >= 0 && phys < p.num_blocks;
          row = static_cast<int64_t>(phys) * p.block_size + key % p.block_size;
        }
        const T* src = v ? kbase + row * kD + unit * 8 : kbase;
        cp_async16(stage + (unit >> 3) * (kKeys * 128) + sw128_offset(r, unit & 7), src, v ? 16u : 0u);
      }
      cp_async_commit();
      if (it >= 1) {
        cp_async_wait<1>();
        fence_proxy_async_smem();
        mbar_arrive(&k_full[(it - 1) % kStages]);
      }
    }
    cp_async_wait<0>();
    if (!use_tma && ok && ntiles_mma > 0) {
      fence_proxy_async_smem();
      mbar_arrive(&k_full[(ntiles_mma - 1) % kStages]);
    }
  } else if (warp == kMmaWarp) {
    // ================================ MMA issuer ====================================================
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kBF16, kKeys, kN, 0, 0);
      for (int it = 0; it < ntiles_mma; ++it) {
        const int s = it % kStages, a = it & 1;
        if (!mbar_wait(&k_full[s], (it / kStages) & 1, p.status)) { ok = false; break; }
        if (it >= 2 && !mbar_wait(&acc_empty[a], ((it >> 1) + 1) & 1, p.status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t stage = sK + s * kKStageBytes;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t da = make_smem_desc(stage + c * (kKeys * 128) + k * 32, 16, 1024, kSwizzle128B);
            const uint64_t db = make_smem_desc(sQ + c * (kN * 128) + k * 32, 16, 1024, kSwizzle128B);
            umma_ss(tmem_base + a * kN, da, db, idesc, (c | k) != 0);
          }
        }
        umma_commit(&k_empty[s]);
        umma_commit(&acc_full[a]);
      }
    }
  } else {
    // ================================ reduce over heads + store ====================================
    // thread = (key, half of the CTA's queries): the accumulator row of its key, the columns of its queries
    const int q4 = warp & 3, half = warp >> 2;
    const int krow = q4 * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
    constexpr int QH = QB / 2;  // queries per thread
    int lim[QH];
#pragma unroll
    for (int i = 0; i < QH; ++i) {
      int dummy;
      const int qi = half * QH + i;
      lim[i] = (q0 + qi < p.S1) ? indexer_limit(p, b, q0 + qi, &dummy) : 0;
    }
    float* out = p.scores + (static_cast<int64_t>(b) * p.S1 + q0 + half * QH) * p.S2;
    for (int it = 0; it < ntiles_all; ++it) {
      const int key = it * kKeys + krow;
      if (it < ntiles_mma) {
        const int a = it & 1;
        if (!mbar_wait(&acc_full[a], (it >> 1) & 1, p.status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tacc = tmem_base + a * kN + half * (kN / 2) + lane_base;
        const float4* w4 = reinterpret_cast<const float4*>(sW + half * (kN / 2));  // weights of this half, 4 per (broadcast) load
        if constexpr (N1 >= 32) {
#pragma unroll
          for (int i = 0; i < QH; ++i) {
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int cc = 0; cc < N1 / 32; ++cc) {
              uint32_t v[32];
              tmem_ld32(tacc + i * N1 + cc * 32, v);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 w = w4[(i * N1 + cc * 32) / 4 + j];
                s0 = fmaf(w.x, fmaxf(__uint_as_float(v[4 * j]), 0.f), s0);
                s1 = fmaf(w.y, fmaxf(__uint_as_float(v[4 * j + 1]), 0.f), s1);
                s0 = fmaf(w.z, fmaxf(__uint_as_float(v[4 * j + 2]), 0.f), s0);
                s1 = fmaf(w.w, fmaxf(__uint_as_float(v[4 * j + 3]), 0.f), s1);
              }
            }
            if (q0 + half * QH + i < p.S1 && key < p.S2) out[static_cast<int64_t>(i) * p.S2 + key] = key < lim[i] ? s0 + s1 : -INFINITY;
          }
        } else {
          constexpr int QPC = 32 / N1;  // queries per 32-column chunk
#pragma unroll
          for (int cc = 0; cc < kN / 64; ++cc) {
            uint32_t v[32];
            tmem_ld32(tacc + cc * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int qq = 0; qq < QPC; ++qq) {
              float sum = 0.f;
#pragma unroll
              for (int j = 0; j < N1 / 4; ++j) {
                const float4 w = w4[(cc * 32 + qq * N1) / 4 + j];
                sum = fmaf(w.x, fmaxf(__uint_as_float(v[qq * N1 + 4 * j]), 0.f), sum);
                sum = fmaf(w.y, fmaxf(__uint_as_float(v[qq * N1 + 4 * j + 1]), 0.f), sum);
                sum = fmaf(w.z, fmaxf(__uint_as_float(v[qq * N1 + 4 * j + 2]), 0.f), sum);
                sum = fmaf(w.w, fmaxf(__uint_as_float(v[qq * N1 + 4 * j + 3]), 0.f), sum);
              }
              const int i = cc * QPC + qq;
              if (q0 + half * QH + i < p.S1 && key < p.S2) out[static_cast<int64_t>(i) * p.S2 + key] = key < lim[i] ? sum : -INFINITY;
            }
          }
        }
        tc_fence_before();
        mbar_arrive(&acc_empty[a]);
      } else if (key < p.S2) {  // tile entirely beyond every limit of this CTA
#pragma unroll
        for (int i = 0; i < QH; ++i)
          if (q0 + half * QH + i < p.S1) out[static_cast<int64_t>(i) * p.S2 + key] = -INFINITY;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem_base, kTmemCols);
}

// -------------------------------------------------------------------------------------------------
// generic CUDA-core kernel: one CTA per (batch, query), one thread per key (strided)
// -------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) indexer_scores_generic_kernel(const IndexerParams p) {
  extern __shared__ float sq[];  // [N1 * D] query heads in fp32, then [N1] weights
  float* sw = sq + p.N1 * p.D;
  const int b = blockIdx.y, s1 = blockIdx.x;
  const T* qrow = reinterpret_cast<const T*>(p.q) + (static_cast<int64_t>(b) * p.S1 + s1) * p.N1 * p.D;
  for (int i = threadIdx.x; i < p.N1 * p.D; i += blockDim.x) sq[i] = static_cast<float>(qrow[i]);
  for (int i = threadIdx.x; i < p.N1; i += blockDim.x) sw[i] = p.w[(static_cast<int64_t>(b) * p.S1 + s1) * p.N1 + i];
  __syncthreads();
  int ak;
  const int lim = indexer_limit(p, b, s1, &ak);
  if (p.limits && threadIdx.x == 0) p.limits[static_cast<int64_t>(b) * p.S1 + s1] = lim;
  float* out = p.scores + (static_cast<int64_t>(b) * p.S1 + s1) * p.S2;
  const int kend = p.fill_masked ? p.S2 : lim;
  for (int key = threadIdx.x; key < kend; key += blockDim.x) {
    float score = -INFINITY;
    if (key < lim) {
      int64_t row = static_cast<int64_t>(b) * p.S2 + key;
      if (p.block_table) {
        const int lb = key / p.block_size;
        const int phys = lb < p.max_blocks ? p.block_table[static_cast<int64_t>(b) * p.max_blocks + lb] : -1;
        if (phys < 0 || phys >= p.num_blocks) { out[key] = 0.f; continue; }  // a candidate key without a block: no contribution
        row = static_cast<int64_t>(phys) * p.block_size + key % p.block_size;
      }
      const T* krow = reinterpret_cast<const T*>(p.k) + row * p.D;
      score = 0.f;
      for (int h = 0; h < p.N1; ++h) {
        float dot = 0.f;
        for (int d = 0; d < p.D; ++d) dot = fmaf(sq[h * p.D + d], static_cast<float>(krow[d]), dot);
        score = fmaf(sw[h], fmaxf(dot, 0.f), score);
      }
    }
    out[key] = score;
  }
}

bool indexer_tc_supported(const IndexerParams& p) {
  return p.D == itc::kD && (p.N1 == 64 || p.N1 == 32 || p.N1 == 16 || p.N1 == 8);
}

namespace {
// k [B * S2, 128] as a tensor map with a box of 64 dims x 128 keys in the 128-byte swizzle; false when that is not
// possible (then the kernel's cp.async producers fetch the tiles)
bool make_k_map(const IndexerParams& p, bool bf16, CUtensorMap* map) {
  // paged cache: all rows of the pool; a box must lie inside one block, so its row count has to divide the block size
  const long long rows = p.block_table ? static_cast<long long>(p.num_blocks) * p.block_size : static_cast<long long>(p.B) * p.S2;
  if (p.block_table && (p.box_rows < 8 || itc::kKeys % p.box_rows != 0 || p.block_size % p.box_rows != 0)) return false;
  return encode_rows_map(p.k, rows, itc::kD, bf16, p.block_table ? p.box_rows : itc::kKeys, map);
}
}  // namespace

template <bool kBF16, int N1>
static int launch_indexer_tc_n1(const IndexerParams& p_in, cudaStream_t stream) {
  IndexerParams p = p_in;
  // rows per TMA box of a paged cache: the largest power of two (8..128) that divides the block size
  p.box_rows = 0;
  if (p.block_table)
    for (int r = itc::kKeys; r >= 8; r >>= 1)
      if (p.block_size % r == 0) { p.box_rows = r; break; }
  auto kern = indexer_scores_tc_kernel<kBF16, N1>;
  int dev = 0, sms = 0;
  cudaError_t e = current_device_sms(&dev, &sms);
  if (e != cudaSuccess) return static_cast<int>(e);
  if ((e = ensure_dynamic_smem(kern, dev, static_cast<int>(itc::kSmemBytes))) != cudaSuccess) return static_cast<int>(e);
  constexpr int QB = itc::kN / N1;
  const int nqb = (p.S1 + QB - 1) / QB;
  alignas(64) CUtensorMap kmap;
  memset(&kmap, 0, sizeof(kmap));
  // DSA_INDEXER_NO_TMA=1 in the environment forces the cp.async producers (used by the tests to cover that path)
  const char* no_tma = getenv("DSA_INDEXER_NO_TMA");
  const int use_tma = (!(no_tma && no_tma[0] == '1') && make_k_map(p, kBF16, &kmap)) ? 1 : 0;
  kern<<<p.B * nqb, itc::kThreads, itc::kSmemBytes, stream>>>(p, kmap, use_tma);
  return static_cast<int>(cudaGetLastError());
}

int launch_indexer_scores_tc(const IndexerParams& p, bool bf16, cudaStream_t stream) {
  switch (p.N1) {
    case 64: return bf16 ? launch_indexer_tc_n1<true, 64>(p, stream) : launch_indexer_tc_n1<false, 64>(p, stream);
    case 32: return bf16 ? launch_indexer_tc_n1<true, 32>(p, stream) : launch_indexer_tc_n1<false, 32>(p, stream);
    case 16: return bf16 ? launch_indexer_tc_n1<true, 16>(p, stream) : launch_indexer_tc_n1<false, 16>(p, stream);
    case 8: return bf16 ? launch_indexer_tc_n1<true, 8>(p, stream) : launch_indexer_tc_n1<false, 8>(p, stream);
    default: return static_cast<int>(cudaErrorInvalidValue);
  }
}

int launch_indexer_scores_generic(const IndexerParams& p, bool bf16, cudaStream_t stream) {
  const size_t smem = (static_cast<size_t>(p.N1) * p.D + p.N1) * sizeof(float);
  dim3 grid(p.S1, p.B);
  cudaError_t e;
  if (bf16) {
    e = cudaFuncSetAttribute(indexer_scores_generic_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    indexer_scores_generic_kernel<__nv_bfloat16><<<grid, 256, smem, stream>>>(p);
  } else {
    e = cudaFuncSetAttribute(indexer_scores_generic_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    indexer_scores_generic_kernel<__half><<<grid, 256, smem, stream>>>(p);
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace dsa
