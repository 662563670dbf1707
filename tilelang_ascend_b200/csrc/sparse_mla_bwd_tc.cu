// Sparse MLA backward on the tensor cores (sm_100a, D = 576, DV = 512).
//
//   P  = exp(sm_scale * Q K^T - lse)            dP = dO V^T             dS = P * (dP - delta) * sm_scale
//   dQ = dS K                                   dKV[idx] += dS^T Q  (576 dims)  +  P^T dO  (first 512 dims)
//
// The five contractions do not fit one CTA's tensor memory (dQ alone is 128 x 576 fp32 = 576 of the 512 columns),
// so the work is cut into four tcgen05 kernels that hand P and dS (input dtype) to each other through a workspace.
// The workspace traffic is small next to the arithmetic (two 16 KB tiles per 64 keys of a query, against 90 MFLOP).
// A pass handles `nq` consecutive queries:
//
//   prep    delta = sum_d dO*O per (query, head); 64-bit validity mask per (query, tile of 64 keys)
//   scores  MODE 0: S = Q K^T   (A = Q of 128 heads in tensor memory, B = gathered KV rows, 9 chunks of 64 dims)  -> P
//           MODE 1: dP = dO V^T (A = dO in tensor memory, B = the first 8 chunks of the same rows)                 -> dS
//   dq      dQ[:, 192 i .. 192 i + 191] = sum over tiles of dS_tile . K_tile   (three CTAs per query, one per 192 dims)
//   dkv     for 128 keys at a time: dS^T Q[:, its 192 dims] + P^T dO[:, its dims]  -> fp32 vector atomics into dKV
//
// P / dS tiles are stored in the workspace as the exact shared-memory image the consumers need ([128 heads x 64 keys],
// rows of 128 bytes in the 128-byte swizzle), so dq and dkv fetch a tile with ONE bulk copy (cp.async.bulk) and use it
// as a K-major A operand (dq: contraction over keys) or an MN-major A operand (dkv: contraction over heads).
// The reference has no sparse-MLA backward; the decomposition (delta preprocess, P recomputed from the saved LSE,
// fp32 atomic accumulation of the key gradient) is the one its dense backward uses
// (examples_experiment/example_gqa_bwd/example_gqa_bwd.py:189-223, 312-556).
#include <type_traits>

#include "params.h"
#include "ptx.cuh"

namespace dsa {

namespace bwdtc {
constexpr int kD = 576, kDV = 512;
constexpr int kM = 128;                        // heads per CTA = UMMA M
constexpr int kBK = 64;                        // keys per tile
constexpr int kMaxTiles = 128;                 // topk <= 8192
constexpr uint32_t kChunkBytes = kBK * 128;    // 64 keys x 64 dims, 128-byte swizzle
constexpr uint32_t kTileBytes = kM * 128;      // one P / dS tile: 128 heads x 64 keys
constexpr int kThreads = 288;                  // warps 0-3 epilogue, 4-7 gather / loads, 8 MMA issuer
constexpr int kMmaWarp = 8;
// Index lists of up to this many entries are copied to shared memory when a CTA starts (one memory latency for the whole
// list); longer lists are read from global memory tile by tile, one exposed latency per tile.
constexpr int kIdxInSmem = 2048;

// Workspace of one pass, carved by the host launcher.
struct Pass {
  uint8_t* p_ws;               // [nq][head_blocks][ntiles2][kTileBytes]
  uint8_t* ds_ws;              // same shape
  unsigned long long* masks;   // [nq][ntiles2]
  float* delta;                // [nq][head_blocks * 128]
  int q0, nq;                  // first query (b * S + t) of the pass and number of queries
  int ntiles, ntiles2;         // tiles of 64 keys per query; rounded up to even
  int head_blocks;
};

__device__ __forceinline__ int64_t kv_row_of(const FwdParams& p, int b, int idx) {
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
template <bool kBF16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (kBF16) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w));
  } else {
    return __half22float2(*reinterpret_cast<__half2*>(&w));
  }
}

// Contiguous global -> shared copy by the copy engine (16-byte aligned addresses, size a multiple of 16); its bytes are
// subtracted from the transaction count of `mbar` (this CTA).
__device__ __forceinline__ void bulk_copy_g2s(uint32_t smem_dst, const void* src, uint32_t bytes, uint64_t* mbar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_dst), "l"(src),
               "r"(bytes), "r"(smem_u32(mbar))
               : "memory");
}

// 16 gathered rows (one per entry of rows[], -1 = zero fill) x kChunks chunks of 64 dims starting at chunk `chunk0` of
// the row, into the K-major / 128-byte-swizzle chunk images of a stage: chunk c at stage + c * kChunkBytes, key
// 16 pw + kk is row 16 pw + kk of every chunk.  Lane = (chunk within a group of four, 16-byte unit).
template <int kChunks>
__device__ __forceinline__ void gather_rows(uint32_t stage, const uint8_t* kv_bytes, int chunk0, const int (&rows)[16], int pw, int lane) {
#pragma unroll
  for (int c0 = 0; c0 < kChunks; c0 += 4) {
    const int c = c0 + (lane >> 3);
    if (c < kChunks) {
      const uint8_t* src = kv_bytes + (chunk0 + c) * 128 + (lane & 7) * 16;
      const uint32_t dst = stage + c * kChunkBytes + pw * 2048;
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) {
        const uint32_t row = static_cast<uint32_t>(rows[kk] < 0 ? 0 : rows[kk]);
        cp_async16(dst + sw128_offset(kk, lane & 7), src + static_cast<size_t>(row) * (kD * 2), rows[kk] < 0 ? 0u : 16u);
      }
    }
  }
}
}  // namespace bwdtc

// -------------------------------------------------------------------------------------------------
// prep: delta and validity masks of a pass
// -------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) sparse_mla_bwd_prep_kernel(const BwdParams bp, const bwdtc::Pass ps) {
  using namespace bwdtc;
  const FwdParams& p = bp.f;
  const int ql = blockIdx.x, bt = ps.q0 + ql;
  const int b = bt / p.S, t = bt - b * p.S;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool active = p.q_len_b ? (t < p.q_len_b[b]) : true;
  const int qs = p.q_start_b ? p.q_start_b[b] : p.q_start;
  const int kv_len = p.kv_len_b ? p.kv_len_b[b] : p.S_kv;
  const int pos_limit = p.causal ? qs + t : 0x7fffffff;
  const int32_t* idx_row = p.indices + static_cast<int64_t>(bt) * p.topk;
  for (int tile = warp; tile < ps.ntiles2; tile += 8) {
    const int s0 = tile * kBK + lane, s1 = s0 + 32;
    const int i0 = (tile < ps.ntiles && s0 < p.topk) ? __ldg(idx_row + s0) : -1;
    const int i1 = (tile < ps.ntiles && s1 < p.topk) ? __ldg(idx_row + s1) : -1;
    const uint32_t lo = __ballot_sync(0xffffffffu, active && i0 >= 0 && i0 < kv_len && i0 <= pos_limit);
    const uint32_t hi = __ballot_sync(0xffffffffu, active && i1 >= 0 && i1 < kv_len && i1 <= pos_limit);
    if (lane == 0) ps.masks[static_cast<int64_t>(ql) * ps.ntiles2 + tile] = (static_cast<unsigned long long>(hi) << 32) | lo;
  }
  // delta[h] = sum over the 512 output dims of dO * O: one warp per head, 16 dims per lane
  const int hpad = ps.head_blocks * kM;
  for (int h = warp; h < hpad; h += 8) {
    float acc = 0.f;
    if (h < p.H) {
      const T* o = reinterpret_cast<const T*>(p.out) + (static_cast<int64_t>(bt) * p.H + h) * kDV + lane * 16;
      const T* g = reinterpret_cast<const T*>(bp.d_out) + (static_cast<int64_t>(bt) * p.H + h) * kDV + lane * 16;
      uint4 ov[2], gv[2];
      ov[0] = __ldg(reinterpret_cast<const uint4*>(o)); ov[1] = __ldg(reinterpret_cast<const uint4*>(o) + 1);
      gv[0] = __ldg(reinterpret_cast<const uint4*>(g)); gv[1] = __ldg(reinterpret_cast<const uint4*>(g) + 1);
      const T* oe = reinterpret_cast<const T*>(ov);
      const T* ge = reinterpret_cast<const T*>(gv);
#pragma unroll
      for (int j = 0; j < 16; ++j) acc += static_cast<float>(oe[j]) * static_cast<float>(ge[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) ps.delta[static_cast<int64_t>(ql) * hpad + h] = acc;
  }
}

// -------------------------------------------------------------------------------------------------
// scores: P (MODE 0) or dS (MODE 1) tiles of one (query, block of 128 heads) per CTA
// -------------------------------------------------------------------------------------------------
namespace bwdtc {
template <int MODE>
struct ScoresCfg {
  static constexpr int kChunks = MODE == 0 ? 9 : 8;          // 64-dim chunks of the contraction: all of D, or the DV dims
  static constexpr int kStages = 3;
  static constexpr uint32_t kStageBytes = kChunks * kChunkBytes;
  static constexpr uint32_t kOffBar = kStages * kStageBytes;
  static constexpr uint32_t kOffMask = kOffBar + 256;
  static constexpr uint32_t kOffIdx = kOffMask + kMaxTiles * 8;             // the query's index list (when it has at most kIdxInSmem entries)
  static constexpr uint32_t kSmemBytes = kOffIdx + kIdxInSmem * 4 + 1024;   // + slack to align the base to 1024 B
  // Tensor memory: the A operand (288 or 256 columns), then a ring of score buffers of 64 columns.  The hand-over of a
  // buffer (commit -> epilogue wakes -> tensor-memory load -> "free" arrive -> issuer wakes) takes longer than the MMAs of a
  // tile, so two buffers leave the tensor pipe idle most of the time; three (four) cover it.
  static constexpr int kSBufs = MODE == 0 ? 3 : 4;
  static constexpr uint32_t kColA = 0, kColS = MODE == 0 ? 288 : 256;
  static_assert(kColS + kSBufs * kBK <= 512, "tensor memory columns");
  static_assert(kSmemBytes <= 232448, "shared memory per CTA");
};
}  // namespace bwdtc

template <bool kBF16, int MODE>
__global__ void __launch_bounds__(bwdtc::kThreads, 1) sparse_mla_bwd_scores_kernel(const BwdParams bp, const bwdtc::Pass ps) {
  using namespace bwdtc;
  using Cfg = ScoresCfg<MODE>;
  constexpr int kChunks = Cfg::kChunks, kStages = Cfg::kStages;
  const FwdParams& p = bp.f;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sBase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBar);
  uint64_t* kv_full = bars;        // [3] count 128: cp.async completion of the gather threads
  uint64_t* kv_empty = bars + 3;   // [3] count 1: commit after the MMAs that read the stage
  uint64_t* s_full = bars + 6;     // [kSBufs] count 1: commit after the MMAs of a tile
  uint64_t* s_free = bars + 10;    // [kSBufs] count 4: the epilogue warps have read the buffer out of tensor memory
  uint64_t* a_ready = bars + 14;   // count 4: the A operand is in tensor memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  constexpr int kSBufs = Cfg::kSBufs;
  unsigned long long* smask = reinterpret_cast<unsigned long long*>(smem + Cfg::kOffMask);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ql = blockIdx.x / ps.head_blocks, hb = blockIdx.x - ql * ps.head_blocks;
  const int bt = ps.q0 + ql, b = bt / p.S, h0 = hb * kM;
  const int64_t tile0 = (static_cast<int64_t>(ql) * ps.head_blocks + hb) * ps.ntiles2;  // first tile of this item in the workspace

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) { mbar_init(&kv_full[i], 128); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < kSBufs; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_free[i], 4); }
    mbar_init(a_ready, 4);
    mbar_init_fence();
  }
  for (int i = tid; i < ps.ntiles; i += kThreads) smask[i] = ps.masks[static_cast<int64_t>(ql) * ps.ntiles2 + i];
  int32_t* sidx = reinterpret_cast<int32_t*>(smem + Cfg::kOffIdx);
  const bool idx_in_smem = p.topk <= kIdxInSmem;
  if (idx_in_smem)
    for (int i = tid; i < p.topk; i += kThreads) sidx[i] = __ldg(p.indices + static_cast<int64_t>(bt) * p.topk + i);
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tA = tmem_base + Cfg::kColA, tS = tmem_base + Cfg::kColS;
  const bool run = *reinterpret_cast<volatile int*>(p.status) == kStatusOk;
  bool ok = true;

  // ---- A operand: rows of Q (MODE 0) or dO (MODE 1) of the 128 heads -> tensor memory, through shared memory -------------
  // A row per lane straight from global memory makes every load instruction touch 32 rows (18 us per CTA, a quarter of its
  // time).  All threads copy the rows -- contiguous in memory -- with whole 128-byte lines into the (still unused) stage ring
  // as chunks of [128 rows x 128 bytes] in the 128-byte swizzle; the thread of a row then reads its row conflict-free.
  {
    constexpr int kRowB = MODE == 0 ? kD * 2 : kDV * 2;
    static_assert(kChunks * 16384u <= Cfg::kStages * Cfg::kStageBytes, "the staged rows fit the stage ring");
    const int nrows = p.H - h0 < kM ? p.H - h0 : kM;
    const uint8_t* abase = (MODE == 0 ? reinterpret_cast<const uint8_t*>(p.q) : reinterpret_cast<const uint8_t*>(bp.d_out)) +
                           (static_cast<int64_t>(bt) * p.H + h0) * kRowB;
    for (int i = tid; i < kChunks * 1024; i += kThreads) {
      const int unit = i & 7, row = (i >> 3) & 127, c = i >> 10;
      const bool v = row < nrows;
      cp_async16(sBase + c * 16384 + sw128_offset(row, unit), v ? abase + static_cast<int64_t>(row) * kRowB + c * 128 + unit * 16 : abase, v ? 16u : 0u);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    if (warp < 4) {
      const int r = warp * 32 + lane;
      const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c) {
        uint32_t w[32];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint4 v = ld_shared_v4(sBase + c * 16384 + sw128_offset(r, j));
          w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
        }
        tmem_st32(tA + lane_base + c * 32, w);   // column c' of the row holds dims 2c', 2c' + 1
      }
      tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();   // the ring is free for the gather; the A operand is in tensor memory
    tc_fence_after();
  }

  if (warp >= 4 && warp < 8) {
    // ================================ gather producers ==============================================
    const int pw = warp - 4;  // keys [16 pw, 16 pw + 16) of every tile
    const uint8_t* kv_bytes = reinterpret_cast<const uint8_t*>(p.kv);
    const int32_t* idx_row = p.indices + static_cast<int64_t>(bt) * p.topk;
    int g = 0;
    for (int tile = 0; run && ok && tile < ps.ntiles; ++tile) {
      const unsigned long long mask = smask[tile];
      if (mask == 0ull) continue;
      const int s = g % kStages;
      const int key = pw * 16 + (lane & 15);
      const bool valid = (mask >> key) & 1ull;
      const int my_idx = valid ? (idx_in_smem ? sidx[tile * kBK + key] : __ldg(idx_row + tile * kBK + key)) : 0;
      const int my_row = valid ? static_cast<int>(kv_row_of(p, b, my_idx)) : -1;
      int rows[16];
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) rows[kk] = __shfl_sync(0xffffffffu, my_row, kk);
      if (g >= kStages && !__all_sync(0xffffffffu, mbar_wait(&kv_empty[s], ((g / kStages) + 1) & 1, p.status))) { ok = false; break; }
      gather_rows<kChunks>(sBase + s * Cfg::kStageBytes, kv_bytes, 0, rows, pw, lane);
      cp_async_arrive_noinc(&kv_full[s]);
      ++g;
    }
    cp_async_wait<0>();
  } else if (warp == kMmaWarp) {
    // ================================ MMA issuer ====================================================
    // the whole warp walks the loop and waits, converged; one elected lane issues through predicated instructions
    if (run) {
      constexpr uint32_t idesc = make_idesc_f16(kBF16, kM, kBK, 0, 0);
      const uint32_t go = elect_one_lane();
      int g = 0;
      ok = __all_sync(0xffffffffu, mbar_wait(a_ready, 0, p.status));
      for (int tile = 0; ok && tile < ps.ntiles; ++tile) {
        if (smask[tile] == 0ull) continue;
        const int s = g % kStages, sb = g % kSBufs;
        const uint32_t stage = sBase + s * Cfg::kStageBytes;
        if (!__all_sync(0xffffffffu, mbar_wait(&kv_full[s], (g / kStages) & 1, p.status))) { ok = false; break; }
        if (g >= kSBufs && !__all_sync(0xffffffffu, mbar_wait(&s_free[sb], ((g / kSBufs) + 1) & 1, p.status))) { ok = false; break; }
        fence_proxy_async_smem();  // the gathered rows were written by cp.async of other threads
        tc_fence_after();
        const uint64_t db0 = make_smem_desc(stage, 16, 1024, kSwizzle128B);
#pragma unroll
        for (int c = 0; c < kChunks; ++c) {
#pragma unroll
          for (int kq = 0; kq < 4; ++kq)
            umma_ts_if(go, tS + sb * kBK, tA + (c * 4 + kq) * 8, db0 + ((c * kChunkBytes + kq * 32) >> 4), idesc, (c | kq) != 0);
        }
        umma_commit_if(go, &s_full[sb]);
        umma_commit_if(go, &kv_empty[s]);
        ++g;
      }
    }
  } else {
    // ================================ A operand + epilogue ==========================================
    // thread = head row r = tensor-memory lane.
    const int r = warp * 32 + lane, h = h0 + r;
    const bool row_ok = h < p.H;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    if (lane == 0) mbar_arrive(a_ready);   // (the rows went to tensor memory before the roles split, see above)
    // MODE 0: lse in log2 units (+inf for rows without a head: P = 0); MODE 1: delta
    float row_c;
    if (MODE == 0) row_c = row_ok ? p.lse[static_cast<int64_t>(bt) * p.H + h] * 1.4426950408889634f : INFINITY;
    else row_c = ps.delta[static_cast<int64_t>(ql) * (ps.head_blocks * kM) + r + h0];
    int g = 0;
    for (int tile = 0; run && ok && tile < ps.ntiles; ++tile) {
      const unsigned long long mask = smask[tile];
      if (mask == 0ull) continue;
      const int sb = g % kSBufs;
      uint32_t sc[64];
      const uint8_t* p_tile = ps.p_ws + (tile0 + tile) * kTileBytes;
      uint4 pv[8];  // MODE 1: this row's P values of the tile, requested before the wait so that their latency hides behind it
      if (MODE == 1) {
#pragma unroll
        for (int u = 0; u < 8; ++u) pv[u] = *reinterpret_cast<const uint4*>(p_tile + sw128_offset(r, u));
      }
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[sb], (g / kSBufs) & 1, p.status))) { ok = false; break; }
      tc_fence_after();
      tmem_ld32(tS + sb * kBK + lane_base, sc);
      tmem_ld32(tS + sb * kBK + 32 + lane_base, sc + 32);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[sb]);
      uint8_t* out_tile = (MODE == 0 ? ps.p_ws : ps.ds_ws) + (tile0 + tile) * kTileBytes;
#pragma unroll
      for (int u = 0; u < 8; ++u) {  // 16-byte unit u = keys 8u .. 8u + 7 of this row
        const uint32_t off = sw128_offset(r, u);
        uint32_t w[4];
        if (MODE == 0) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int k0 = 8 * u + 2 * j;
            float e0 = exp2f(__uint_as_float(sc[k0]) * p.scale_log2 - row_c);
            float e1 = exp2f(__uint_as_float(sc[k0 + 1]) * p.scale_log2 - row_c);
            e0 = ((mask >> k0) & 1ull) ? e0 : 0.f;
            e1 = ((mask >> (k0 + 1)) & 1ull) ? e1 : 0.f;
            w[j] = pack2<kBF16>(e0, e1);
          }
        } else {
          const uint32_t pw4[4] = {pv[u].x, pv[u].y, pv[u].z, pv[u].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int k0 = 8 * u + 2 * j;
            const float2 pp = unpack2<kBF16>(pw4[j]);
            w[j] = pack2<kBF16>(pp.x * (__uint_as_float(sc[k0]) - row_c) * bp.sm_scale, pp.y * (__uint_as_float(sc[k0 + 1]) - row_c) * bp.sm_scale);
          }
        }
        *reinterpret_cast<uint4*>(out_tile + off) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      ++g;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem_base, 512);
}

// -------------------------------------------------------------------------------------------------
// dq: dQ[:, 192 i .. 192 i + 191] of one (query, block of 128 heads) per CTA, two CTAs per SM
// -------------------------------------------------------------------------------------------------
namespace bwdtc {
constexpr int kDimsPerCta = 192;                                // three 64-dim chunks
constexpr int kDimSplits = kD / kDimsPerCta;                    // 3
namespace dq {
constexpr int kStages = 2;
constexpr uint32_t kBBytes = 3 * kChunkBytes;                   // gathered rows: 64 keys x 192 dims
constexpr uint32_t kStageBytes = kTileBytes + kBBytes;          // dS tile + rows
constexpr uint32_t kOffBar = kStages * kStageBytes;
constexpr uint32_t kOffMask = kOffBar + 128;
constexpr uint32_t kOffIdx = kOffMask + kMaxTiles * 8;
constexpr uint32_t kSmemBytes = kOffIdx + kIdxInSmem * 4 + 1024;
constexpr uint32_t kTmemCols = 256;
static_assert(2 * kSmemBytes <= 232448 - 2048, "two CTAs per SM");
}  // namespace dq
}  // namespace bwdtc

template <bool kBF16>
__global__ void __launch_bounds__(bwdtc::kThreads, 2) sparse_mla_bwd_dq_kernel(const BwdParams bp, const bwdtc::Pass ps) {
  using namespace bwdtc;
  using namespace bwdtc::dq;
  const FwdParams& p = bp.f;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sBase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
  uint64_t* kv_full = bars;        // [2] count 128: gathered rows landed
  uint64_t* a_full = bars + 2;     // [2] count 1 + 16384 transaction bytes: the dS tile landed
  uint64_t* empty = bars + 4;      // [2] count 1: commit after the MMAs that read the stage
  uint64_t* done = bars + 6;       // count 1: commit after the last MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
  unsigned long long* smask = reinterpret_cast<unsigned long long*>(smem + kOffMask);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int part = blockIdx.x % kDimSplits;
  const int item = blockIdx.x / kDimSplits;
  const int ql = item / ps.head_blocks, hb = item - ql * ps.head_blocks;
  const int bt = ps.q0 + ql, b = bt / p.S, h0 = hb * kM;
  const int64_t tile0 = (static_cast<int64_t>(ql) * ps.head_blocks + hb) * ps.ntiles2;

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) { mbar_init(&kv_full[i], 128); mbar_init(&a_full[i], 1); mbar_init(&empty[i], 1); }
    mbar_init(done, 1);
    mbar_init_fence();
  }
  for (int i = tid; i < ps.ntiles; i += kThreads) smask[i] = ps.masks[static_cast<int64_t>(ql) * ps.ntiles2 + i];
  int32_t* sidx = reinterpret_cast<int32_t*>(smem + kOffIdx);
  const bool idx_in_smem = p.topk <= kIdxInSmem;
  if (idx_in_smem)
    for (int i = tid; i < p.topk; i += kThreads) sidx[i] = __ldg(p.indices + static_cast<int64_t>(bt) * p.topk + i);
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tD = *tmem_slot;
  const bool run = *reinterpret_cast<volatile int*>(p.status) == kStatusOk;
  bool ok = true;
  int ntl = 0;  // tiles with at least one key taking part
  for (int tile = 0; tile < ps.ntiles; ++tile) ntl += smask[tile] != 0ull;

  if (warp >= 4 && warp < 8) {
    // ================================ gather producers + dS tile loads ==============================
    const int pw = warp - 4;
    const uint8_t* kv_bytes = reinterpret_cast<const uint8_t*>(p.kv);
    const int32_t* idx_row = p.indices + static_cast<int64_t>(bt) * p.topk;
    int g = 0;
    for (int tile = 0; run && ok && tile < ps.ntiles; ++tile) {
      const unsigned long long mask = smask[tile];
      if (mask == 0ull) continue;
      const int s = g % kStages;
      const int key = pw * 16 + (lane & 15);
      const bool valid = (mask >> key) & 1ull;
      const int my_idx = valid ? (idx_in_smem ? sidx[tile * kBK + key] : __ldg(idx_row + tile * kBK + key)) : 0;
      const int my_row = valid ? static_cast<int>(kv_row_of(p, b, my_idx)) : -1;
      int rows[16];
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) rows[kk] = __shfl_sync(0xffffffffu, my_row, kk);
      if (g >= kStages && !__all_sync(0xffffffffu, mbar_wait(&empty[s], ((g / kStages) + 1) & 1, p.status))) { ok = false; break; }
      const uint32_t stage = sBase + s * kStageBytes;
      if (pw == 0 && lane == 0) {
        mbar_arrive_expect_tx(&a_full[s], kTileBytes);
        bulk_copy_g2s(stage, ps.ds_ws + (tile0 + tile) * kTileBytes, kTileBytes, &a_full[s]);
      }
      gather_rows<3>(stage + kTileBytes, kv_bytes, 3 * part, rows, pw, lane);
      cp_async_arrive_noinc(&kv_full[s]);
      ++g;
    }
    cp_async_wait<0>();
  } else if (warp == kMmaWarp) {
    // ================================ MMA issuer ====================================================
    // D[128 heads x 192 dims] += dS[128 x 64 keys] (K-major, 16 keys = 32 bytes per step) . rows[64 keys x 192 dims] (MN-major)
    if (run) {  // converged warp, one elected lane issues
      constexpr uint32_t idesc = make_idesc_f16(kBF16, kM, kDimsPerCta, 0, 1);
      const uint32_t go = elect_one_lane();
      int g = 0;
      for (int tile = 0; ok && tile < ps.ntiles; ++tile) {
        if (smask[tile] == 0ull) continue;
        const int s = g % kStages;
        const uint32_t stage = sBase + s * kStageBytes;
        if (!__all_sync(0xffffffffu, mbar_wait(&a_full[s], (g / kStages) & 1, p.status))) { ok = false; break; }
        if (!__all_sync(0xffffffffu, mbar_wait(&kv_full[s], (g / kStages) & 1, p.status))) { ok = false; break; }
        fence_proxy_async_smem();
        tc_fence_after();
        const uint64_t da0 = make_smem_desc(stage, 16, 1024, kSwizzle128B);
        const uint64_t db0 = make_smem_desc(stage + kTileBytes, kChunkBytes, 1024, kSwizzle128B);
#pragma unroll
        for (int ks = 0; ks < kBK / 16; ++ks)
          umma_ss_if(go, tD, da0 + ((ks * 32) >> 4), db0 + ((ks * 2048) >> 4), idesc, (g | ks) != 0);
        umma_commit_if(go, &empty[s]);
        ++g;
      }
      if (ok && g > 0) umma_commit_if(go, done);
    }
  } else {
    // ================================ epilogue ======================================================
    const int r = warp * 32 + lane, h = h0 + r;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;
    T* drow = reinterpret_cast<T*>(bp.d_q) + (static_cast<int64_t>(bt) * p.H + h) * kD + part * kDimsPerCta;
    if (ntl == 0) {
      if (h < p.H)
        for (int j = 0; j < kDimsPerCta / 8; ++j) reinterpret_cast<uint4*>(drow)[j] = make_uint4(0, 0, 0, 0);
    } else if (run) {
      ok = __all_sync(0xffffffffu, mbar_wait<true>(done, 0, p.status));
      tc_fence_after();
      if (ok) {
#pragma unroll 1
        for (int cc = 0; cc < kDimsPerCta / 32; ++cc) {
          uint32_t v[32];
          tmem_ld32(tD + lane_base + cc * 32, v);
          tmem_wait_ld();
          if (h < p.H) {
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
              uint4 w;
              w.x = pack2<kBF16>(__uint_as_float(v[8 * gq + 0]), __uint_as_float(v[8 * gq + 1]));
              w.y = pack2<kBF16>(__uint_as_float(v[8 * gq + 2]), __uint_as_float(v[8 * gq + 3]));
              w.z = pack2<kBF16>(__uint_as_float(v[8 * gq + 4]), __uint_as_float(v[8 * gq + 5]));
              w.w = pack2<kBF16>(__uint_as_float(v[8 * gq + 6]), __uint_as_float(v[8 * gq + 7]));
              reinterpret_cast<uint4*>(drow + cc * 32)[gq] = w;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tD, kTmemCols);
}

// -------------------------------------------------------------------------------------------------
// dkv: key gradient of one (query, block of 128 heads, 192 dims) per CTA, 128 keys (two tiles) at a time
// -------------------------------------------------------------------------------------------------
namespace bwdtc {
namespace dkv {
constexpr int kStages = 3;
constexpr uint32_t kPairBytes = 2 * kTileBytes;                 // dS or P of 128 keys: two consecutive workspace tiles
constexpr uint32_t kOperandBytes = 3 * kTileBytes;              // Q (or dO) of 128 heads x 192 dims: three [128 x 128 B] chunks
constexpr uint32_t kOffQ = kStages * kPairBytes;                // 98304
constexpr uint32_t kOffDO = kOffQ + kOperandBytes;              // 147456
constexpr uint32_t kOffBar = kOffDO + kOperandBytes;            // 196608
constexpr uint32_t kOffMask = kOffBar + 128;
constexpr uint32_t kOffXpose = kOffMask + kMaxTiles * 8;        // per epilogue warp: [32 keys x 16 dims] fp32 + 32 row numbers
constexpr uint32_t kXposeBytes = 32 * 64 + 128;
constexpr int kEpilogueWarps = 8;                               // warp w: tensor-memory lanes 32 (w & 3) .., columns 96 (w >> 2) .. + 95
constexpr int kLoadWarp = 8, kIssueWarp = 9;
constexpr int kThreadsDkv = 320;
constexpr uint32_t kSmemBytes = kOffXpose + kEpilogueWarps * kXposeBytes + 1024;
constexpr uint32_t kTmemCols = 512;                             // two accumulators of 192 columns
static_assert(kSmemBytes <= 232448, "shared memory per CTA");
}  // namespace dkv
}  // namespace bwdtc

template <bool kBF16>
__global__ void __launch_bounds__(bwdtc::dkv::kThreadsDkv, 1) sparse_mla_bwd_dkv_kernel(const BwdParams bp, const bwdtc::Pass ps) {
  using namespace bwdtc;
  using namespace bwdtc::dkv;
  const FwdParams& p = bp.f;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sBase = smem_u32(smem);
  const uint32_t sQ = sBase + kOffQ, sDO = sBase + kOffDO;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
  uint64_t* full = bars;           // [3] count 1 + 32768 transaction bytes: a dS or P pair of tiles landed
  uint64_t* empty = bars + 3;      // [3] count 1: commit after the MMAs that read the stage
  uint64_t* acc_full = bars + 6;   // [2] count 1: commit after the MMAs of a key pair
  uint64_t* acc_free = bars + 8;   // [2] count 8: the epilogue warps have read the accumulator
  uint64_t* b_ready = bars + 10;   // count 128: Q / dO columns are in shared memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  unsigned long long* smask = reinterpret_cast<unsigned long long*>(smem + kOffMask);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int part = blockIdx.x % kDimSplits;
  const int item = blockIdx.x / kDimSplits;
  const int ql = item / ps.head_blocks, hb = item - ql * ps.head_blocks;
  const int bt = ps.q0 + ql, b = bt / p.S, h0 = hb * kM;
  const int64_t tile0 = (static_cast<int64_t>(ql) * ps.head_blocks + hb) * ps.ntiles2;
  const int npairs = ps.ntiles2 >> 1;
  // dO columns of this CTA: dims [192 part, 192 part + 192) clipped to the 512 value dims -> 3, 3, 2 chunks
  const int do_chunks = part < 2 ? 3 : 2;

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_free[i], kEpilogueWarps); }
    mbar_init(b_ready, 128);
    mbar_init_fence();
  }
  for (int i = tid; i < ps.ntiles2; i += kThreadsDkv) smask[i] = i < ps.ntiles ? ps.masks[static_cast<int64_t>(ql) * ps.ntiles2 + i] : 0ull;
  if (warp == kIssueWarp) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tAcc = *tmem_slot;
  const bool run = *reinterpret_cast<volatile int*>(p.status) == kStatusOk;
  bool ok = true;

  if (warp == kLoadWarp) {
    // ================================ tile loads ====================================================
    // per key pair two loads into consecutive slots of the ring: dS (tiles 2 tp, 2 tp + 1), then P
    if (lane == 0 && run) {
      int j = 0;
      for (int tp = 0; ok && tp < npairs; ++tp) {
        if ((smask[2 * tp] | smask[2 * tp + 1]) == 0ull) continue;
#pragma unroll 1
        for (int which = 0; which < 2; ++which, ++j) {
          const int s = j % kStages;
          if (j >= kStages && !mbar_wait(&empty[s], ((j / kStages) + 1) & 1, p.status)) { ok = false; break; }
          mbar_arrive_expect_tx(&full[s], kPairBytes);
          bulk_copy_g2s(sBase + s * kPairBytes, (which == 0 ? ps.ds_ws : ps.p_ws) + (tile0 + 2 * tp) * kTileBytes, kPairBytes, &full[s]);
        }
      }
    }
  } else if (warp == kIssueWarp) {
    // ================================ MMA issuer ====================================================
    // acc[128 keys x 192 dims] = dS^T[128 keys x 128 heads] . Q[128 heads x 192 dims] + P^T . dO[128 heads x its dims]:
    // both operands MN-major (contraction over heads = rows of the shared-memory images), 16 heads = 2048 bytes per step.
    if (run) {  // converged warp, one elected lane issues
      constexpr uint32_t idesc_q = make_idesc_f16(kBF16, kM, kDimsPerCta, 1, 1);
      constexpr uint32_t idesc_o2 = make_idesc_f16(kBF16, kM, 128, 1, 1);
      const uint32_t idesc_o = do_chunks == 3 ? idesc_q : idesc_o2;
      const uint32_t go = elect_one_lane();
      ok = __all_sync(0xffffffffu, mbar_wait(b_ready, 0, p.status));
      const uint64_t dq0 = make_smem_desc(sQ, kTileBytes, 1024, kSwizzle128B);
      const uint64_t do0 = make_smem_desc(sDO, kTileBytes, 1024, kSwizzle128B);
      int g = 0, j = 0;
      for (int tp = 0; ok && tp < npairs; ++tp) {
        if ((smask[2 * tp] | smask[2 * tp + 1]) == 0ull) continue;
        const int ab = g & 1;
        if (g >= 2 && !__all_sync(0xffffffffu, mbar_wait(&acc_free[ab], ((g >> 1) + 1) & 1, p.status))) { ok = false; break; }
#pragma unroll 1
        for (int which = 0; which < 2; ++which, ++j) {
          const int s = j % kStages;
          if (!__all_sync(0xffffffffu, mbar_wait(&full[s], (j / kStages) & 1, p.status))) { ok = false; break; }
          tc_fence_after();
          const uint64_t da0 = make_smem_desc(sBase + s * kPairBytes, kTileBytes, 1024, kSwizzle128B);
          const uint64_t db0 = which == 0 ? dq0 : do0;
          const uint32_t idesc = which == 0 ? idesc_q : idesc_o;
#pragma unroll
          for (int ks = 0; ks < kM / 16; ++ks)
            umma_ss_if(go, tAcc + ab * kDimsPerCta, da0 + ((ks * 2048) >> 4), db0 + ((ks * 2048) >> 4), idesc, (which | ks) != 0);
          umma_commit_if(go, &empty[s]);
        }
        if (!ok) break;
        umma_commit_if(go, &acc_full[ab]);
        ++g;
      }
    }
  } else if (warp < kEpilogueWarps) {
    // ================================ operand columns + epilogue ====================================
    // the first four warps copy the 128 head rows' 192 Q dims and dO dims into the [128 heads x 128 B] chunk
    // images.  Then thread (r, half) owns key r of every pair: tensor-memory lane r holds that key's 192 gradient values,
    // of which this thread takes columns [96 half, 96 half + 96).
    const int q4 = warp & 3, half = warp >> 2;
    const int r = q4 * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
    if (half == 0) {
      // whole 128-byte lines: eight lanes copy one row's 64 dims of a chunk, a warp instruction covers four rows (a row per
      // lane would make every instruction touch 32 rows)
      const int nrows = p.H - h0 < kM ? p.H - h0 : kM;
      const uint8_t* qbase = reinterpret_cast<const uint8_t*>(p.q) + (static_cast<int64_t>(bt) * p.H + h0) * (kD * 2) + part * (kDimsPerCta * 2);
      const uint8_t* dobase = reinterpret_cast<const uint8_t*>(bp.d_out) + (static_cast<int64_t>(bt) * p.H + h0) * (kDV * 2) + part * (kDimsPerCta * 2);
#pragma unroll 4
      for (int i = r; i < 3 * 1024; i += 128) {
        const int u = i & 7, row = (i >> 3) & 127, c = i >> 10;
        const bool row_ok = row < nrows;
        cp_async16(sQ + c * kTileBytes + sw128_offset(row, u), row_ok ? qbase + static_cast<int64_t>(row) * (kD * 2) + c * 128 + u * 16 : qbase, row_ok ? 16u : 0u);
        // (the last CTA's third dO chunk would be dims 512 .. 575, which do not exist: zero fill)
        const bool do_ok = row_ok && c < do_chunks;
        cp_async16(sDO + c * kTileBytes + sw128_offset(row, u), do_ok ? dobase + static_cast<int64_t>(row) * (kDV * 2) + c * 128 + u * 16 : dobase, do_ok ? 16u : 0u);
      }
      cp_async_commit();
      cp_async_wait<0>();
      fence_proxy_async_smem();
      mbar_arrive(b_ready);
    }
    const int32_t* idx_row = p.indices + static_cast<int64_t>(bt) * p.topk;
    uint8_t* xbuf_ptr = smem + kOffXpose + warp * kXposeBytes;
    const uint32_t xbuf = smem_u32(xbuf_ptr);
    int* xrows = reinterpret_cast<int*>(xbuf_ptr + 32 * 64);
    int g = 0;
    for (int tp = 0; run && ok && tp < npairs; ++tp) {
      const unsigned long long m0 = smask[2 * tp], m1 = smask[2 * tp + 1];
      if ((m0 | m1) == 0ull) continue;
      const int ab = g & 1;
      const bool valid = ((r < 64 ? m0 >> r : m1 >> (r - 64)) & 1ull) != 0ull;
      const int idx = valid ? __ldg(idx_row + tp * 128 + r) : 0;
      // row number inside dKV of this thread's key (-1: takes no part), shared with the warp for the transposed atomics
      __syncwarp();
      xrows[lane] = valid ? static_cast<int>(kv_row_of(p, b, idx)) : -1;
      if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[ab], (g >> 1) & 1, p.status))) { ok = false; break; }
      tc_fence_after();
      // this thread's 96 columns leave tensor memory at once, so that the accumulator goes back to the MMA issuer before
      // the (slow) atomics start
      uint32_t v[96];
#pragma unroll
      for (int c3 = 0; c3 < 3; ++c3) tmem_ld32(tAcc + ab * kDimsPerCta + lane_base + half * 96 + c3 * 32, v + 32 * c3);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_free[ab]);
      int rows4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) rows4[i] = xrows[i * 8 + (lane >> 2)];
#pragma unroll
      for (int cc = 0; cc < 6; ++cc) {  // chunks of 16 columns
        // The warp holds [32 keys x 16 dims] with one key per lane.  Through shared memory (16-byte units XOR-swizzled by the
        // row, conflict-free both ways) it is turned so that 4 consecutive lanes cover the 64 contiguous bytes of ONE key:
        // an atomic instruction then touches 16 full sectors instead of 32 half-used ones.
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j)
          st_shared_v4(xbuf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4), v[16 * cc + 4 * j], v[16 * cc + 4 * j + 1], v[16 * cc + 4 * j + 2],
                       v[16 * cc + 4 * j + 3]);
        __syncwarp();
        float4 val[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int key = i * 8 + (lane >> 2);
          val[i] = *reinterpret_cast<const float4*>(xbuf_ptr + key * 64 + (((lane & 3) ^ ((key >> 1) & 3)) << 4));
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (rows4[i] >= 0)
            atomicAdd(reinterpret_cast<float4*>(bp.d_kv + static_cast<int64_t>(rows4[i]) * kD + part * kDimsPerCta + half * 96 + cc * 16) + (lane & 3),
                      val[i]);
      }
      ++g;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kIssueWarp) tmem_dealloc(tAcc, kTmemCols);
}

// -------------------------------------------------------------------------------------------------
// host side
// -------------------------------------------------------------------------------------------------
bool sparse_mla_bwd_tc_supported(const FwdParams& p) {
  return p.D == bwdtc::kD && p.DV == bwdtc::kDV && p.topk <= bwdtc::kMaxTiles * bwdtc::kBK;
}

// Workspace bytes one query of a pass needs: P and dS tiles, validity masks, delta (rounded up to 256 bytes).
size_t sparse_mla_bwd_tc_bytes_per_query(int H, int topk) {
  using namespace bwdtc;
  const size_t hbs = static_cast<size_t>((H + kM - 1) / kM);
  const size_t ntiles2 = (static_cast<size_t>((topk + kBK - 1) / kBK) + 1) & ~static_cast<size_t>(1);
  const size_t bytes = 2 * hbs * ntiles2 * kTileBytes + ntiles2 * 8 + hbs * kM * 4;
  return (bytes + 255) & ~static_cast<size_t>(255);
}

namespace {
template <bool kBF16>
int run_bwd_tc_passes(const BwdParams& bp, bwdtc::Pass ps, int nq_max, cudaStream_t stream) {
  using namespace bwdtc;
  using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;
  const FwdParams& p = bp.f;
  cudaError_t e;
  auto k_p = sparse_mla_bwd_scores_kernel<kBF16, 0>;
  auto k_ds = sparse_mla_bwd_scores_kernel<kBF16, 1>;
  auto k_dq = sparse_mla_bwd_dq_kernel<kBF16>;
  auto k_dkv = sparse_mla_bwd_dkv_kernel<kBF16>;
  if ((e = cudaFuncSetAttribute(k_p, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(ScoresCfg<0>::kSmemBytes))) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(k_ds, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(ScoresCfg<1>::kSmemBytes))) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(k_dq, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(dq::kSmemBytes))) != cudaSuccess) return e;
  if ((e = cudaFuncSetAttribute(k_dkv, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(dkv::kSmemBytes))) != cudaSuccess) return e;
  const int total = p.B * p.S;
  for (int q0 = 0; q0 < total; q0 += nq_max) {
    ps.q0 = q0;
    ps.nq = total - q0 < nq_max ? total - q0 : nq_max;
    const unsigned items = static_cast<unsigned>(ps.nq) * ps.head_blocks;
    sparse_mla_bwd_prep_kernel<T><<<static_cast<unsigned>(ps.nq), 256, 0, stream>>>(bp, ps);
    k_p<<<items, kThreads, ScoresCfg<0>::kSmemBytes, stream>>>(bp, ps);
    k_ds<<<items, kThreads, ScoresCfg<1>::kSmemBytes, stream>>>(bp, ps);
    k_dq<<<items * kDimSplits, kThreads, dq::kSmemBytes, stream>>>(bp, ps);
    k_dkv<<<items * kDimSplits, dkv::kThreadsDkv, dkv::kSmemBytes, stream>>>(bp, ps);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
  }
  return 0;
}
}  // namespace

// `queries_per_pass` <= 0: as many as the workspace holds (a multiple of the SM count when it holds that many).
int launch_sparse_mla_bwd_tc(const BwdParams& bp, bool bf16, void* workspace, size_t workspace_bytes, int queries_per_pass, cudaStream_t stream) {
  using namespace bwdtc;
  const FwdParams& p = bp.f;
  const size_t per_q = sparse_mla_bwd_tc_bytes_per_query(p.H, p.topk);
  size_t nq_max = workspace_bytes / per_q;
  const size_t total = static_cast<size_t>(p.B) * p.S;
  if (nq_max > total) nq_max = total;
  if (queries_per_pass > 0 && static_cast<size_t>(queries_per_pass) < nq_max) nq_max = queries_per_pass;
  if (nq_max == 0) return static_cast<int>(cudaErrorInvalidValue);
  if (queries_per_pass <= 0 && nq_max < total) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0 &&
        nq_max >= static_cast<size_t>(sms))
      nq_max = nq_max / sms * sms;
  }
  Pass ps;
  ps.head_blocks = (p.H + kM - 1) / kM;
  ps.ntiles = (p.topk + kBK - 1) / kBK;
  ps.ntiles2 = (ps.ntiles + 1) & ~1;
  const size_t tile_bytes = nq_max * ps.head_blocks * ps.ntiles2 * kTileBytes;
  uint8_t* w = static_cast<uint8_t*>(workspace);
  ps.p_ws = w;
  ps.ds_ws = w + tile_bytes;
  ps.masks = reinterpret_cast<unsigned long long*>(w + 2 * tile_bytes);
  ps.delta = reinterpret_cast<float*>(w + 2 * tile_bytes + nq_max * ps.ntiles2 * 8);
  ps.q0 = 0; ps.nq = 0;
  return bf16 ? run_bwd_tc_passes<true>(bp, ps, static_cast<int>(nq_max), stream) : run_bwd_tc_passes<false>(bp, ps, static_cast<int>(nq_max), stream);
}

}  // namespace dsa
