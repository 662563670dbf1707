// Row-wise top-k selector: radix select + bitonic sort of the survivors.
//
// For each fp32 row the kernel emits the indices of the `top_k` largest candidates in descending
// score order, equal scores in ascending index order (the stable-sort rule of
// cpu_lightning_indexer, examples/deepseek_v4/lightning_indexer.py:316-325); candidates are the first
// `limit[row]` entries whose score is > -1e30; slots left over hold -1 (value -inf).  For rows of
// distinct values this is also torch.topk's answer (examples/topk_selector/example_topk_selector.py:57-58).
//
// One CTA per row.  The row is converted to order-preserving 32-bit keys in shared memory, four
// 8-bit most-significant-digit-first histogram passes find the k-th largest key, an index-ordered
// compaction (per-warp counts, prefix over warps, ordered write) takes everything above it plus the
// lowest-index ties, and a stable least-significant-digit radix sort (four 8-bit passes, descending) of the
// <= k survivors fixes the output order: the compaction leaves equal keys in ascending index order and
// a stable sort keeps them so.  With ordered = 0 the sort is left out and the selected SET comes out in ascending index
// order (what the sparse attention after the indexer needs, and the order in which its row gather is most local).
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "launch_util.h"

namespace dsa {

namespace topk {
constexpr int kThreads = 512;                     // 4 rows (CTAs) per SM hide each other's barrier phases
constexpr int kWarps = kThreads / 32;
constexpr size_t kMaxSmemBytes = 220 * 1024;       // rows whose keys do not fit are streamed from global memory
}  // namespace topk

__device__ __forceinline__ uint32_t float_to_key(float f) {
  uint32_t u = __float_as_uint(f);
  if (u == 0x80000000u) u = 0u;  // -0.0 ties with +0.0, as in a floating-point comparison
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

// scores [rows, row_stride]; limits [rows] or null; out_idx [rows, top_k]; out_val [rows, top_k] or null.
// Dynamic shared memory: max(kpow2 * 8 (sort buffer), kWarps * 256 * 4 (per-warp first-digit histograms, used before the
// sort buffer)) + max(n * 4 (keys), kpow2 * 8 + kWarps * 256 * 2 (second sort buffer + digit counters, used after the keys)).
// kMaxRounds: 32-element rounds per warp in the sort, top_k <= kWarps * 32 * kMaxRounds.
// kStream: rows too long for shared memory (more than about 52 k candidates).  The keys are not kept: every pass -- the
// first-digit histogram, the three further select passes, the two passes of the compaction -- converts the scores again
// from global memory (six reads of a row that stays in L2 instead of one); the shared memory then holds the sort buffers
// only.  Same results bit for bit.
template <int kMaxRounds, bool kStream>
__global__ void __launch_bounds__(topk::kThreads, kMaxRounds <= 4 ? 4 : 1) topk_select_kernel(const float* __restrict__ scores, int64_t row_stride, int n,
                                                                     const int32_t* __restrict__ limits, int top_k, int kpow2,
                                                                     int32_t* __restrict__ out_idx, float* __restrict__ out_val, int ordered) {
  using namespace topk;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const size_t front = max(static_cast<size_t>(kpow2) * 8, static_cast<size_t>(kWarps) * 256 * 4);
  unsigned long long* sortbuf = reinterpret_cast<unsigned long long*>(smem_raw);  // [kpow2]
  uint32_t* whist = reinterpret_cast<uint32_t*>(smem_raw);                         // [kWarps][256], dead before sortbuf is written
  uint32_t* keys = reinterpret_cast<uint32_t*>(smem_raw + front);                  // [n]
  __shared__ uint32_t hist[256], dbase[256];
  __shared__ uint32_t warp_sums[kWarps], warp_ties[kWarps];
  __shared__ uint32_t s_prefix, s_remaining, s_nvalid;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row = blockIdx.x;
  const float* x = scores + static_cast<int64_t>(row) * row_stride;
  const bool whole_groups = (n & 3) == 0;  // 16-byte groups never reach past the end of the row
  int lim = limits ? limits[row] : n;
  lim = lim < 0 ? 0 : (lim > n ? n : lim);
  n = lim;  // entries at or beyond the limit are not candidates: none of the passes below looks at them
  // key of candidate i (0 = not a candidate), from shared memory or again from the scores
  auto key_at = [&](int i) -> uint32_t {
    if constexpr (kStream) {
      const float f = __ldg(x + i);
      return f > -1e30f ? float_to_key(f) : 0u;
    } else {
      return keys[i];
    }
  };

  if (tid == 0) s_nvalid = 0;
  for (int i = tid; i < kWarps * 256; i += kThreads) whist[i] = 0;
  __syncthreads();

  // ---- load, convert, count candidates, first-digit histogram ---------------------------------------
  uint32_t my_valid = 0;
  auto take = [&](int i, float f) {
    uint32_t k = 0;
    if (i < lim && f > -1e30f) { k = float_to_key(f); ++my_valid; }
    if (!kStream && i < n) keys[i] = k;  // 0 marks "not a candidate" (a real key is never 0 for a score > -1e30)
    // sign + exponent bits crowd into a few bins: a private histogram per warp keeps the atomics apart
    if (k) atomicAdd(&whist[warp * 256 + (k >> 24)], 1u);
  };
  if (whole_groups && (reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
    // 16-byte loads, four of them in flight per thread before the first is used: a row of 8192 scores is two round
    // trips to memory instead of sixteen
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const int n4 = (n + 3) >> 2;
    for (int base = 0; base < n4; base += 4 * kThreads) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i4 = base + u * kThreads + tid;
        v[u] = i4 < n4 ? __ldg(x4 + i4) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = (base + u * kThreads + tid) * 4;
        take(i, v[u].x); take(i + 1, v[u].y); take(i + 2, v[u].z); take(i + 3, v[u].w);
      }
    }
  } else {
    for (int base = 0; base < n; base += kThreads) {
      const int i = base + tid;
      take(i, i < lim ? x[i] : 0.f);
    }
  }
  for (int o = 16; o > 0; o >>= 1) my_valid += __shfl_xor_sync(0xffffffffu, my_valid, o);
  if (lane == 0 && my_valid) atomicAdd(&s_nvalid, my_valid);
  __syncthreads();
  if (tid < 256) {
    uint32_t t = 0;
#pragma unroll 8
    for (int w = 0; w < kWarps; ++w) t += whist[w * 256 + tid];
    hist[tid] = t;
  }
  __syncthreads();
  const uint32_t nvalid = s_nvalid;
  const uint32_t kk = nvalid < static_cast<uint32_t>(top_k) ? nvalid : static_cast<uint32_t>(top_k);

  // ---- radix select: threshold key T = kk-th largest candidate key -----------------------------------
  uint32_t thresh = 0;     // everything is taken when nvalid <= top_k
  uint32_t need_ties = 0;  // how many keys equal to T are taken (lowest indices first)
  if (nvalid > static_cast<uint32_t>(top_k)) {
    if (tid == 0) { s_prefix = 0; s_remaining = kk; }
    __syncthreads();
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (pass > 0) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        const uint32_t pmask = 0xffffffffu << (shift + 8);
        for (int base = 0; base < n; base += kThreads) {
          const int i = base + tid;
          const uint32_t k = i < n ? key_at(i) : 0u;
          if (k && (k & pmask) == prefix) atomicAdd(&hist[(k >> shift) & 0xffu], 1u);  // few survivors, spread digits
        }
        __syncthreads();
      }
      // warp 0 walks the 256 bins from the top: find digit dsel with  sum(bins > dsel) < remaining <= sum(bins >= dsel)
      if (warp == 0) {
        const uint32_t remaining = s_remaining;
        uint32_t c[8], tot = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) { c[j] = hist[255 - (lane * 8 + j)]; tot += c[j]; }  // lane 0 holds the top 8 bins
        uint32_t incl = tot;
        for (int o = 1; o < 32; o <<= 1) {
          const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += t;
        }
        uint32_t above = incl - tot;  // candidates in bins above this lane's 8 bins
        const bool mine = above < remaining && remaining <= incl;
        if (mine) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (above < remaining && remaining <= above + c[j]) {
              s_prefix = s_prefix | ((255u - (lane * 8 + j)) << shift);
              s_remaining = remaining - above;
            }
            above += c[j];
          }
        }
      }
      __syncthreads();
    }
    thresh = s_prefix;
    need_ties = s_remaining;
  }

  // ---- ordered compaction: keys > T in any order, keys == T by ascending index until need_ties ----------
  const bool take_all = nvalid <= static_cast<uint32_t>(top_k);
  {
    // warp w owns the contiguous index range [w * per, w * per + per): count, prefix over warps, then write in order
    const int per = ((n + kWarps - 1) / kWarps + 31) & ~31;
    const int beg = warp * per, end = min(n, beg + per);
    uint32_t n_gt = 0, n_eq = 0;
    for (int base = beg; base < end; base += 32) {
      const int i = base + lane;
      const uint32_t k = i < end ? key_at(i) : 0u;
      n_gt += __popc(__ballot_sync(0xffffffffu, k != 0 && (take_all || k > thresh)));
      n_eq += __popc(__ballot_sync(0xffffffffu, !take_all && k != 0 && k == thresh));
    }
    if (lane == 0) { warp_sums[warp] = n_gt; warp_ties[warp] = n_eq; }
    __syncthreads();
    uint32_t tie_rank = 0, out_pos = 0;  // ties / selected elements in the warps before this one
    for (int w = 0; w < warp; ++w) {
      const uint32_t e = warp_ties[w];
      const uint32_t taken = tie_rank >= need_ties ? 0u : min(e, need_ties - tie_rank);
      out_pos += warp_sums[w] + taken;
      tie_rank += e;
    }
    for (int base = beg; base < end; base += 32) {
      const int i = base + lane;
      const uint32_t k = i < end ? key_at(i) : 0u;
      const bool gt = k != 0 && (take_all || k > thresh);
      const bool eq = !take_all && k != 0 && k == thresh;
      const uint32_t bal_eq = __ballot_sync(0xffffffffu, eq);
      const bool take = gt || (eq && tie_rank + __popc(bal_eq & ((1u << lane) - 1u)) < need_ties);
      const uint32_t bal = __ballot_sync(0xffffffffu, take);
      if (take)
        sortbuf[out_pos + __popc(bal & ((1u << lane) - 1u))] =
            (static_cast<unsigned long long>(k) << 32) | static_cast<unsigned long long>(0xffffffffu - static_cast<uint32_t>(i));
      out_pos += __popc(bal);
      tie_rank += __popc(bal_eq);
    }
  }
  __syncthreads();

  // ---- stable radix sort of the kk survivors, descending by key --------------------------------------------------
  // Four passes over 8-bit digits, least significant first, ping-pong between the sort buffer and the (now free) key
  // array.  Warp w owns the contiguous slice [w * per, w * per + per) of the current order.  Rank of an element inside
  // its digit = (elements of that digit in earlier warps) + (in earlier 32-element rounds of this warp) + (in lower
  // lanes of this round, from match_any).  Per-warp digit counters are 16-bit and only ever touched by their own warp.
  unsigned long long* src = sortbuf;
  unsigned long long* dst = reinterpret_cast<unsigned long long*>(keys);
  uint16_t* wcnt = reinterpret_cast<uint16_t*>(keys) + static_cast<size_t>(kpow2) * 4;  // [kWarps][256], behind the second buffer
  if (!ordered) {
    // the caller wants the index SET only: the survivors stay as the compaction left them, in ascending index order
  } else if (kk <= 64u) {
    // up to 64 survivors: one warp sorts them in registers (two per lane, bitonic network, descending on the whole
    // 64-bit element = key, then lower index), no block barriers
    if (warp == 0) {
      const int i0 = lane, i1 = lane + 32;
      unsigned long long a = i0 < static_cast<int>(kk) ? sortbuf[i0] : 0ull, b = i1 < static_cast<int>(kk) ? sortbuf[i1] : 0ull;
      for (int size = 2; size <= 64; size <<= 1) {
        const bool d0 = (i0 & size) == 0, d1 = (i1 & size) == 0;
        int stride = min(size >> 1, 32);
        if (stride == 32) {
          if ((a < b) == d0) { const unsigned long long t = a; a = b; b = t; }
          stride = 16;
        }
        for (; stride > 0; stride >>= 1) {
          const bool lower = (lane & stride) == 0;
          const unsigned long long oa = __shfl_xor_sync(0xffffffffu, a, stride), ob = __shfl_xor_sync(0xffffffffu, b, stride);
          a = (lower == d0) ? (a > oa ? a : oa) : (a < oa ? a : oa);
          b = (lower == d1) ? (b > ob ? b : ob) : (b < ob ? b : ob);
        }
      }
      sortbuf[i0] = a;
      sortbuf[i1] = b;
    }
    __syncthreads();
  } else
  {
    const int cnt = static_cast<int>(kk);
    const int per = ((cnt + kWarps - 1) / kWarps + 31) & ~31;
    const int rounds = per >> 5;  // <= kMaxRounds (checked by the launcher)
    const int beg = warp * per;
    const int nw = (cnt + per - 1) / per;  // warps that own elements: the counters of the others are never looked at
    for (int pass = 0; pass < 4 && cnt > 1; ++pass) {
      const int shift = 32 + 8 * pass;  // the key is the upper word of the element
      for (int i = tid; i < nw * 256; i += kThreads) wcnt[i] = 0;
      __syncthreads();
      unsigned long long e[kMaxRounds];
      uint32_t dig[kMaxRounds], rk[kMaxRounds];
#pragma unroll
      for (int j = 0; j < kMaxRounds; ++j) {
        if (j < rounds) {
          const int i = beg + j * 32 + lane;
          const bool live = i < cnt;
          e[j] = live ? src[i] : 0ull;
          dig[j] = live ? static_cast<uint32_t>(e[j] >> shift) & 0xffu : 0x100u + lane;  // dead lanes match nobody
          const uint32_t peers = __match_any_sync(0xffffffffu, dig[j]);
          uint32_t old = 0;
          if (live) old = wcnt[warp * 256 + dig[j]];
          __syncwarp();
          if (live && (__ffs(peers) - 1) == lane) wcnt[warp * 256 + dig[j]] = static_cast<uint16_t>(old + __popc(peers));
          __syncwarp();
          rk[j] = old + __popc(peers & ((1u << lane) - 1u));
        }
      }
      __syncthreads();
      // per digit: exclusive prefix over the warps, total
      if (tid < 256) {
        uint32_t run = 0;
#pragma unroll 4
        for (int w = 0; w < nw; ++w) {
          const uint32_t c = wcnt[w * 256 + tid];
          wcnt[w * 256 + tid] = static_cast<uint16_t>(run);
          run += c;
        }
        hist[tid] = run;
      }
      __syncthreads();
      // descending order: digit d starts after all larger digits (warp 0, lane l holds digits 255 - 8l .. 248 - 8l)
      if (warp == 0) {
        uint32_t c[8], tot = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) { c[j] = hist[255 - (lane * 8 + j)]; tot += c[j]; }
        uint32_t incl = tot;
        for (int o = 1; o < 32; o <<= 1) {
          const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += t;
        }
        uint32_t above = incl - tot;
#pragma unroll
        for (int j = 0; j < 8; ++j) { dbase[255 - (lane * 8 + j)] = above; above += c[j]; }
      }
      __syncthreads();
#pragma unroll
      for (int j = 0; j < kMaxRounds; ++j) {
        if (j < rounds) {
          const int i = beg + j * 32 + lane;
          if (i < cnt) dst[dbase[dig[j]] + wcnt[warp * 256 + dig[j]] + rk[j]] = e[j];
        }
      }
      __syncthreads();
      unsigned long long* t = src; src = dst; dst = t;
    }
  }
  const unsigned long long* sorted = src;

  // ---- output ---------------------------------------------------------------------------------------------
  int32_t* oi = out_idx + static_cast<int64_t>(row) * top_k;
  float* ov = out_val ? out_val + static_cast<int64_t>(row) * top_k : nullptr;
  for (int i = tid; i < top_k; i += kThreads) {
    if (static_cast<uint32_t>(i) < kk) {
      const unsigned long long e = sorted[i];
      oi[i] = static_cast<int32_t>(0xffffffffu - static_cast<uint32_t>(e & 0xffffffffull));
      if (ov) ov[i] = key_to_float(static_cast<uint32_t>(e >> 32));
    } else {
      oi[i] = -1;
      if (ov) ov[i] = -INFINITY;
    }
  }
}

// Shared memory of the kernel that keeps a row's keys (n > 0) or of the streaming kernel (n = 0).
size_t topk_smem_bytes(int n, int top_k, int* kpow2_out) {
  int kp = 32;  // buffer length: top_k rounded up to a multiple of 32 (name kept from the power-of-two days of a bitonic sort)
  while (kp < top_k) kp += 32;
  if (kpow2_out) *kpow2_out = kp;
  const size_t front = static_cast<size_t>(kp) * 8 > static_cast<size_t>(topk::kWarps) * 256 * 4 ? static_cast<size_t>(kp) * 8 : static_cast<size_t>(topk::kWarps) * 256 * 4;
  const size_t back_sort = static_cast<size_t>(kp) * 8 + static_cast<size_t>(topk::kWarps) * 256 * 2;
  const size_t back = static_cast<size_t>(n) * 4 > back_sort ? static_cast<size_t>(n) * 4 : back_sort;
  return front + back;
}

int launch_topk_select(const float* scores, int64_t rows, int n, int64_t row_stride, const int32_t* limits, int top_k,
                       int32_t* out_idx, float* out_val, cudaStream_t stream, int ordered) {
  int kp = 0;
  const bool stream_rows = topk_smem_bytes(n, top_k, nullptr) > topk::kMaxSmemBytes;
  const size_t smem = topk_smem_bytes(stream_rows ? 0 : n, top_k, &kp);
  if (top_k > topk::kWarps * 32 * 16) return static_cast<int>(cudaErrorInvalidValue);
  const bool small = top_k <= topk::kWarps * 32 * 4;
  auto kern = stream_rows ? (small ? topk_select_kernel<4, true> : topk_select_kernel<16, true>)
                          : (small ? topk_select_kernel<4, false> : topk_select_kernel<16, false>);
  int dev = 0, sms = 0;
  cudaError_t e = current_device_sms(&dev, &sms);
  if (e != cudaSuccess) return static_cast<int>(e);
  if ((e = ensure_dynamic_smem(kern, dev, static_cast<int>(smem))) != cudaSuccess) return static_cast<int>(e);
  kern<<<static_cast<unsigned>(rows), topk::kThreads, smem, stream>>>(scores, row_stride, n, limits, top_k, kp, out_idx, out_val, ordered);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace dsa
