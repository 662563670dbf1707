// Combines up to two partial attention results over disjoint key sets with a per-head attention sink.
//
// DeepSeek-V4's sparse_flash_mla attends, per query, to a sliding window of the original KV cache and to a set of
// compressed KV tokens, and adds a learned per-head "sink" logit to the softmax denominator (it has no value row):
// the reference golden starts its online softmax with row_max = sink, row_sum = 1
// (examples/deepseek_v4/sparse_flash_mla/sparse_flash_mla_golden.py:121-153).  Here the two key sets are run as two
// calls of the sparse forward kernel, each giving a normalised output and its natural-log LSE; this kernel merges them:
//   lse = log(exp(lse_a) + exp(lse_b) + exp(sink)),   out = exp(lse_a - lse) out_a + exp(lse_b - lse) out_b.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dsa {

template <typename T>
__global__ void __launch_bounds__(256) sink_combine_kernel(const T* __restrict__ out_a, const float* __restrict__ lse_a, const T* __restrict__ out_b,
                                                           const float* __restrict__ lse_b, const float* __restrict__ sinks, T* __restrict__ out,
                                                           float* __restrict__ lse, int64_t rows, int H, int DV) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);  // one warp per (token, head)
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float la = lse_a[row];
  const float lb = out_b ? lse_b[row] : -INFINITY;
  const float sk = sinks ? sinks[row % H] : -INFINITY;
  const float m = fmaxf(fmaxf(la, lb), sk);
  float wa = 0.f, wb = 0.f, total = -INFINITY;
  if (m > -INFINITY) {
    const float ea = __expf(la - m), eb = __expf(lb - m), es = __expf(sk - m);
    const float den = ea + eb + es;
    wa = ea / den; wb = eb / den;
    total = m + __logf(den);
  }
  const T* pa = out_a + row * DV;
  const T* pb = out_b ? out_b + row * DV : nullptr;
  T* po = out + row * DV;
  for (int d = lane; d < DV; d += 32) {
    float v = wa * static_cast<float>(pa[d]);
    if (pb) v += wb * static_cast<float>(pb[d]);
    po[d] = static_cast<T>(v);
  }
  if (lane == 0 && lse) lse[row] = total;
}

int launch_sink_combine(const void* out_a, const float* lse_a, const void* out_b, const float* lse_b, const float* sinks, void* out, float* lse,
                        int64_t rows, int H, int DV, bool bf16, cudaStream_t stream) {
  const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
  if (bf16)
    sink_combine_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(out_a), lse_a, static_cast<const __nv_bfloat16*>(out_b),
                                                                 lse_b, sinks, static_cast<__nv_bfloat16*>(out), lse, rows, H, DV);
  else
    sink_combine_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(out_a), lse_a, static_cast<const __half*>(out_b), lse_b, sinks,
                                                          static_cast<__half*>(out), lse, rows, H, DV);
  return static_cast<int>(cudaGetLastError());
}

// Index lists of sparse_flash_mla, one CTA per query token: physical row numbers (into the paged pools) of the sliding
// window of the original cache and of the token's compressed keys, -1 for slots that take no part.  Rules as in the
// reference golden (examples/deepseek_v4/sparse_flash_mla/sparse_flash_mla_golden.py:16-53, 95-118): token s of sequence b
// sits at p = seqused_kv[b] - len_q[b] + s; window [max(p - win_left, 0), p]; compressed tokens below
// threshold = floor((p + 1) / ratio): scenario 3 takes the caller's list, cut at min(K, threshold) entries and at the first
// -1, entries >= min(threshold, floor(seqused_kv[b] / ratio)) skipped; scenario 2 takes all tokens below the threshold.
struct V4IndexParams {
  const int32_t* cu_q;        // [B + 1] or null (every sequence has S queries)
  const int32_t* seqused_kv;  // [B]
  const int32_t* ori_bt;      // [B, ori_table_len]
  const int32_t* cmp_bt;      // [B, cmp_table_len] or null
  const int32_t* cmp_idx;     // [T, K] or null
  int32_t* ori_rows;          // [T, win_left + 1]
  int32_t* cmp_rows;          // [T, K] or null
  int B, T, S, tnd;           // tnd: tokens are packed (sequence found from cu_q); else token = b * S + s
  int ori_table_len, ori_bs, win_left;
  int cmp_table_len, cmp_bs, ratio, scenario, K;
};

__global__ void __launch_bounds__(128) v4_build_indices_kernel(const V4IndexParams p) {
  const int t = blockIdx.x, tid = threadIdx.x;
  __shared__ int s_first_end;
  int b, s_local, len_q;
  if (p.tnd) {
    b = 0;
    while (b + 1 < p.B && t >= p.cu_q[b + 1]) ++b;
    s_local = t - p.cu_q[b];
    len_q = p.cu_q[b + 1] - p.cu_q[b];
  } else {
    b = t / p.S;
    s_local = t - b * p.S;
    len_q = p.cu_q ? p.cu_q[b + 1] - p.cu_q[b] : p.S;
  }
  const int act_kv = p.seqused_kv[b];
  const int pos = act_kv - len_q + s_local;
  const bool exists = s_local < len_q && pos >= 0;
  const int W = p.win_left + 1;
  for (int i = tid; i < W; i += 128) {
    const int w = pos - p.win_left + i;
    int row = -1;
    if (exists && w >= 0) row = p.ori_bt[static_cast<int64_t>(b) * p.ori_table_len + w / p.ori_bs] * p.ori_bs + w % p.ori_bs;
    p.ori_rows[static_cast<int64_t>(t) * W + i] = row;
  }
  if (p.scenario == 1 || !p.cmp_rows) return;
  const int threshold = exists ? (pos + 1) / p.ratio : 0;
  const int limit = min(threshold, act_kv / p.ratio);
  if (tid == 0) s_first_end = p.K;
  __syncthreads();
  if (p.scenario == 3) {
    for (int i = tid; i < p.K; i += 128)
      if (p.cmp_idx[static_cast<int64_t>(t) * p.K + i] == -1) atomicMin(&s_first_end, i);
    __syncthreads();
  }
  const int first_end = s_first_end;
  for (int i = tid; i < p.K; i += 128) {
    int c = -1;
    if (p.scenario == 3) {
      const int v = p.cmp_idx[static_cast<int64_t>(t) * p.K + i];
      if (i < threshold && i < first_end && v >= 0 && v < limit) c = v;
    } else if (i < threshold) {
      c = i;
    }
    int row = -1;
    if (c >= 0) row = p.cmp_bt[static_cast<int64_t>(b) * p.cmp_table_len + c / p.cmp_bs] * p.cmp_bs + c % p.cmp_bs;
    p.cmp_rows[static_cast<int64_t>(t) * p.K + i] = row;
  }
}

int launch_v4_build_indices(const int32_t* cu_q, const int32_t* seqused_kv, const int32_t* ori_bt, const int32_t* cmp_bt, const int32_t* cmp_idx,
                            int32_t* ori_rows, int32_t* cmp_rows, int B, int T, int S, int tnd, int ori_table_len, int ori_bs, int win_left,
                            int cmp_table_len, int cmp_bs, int ratio, int scenario, int K, cudaStream_t stream) {
  V4IndexParams p{cu_q, seqused_kv, ori_bt, cmp_bt, cmp_idx, ori_rows, cmp_rows, B, T, S, tnd, ori_table_len, ori_bs, win_left,
                  cmp_table_len, cmp_bs, ratio, scenario, K};
  v4_build_indices_kernel<<<static_cast<unsigned>(T), 128, 0, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace dsa
