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

}  // namespace dsa
