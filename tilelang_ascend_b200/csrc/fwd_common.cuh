// Helpers shared by the sparse MLA forward kernels: which indices take part, where a key's row lives, packed fp32 arithmetic.
#pragma once
#include <type_traits>

#include "params.h"
#include "ptx.cuh"

namespace dsa {

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

// Packed pairs of fp32 (one instruction for two values) and the three-input maximum of sm_100.
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tadd.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
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

}  // namespace dsa
