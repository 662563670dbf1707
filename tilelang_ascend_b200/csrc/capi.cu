// C ABI of the library: argument validation, parameter blocks, kernel launches.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <mutex>
#include <string>

#include "../../include/dsa_b200.h"
#include "launch_util.h"
#include "params.h"

namespace dsa {
// launchers defined in the kernel translation units
bool sparse_mla_fwd_tc_supported(const FwdParams& p);
int launch_sparse_mla_fwd_tc(const FwdParams& p, bool bf16, cudaStream_t stream);
bool sparse_mla_fwd_pair_supported(const FwdParams& p);
int launch_sparse_mla_fwd_pair_combined(const FwdParams& p, bool bf16, cudaStream_t stream);
int launch_sparse_mla_fwd_generic(const FwdParams& p, bool bf16, cudaStream_t stream);
int sparse_mla_fwd_auto_nsplit(const FwdParams& p, int sms);
size_t topk_smem_bytes(int n, int top_k, int* kpow2_out);
int launch_topk_select(const float* scores, int64_t rows, int n, int64_t row_stride, const int32_t* limits, int top_k,
                       int32_t* out_idx, float* out_val, cudaStream_t stream, int ordered = 1);
bool indexer_tc_supported(const IndexerParams& p);
int launch_indexer_scores_tc(const IndexerParams& p, bool bf16, cudaStream_t stream);
int launch_indexer_scores_generic(const IndexerParams& p, bool bf16, cudaStream_t stream);
int launch_sparse_mla_bwd(const BwdParams& bp, bool bf16, cudaStream_t stream);
int launch_sink_combine(const void* out_a, const float* lse_a, const void* out_b, const float* lse_b, const float* sinks, void* out, float* lse,
                        int64_t rows, int H, int DV, bool bf16, cudaStream_t stream);
int launch_v4_build_indices(const int32_t* cu_q, const int32_t* seqused_kv, const int32_t* ori_bt, const int32_t* cmp_bt, const int32_t* cmp_idx,
                            int32_t* ori_rows, int32_t* cmp_rows, int B, int T, int S, int tnd, int ori_table_len, int ori_bs, int win_left,
                            int cmp_table_len, int cmp_bs, int ratio, int scenario, int K, cudaStream_t stream);
bool block_sparse_logits_supported(const BlockSparseLogitsParams& p);
bool block_sparse_logits_tc_supported(const BlockSparseLogitsParams& p);
int launch_block_sparse_logits_tc(const BlockSparseLogitsParams& p, bool bf16, cudaStream_t stream);
int launch_block_sparse_logits(const BlockSparseLogitsParams& p, bool bf16, cudaStream_t stream);
int launch_bounded_wait_selftest(int* status, long long budget_cycles, int* gave_up, cudaStream_t stream);
bool sparse_mla_bwd_tc_supported(const FwdParams& p);
size_t sparse_mla_bwd_tc_bytes_per_query(int H, int topk);
int launch_sparse_mla_bwd_tc(const BwdParams& bp, bool bf16, void* workspace, size_t workspace_bytes, int queries_per_pass, cudaStream_t stream);
}  // namespace dsa

namespace {

thread_local std::string g_last_error;

}  // namespace

namespace dsa {
// Lets the other translation units of the library report through dsa_get_last_error().
void set_last_error(const std::string& msg) { g_last_error = msg; }
}  // namespace dsa

namespace {

int fail(const std::string& msg) {
  g_last_error = msg;
  return 1;
}
int fail_cuda(const char* what, int err) {
  g_last_error = std::string(what) + ": " + cudaGetErrorString(static_cast<cudaError_t>(err));
  return 1;
}

constexpr int kMaxDevices = 64;
int* g_status[kMaxDevices] = {nullptr};
std::mutex g_status_mutex;

// Device status word of the current device (allocated and cleared on first use).
int get_status_word(int** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda("cudaGetDevice", e);
  if (dev < 0 || dev >= kMaxDevices) return fail("device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (!g_status[dev]) {
    int* ptr = nullptr;
    e = cudaMalloc(&ptr, sizeof(int));
    if (e != cudaSuccess) return fail_cuda("cudaMalloc(status word)", e);
    e = cudaMemset(ptr, 0, sizeof(int));
    if (e != cudaSuccess) return fail_cuda("cudaMemset(status word)", e);
    g_status[dev] = ptr;
  }
  *out = g_status[dev];
  return 0;
}

#ifdef DSA_TRACE
long long* g_trace = nullptr;  // development builds only: device buffer the forward kernel's clock samples go to
#endif

bool dtype_ok(int dtype) { return dtype == DSA_DTYPE_BF16 || dtype == DSA_DTYPE_FP16; }

int fill_fwd_params(dsa::FwdParams* p, const void* q, const void* kv, const int32_t* indices, void* out, float* lse, int32_t B,
                    int32_t S, int32_t S_kv, int32_t H, int32_t D, int32_t DV, int32_t topk, float sm_scale, int32_t q_start,
                    int32_t causal, int32_t dtype, const int32_t* q_start_b, const int32_t* kv_len_b, const int32_t* q_len_b,
                    const int32_t* block_table, int32_t block_size, int32_t max_blocks) {
  if (!q || !kv || !indices || !out) return fail("null tensor pointer");
  if (!dtype_ok(dtype)) return fail("dtype must be 0 (bfloat16) or 1 (float16)");
  if (B <= 0 || S <= 0 || S_kv <= 0 || H <= 0 || topk <= 0) return fail("B, S, S_kv, H and topk must be positive");
  if (D <= 0 || D % 8 != 0 || D > 640) return fail("D must be a positive multiple of 8, at most 640");
  if (DV <= 0 || DV > D || DV > 512) return fail("DV must be in [1, min(D, 512)]");
  if (static_cast<int64_t>(B) * S > 0x7fffffffLL / 2) return fail("B * S too large");
  if (block_table && (block_size <= 0 || max_blocks <= 0)) return fail("block_size and max_blocks must be positive with a block table");
  if (!(sm_scale > 0.f) || !std::isfinite(sm_scale)) return fail("sm_scale must be positive and finite");
  p->q = q; p->kv = kv; p->indices = indices; p->out = out; p->lse = lse;
  p->B = B; p->S = S; p->S_kv = S_kv; p->H = H; p->topk = topk; p->D = D; p->DV = DV;
  p->q_start = q_start; p->causal = causal ? 1 : 0;
  p->q_start_b = q_start_b; p->kv_len_b = kv_len_b; p->q_len_b = q_len_b;
  p->block_table = block_table; p->block_size = block_size; p->max_blocks = max_blocks;
  p->scale_log2 = sm_scale * 1.4426950408889634f;
  p->nsplit = 1; p->part_out = nullptr; p->part_lse = nullptr; p->kv_rope = nullptr; p->split_queries = 0;
#ifdef DSA_TRACE
  p->trace = g_trace;
#endif
  return get_status_word(&p->status);
}

}  // namespace

extern "C" {

#ifdef DSA_TRACE
void dsa_set_trace(long long* device_buffer) { g_trace = device_buffer; }
#endif

int dsa_init(void) {
  int* s = nullptr;
  return get_status_word(&s);
}

const char* dsa_get_last_error(void) { return g_last_error.c_str(); }

int dsa_kernel_status(int* status) {
  int* s = nullptr;
  if (get_status_word(&s)) return 1;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail_cuda("cudaDeviceSynchronize", e);
  int host = 0;
  e = cudaMemcpy(&host, s, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail_cuda("cudaMemcpy(status word)", e);
  if (host != 0) {
    e = cudaMemset(s, 0, sizeof(int));
    if (e != cudaSuccess) return fail_cuda("cudaMemset(status word)", e);
  }
  if (status) *status = host;
  return 0;
}

int dsa_selftest_bounded_wait(int64_t budget_cycles, int32_t* gave_up, void* stream) {
  if (budget_cycles < 1 || budget_cycles > 2000000000LL) return fail("budget_cycles must be in [1, 2e9]");
  int* s = nullptr;
  if (get_status_word(&s)) return 1;
  int err = dsa::launch_bounded_wait_selftest(s, budget_cycles, gave_up, static_cast<cudaStream_t>(stream));
  return err ? fail_cuda("bounded_wait_selftest launch", err) : 0;
}

static int topk_select_impl(const float* scores, int64_t rows, int64_t n, int64_t row_stride, const int32_t* limits, int32_t top_k,
                            int32_t* out_idx, float* out_val, void* stream, int ordered) {
  if (!scores || !out_idx) return fail("null tensor pointer");
  if (rows < 0 || n <= 0 || top_k <= 0 || row_stride < n) return fail("need rows >= 0, n > 0, top_k > 0, row_stride >= n");
  if (rows == 0) return 0;
  if (rows > 0x7fffffffLL) return fail("too many rows");
  if (top_k > 8192) return fail("top_k must be at most 8192");
  if (n > 0x7fffffffLL) return fail("row too long");
  int err = dsa::launch_topk_select(scores, rows, static_cast<int>(n), row_stride, limits, top_k, out_idx, out_val,
                                    static_cast<cudaStream_t>(stream), ordered);
  return err ? fail_cuda("topk_select launch", err) : 0;
}

int dsa_topk_select(const float* scores, int64_t rows, int64_t n, int64_t row_stride, const int32_t* limits, int32_t top_k,
                    int32_t* out_idx, float* out_val, void* stream) {
  return topk_select_impl(scores, rows, n, row_stride, limits, top_k, out_idx, out_val, stream, 1);
}

int dsa_topk_select_unordered(const float* scores, int64_t rows, int64_t n, int64_t row_stride, const int32_t* limits, int32_t top_k,
                              int32_t* out_idx, float* out_val, void* stream) {
  return topk_select_impl(scores, rows, n, row_stride, limits, top_k, out_idx, out_val, stream, 0);
}

// Paged keys of the indexer: block table [B, max_blocks] over a cache of num_blocks blocks of block_size rows (all zero = dense k).
struct PagedKeys {
  const int32_t* block_table = nullptr;
  int32_t block_size = 0, max_blocks = 0, num_blocks = 0;
};

static int indexer_scores_impl(const void* q, const void* k, const float* w, float* scores, int32_t B, int32_t S1, int32_t S2,
                               int32_t N1, int32_t D, int32_t dtype, int32_t sparse_mode, const int32_t* q_len_b,
                               const int32_t* k_len_b, int32_t* limits_out, int32_t fill_masked, void* stream,
                               const PagedKeys& paged = PagedKeys()) {
  if (!q || !k || !w || !scores) return fail("null tensor pointer");
  if (!dtype_ok(dtype)) return fail("dtype must be 0 (bfloat16) or 1 (float16)");
  if (B <= 0 || S1 <= 0 || S2 <= 0 || N1 <= 0 || D <= 0) return fail("B, S1, S2, N1 and D must be positive");
  if (sparse_mode != 0 && sparse_mode != 3) return fail("sparse_mode must be 0 or 3");
  if (D % 8 != 0) return fail("D must be a multiple of 8");
  dsa::IndexerParams p{};
  p.q = q; p.k = k; p.w = w; p.scores = scores;
  p.B = B; p.S1 = S1; p.S2 = S2; p.N1 = N1; p.D = D;
  p.sparse_mode = sparse_mode; p.q_len_b = q_len_b; p.k_len_b = k_len_b; p.limits = limits_out;
  p.fill_masked = fill_masked ? 1 : 0;
  if (paged.block_table) {
    if (paged.block_size <= 0 || paged.max_blocks <= 0 || paged.num_blocks <= 0) return fail("block_size, max_blocks and num_blocks must be positive with a block table");
    if (static_cast<int64_t>(paged.max_blocks) * paged.block_size < S2) return fail("the block table covers fewer than S2 keys");
    if (static_cast<int64_t>(paged.num_blocks) * paged.block_size > 0x7fffffffLL) return fail("paged key cache too large");
    p.block_table = paged.block_table; p.block_size = paged.block_size; p.max_blocks = paged.max_blocks; p.num_blocks = paged.num_blocks;
  }
  if (get_status_word(&p.status)) return 1;
  int err;
  if (dsa::indexer_tc_supported(p)) {
    err = dsa::launch_indexer_scores_tc(p, dtype == DSA_DTYPE_BF16, static_cast<cudaStream_t>(stream));
  } else {
    if ((static_cast<size_t>(N1) * D + N1) * 4 > 200 * 1024) return fail("N1 * D too large for the generic indexer kernel");
    err = dsa::launch_indexer_scores_generic(p, dtype == DSA_DTYPE_BF16, static_cast<cudaStream_t>(stream));
  }
  return err ? fail_cuda("indexer_scores launch", err) : 0;
}

int dsa_indexer_scores(const void* q, const void* k, const float* w, float* scores, int32_t B, int32_t S1, int32_t S2, int32_t N1,
                       int32_t D, int32_t dtype, int32_t sparse_mode, const int32_t* q_len_b, const int32_t* k_len_b,
                       int32_t* limits_out, int32_t fill_masked, void* stream) {
  return indexer_scores_impl(q, k, w, scores, B, S1, S2, N1, D, dtype, sparse_mode, q_len_b, k_len_b, limits_out, fill_masked,
                             stream);
}

size_t dsa_lightning_indexer_workspace_bytes(int32_t B, int32_t S1, int32_t S2) {
  const size_t rows = static_cast<size_t>(B) * S1;
  const size_t scores = (rows * S2 * sizeof(float) + 255) & ~static_cast<size_t>(255);
  return scores + rows * sizeof(int32_t);
}

static int lightning_indexer_impl(const void* q, const void* k, const float* w, int32_t B, int32_t S1, int32_t S2, int32_t N1, int32_t D,
                                  int32_t dtype, int32_t sparse_mode, const int32_t* q_len_b, const int32_t* k_len_b, int32_t top_k,
                                  int32_t* out_idx, float* out_val, void* workspace, size_t workspace_bytes, void* stream,
                                  const PagedKeys& paged, int ordered) {
  if (!workspace || workspace_bytes < dsa_lightning_indexer_workspace_bytes(B, S1, S2)) return fail("workspace missing or too small");
  if (!out_idx) return fail("null tensor pointer");
  const size_t rows = static_cast<size_t>(B) * S1;
  float* scores = static_cast<float*>(workspace);
  int32_t* limits = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + ((rows * S2 * sizeof(float) + 255) & ~static_cast<size_t>(255)));
  int rc = indexer_scores_impl(q, k, w, scores, B, S1, S2, N1, D, dtype, sparse_mode, q_len_b, k_len_b, limits, 0, stream, paged);
  if (rc) return rc;
  return topk_select_impl(scores, static_cast<int64_t>(rows), S2, S2, limits, top_k, out_idx, out_val, stream, ordered);
}

int dsa_lightning_indexer(const void* q, const void* k, const float* w, int32_t B, int32_t S1, int32_t S2, int32_t N1, int32_t D,
                          int32_t dtype, int32_t sparse_mode, const int32_t* q_len_b, const int32_t* k_len_b, int32_t top_k,
                          int32_t* out_idx, float* out_val, void* workspace, size_t workspace_bytes, void* stream) {
  return lightning_indexer_impl(q, k, w, B, S1, S2, N1, D, dtype, sparse_mode, q_len_b, k_len_b, top_k, out_idx, out_val, workspace,
                                workspace_bytes, stream, PagedKeys(), 1);
}

int dsa_lightning_indexer_unordered(const void* q, const void* k, const float* w, int32_t B, int32_t S1, int32_t S2, int32_t N1, int32_t D,
                                    int32_t dtype, int32_t sparse_mode, const int32_t* q_len_b, const int32_t* k_len_b, int32_t top_k,
                                    int32_t* out_idx, float* out_val, void* workspace, size_t workspace_bytes, void* stream) {
  return lightning_indexer_impl(q, k, w, B, S1, S2, N1, D, dtype, sparse_mode, q_len_b, k_len_b, top_k, out_idx, out_val, workspace,
                                workspace_bytes, stream, PagedKeys(), 0);
}

int dsa_lightning_indexer_paged(const void* q, const void* k_cache, const float* w, int32_t B, int32_t S1, int32_t S2, int32_t N1, int32_t D,
                                int32_t dtype, int32_t sparse_mode, const int32_t* q_len_b, const int32_t* k_len_b, const int32_t* block_table,
                                int32_t block_size, int32_t max_blocks, int32_t num_blocks, int32_t top_k, int32_t* out_idx, float* out_val,
                                void* workspace, size_t workspace_bytes, void* stream) {
  if (!block_table) return fail("null tensor pointer");
  PagedKeys paged;
  paged.block_table = block_table; paged.block_size = block_size; paged.max_blocks = max_blocks; paged.num_blocks = num_blocks;
  return lightning_indexer_impl(q, k_cache, w, B, S1, S2, N1, D, dtype, sparse_mode, q_len_b, k_len_b, top_k, out_idx, out_val, workspace,
                                workspace_bytes, stream, paged, 1);
}

int dsa_sparse_mla_fwd(const void* q, const void* kv, const int32_t* indices, void* out, float* lse, int32_t B, int32_t S,
                       int32_t S_kv, int32_t H, int32_t D, int32_t DV, int32_t topk, float sm_scale, int32_t q_start, int32_t causal,
                       int32_t dtype, const int32_t* q_start_b, const int32_t* kv_len_b, const int32_t* q_len_b,
                       const int32_t* block_table, int32_t block_size, int32_t max_blocks, int32_t impl, void* stream) {
  dsa::FwdParams p;
  if (fill_fwd_params(&p, q, kv, indices, out, lse, B, S, S_kv, H, D, DV, topk, sm_scale, q_start, causal, dtype, q_start_b,
                      kv_len_b, q_len_b, block_table, block_size, max_blocks))
    return 1;
  const bool tc_ok = dsa::sparse_mla_fwd_tc_supported(p);
  if (impl == DSA_IMPL_TENSOR_CORE && !tc_ok) return fail("the tensor-core kernel needs D = 576 or 512, DV = 512 and topk <= 8192");
  if (impl != DSA_IMPL_AUTO && impl != DSA_IMPL_GENERIC && impl != DSA_IMPL_TENSOR_CORE) return fail("unknown impl");
  const bool use_tc = impl == DSA_IMPL_TENSOR_CORE || (impl == DSA_IMPL_AUTO && tc_ok);
  int err = use_tc ? dsa::launch_sparse_mla_fwd_tc(p, dtype == DSA_DTYPE_BF16, static_cast<cudaStream_t>(stream))
                   : dsa::launch_sparse_mla_fwd_generic(p, dtype == DSA_DTYPE_BF16, static_cast<cudaStream_t>(stream));
  return err ? fail_cuda("sparse_mla_fwd launch", err) : 0;
}

int dsa_sparse_mla_fwd_two_part(const void* q, const void* kv_latent, const void* kv_rope, const int32_t* indices, void* out, float* lse,
                                int32_t B, int32_t S, int32_t S_kv, int32_t H, int32_t D, int32_t DV, int32_t topk, float sm_scale,
                                int32_t q_start, int32_t causal, int32_t dtype, const int32_t* q_start_b, const int32_t* kv_len_b,
                                const int32_t* q_len_b, const int32_t* block_table, int32_t block_size, int32_t max_blocks, int32_t nsplit,
                                void* workspace, size_t workspace_bytes, void* stream) {
  if (!kv_rope) return fail("null tensor pointer");
  if (D != 576 || DV != 512) return fail("key rows in two parts need D = 576 and DV = 512");
  if ((reinterpret_cast<uintptr_t>(kv_latent) | reinterpret_cast<uintptr_t>(kv_rope)) & 15u) return fail("key tensors must be 16-byte aligned");
  dsa::FwdParams p;
  if (fill_fwd_params(&p, q, kv_latent, indices, out, lse, B, S, S_kv, H, D, DV, topk, sm_scale, q_start, causal, dtype, q_start_b,
                      kv_len_b, q_len_b, block_table, block_size, max_blocks))
    return 1;
  if (!dsa::sparse_mla_fwd_pair_supported(p)) return fail("key rows in two parts need topk <= 8192");
  p.kv_rope = kv_rope;
  if (nsplit < 1 || nsplit > 64) return fail("nsplit must be in [1, 64]");
  if (nsplit > 1) {
    const size_t need = dsa_sparse_mla_fwd_splitkv_workspace_bytes(B, S, H, DV, nsplit);
    if (!workspace || workspace_bytes < need) return fail("workspace too small (see dsa_sparse_mla_fwd_splitkv_workspace_bytes)");
    if (reinterpret_cast<uintptr_t>(workspace) & 15u) return fail("workspace must be 16-byte aligned");
    p.nsplit = nsplit;
    p.part_out = static_cast<float*>(workspace);
    p.part_lse = p.part_out + static_cast<size_t>(nsplit) * B * S * H * DV;
  }
  int err = dsa::launch_sparse_mla_fwd_pair_combined(p, dtype == DSA_DTYPE_BF16, static_cast<cudaStream_t>(stream));
  return err ? fail_cuda("sparse_mla_fwd_two_part launch", err) : 0;
}

int dsa_sparse_mla_fwd_splitkv_nsplit(int32_t B, int32_t S, int32_t H, int32_t topk) {
  int dev = 0, sms = 0;
  if (dsa::current_device_sms(&dev, &sms) != cudaSuccess) return 1;
  dsa::FwdParams p{};
  p.B = B; p.S = S; p.H = H; p.topk = topk;
  return dsa::sparse_mla_fwd_auto_nsplit(p, sms);
}

size_t dsa_sparse_mla_fwd_splitkv_workspace_bytes(int32_t B, int32_t S, int32_t H, int32_t DV, int32_t nsplit) {
  if (B <= 0 || S <= 0 || H <= 0 || DV <= 0 || nsplit <= 1) return 0;
  const size_t rows = static_cast<size_t>(B) * S * H;
  return static_cast<size_t>(nsplit) * rows * (static_cast<size_t>(DV) + 1) * sizeof(float);
}

int dsa_sparse_mla_fwd_splitkv(const void* q, const void* kv, const int32_t* indices, void* out, float* lse, int32_t B, int32_t S,
                               int32_t S_kv, int32_t H, int32_t D, int32_t DV, int32_t topk, float sm_scale, int32_t q_start,
                               int32_t causal, int32_t dtype, const int32_t* q_start_b, const int32_t* kv_len_b, const int32_t* q_len_b,
                               const int32_t* block_table, int32_t block_size, int32_t max_blocks, int32_t nsplit, void* workspace,
                               size_t workspace_bytes, void* stream) {
  dsa::FwdParams p;
  if (fill_fwd_params(&p, q, kv, indices, out, lse, B, S, S_kv, H, D, DV, topk, sm_scale, q_start, causal, dtype, q_start_b,
                      kv_len_b, q_len_b, block_table, block_size, max_blocks))
    return 1;
  if (!dsa::sparse_mla_fwd_tc_supported(p)) return fail("split-KV needs the tensor-core kernel: D = 576 or 512, DV = 512 and topk <= 8192");
  if (nsplit < 1 || nsplit > 64) return fail("nsplit must be in [1, 64]");
  if (nsplit > 1) {
    const size_t need = dsa_sparse_mla_fwd_splitkv_workspace_bytes(B, S, H, DV, nsplit);
    if (!workspace || workspace_bytes < need) return fail("workspace too small (see dsa_sparse_mla_fwd_splitkv_workspace_bytes)");
    if (reinterpret_cast<uintptr_t>(workspace) & 15u) return fail("workspace must be 16-byte aligned");
    p.nsplit = nsplit;
    p.part_out = static_cast<float*>(workspace);
    p.part_lse = p.part_out + static_cast<size_t>(nsplit) * B * S * H * DV;
  }
  int err = dsa::launch_sparse_mla_fwd_tc(p, dtype == DSA_DTYPE_BF16, static_cast<cudaStream_t>(stream));
  return err ? fail_cuda("sparse_mla_fwd_splitkv launch", err) : 0;
}

int dsa_sparse_mla_fwd_split_tail(const void* q, const void* kv, const int32_t* indices, void* out, float* lse, int32_t B, int32_t S,
                                  int32_t S_kv, int32_t H, int32_t D, int32_t DV, int32_t topk, float sm_scale, int32_t q_start,
                                  int32_t causal, int32_t dtype, const int32_t* q_start_b, const int32_t* kv_len_b, const int32_t* q_len_b,
                                  const int32_t* block_table, int32_t block_size, int32_t max_blocks, int32_t split_queries, int32_t nsplit,
                                  void* workspace, size_t workspace_bytes, void* stream) {
  dsa::FwdParams p;
  if (fill_fwd_params(&p, q, kv, indices, out, lse, B, S, S_kv, H, D, DV, topk, sm_scale, q_start, causal, dtype, q_start_b,
                      kv_len_b, q_len_b, block_table, block_size, max_blocks))
    return 1;
  if (!dsa::sparse_mla_fwd_pair_supported(p)) return fail("a split tail needs D = 576 or 512, DV = 512 and topk <= 8192");
  if (nsplit < 2 || nsplit > 64) return fail("nsplit must be in [2, 64]");
  if (split_queries < 1 || static_cast<int64_t>(split_queries) >= static_cast<int64_t>(B) * S) return fail("split_queries must be in [1, B * S)");
  const size_t need = dsa_sparse_mla_fwd_splitkv_workspace_bytes(1, split_queries, H, DV, nsplit);
  if (!workspace || workspace_bytes < need) return fail("workspace too small (dsa_sparse_mla_fwd_splitkv_workspace_bytes(1, split_queries, H, DV, nsplit))");
  if (reinterpret_cast<uintptr_t>(workspace) & 15u) return fail("workspace must be 16-byte aligned");
  p.nsplit = nsplit;
  p.split_queries = split_queries;
  p.part_out = static_cast<float*>(workspace);
  p.part_lse = p.part_out + static_cast<size_t>(nsplit) * split_queries * H * DV;
  int err = dsa::launch_sparse_mla_fwd_pair_combined(p, dtype == DSA_DTYPE_BF16, static_cast<cudaStream_t>(stream));
  return err ? fail_cuda("sparse_mla_fwd_split_tail launch", err) : 0;
}

int dsa_sparse_mla_bwd(const void* q, const void* kv, const int32_t* indices, const void* out, const float* lse, const void* d_out,
                       void* d_q, float* d_kv, int32_t B, int32_t S, int32_t S_kv, int32_t H, int32_t D, int32_t DV, int32_t topk,
                       float sm_scale, int32_t q_start, int32_t causal, int32_t dtype, const int32_t* q_start_b,
                       const int32_t* kv_len_b, const int32_t* q_len_b, const int32_t* block_table, int32_t block_size,
                       int32_t max_blocks, void* stream) {
  if (!lse || !d_out || !d_q || !d_kv) return fail("null tensor pointer");
  dsa::BwdParams bp;
  if (fill_fwd_params(&bp.f, q, kv, indices, const_cast<void*>(out), const_cast<float*>(lse), B, S, S_kv, H, D, DV, topk, sm_scale,
                      q_start, causal, dtype, q_start_b, kv_len_b, q_len_b, block_table, block_size, max_blocks))
    return 1;
  bp.d_out = d_out; bp.d_q = d_q; bp.d_kv = d_kv; bp.sm_scale = sm_scale;
  int err = dsa::launch_sparse_mla_bwd(bp, dtype == DSA_DTYPE_BF16, static_cast<cudaStream_t>(stream));
  return err ? fail_cuda("sparse_mla_bwd launch", err) : 0;
}

size_t dsa_sparse_mla_bwd_tc_workspace_bytes(int32_t B, int32_t S, int32_t H, int32_t topk, int32_t queries_per_pass) {
  if (B <= 0 || S <= 0 || H <= 0 || topk <= 0) return 0;
  size_t nq = static_cast<size_t>(B) * S;
  if (queries_per_pass > 0 && static_cast<size_t>(queries_per_pass) < nq) nq = queries_per_pass;
  return nq * dsa::sparse_mla_bwd_tc_bytes_per_query(H, topk);
}

int dsa_sparse_mla_bwd_tc(const void* q, const void* kv, const int32_t* indices, const void* out, const float* lse, const void* d_out,
                          void* d_q, float* d_kv, int32_t B, int32_t S, int32_t S_kv, int32_t H, int32_t D, int32_t DV, int32_t topk,
                          float sm_scale, int32_t q_start, int32_t causal, int32_t dtype, const int32_t* q_start_b,
                          const int32_t* kv_len_b, const int32_t* q_len_b, const int32_t* block_table, int32_t block_size,
                          int32_t max_blocks, void* workspace, size_t workspace_bytes, int32_t queries_per_pass, void* stream) {
  if (!lse || !d_out || !d_q || !d_kv) return fail("null tensor pointer");
  dsa::BwdParams bp;
  if (fill_fwd_params(&bp.f, q, kv, indices, const_cast<void*>(out), const_cast<float*>(lse), B, S, S_kv, H, D, DV, topk, sm_scale,
                      q_start, causal, dtype, q_start_b, kv_len_b, q_len_b, block_table, block_size, max_blocks))
    return 1;
  if (!dsa::sparse_mla_bwd_tc_supported(bp.f)) return fail("the tensor-core backward needs D = 576, DV = 512 and topk <= 8192");
  const uintptr_t all = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kv) | reinterpret_cast<uintptr_t>(out) |
                        reinterpret_cast<uintptr_t>(d_out) | reinterpret_cast<uintptr_t>(d_q) | reinterpret_cast<uintptr_t>(d_kv);
  if (all & 15u) return fail("q, kv, out, d_out, d_q and d_kv must be 16-byte aligned");
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return fail("workspace must be non-null and 256-byte aligned");
  if (workspace_bytes < dsa::sparse_mla_bwd_tc_bytes_per_query(H, topk))
    return fail("workspace too small: it must hold at least one query (see dsa_sparse_mla_bwd_tc_workspace_bytes)");
  bp.d_out = d_out; bp.d_q = d_q; bp.d_kv = d_kv; bp.sm_scale = sm_scale;
  int err = dsa::launch_sparse_mla_bwd_tc(bp, dtype == DSA_DTYPE_BF16, workspace, workspace_bytes, queries_per_pass, static_cast<cudaStream_t>(stream));
  return err ? fail_cuda("sparse_mla_bwd_tc launch", err) : 0;
}

int dsa_sink_combine(const void* out_a, const float* lse_a, const void* out_b, const float* lse_b, const float* sinks, void* out, float* lse,
                     int64_t rows, int32_t H, int32_t DV, int32_t dtype, void* stream) {
  if (!out_a || !lse_a || !out) return fail("null tensor pointer");
  if ((out_b == nullptr) != (lse_b == nullptr)) return fail("out_b and lse_b must both be given or both be null");
  if (!dtype_ok(dtype)) return fail("dtype must be 0 (bfloat16) or 1 (float16)");
  if (rows <= 0 || H <= 0 || DV <= 0 || rows % H != 0) return fail("rows must be a positive multiple of H; DV positive");
  int err = dsa::launch_sink_combine(out_a, lse_a, out_b, lse_b, sinks, out, lse, rows, H, DV, dtype == DSA_DTYPE_BF16, static_cast<cudaStream_t>(stream));
  return err ? fail_cuda("sink_combine launch", err) : 0;
}

int dsa_block_sparse_logits(const void* q, const void* k, const int32_t* block_indices, const void* weights, const int32_t* ks,
                            const int32_t* ke, float* logits, int32_t S, int32_t S_kv, int32_t H, int32_t D, int32_t kv_block_size,
                            int32_t topk, int32_t dtype, int32_t weights_dtype, int32_t impl, const int32_t* block_table, int32_t max_blocks,
                            int32_t tokens_per_seq, void* stream) {
  if (!q || !k || !block_indices || !weights || !ks || !ke || !logits) return fail("null tensor pointer");
  if (!dtype_ok(dtype)) return fail("dtype must be 0 (bfloat16) or 1 (float16)");
  if (weights_dtype < 0 || weights_dtype > 2) return fail("weights_dtype must be 0 (bfloat16), 1 (float16) or 2 (float32)");
  if (S <= 0 || S_kv <= 0 || kv_block_size <= 0 || topk <= 0) return fail("S, S_kv, kv_block_size and topk must be positive");
  if (block_table && (max_blocks <= 0 || tokens_per_seq <= 0)) return fail("max_blocks and tokens_per_seq must be positive with a block table");
  dsa::BlockSparseLogitsParams p{q, k, block_indices, weights, ks, ke, logits, S, S_kv, H, D, kv_block_size, topk, weights_dtype,
                                 block_table, max_blocks, tokens_per_seq, nullptr};
  if (get_status_word(&p.status)) return 1;
  if (!dsa::block_sparse_logits_supported(p)) return fail("block-sparse logits need 1 <= heads <= 64 and index_dim a multiple of 8, at most 256");
  if ((reinterpret_cast<uintptr_t>(k) & 15u) || (reinterpret_cast<uintptr_t>(q) & 15u)) return fail("q and k must be 16-byte aligned");
  // blocks of 128 keys with index_dim 128 and up to 64 heads go to the tensor cores (impl = DSA_IMPL_GENERIC keeps them off)
  const bool use_tc = impl != DSA_IMPL_GENERIC && dsa::block_sparse_logits_tc_supported(p);
  if (impl == DSA_IMPL_TENSOR_CORE && !use_tc) return fail("the tensor-core kernel needs kv_block_size = 128, index_dim = 128 and at most 64 heads");
  int err = use_tc ? dsa::launch_block_sparse_logits_tc(p, dtype == DSA_DTYPE_BF16, static_cast<cudaStream_t>(stream))
                   : dsa::launch_block_sparse_logits(p, dtype == DSA_DTYPE_BF16, static_cast<cudaStream_t>(stream));
  return err ? fail_cuda("block_sparse_logits launch", err) : 0;
}

int dsa_v4_build_indices(const int32_t* cu_seqlens_q, const int32_t* seqused_kv, const int32_t* ori_block_table, const int32_t* cmp_block_table,
                         const int32_t* cmp_sparse_indices, int32_t* ori_rows, int32_t* cmp_rows, int32_t B, int32_t T, int32_t S, int32_t tnd,
                         int32_t ori_table_len, int32_t ori_block_size, int32_t ori_win_left, int32_t cmp_table_len, int32_t cmp_block_size,
                         int32_t cmp_ratio, int32_t scenario, int32_t K, void* stream) {
  if (!seqused_kv || !ori_block_table || !ori_rows) return fail("null tensor pointer");
  if (B <= 0 || T <= 0 || ori_table_len <= 0 || ori_block_size <= 0 || ori_win_left < 0) return fail("B, T, table length and block size must be positive");
  if (tnd ? !cu_seqlens_q : (S <= 0 || T != B * S)) return fail("packed tokens need cu_seqlens_q; otherwise T must equal B * S");
  if (scenario < 1 || scenario > 3) return fail("scenario must be 1 (window only), 2 (all compressed tokens) or 3 (selected compressed tokens)");
  if (scenario != 1 && (!cmp_block_table || !cmp_rows || cmp_table_len <= 0 || cmp_block_size <= 0 || cmp_ratio <= 0 || K <= 0))
    return fail("compressed-token scenarios need the compressed block table, an output buffer, a positive ratio and K");
  if (scenario == 3 && !cmp_sparse_indices) return fail("scenario 3 needs cmp_sparse_indices");
  int err = dsa::launch_v4_build_indices(cu_seqlens_q, seqused_kv, ori_block_table, cmp_block_table, cmp_sparse_indices, ori_rows, cmp_rows, B, T, S, tnd,
                                         ori_table_len, ori_block_size, ori_win_left, cmp_table_len, cmp_block_size, cmp_ratio, scenario, K,
                                         static_cast<cudaStream_t>(stream));
  return err ? fail_cuda("v4_build_indices launch", err) : 0;
}

}  // extern "C"
