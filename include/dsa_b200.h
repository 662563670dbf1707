/* C ABI of the B200 (sm_100a) DeepSeek-sparse-attention kernels.
 *
 * Conventions (every entry point):
 *   - plain pointers and sizes; all data pointers are DEVICE pointers on the current CUDA device;
 *   - tensors are contiguous row-major in the layouts stated per function;
 *   - returns 0 on success, non-zero on error with a message available from dsa_get_last_error();
 *   - launches asynchronously on `stream` (a cudaStream_t passed as void*; NULL = default stream),
 *     never synchronises, and allocates nothing except one 4-byte status word per device on the
 *     first call on that device; workspaces are passed in by the caller;
 *   - dtype: 0 = bfloat16, 1 = float16.
 *
 * These replace, for this path, the `extern "C" void call(uint8_t* arg0, ..., int64_t dyn0, ...,
 * aclrtStream stream)` launcher that the reference's code generator emits per kernel
 * (src/target/codegen_ascend.cc:1141-1226) and that its adapter binds
 * (tilelang/jit/adapter/cython/cython_wrapper.pyx:75-203).  The `int` status + message convention is
 * the one of the reference's CUDA wrapper, `init / get_last_error / call`
 * (tilelang/jit/adapter/wrapper.py:30-50).
 */
#ifndef DSA_B200_H_
#define DSA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSA_DTYPE_BF16 0
#define DSA_DTYPE_FP16 1

/* Kernel choice for dsa_sparse_mla_fwd: the tensor-core kernel needs DV = 512 and D = 576 (512 latent + 64 rope dims) or
 * D = 512 (no rope dims: keys and values are the same rows). */
#define DSA_IMPL_AUTO 0
#define DSA_IMPL_GENERIC 1
#define DSA_IMPL_TENSOR_CORE 2

/* Prepares the current device (allocates and clears its status word).  Optional: every entry point
 * does this on first use.  Mirrors `init()` of tilelang/jit/adapter/wrapper.py:30-50. */
int dsa_init(void);

/* Message of the last failed call on this thread (empty string if none).
 * Mirrors `get_last_error()` of tilelang/jit/adapter/wrapper.py:30-50. */
const char* dsa_get_last_error(void);

/* Synchronises the current device, reads the device status word into *status (0 = every kernel ran
 * to completion, 1 = a bounded in-kernel wait gave up) and clears it.  No reference counterpart: the
 * reference launcher returns void and faults surface at the next synchronisation. */
int dsa_kernel_status(int* status);

/* Self-test of the kernels' bounded waits: launches one tiny kernel whose single waiting thread waits, for at most
 * budget_cycles SM clock cycles (1 .. 2e9; a million is about half a millisecond), on a barrier that nothing completes.
 * The wait runs out, the kernel sets the device status word to 1 and ends normally -- the mechanism by which every
 * tcgen05 kernel of this library turns a lost hand-over into a status instead of a hang.  gave_up: device int32 or
 * NULL, receives 1.  Afterwards dsa_kernel_status reports 1 (and clears the word); kernels launched while the word
 * is set return at once without writing results.  No reference counterpart. */
int dsa_selftest_bounded_wait(int64_t budget_cycles, int32_t* gave_up, void* stream);

/* Row-wise top-k.  scores [rows, row_stride] fp32 (n <= row_stride entries per row are looked at);
 * limits [rows] int32 or NULL: number of leading entries of each row that are candidates;
 * out_idx [rows, top_k] int32; out_val [rows, top_k] fp32 or NULL.
 * Order: descending score, equal scores by ascending index; candidates need score > -1e30; unused
 * slots hold -1 / -inf.  Replaces the kernel of simple_topk_selector
 * (examples/topk_selector/example_topk_selector.py:10-54) and the sort/merge phase of the
 * production indexer (examples/deepseek_v4/lightning_indexer.py:945-1081). */
int dsa_topk_select(const float* scores, int64_t rows, int64_t n, int64_t row_stride, const int32_t* limits,
                    int32_t top_k, int32_t* out_idx, float* out_val, void* stream);

/* dsa_topk_select without the final sort: the same SET of top_k indices per row (the same lowest-index tie rule at the
 * threshold), written in ASCENDING INDEX order instead of descending score order.  For consumers that only need the set --
 * the sparse attention that follows the indexer -- at about half the selector's time.  No reference counterpart (the reference
 * selector always sorts). */
int dsa_topk_select_unordered(const float* scores, int64_t rows, int64_t n, int64_t row_stride, const int32_t* limits,
                              int32_t top_k, int32_t* out_idx, float* out_val, void* stream);

/* Lightning-indexer scores: scores[b,s1,s2] = sum_h w[b,s1,h] * relu(q[b,s1,h,:] . k[b,s2,0,:]).
 * q [B,S1,N1,D], k [B,S2,1,D] (dtype), w [B,S1,N1] fp32, scores [B,S1,S2] fp32.
 * sparse_mode 3 = causal (key s2 is a candidate iff s2 < ak - aq + s1 + 1), 0 = all ak keys.
 * q_len_b / k_len_b: per-batch actual lengths [B] int32 or NULL.  limits_out [B,S1] int32 or NULL
 * receives the candidate count per row.  fill_masked != 0 writes -inf into every non-candidate entry
 * (needed when `scores` is read as a full matrix; dsa_topk_select with limits does not need it).
 * Replaces the cube + vector phases of make_lightning_indexer_kernel
 * (examples/deepseek_v4/lightning_indexer.py:661-940) and the `indexer` kernel
 * (examples/lightning_indexer/example_lightning_indexer.py:19-125). */
int dsa_indexer_scores(const void* q, const void* k, const float* w, float* scores, int32_t B, int32_t S1, int32_t S2,
                       int32_t N1, int32_t D, int32_t dtype, int32_t sparse_mode, const int32_t* q_len_b,
                       const int32_t* k_len_b, int32_t* limits_out, int32_t fill_masked, void* stream);

/* Bytes of workspace dsa_lightning_indexer needs (fp32 score matrix + per-row limits). */
size_t dsa_lightning_indexer_workspace_bytes(int32_t B, int32_t S1, int32_t S2);

/* Fused front door of the production indexer: scores + causal limits + top-k in one call.
 * out_idx [B,S1,1,top_k] int32, out_val [B,S1,1,top_k] fp32 or NULL, workspace as sized above.
 * Replaces the kernel launched by lightning_indexer(...)
 * (examples/deepseek_v4/lightning_indexer.py:1202-1370). */
int dsa_lightning_indexer(const void* q, const void* k, const float* w, int32_t B, int32_t S1, int32_t S2, int32_t N1,
                          int32_t D, int32_t dtype, int32_t sparse_mode, const int32_t* q_len_b, const int32_t* k_len_b,
                          int32_t top_k, int32_t* out_idx, float* out_val, void* workspace, size_t workspace_bytes,
                          void* stream);

/* dsa_lightning_indexer with the selector of dsa_topk_select_unordered: index sets in ascending index order. */
int dsa_lightning_indexer_unordered(const void* q, const void* k, const float* w, int32_t B, int32_t S1, int32_t S2, int32_t N1,
                                    int32_t D, int32_t dtype, int32_t sparse_mode, const int32_t* q_len_b, const int32_t* k_len_b,
                                    int32_t top_k, int32_t* out_idx, float* out_val, void* workspace, size_t workspace_bytes,
                                    void* stream);

/* dsa_lightning_indexer over a PAGED key cache: k_cache [num_blocks, block_size, 1, D] (dtype), block_table [B, max_blocks]
 * int32; logical key j of batch b is cache row block_table[b, j / block_size] * block_size + j % block_size.  S2 is the
 * largest logical key count (max_blocks * block_size >= S2); k_len_b [B] gives each sequence's count.  Table entries that
 * are padding (negative, or >= num_blocks) are never dereferenced; keys they would name lie beyond k_len_b in a well-formed
 * call.  The tensor-core kernel addresses the cache through the table tile by tile (TMA boxes inside one block when the
 * block size has a power-of-two factor >= 8, per-row copies otherwise): no dense copy of the keys is made.
 * Replaces the PA_BSND path of the kernel launched by lightning_indexer(..., layout_key="PA_BSND", block_table=...)
 * (examples/deepseek_v4/lightning_indexer.py:1256-1305; paged cube loads :661-793). */
int dsa_lightning_indexer_paged(const void* q, const void* k_cache, const float* w, int32_t B, int32_t S1, int32_t S2, int32_t N1,
                                int32_t D, int32_t dtype, int32_t sparse_mode, const int32_t* q_len_b, const int32_t* k_len_b,
                                const int32_t* block_table, int32_t block_size, int32_t max_blocks, int32_t num_blocks,
                                int32_t top_k, int32_t* out_idx, float* out_val, void* workspace, size_t workspace_bytes,
                                void* stream);

/* Size in bytes of the scratch array built into the library image (per GPU, held until the process exits). */
#define DSA_NOALLOC_SCRATCH_BYTES (32u << 20)
size_t dsa_lightning_indexer_noalloc_max_bytes(void);

/* dsa_lightning_indexer for callers that cannot allocate device memory -- a process whose own pool already owns
 * all free GPU memory, or a loop that cannot take the device-wide synchronisation an allocation may cause.
 * NO COUNTERPART IN THE REFERENCE (its adapter allocates workspaces with torch.empty on every call).
 * Same arguments and results as dsa_lightning_indexer, minus the workspace: scores and per-row limits live in
 * a DSA_NOALLOC_SCRATCH_BYTES array inside the library, and the kernels' status word too (this entry point
 * never calls cudaMalloc / cudaFree and creates no status word of its own).  status_out: device int32 or NULL;
 * receives the status word of this call (0 = ok) in stream order -- dsa_kernel_status does not see it.
 * Limits: 256 + round256(4 B S1) + 4 B S1 S2 bytes must fit the array, otherwise the call fails with a
 * message and launches nothing.  The first call on each device resolves the array's device address
 * (cudaGetSymbolAddress) with that device current: make that first call before any stream capture begins.
 * The array itself is reserved on a GPU when the library's device code is loaded there, which with CUDA's lazy loading
 * is the first call into the library on that device: a caller that then takes all remaining device memory for its own
 * pool must make that first call BEFORE the grab, or the load will fail for lack of memory.
 * All calls on a device share the one array and it keeps the previous call's contents (the call clears the
 * status word itself; nothing else needs to start at zero).  Two calls that overlap on the GPU -- different
 * streams, or different host threads -- race on it: serialise them. */
int dsa_lightning_indexer_noalloc(const void* q, const void* k, const float* w, int32_t B, int32_t S1, int32_t S2,
                                  int32_t N1, int32_t D, int32_t dtype, int32_t sparse_mode, const int32_t* q_len_b,
                                  const int32_t* k_len_b, int32_t top_k, int32_t* out_idx, float* out_val,
                                  int32_t* status_out, void* stream);

/* Sparse MLA forward.  q [B,S,H,D], kv [B,S_kv,1,D] (or [num_blocks,block_size,1,D] with a block
 * table), indices [B,S,1,topk] int32, out [B,S,H,DV] (dtype), lse [B,S,H] fp32 or NULL.
 * An index takes part iff 0 <= idx < kv_len and (not causal or idx <= q_start + t); -1 and S_kv are
 * therefore both padding.  Indices of one query must be distinct.  q_start_b / kv_len_b / q_len_b:
 * per-batch [B] int32 overrides or NULL.  sm_scale multiplies q.k before the softmax; lse is
 * natural-log.  Replaces the kernels of sparse_attention_fwd
 * (examples/sparse_flash_attention/example_sparse_flash_attn.py:18-243, _mask_pa.py:13-333) and of
 * sparse_attn_tilelang (bench_sfa/sparse_flash_attn_pa_no_cv_pipeline.py:27-419). */
int dsa_sparse_mla_fwd(const void* q, const void* kv, const int32_t* indices, void* out, float* lse, int32_t B,
                       int32_t S, int32_t S_kv, int32_t H, int32_t D, int32_t DV, int32_t topk, float sm_scale,
                       int32_t q_start, int32_t causal, int32_t dtype, const int32_t* q_start_b,
                       const int32_t* kv_len_b, const int32_t* q_len_b, const int32_t* block_table, int32_t block_size,
                       int32_t max_blocks, int32_t impl, void* stream);

/* The same forward with the keys of every query split over `nsplit` work units (tensor-core kernel only: D = 576,
 * DV = 512): for calls with fewer (query, block of 128 heads) items than SM pairs -- decode with a handful of
 * sequences per GPU -- where one unit per query would leave most of the GPU idle.  Each unit writes a normalised
 * partial output and its log-sum-exp into `workspace` (fp32, size from dsa_sparse_mla_fwd_splitkv_workspace_bytes,
 * 16-byte aligned, owned by the caller); a second kernel on the same stream combines them into out / lse.
 * nsplit = 1 is dsa_sparse_mla_fwd with impl = DSA_IMPL_TENSOR_CORE; dsa_sparse_mla_fwd_splitkv_nsplit suggests a
 * value for the current device (1 = do not split).  Queries that do not exist (q_len_b) get out = 0, lse = -inf.
 * Replaces the same reference kernels as dsa_sparse_mla_fwd (their decode shape:
 * bench_sfa/sparse_flash_attn_pa_no_cv_pipeline.py:384-419, T = 1). */
/* The forward with only the FIRST split_queries of the B * S queries (memory order) split into nsplit shares each, the
 * others handled whole: for launches whose last round of work units fills the SM pairs only partly (e.g. one GPU's block
 * of a sharded prefill: a persistent kernel reaches the first queries last) -- the split queries' shares then fill that
 * round.  workspace: dsa_sparse_mla_fwd_splitkv_workspace_bytes(1, split_queries, H, DV, nsplit) bytes.  Results of the
 * split queries are combined from fp32 partial results (same tolerance as dsa_sparse_mla_fwd_splitkv, not bit-equal to the
 * unsplit kernel); all other rows are bit-equal to dsa_sparse_mla_fwd. */
int dsa_sparse_mla_fwd_split_tail(const void* q, const void* kv, const int32_t* indices, void* out, float* lse, int32_t B, int32_t S,
                                  int32_t S_kv, int32_t H, int32_t D, int32_t DV, int32_t topk, float sm_scale, int32_t q_start,
                                  int32_t causal, int32_t dtype, const int32_t* q_start_b, const int32_t* kv_len_b, const int32_t* q_len_b,
                                  const int32_t* block_table, int32_t block_size, int32_t max_blocks, int32_t split_queries, int32_t nsplit,
                                  void* workspace, size_t workspace_bytes, void* stream);
/* The same forward with the key rows in TWO tensors addressed by the same row numbers: kv_latent [B, S_kv, 1, DV] (or paged
 * blocks) and kv_rope [B, S_kv, 1, D - DV] -- the KV and K_pe arguments of the reference's dense MLA decode kernels
 * (examples_experiment/deepseek_mla/example_mla_decode/example_mla_decode.py:46-249, example_mla_decode_paged.py:41-53),
 * used in place instead of being concatenated into rows of D values first.  D = 576, DV = 512, topk <= 8192 only; nsplit /
 * workspace as for dsa_sparse_mla_fwd_splitkv (nsplit = 1: no workspace). */
int dsa_sparse_mla_fwd_two_part(const void* q, const void* kv_latent, const void* kv_rope, const int32_t* indices, void* out, float* lse,
                                int32_t B, int32_t S, int32_t S_kv, int32_t H, int32_t D, int32_t DV, int32_t topk, float sm_scale,
                                int32_t q_start, int32_t causal, int32_t dtype, const int32_t* q_start_b, const int32_t* kv_len_b,
                                const int32_t* q_len_b, const int32_t* block_table, int32_t block_size, int32_t max_blocks, int32_t nsplit,
                                void* workspace, size_t workspace_bytes, void* stream);
int dsa_sparse_mla_fwd_splitkv_nsplit(int32_t B, int32_t S, int32_t H, int32_t topk);
size_t dsa_sparse_mla_fwd_splitkv_workspace_bytes(int32_t B, int32_t S, int32_t H, int32_t DV, int32_t nsplit);
int dsa_sparse_mla_fwd_splitkv(const void* q, const void* kv, const int32_t* indices, void* out, float* lse, int32_t B,
                               int32_t S, int32_t S_kv, int32_t H, int32_t D, int32_t DV, int32_t topk, float sm_scale,
                               int32_t q_start, int32_t causal, int32_t dtype, const int32_t* q_start_b,
                               const int32_t* kv_len_b, const int32_t* q_len_b, const int32_t* block_table,
                               int32_t block_size, int32_t max_blocks, int32_t nsplit, void* workspace,
                               size_t workspace_bytes, void* stream);

/* Sparse MLA backward.  Inputs as the forward plus out / lse of the forward and d_out [B,S,H,DV];
 * outputs d_q [B,S,H,D] (dtype) and d_kv (fp32, same shape as kv, ACCUMULATED INTO: zero it first).
 * The reference has no counterpart kernel; the decomposition follows its dense backward
 * (examples_experiment/example_gqa_bwd/example_gqa_bwd.py:189-556). */
int dsa_sparse_mla_bwd(const void* q, const void* kv, const int32_t* indices, const void* out, const float* lse,
                       const void* d_out, void* d_q, float* d_kv, int32_t B, int32_t S, int32_t S_kv, int32_t H,
                       int32_t D, int32_t DV, int32_t topk, float sm_scale, int32_t q_start, int32_t causal,
                       int32_t dtype, const int32_t* q_start_b, const int32_t* kv_len_b, const int32_t* q_len_b,
                       const int32_t* block_table, int32_t block_size, int32_t max_blocks, void* stream);

/* Sparse MLA backward on the tensor cores (D = 576, DV = 512, topk <= 8192): same arguments and results as
 * dsa_sparse_mla_bwd, plus a caller-owned workspace (256-byte aligned).  The work is done in passes over consecutive
 * queries; a pass keeps P and dS of its queries in the workspace (dsa_sparse_mla_bwd_tc_workspace_bytes(B, S, H, topk, n)
 * bytes hold n queries per pass; n <= 0 or n >= B * S = all queries in one pass).  queries_per_pass <= 0 lets the
 * library use as many as the workspace holds.  d_kv is accumulated into with fp32 atomics: zero it first.
 * No counterpart in the reference (see dsa_sparse_mla_bwd). */
size_t dsa_sparse_mla_bwd_tc_workspace_bytes(int32_t B, int32_t S, int32_t H, int32_t topk, int32_t queries_per_pass);
int dsa_sparse_mla_bwd_tc(const void* q, const void* kv, const int32_t* indices, const void* out, const float* lse,
                          const void* d_out, void* d_q, float* d_kv, int32_t B, int32_t S, int32_t S_kv, int32_t H,
                          int32_t D, int32_t DV, int32_t topk, float sm_scale, int32_t q_start, int32_t causal,
                          int32_t dtype, const int32_t* q_start_b, const int32_t* kv_len_b, const int32_t* q_len_b,
                          const int32_t* block_table, int32_t block_size, int32_t max_blocks, void* workspace,
                          size_t workspace_bytes, int32_t queries_per_pass, void* stream);

/* Merges one or two partial attention results over disjoint key sets with a per-head sink logit:
 * lse = log(exp(lse_a) + exp(lse_b) + exp(sinks[h])), out = exp(lse_a - lse) out_a + exp(lse_b - lse) out_b.
 * out_a / out_b / out [rows, DV] (dtype), lse_a / lse_b / lse [rows] fp32 with rows = tokens * H (head fastest), sinks [H]
 * fp32 or NULL (no sink); out_b / lse_b may be NULL (one partial); lse may be NULL; out may alias out_a.
 * Together with two dsa_sparse_mla_fwd calls (sliding window of the original cache; selected compressed tokens) this replaces
 * the kernel of sparse_flash_mla (examples/deepseek_v4/sparse_flash_mla/sparse_flash_mla_kernel.py; sink and LSE handling
 * :1053-1064, golden sparse_flash_mla_golden.py:121-153). */
int dsa_sink_combine(const void* out_a, const float* lse_a, const void* out_b, const float* lse_b, const float* sinks,
                     void* out, float* lse, int64_t rows, int32_t H, int32_t DV, int32_t dtype, void* stream);

/* Block-sparse indexer logits (HISA): logits[s, j, b] = sum_h w[s,h] * relu(q[s,h,:] . k[block_indices[s,j] * kv_block_size + b, :]),
 * -inf where that position is outside [0, S_kv) or outside [ks[s], ke[s]).  q [S,H,D], k [S_kv,D] (dtype), block_indices
 * [S,topk] int32, weights [S,H] (weights_dtype: 0 bf16, 1 fp16, 2 fp32), ks / ke [S] int32, logits [S,topk,kv_block_size] fp32.
 * Paged keys: with block_table [B, max_blocks] (else NULL) k is the cache [num_phys_blocks, kv_block_size, 1, D], the indices
 * name LOGICAL blocks of the sequence of query s (sequence = s / tokens_per_seq) and S_kv = num_phys_blocks * kv_block_size (the
 * rows of the cache).  A table entry is read only for positions inside [ks[s], ke[s]) -- entries of blocks past a sequence's
 * context may be padding such as -1 -- and an entry outside [0, num_phys_blocks) is not dereferenced (its logits are -inf); this is the kernel of
 * paged_block_sparse_mqa_attn_return_logits (examples/HISA/paged_block_sparse_mqa_attn_expert.py:54-420, golden :425-468)
 * with ks = 0 and ke = the sequence's context length.
 * impl: DSA_IMPL_AUTO = the tcgen05 kernel when kv_block_size = 128, D = 128 and H <= 64, else CUDA cores; DSA_IMPL_GENERIC /
 * DSA_IMPL_TENSOR_CORE force one.
 * Replaces the kernel of block_sparse_mqa_attn_return_logits (examples/HISA/block_sparse_mqa_attn_expert_test.py:24-545;
 * golden ref_block_sparse_mqa_attn :548-587). */
int dsa_block_sparse_logits(const void* q, const void* k, const int32_t* block_indices, const void* weights, const int32_t* ks,
                            const int32_t* ke, float* logits, int32_t S, int32_t S_kv, int32_t H, int32_t D,
                            int32_t kv_block_size, int32_t topk, int32_t dtype, int32_t weights_dtype, int32_t impl,
                            const int32_t* block_table, int32_t max_blocks, int32_t tokens_per_seq, void* stream);

/* Index lists of sparse_flash_mla for T query tokens: ori_rows [T, ori_win_left + 1] and cmp_rows [T, K] int32 receive the
 * physical row numbers (block_table[b, pos / block_size] * block_size + pos % block_size) of each token's sliding window
 * of the original cache and of its compressed keys, -1 where a slot takes no part; they are the `indices` of two
 * dsa_sparse_mla_fwd calls over the flattened pools.  tnd != 0: tokens are packed and cu_seqlens_q [B + 1] gives the sequence
 * starts; tnd == 0: token = b * S + s (cu_seqlens_q optional: actual lengths, padded tokens get empty lists).
 * scenario 1: window only (cmp_* unused); 2: every compressed token below floor((p + 1) / cmp_ratio); 3: the caller's
 * cmp_sparse_indices [T, K], cut at the first -1.  Replaces the per-token key selection inside the reference kernel
 * (examples/deepseek_v4/sparse_flash_mla/sparse_flash_mla_kernel.py; rules restated from sparse_flash_mla_golden.py:16-53, 95-118). */
int dsa_v4_build_indices(const int32_t* cu_seqlens_q, const int32_t* seqused_kv, const int32_t* ori_block_table,
                         const int32_t* cmp_block_table, const int32_t* cmp_sparse_indices, int32_t* ori_rows, int32_t* cmp_rows,
                         int32_t B, int32_t T, int32_t S, int32_t tnd, int32_t ori_table_len, int32_t ori_block_size,
                         int32_t ori_win_left, int32_t cmp_table_len, int32_t cmp_block_size, int32_t cmp_ratio, int32_t scenario,
                         int32_t K, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DSA_B200_H_ */
