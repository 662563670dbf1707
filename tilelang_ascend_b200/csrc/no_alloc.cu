// Lightning indexer + top-k for callers that must not allocate device memory.
//
// dsa_lightning_indexer needs a workspace (the fp32 score matrix and the per-row candidate counts) and the
// library's other entry points create a status word with cudaMalloc the first time a device is used.  Some
// callers can do neither: a serving process that handed every free byte of the GPU to its own memory pool
// at start-up (a later cudaMalloc simply fails), or a latency-bound loop that cannot accept the implicit
// device-wide synchronisation cudaMalloc / cudaFree may perform.  For them the scratch lives in the library
// image itself: a file-scope __device__ array that every GPU loading the library holds until the process
// exits.  Its size is the price of the convenience, so it is kept modest and larger problems are refused.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "../../include/dsa_b200.h"
#include "params.h"

namespace dsa {
void set_last_error(const std::string& msg);
size_t topk_smem_bytes(int n, int top_k, int* kpow2_out);
int launch_topk_select(const float* scores, int64_t rows, int n, int64_t row_stride, const int32_t* limits, int top_k,
                       int32_t* out_idx, float* out_val, cudaStream_t stream, int ordered = 1);
bool indexer_tc_supported(const IndexerParams& p);
int launch_indexer_scores_tc(const IndexerParams& p, bool bf16, cudaStream_t stream);
int launch_indexer_scores_generic(const IndexerParams& p, bool bf16, cudaStream_t stream);
}  // namespace dsa

namespace {

// Layout of the built-in scratch: [0, 256) status word of the kernels, then the per-row candidate counts,
// then the score matrix.  In host code `g_noalloc_scratch` is only a handle for cudaGetSymbolAddress --
// it is NOT a device address and must never be handed to a kernel directly.
static __device__ __align__(256) unsigned char g_noalloc_scratch[DSA_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_dev[kMaxDevices] = {nullptr};  // device address of the array, per device
std::mutex g_setup_mutex;

int fail(const std::string& msg) {
  dsa::set_last_error(msg);
  return 1;
}

// Once per device, with that device current: resolve the device address of the scratch array.
int scratch_address(unsigned char** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail("device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_dev[dev]) {
    unsigned char* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(std::string("cudaGetSymbolAddress(built-in scratch): ") + cudaGetErrorString(e));
    g_scratch_dev[dev] = ptr;
  }
  *out = g_scratch_dev[dev];
  return 0;
}

size_t round256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

}  // namespace

extern "C" {

size_t dsa_lightning_indexer_noalloc_max_bytes(void) { return DSA_NOALLOC_SCRATCH_BYTES; }

int dsa_lightning_indexer_noalloc(const void* q, const void* k, const float* w, int32_t B, int32_t S1, int32_t S2, int32_t N1,
                                  int32_t D, int32_t dtype, int32_t sparse_mode, const int32_t* q_len_b, const int32_t* k_len_b,
                                  int32_t top_k, int32_t* out_idx, float* out_val, int32_t* status_out, void* stream) {
  if (!q || !k || !w || !out_idx) return fail("null tensor pointer");
  if (dtype != DSA_DTYPE_BF16 && dtype != DSA_DTYPE_FP16) return fail("dtype must be 0 (bfloat16) or 1 (float16)");
  if (B <= 0 || S1 <= 0 || S2 <= 0 || N1 <= 0 || D <= 0 || D % 8 != 0) return fail("B, S1, S2, N1 must be positive and D a positive multiple of 8");
  if (sparse_mode != 0 && sparse_mode != 3) return fail("sparse_mode must be 0 or 3");
  if (top_k <= 0 || top_k > 8192) return fail("top_k must be in [1, 8192]");
  const size_t rows = static_cast<size_t>(B) * S1;
  const size_t off_limits = 256;
  const size_t off_scores = off_limits + round256(rows * sizeof(int32_t));
  const size_t need = off_scores + rows * static_cast<size_t>(S2) * sizeof(float);
  if (need > DSA_NOALLOC_SCRATCH_BYTES)
    return fail("problem too large for the built-in scratch: " + std::to_string(need) + " bytes needed, " +
                std::to_string(static_cast<size_t>(DSA_NOALLOC_SCRATCH_BYTES)) +
                " available (use dsa_lightning_indexer with a caller-provided workspace)");
  unsigned char* base = nullptr;
  if (scratch_address(&base)) return 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int* status = reinterpret_cast<int*>(base);
  int32_t* limits = reinterpret_cast<int32_t*>(base + off_limits);
  float* scores = reinterpret_cast<float*>(base + off_scores);
  // the array keeps whatever the previous call left: the status word must start at zero, everything else that is
  // read below (the candidate part of each score row, the limits) is rewritten by this call before it is read
  cudaError_t e = cudaMemsetAsync(status, 0, sizeof(int), st);
  if (e != cudaSuccess) return fail(std::string("cudaMemsetAsync(status word): ") + cudaGetErrorString(e));

  dsa::IndexerParams p{};  // (no paged keys on this path)
  p.q = q; p.k = k; p.w = w; p.scores = scores;
  p.B = B; p.S1 = S1; p.S2 = S2; p.N1 = N1; p.D = D;
  p.sparse_mode = sparse_mode; p.q_len_b = q_len_b; p.k_len_b = k_len_b; p.limits = limits;
  p.fill_masked = 0;
  p.status = status;
  int err;
  if (dsa::indexer_tc_supported(p)) {
    err = dsa::launch_indexer_scores_tc(p, dtype == DSA_DTYPE_BF16, st);
  } else {
    if ((static_cast<size_t>(N1) * D + N1) * 4 > 200 * 1024) return fail("N1 * D too large for the generic indexer kernel");
    err = dsa::launch_indexer_scores_generic(p, dtype == DSA_DTYPE_BF16, st);
  }
  if (err) return fail(std::string("indexer_scores launch: ") + cudaGetErrorString(static_cast<cudaError_t>(err)));
  err = dsa::launch_topk_select(scores, static_cast<int64_t>(rows), S2, S2, limits, top_k, out_idx, out_val, st);
  if (err) return fail(std::string("topk_select launch: ") + cudaGetErrorString(static_cast<cudaError_t>(err)));
  if (status_out) {
    e = cudaMemcpyAsync(status_out, status, sizeof(int), cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return fail(std::string("cudaMemcpyAsync(status word): ") + cudaGetErrorString(e));
  }
  return 0;
}

}  // extern "C"
