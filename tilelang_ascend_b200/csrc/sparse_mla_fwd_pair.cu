// Sparse MLA forward for sm_100a on PAIRS of SMs: every MMA is a tcgen05 cta_group::2 instruction that runs on both CTAs of a
// 2-CTA cluster.  Same semantics as the kernels in sparse_mla_fwd.cu (ref_sparse_attention_fwd_interface,
// examples/sparse_flash_attention/example_sparse_flash_attn.py:255-292; -1 / length rules of
// example_sparse_flash_attn_mask_pa.py:221-238), for D = 576 (or 512, rows without rope dims) and DV = 512.
//
// A cluster handles one (query, block of 128 heads) item at a time, persistent over items.  The pair splits an item by HEADS
// and every tile of 64 gathered keys by KEYS:
//   CTA r owns heads [64 r, 64 r + 64) and gathers keys [32 r, 32 r + 32) of each tile -- whole rows of 1152 bytes.
//   * S = Q K^T: M = 128 heads, N = 64 keys.  Each CTA supplies its 64 rows of Q and its 32 keys as the halves of A and B and
//     receives the COMPLETE scores of its 64 heads against all 64 keys: nothing is summed across CTAs and each CTA runs the
//     softmax of its own 64 rows only.
//   * O = P V: M = 128 heads, N = 512 output dims as two MMAs of N = 256.  CTA r supplies P of its 64 heads and, as its half of
//     B, the value dims [256 r, 256 r + 256) of ALL 64 keys of the tile -- so it needs those dims of the peer's 32 keys.  They
//     take the place of the dims of its own keys that it does not need after Q K^T (dims [256 (1 - r), +256)): once the
//     Q K^T of a tile is complete the two CTAs SWAP those 16 KB regions of the stage (exchange warps: read the own region into
//     registers, tell the peer, wait for the peer to have read its region, write the registers into the peer's region with
//     st.async).  Both CTAs then hold [64 keys x their 256 dims] at the same shared-memory offsets, as cta_group::2 requires.
//   Per CTA: O = 64 heads x 512 dims fp32 in 128 lanes x 256 columns of tensor memory (lanes 0..63: dims 0..255, lanes 64..127:
//   dims 256..511), two score buffers of 32 columns (lanes 0..63: keys 0..31, lanes 64..127: keys 32..63), Q dims 0..383 as the
//   tensor-memory A operand (192 columns, the same row in lanes m and m + 64), Q dims 384..575 in shared memory.
// A unit's Q rows travel through two slots of the stage ring ahead of the unit's tiles (see the gather warps).
// Warp roles (20 warps): 8 softmax warps (two per 32 lanes: 16 score columns each), 4 gather warps (they also build the units'
// tile lists and send Q), 4 exchange warps (the swap; they also move Q from its ring slots to tensor memory and the Q buffer),
// and four issuing warps in the EVEN CTA: Q K^T of the even tiles, Q K^T of the odd tiles, and one P V issuer per N = 256
// half.  Issuing warps stay converged -- all lanes walk the loops and waits, one elected lane issues through predicated
// instructions.  In the odd CTA lane 0 of the same four warps forwards "my gather landed" / "my softmax warps are past the
// scores" / "my half of the swap landed" / "my P is written" to the even CTA.
// Barriers the issuers wait for live in the even CTA and count arrivals from both CTAs; completions (tcgen05.commit) are
// broadcast to the same barrier in both CTAs.  Every wait is bounded; a wait that gives up records status 1 and all roles
// fall through to the teardown.
#include "fwd_common.cuh"
#include "launch_util.h"
#include "params.h"
#include "ptx.cuh"

namespace dsa {

namespace pr {
constexpr int kD = 576, kDV = 512;
constexpr int kM = 128;                                // heads per cluster
constexpr int kHeads = 64;                             // heads per CTA
constexpr int kBK = 64;                                // keys per tile
constexpr int kKeys = 32;                              // keys per tile and CTA
constexpr int kStages = 5;
constexpr int kMaxTiles = 128;                         // topk <= 8192
constexpr uint32_t kChunk = kKeys * 128;               // 4096: 32 keys x 64 dims, 128-byte swizzle
constexpr uint32_t kStageBytes = 9 * kChunk;           // 36864: 8 latent chunks + the rope chunk
constexpr uint32_t kSwapBytes = 4 * kChunk;            // 16384: four chunks trade places with the peer's
constexpr uint32_t kQChunk = kHeads * 128;             // 8192: 64 heads x 64 dims
constexpr uint32_t kQBytes = 3 * kQChunk;              // Q dims 384..575 in shared memory
constexpr uint32_t kQPiece = kHeads * 64;              // 4096: 64 heads x 32 dims, the unit in which those dims ride the stage ring
constexpr uint32_t kQPieceOff = 3 * kQChunk;           // pieces sit behind the three tensor-memory chunks of a ring slot
constexpr uint32_t kPBytes = kHeads * kBK * 2;         // 8192: P of one tile [64 heads x 64 keys]
constexpr uint32_t kOffQ = kStages * kStageBytes;      // 184320
constexpr uint32_t kOffP = kOffQ + kQBytes;            // the Q buffer, then two P buffers
constexpr uint32_t kOffBar = kOffP + 2 * kPBytes;
constexpr uint32_t kOffRowMax = kOffBar + 512;         // [2][4][64] floats: row maxima of the four threads of a row, by tile parity
constexpr uint32_t kOffRowSum = kOffRowMax + 2 * 4 * 64 * 4;   // [4][64] floats
constexpr uint32_t kOffMask = kOffRowSum + 4 * 64 * 4;         // [2][kMaxTiles] 64-bit validity masks (per item parity)
constexpr uint32_t kOffList = kOffMask + 2 * kMaxTiles * 8;    // [2][kMaxTiles] 16-bit tile ids
constexpr uint32_t kOffInfo = kOffList + 2 * kMaxTiles * 2;    // [2] {tile count, run flag}; scratch words of the warps behind it
// No slack to align the base: the kernel's only shared memory is this dynamic array, declared with 1024-byte alignment (the
// swizzled operand tiles need it); the kernel checks the base and reports kStatusBadLayout instead of running misaligned.
constexpr uint32_t kSmemBytes = kOffInfo + 256;
static_assert(kSmemBytes <= 232448, "shared memory per CTA");
static_assert(kQPieceOff + 3 * kQPiece <= kStageBytes, "a ring slot holds half of Q");
constexpr int kSoftmaxWarps = 8;                       // warp w: lanes 32 (w & 3) .. +31, score columns 16 (w >> 2) .. +15
constexpr int kFirstGatherWarp = 8;
constexpr int kFirstExchangeWarp = 12;                 // 12..15: (w & 3) is also the lane quarter of their tensor-memory stores
// The four issuing warps sit on the four sub-partitions of the SM (warp % 4); the two Q K^T issuers, which issue nine times
// as many instructions as the P V issuers, share theirs with softmax warps of DIFFERENT 32-head blocks (warp % 2), so that
// neither block of softmax warps is the slower one.
constexpr int kQkWarp = 16;                            // even CTA: Q K^T issuer of the even tiles; odd CTA: forwards kv_full
constexpr int kQkWarpB = 17;                           // even CTA: Q K^T issuer of the odd tiles; odd CTA: forwards s_free
constexpr int kPvWarp = 18;                            // even CTA: first P V issuer; odd CTA: forwards v_full
constexpr int kRelayWarp = 19;                         // even CTA: second P V issuer; odd CTA: forwards p_ready
constexpr int kThreads = 640;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 0, kColS = 256, kColQ = 320;  // O 256 | S0 32 | S1 32 | Q 192
constexpr float kRescaleThreshold = 8.0f;              // log2 units: P stays below 2^8
constexpr uint32_t kGatherBarrier = 5;                 // named barrier of the 128 gather threads
// barrier slots (8 bytes each).  "even CTA" barriers receive one remote arrival per event from a forwarding thread of the odd CTA:
// a remote arrive with release semantics costs its issuer about a thousand clocks, which the softmax warps cannot afford per
// tile -- they arrive on barriers of their own CTA and a dedicated thread passes the completed phase on.
constexpr int kBarKvFull = 0;                     // [kStages] count 128: cp.async completion of this CTA's gather threads
constexpr int kBarPeerKvFull = kStages;           // [kStages] count 1, even CTA: the odd CTA's gather of the stage landed
constexpr int kBarKvEmpty = 2 * kStages;          // [kStages] count 2: commits of the two P V issuers after their MMAs of the stage
constexpr int kBarPeerRead = 3 * kStages;         // [kStages] count 4: the peer's exchange warps hold their swap region in registers
constexpr int kBarVFull = 4 * kStages;            // [kStages] count 1 + 16384 bytes: the peer's half of the swap landed here
constexpr int kBarPeerVFull = 5 * kStages;        // [kStages] count 1, even CTA: ... landed in the odd CTA
constexpr int kBarSFull = 6 * kStages;            // [2] count 1: commit after the Q K^T MMAs
constexpr int kBarSFree = kBarSFull + 2;          // [2] count 12: this CTA's softmax (and exchange) warps are past the scores
constexpr int kBarPeerSFree = kBarSFull + 4;      // [2] count 1, even CTA: ... the odd CTA's
constexpr int kBarPReady = kBarSFull + 6;         // [2] count 8: this CTA's softmax warps wrote P
constexpr int kBarPeerPReady = kBarSFull + 8;     // [2] count 1, even CTA: ... the odd CTA's
constexpr int kBarPFree = kBarSFull + 10;         // [2] count 2: commits of the two P V issuers after their MMAs that read this P buffer
constexpr int kBarQReady = kBarSFull + 12;        // count 8, even CTA: the exchange warps of both CTAs loaded the item's Q
constexpr int kBarQFree = kBarSFull + 13;         // count 2: both Q K^T issuers are done with the item's Q (commit after their last MMAs of the item)
constexpr int kBarOFree = kBarSFull + 14;         // count 16, even CTA: the softmax warps drained the previous item's output
constexpr int kBarInfoFull = kBarSFull + 15;      // [2] count 1: tile list of an item published by the gather warps
constexpr int kBarInfoEmpty = kBarSFull + 17;     // [2] count 16: softmax, exchange, issuer / forwarding warps are done with the list
constexpr int kBarQRead = kBarSFull + 19;         // count 4: the exchange warps have emptied a Q slot of the ring
constexpr int kBarCount = kBarSFull + 20;
static_assert(kBarCount * 8 + 16 <= 512, "barrier region");
}  // namespace pr

// Remote arrives in this kernel are RELAXED: an arrive with release semantics at cluster scope costs its thread about 1100
// clocks here (measured), far too much per tile.  None of them publishes data that another SM reads through the memory
// system: what they announce -- rows landed in this SM's shared memory, tensor-memory loads / stores of this SM finished,
// shared-memory loads finished -- is complete on THIS SM before the arrive is issued (observed on a local barrier, or held
// back by a dependent instruction), and the consumers are this SM's tensor core, started by the even CTA's issuing thread
// only after it has seen the arrival, or the peer's st.async writes, issued only after it has seen the arrival.
// Arrive (count 1) on the barrier at `local_addr` of CTA `target` of the cluster: a plain arrive when that is this CTA.
__device__ __forceinline__ void arrive_at(uint32_t local_addr, uint32_t target, uint32_t my_rank) {
  if (target == my_rank) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(local_addr) : "memory");
  } else {
    mbar_arrive_cluster_relaxed(map_to_cta(local_addr, target));
  }
}
__device__ __forceinline__ void st_async_v4_b32(uint32_t cluster_addr, uint32_t cluster_mbar, uint4 v) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(cluster_addr), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w), "r"(cluster_mbar)
               : "memory");
}

template <bool kBF16, bool kRope>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pr::kThreads, 1) sparse_mla_fwd_pair_kernel(const FwdParams p) {
  using namespace pr;
  constexpr int kRowBytes = kRope ? kD * 2 : kDV * 2;
  constexpr int kChunks = kRope ? 9 : 8;               // 64-dim chunks of a key row
  constexpr int kQSmemChunks = kChunks - 6;            // Q chunks 6.. in shared memory
  constexpr int kQPiecesPerSlot = kQSmemChunks;        // ... as 2 kQSmemChunks pieces of 32 dims, half of them in each of the two ring slots
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sBase = smem_u32(smem);
  if (sBase & 1023u) {  // same in every CTA of the launch: nobody runs, nobody waits
    if (threadIdx.x == 0) atomicCAS(p.status, kStatusOk, kStatusBadLayout);
    return;
  }
  const uint32_t sQ = sBase + kOffQ;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
  const uint32_t sBars = sBase + kOffBar;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kBarCount);
  int* start_status = reinterpret_cast<int*>(bars + kBarCount + 1);
  float* rowmax = reinterpret_cast<float*>(smem + kOffRowMax);
  float* rowsum = reinterpret_cast<float*>(smem + kOffRowSum);
  unsigned long long* masks = reinterpret_cast<unsigned long long*>(smem + kOffMask);
  uint16_t* tile_list = reinterpret_cast<uint16_t*>(smem + kOffList);
  int* info = reinterpret_cast<int*>(smem + kOffInfo);  // [2][2]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();   // which 64 heads, which 32 keys of a tile
  const uint32_t peer = rank ^ 1u;
  const int num_clusters = gridDim.x >> 1, cluster_id = blockIdx.x >> 1;
  const int head_blocks = (p.H + kM - 1) / kM;
  const int nsplit = p.nsplit > 1 ? p.nsplit : 1;
  // Work units: a (query, head block) item, or one of the nsplit shares of its key tiles.  The first split_rows queries are
  // split (all of them unless the caller names fewer: the tail of a launch, which the clusters reach last and which fills
  // their last round only partly), the others are one unit each.  Units are numbered with the split items first.
  const int split_rows = nsplit > 1 ? ((p.split_queries > 0 && p.split_queries < p.B * p.S) ? p.split_queries : p.B * p.S) : 0;
  const int split_units = split_rows * head_blocks * nsplit;
  const int num_items = split_units + (p.B * p.S - split_rows) * head_blocks;
  const int ntiles = (p.topk + kBK - 1) / kBK;
  using T = typename std::conditional<kBF16, __nv_bfloat16, __half>::type;
  // k-th work unit of this cluster (late queries first), or negative
  auto item_of = [&](int k) { return num_items - 1 - cluster_id - k * num_clusters; };
  // unit -> (query, head block) item, its share and the number of shares of that item
  auto item_and_share = [&](int u, int* share, int* shares) {
    if (u < split_units) {
      const int it = u / nsplit;
      *share = u - it * nsplit;
      *shares = nsplit;
      return it;
    }
    *share = 0;
    *shares = 1;
    return split_rows * head_blocks + (u - split_units);
  };
#ifdef DSA_TRACE
#ifndef DSA_TRACE_MASK
#define DSA_TRACE_MASK 0xffffffu   // which events are compiled in: every sample point slows its role, a build with few is closer to the product
#endif
  auto tr = [&](int ev, int g) {
    if (((DSA_TRACE_MASK >> ev) & 1u) && cluster_id == 0 && g < 64 && p.trace) p.trace[(rank * 24 + ev) * 64 + g] = clock64();
  };
#else
  auto tr = [&](int, int) {};
#endif
  auto bar = [&](int slot) { return bars + slot; };
  auto bar_addr = [&](int slot) { return sBars + static_cast<uint32_t>(slot) * 8u; };

  // First Q row (head 64 r of the unit's head block) of work unit `u` and the number of this CTA's 64 rows that exist
  // (nullptr / 0 when the unit does not exist).  The 64 rows are contiguous in q: 64 x kRowBytes bytes.
  auto q_rows_of = [&](int u, int* nrows) -> const uint8_t* {
    *nrows = 0;
    if (u < 0) return nullptr;
    int sh_unused, ns_unused;
    const int it_item = item_and_share(u, &sh_unused, &ns_unused);
    const int nbt = it_item / head_blocks, nh0 = (it_item - nbt * head_blocks) * kM + static_cast<int>(rank) * kHeads;
    if (nh0 >= p.H) return nullptr;
    *nrows = p.H - nh0 < kHeads ? p.H - nh0 : kHeads;
    return reinterpret_cast<const uint8_t*>(p.q) + (static_cast<int64_t>(nbt) * p.H + nh0) * kRowBytes;
  };

  // ---- setup ------------------------------------------------------------------------------------------
  if (tid == 0) {
    *start_status = *reinterpret_cast<volatile int*>(p.status);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar(kBarKvFull + i), 128); mbar_init(bar(kBarPeerKvFull + i), 1); mbar_init(bar(kBarKvEmpty + i), 2);
      mbar_init(bar(kBarPeerRead + i), 4); mbar_init(bar(kBarVFull + i), 1); mbar_init(bar(kBarPeerVFull + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(kBarSFull + i), 1); mbar_init(bar(kBarSFree + i), kSoftmaxWarps + 4); mbar_init(bar(kBarPeerSFree + i), 1);
      mbar_init(bar(kBarPReady + i), kSoftmaxWarps); mbar_init(bar(kBarPeerPReady + i), 1); mbar_init(bar(kBarPFree + i), 2);
      mbar_init(bar(kBarInfoFull + i), 1); mbar_init(bar(kBarInfoEmpty + i), kSoftmaxWarps + 4 + 4);
    }
    mbar_init(bar(kBarQReady), 8); mbar_init(bar(kBarQFree), 2); mbar_init(bar(kBarOFree), 2 * kSoftmaxWarps);
    mbar_init(bar(kBarQRead), 4);
    for (int i = 0; i < 4; ++i) info[i] = 0;
    mbar_init_fence();
  }
  if (warp == kQkWarp) {  // the same warp of both CTAs allocates the pair's tensor memory
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tO = tmem_base + kColO, tS = tmem_base + kColS, tQ = tmem_base + kColQ;
  // both CTAs must have their barriers initialised before any remote arrive; every thread takes part
  cluster_sync_all();
  const bool run_all = *start_status == kStatusOk;
  bool ok = true;

  if (warp < kSoftmaxWarps) {
    // ================================ softmax + epilogue ============================================
    // thread = (tensor-memory lane L, column half ch): head m = L % 64 of this CTA, keys 32 (L / 64) + 16 ch .. + 15 of a tile,
    // output dims 256 (L / 64) + 128 ch .. + 127.  The four threads of a head combine their maxima (and at the end their sums)
    // through shared memory and a 128-thread named barrier per block of 32 heads.  A failed wait clears `ok` but does not leave
    // the loops (the partner warps would wait at the named barrier): the remaining tiles are walked without waiting.
    const int q4 = warp & 3, ch = warp >> 2;
    const int L = q4 * 32 + lane, m = L & 63, kh = L >> 6;
    const int part = 2 * kh + ch;
    const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
    const uint32_t named = 1 + (q4 & 1);
    int g = 0;
    for (int k = 0; run_all; ++k) {
      const int unit = item_of(k);
      if (unit < 0) break;
      int share, shares;
      const int item = item_and_share(unit, &share, &shares);
      const int qp = k & 1;
      const int bt = item / head_blocks, h0 = (item - bt * head_blocks) * kM;
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(kBarInfoFull + qp), (k >> 1) & 1, p.status));
      const int nvt = info[qp * 2];  // read unconditionally: all warps of a head block must walk the same number of tiles
      float m_used = -INFINITY, l = 0.f;
      for (int it = 0; it < nvt; ++it, ++g) {
        const uint32_t mask = static_cast<uint32_t>(masks[qp * kMaxTiles + tile_list[qp * kMaxTiles + it]] >> (32 * kh + 16 * ch)) & 0xffffu;
        const int sb = g & 1;
        uint32_t sc[16];  // scores as raw bits (tensor-memory loads), used as floats below
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(kBarSFull + sb), (g >> 1) & 1, p.status));
        if (tid == 0) tr(3, g);
        tc_fence_after();
        tmem_ld16(tS + sb * 32 + ch * 16 + lane_base, sc);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(kBarSFree + sb));  // the Q K^T of tile g+2 may overwrite the buffer
        float mx;
        {
          // scores of keys that do not take part count as -inf from here on: their exponentials are exact zeros.  (One code
          // path for full and partly filled tiles: a separate fast path for full tiles made the loop longer and the kernel slower.)
#pragma unroll
          for (int j = 0; j < 16; ++j) sc[j] = ((mask >> j) & 1u) ? sc[j] : 0xff800000u;
          float m4[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) m4[j] = fmaxf(__uint_as_float(sc[2 * j]), __uint_as_float(sc[2 * j + 1]));
#pragma unroll
          for (int j = 4; j < 8; ++j) m4[j & 3] = fmax3(m4[j & 3], __uint_as_float(sc[2 * j]), __uint_as_float(sc[2 * j + 1]));
          mx = fmaxf(fmax3(m4[0], m4[1], m4[2]), m4[3]);
        }
        float* slot = rowmax + (g & 1) * 256;
        slot[part * 64 + m] = mx;
        // exponentials relative to this thread's own maximum, before the barrier: the MUFU work overlaps the wait for the
        // partner warps, and only one correction factor per thread is left for afterwards
        const float m_loc = mx * p.scale_log2;                      // -inf when no key of this thread takes part
        const float neg_loc = (mx == -INFINITY) ? 0.f : -m_loc;
        float pe[16];
        float2 sum2 = make_float2(0.f, 0.f);
        const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), neg2 = make_float2(neg_loc, neg_loc);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 x = ffma2(make_float2(__uint_as_float(sc[2 * j]), __uint_as_float(sc[2 * j + 1])), scale2, neg2);
          float2 e = make_float2(exp2f(x.x), exp2f(x.y));
          pe[2 * j] = e.x; pe[2 * j + 1] = e.y;
          sum2 = fadd2(sum2, e);
        }
        named_bar_sync(named, 128);
        mx = fmaxf(fmaxf(slot[m], slot[64 + m]), fmaxf(slot[128 + m], slot[192 + m])) * p.scale_log2;
        // ---- online softmax with a lazily updated reference maximum (identical in the four threads of the head) ----
        float factor = 1.f;
        if (mx > m_used + kRescaleThreshold || m_used == -INFINITY) {
          factor = (m_used == -INFINITY) ? 0.f : exp2f(m_used - mx);
          m_used = mx;
        }
        if (it > 0 && __any_sync(0xffffffffu, factor != 1.f)) {
          // O must be quiescent: the P V MMAs of the previous tile are done.  (Waited for on that tile's P buffer barrier:
          // its phase before -- tile g-3 -- was already waited for when P of tile g-1 was written, so the parity
          // test cannot be fooled by a barrier that is two phases behind.)
          if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(kBarPFree + ((g - 1) & 1)), ((g - 1) >> 1) & 1, p.status));
          tc_fence_after();
          uint32_t o[32];
#pragma unroll 1
          for (int cc = 4 * ch; cc < 4 * ch + 4; ++cc) {  // this thread's half of the lane's output columns
            tmem_ld32(tO + lane_base + cc * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * factor);
            tmem_st32(tO + lane_base + cc * 32, o);
          }
          tmem_wait_st();
          tc_fence_before();
        }
        const float corr = exp2f(m_loc - m_used);                  // <= 2^8; 0 for a thread without keys
        l = l * factor + (sum2.x + sum2.y) * corr;
        uint32_t pk[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 v = fmul2(make_float2(pe[2 * j], pe[2 * j + 1]), make_float2(corr, corr));
          pk[j] = pack2<kBF16>(v.x, v.y);
        }
        // P goes to shared memory as the K-major A operand of the P V MMAs: row m, keys 32 kh + 16 ch .. + 15 = two 16-byte
        // units.  The buffer was last read by the P V MMAs of tile g-2.
        if (tid == 0) tr(11, g);
        if (g >= 2 && ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(kBarPFree + sb), ((g >> 1) + 1) & 1, p.status));
        if (tid == 0) tr(12, g);
        const uint32_t prow = sBase + kOffP + sb * kPBytes;
        st_shared_v4(prow + sw128_offset(m, 4 * kh + 2 * ch), pk[0], pk[1], pk[2], pk[3]);
        st_shared_v4(prow + sw128_offset(m, 4 * kh + 2 * ch + 1), pk[4], pk[5], pk[6], pk[7]);
        // (No proxy fence here: the P V issuers -- and in the odd CTA the thread that forwards this barrier -- execute it after
        // they have seen the barrier, as the Q K^T issuers do for the gathered rows.  A fence issued from these warps waits
        // behind the tensor-core work queued on this SM: 800 clocks per tile in the even CTA, measured.)
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(kBarPReady + sb));
        if (tid == 0) tr(4, g);
      }
      if (tid == 0) tr(18, k);
      // ---- epilogue: each thread normalises and stores 128 of its head's 512 output dims ----
      if (nvt > 0) {  // row sum = sum over the four threads of the head
        rowsum[part * 64 + m] = l;
        named_bar_sync(named, 128);
        l = (rowsum[m] + rowsum[64 + m]) + (rowsum[128 + m] + rowsum[192 + m]);  // (rewritten only after the next item's barriers)
      }
      const int h = h0 + static_cast<int>(rank) * kHeads + m;
      const int dim0 = 256 * kh + 128 * ch;
      T* orow = reinterpret_cast<T*>(p.out) + (static_cast<int64_t>(bt) * p.H + h) * kDV + dim0;
      // split-KV: this unit's normalised partial result and its log-sum-exp go to the workspace instead
      const int64_t prow_index = (static_cast<int64_t>(share) * split_rows + bt) * p.H + h;
      float* part_row = shares > 1 ? p.part_out + prow_index * kDV + dim0 : nullptr;
      const bool lse_writer = kh == 0 && ch == 0;
      // scratch of this warp for the output transposition: inside the P rows of its own block of 32 heads (both P buffers), so
      // that only warps of the same block -- which meet at a named barrier when they are done -- can write P over it
      const uint32_t out_scratch = sBase + kOffP + (part < 2 ? 0u : kPBytes) + (q4 & 1) * 4096u + (part & 1) * 2048u;
      if (shares > 1 && nvt == 0) {
        if (h < p.H) {  // nothing to add from this share (also for queries that do not exist: the combine step writes zeros)
          for (int j = 0; j < 32; ++j) reinterpret_cast<float4*>(part_row)[j] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (lse_writer) p.part_lse[prow_index] = -INFINITY;
        }
      } else if (nvt == 0) {  // no key takes part, or the query does not exist (beyond q_len_b): out = 0, lse = -inf
        if (h < p.H) {
          for (int j = 0; j < 16; ++j) reinterpret_cast<uint4*>(orow)[j] = make_uint4(0, 0, 0, 0);
          if (lse_writer && p.lse) p.lse[static_cast<int64_t>(bt) * p.H + h] = -INFINITY;
        }
      } else {
        // the last P V of the item is complete (same barrier and argument as for the rescale above)
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(kBarPFree + ((g - 1) & 1)), ((g - 1) >> 1) & 1, p.status));
        tc_fence_after();
        const float inv_l = 1.f / l;
        uint32_t v[32];
#pragma unroll 1
        for (int cc = 0; cc < 4; ++cc) {
          tmem_ld32(tO + lane_base + (4 * ch + cc) * 32, v);
          tmem_wait_ld();
          if (shares > 1) {
            // fp32 partial rows: the same detour through the warp's scratch as below, 16 columns (64 bytes per row) at a time
#pragma unroll
            for (int hq = 0; hq < 2; ++hq) {
#pragma unroll
              for (int gq = 0; gq < 4; ++gq)
                st_shared_v4(out_scratch + lane * 64 + ((gq ^ ((lane >> 1) & 3)) << 4), __float_as_uint(__uint_as_float(v[16 * hq + 4 * gq]) * inv_l),
                             __float_as_uint(__uint_as_float(v[16 * hq + 4 * gq + 1]) * inv_l), __float_as_uint(__uint_as_float(v[16 * hq + 4 * gq + 2]) * inv_l),
                             __float_as_uint(__uint_as_float(v[16 * hq + 4 * gq + 3]) * inv_l));
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int r = 8 * i + (lane >> 2), u = lane & 3;
                const uint4 x = ld_shared_v4(out_scratch + r * 64 + ((u ^ ((r >> 1) & 3)) << 4));
                if (ok && h - lane + r < p.H) *reinterpret_cast<uint4*>(part_row + static_cast<int64_t>(r - lane) * kDV + cc * 32 + hq * 16 + u * 4) = x;
              }
              __syncwarp();
            }
          } else {
            // A row per lane would make every store instruction touch 32 lines.  The warp's 32 rows x 64 bytes go through its
            // scratch (a quarter of the P buffers, which are idle: the item's last P V is complete) and leave as 64 contiguous
            // bytes of each of 8 rows per instruction.
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
              const uint32_t w0 = pack2<kBF16>(__uint_as_float(v[8 * gq + 0]) * inv_l, __uint_as_float(v[8 * gq + 1]) * inv_l);
              const uint32_t w1 = pack2<kBF16>(__uint_as_float(v[8 * gq + 2]) * inv_l, __uint_as_float(v[8 * gq + 3]) * inv_l);
              const uint32_t w2 = pack2<kBF16>(__uint_as_float(v[8 * gq + 4]) * inv_l, __uint_as_float(v[8 * gq + 5]) * inv_l);
              const uint32_t w3 = pack2<kBF16>(__uint_as_float(v[8 * gq + 6]) * inv_l, __uint_as_float(v[8 * gq + 7]) * inv_l);
              st_shared_v4(out_scratch + lane * 64 + ((gq ^ ((lane >> 1) & 3)) << 4), w0, w1, w2, w3);
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int r = 8 * i + (lane >> 2), u = lane & 3;
              const uint4 x = ld_shared_v4(out_scratch + r * 64 + ((u ^ ((r >> 1) & 3)) << 4));
              const int hr = h - lane + r;   // head of row r of this warp (the warp's rows are consecutive heads)
              if (ok && hr < p.H) *reinterpret_cast<uint4*>(orow + static_cast<int64_t>(r - lane) * kDV + cc * 32 + u * 8) = x;
            }
            __syncwarp();
          }
        }
        if (ok && lse_writer && h < p.H) {
          const float lse_v = m_used * 0.6931471805599453f + logf(l);
          if (shares > 1) p.part_lse[prow_index] = lse_v;
          else if (p.lse) p.lse[static_cast<int64_t>(bt) * p.H + h] = lse_v;
        }
      }
      if (tid == 0) tr(19, k);
      if (nvt > 0) named_bar_sync(named, 128);  // the block's warps are done with their scratch: P may be written again
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (nvt > 0) arrive_at(bar_addr(kBarOFree), 0, rank);  // the output tile may be overwritten by the next item's first P V
        mbar_arrive(bar(kBarInfoEmpty + qp));                  // the item's tile list is no longer needed here
      }
    }
  } else if (warp < kFirstExchangeWarp) {
    // ================================ tile lists + gather producers =================================
    // These warps never leave their loops early: they meet at a named barrier twice per item.  Both CTAs build the same
    // list (it decides how many tiles every role of the pair walks); each gathers its own 32 keys of a tile.
    const int pw = warp - kFirstGatherWarp;  // keys [8 pw, 8 pw + 8) of the CTA's 32
    const uint8_t* kv_bytes = reinterpret_cast<const uint8_t*>(p.kv);
    // key rows in one piece (kRowBytes each) or in two parts (latent rows of 1024 bytes in kv, rope rows of 128 bytes in kv_rope):
    // the first eight chunks come from kv at the row stride, the rope chunk from its own base and stride
    const size_t row_stride = (kRope && p.kv_rope) ? static_cast<size_t>(kDV * 2) : static_cast<size_t>(kRowBytes);
    const uint8_t* last_base = (kRope && p.kv_rope) ? reinterpret_cast<const uint8_t*>(p.kv_rope) : kv_bytes + 8 * 128;
    const size_t last_stride = (kRope && p.kv_rope) ? static_cast<size_t>((kD - kDV) * 2) : static_cast<size_t>(kRowBytes);
    int g = 0, qslots = 0;  // tiles so far; ring slots so far that carried Q rows instead of a tile (two per non-empty item)
    for (int k = 0; run_all; ++k) {
      const int unit = item_of(k);
      if (unit < 0) break;
      int share, shares;
      const int item = item_and_share(unit, &share, &shares);
      const int qp = k & 1;
      const int bt = item / head_blocks;
      const RowCtx ctx = make_row_ctx(p, bt);
      if (k >= 2 && ok) ok = __all_sync(0xffffffffu, mbar_wait<true>(bar(kBarInfoEmpty + qp), ((k >> 1) + 1) & 1, p.status));
      // validity masks of all tiles of the item, then the list of tiles with at least one key taking part.  The indices
      // of eight tiles are loaded before the first of them is used, so that their latencies overlap.
      for (int t0 = pw; t0 < ntiles; t0 += 32) {
        int i0[8], i1[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int tile = t0 + 4 * u;
          const int s0 = tile * kBK + lane, s1 = s0 + 32;
          i0[u] = (tile < ntiles && s0 < p.topk) ? __ldg(ctx.idx_row + s0) : -1;
          i1[u] = (tile < ntiles && s1 < p.topk) ? __ldg(ctx.idx_row + s1) : -1;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int tile = t0 + 4 * u;
          const uint32_t lo = __ballot_sync(0xffffffffu, ctx.active && index_valid(ctx, i0[u]));
          const uint32_t hi = __ballot_sync(0xffffffffu, ctx.active && index_valid(ctx, i1[u]));
          if (lane == 0 && tile < ntiles) masks[qp * kMaxTiles + tile] = (static_cast<unsigned long long>(hi) << 32) | lo;
        }
      }
      named_bar_sync(kGatherBarrier, 128);
      if (pw == 0) {
        int n = 0;
        for (int base = 0; base < ntiles; base += 32) {
          const int tile = base + lane;
          const bool nonempty = tile < ntiles && masks[qp * kMaxTiles + tile] != 0ull;
          const uint32_t bal = __ballot_sync(0xffffffffu, nonempty);
          if (nonempty) tile_list[qp * kMaxTiles + n + __popc(bal & ((1u << lane) - 1u))] = static_cast<uint16_t>(tile);
          n += __popc(bal);
        }
        if (shares > 1) {
          // this unit's share of the list: entries [lo, hi) move to the front (in chunks of 32, reading before writing)
          const int lo = static_cast<int>(static_cast<long long>(n) * share / shares);
          const int hi = static_cast<int>(static_cast<long long>(n) * (share + 1) / shares);
          __syncwarp();
          for (int base = 0; base < hi - lo; base += 32) {
            const int i = base + lane;
            const uint16_t v = i < hi - lo ? tile_list[qp * kMaxTiles + lo + i] : 0;
            __syncwarp();
            if (i < hi - lo) tile_list[qp * kMaxTiles + i] = v;
            __syncwarp();
          }
          n = hi - lo;
        }
        if (lane == 0) { info[qp * 2] = n; info[qp * 2 + 1] = ctx.active ? 1 : 0; }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(kBarInfoFull + qp));
        if (lane == 0) tr(20, k);
      }
      named_bar_sync(kGatherBarrier, 128);
      const int nvt = info[qp * 2];
      if (nvt > 0) {
        // The item's Q rows travel through the stage ring as two slots AHEAD of the item's
        // tiles -- requested as soon as stages come free, i.e. while the previous item is still being worked on -- so that at
        // the item boundary the exchange warps only move them from shared memory to tensor memory.  Slot j: dims 192 j ..
        // 192 j + 191 as three chunks of [64 rows x 128 bytes] (128-byte swizzle); one instruction copies 128 bytes of four rows.
        int nrows;
        const uint8_t* q0 = q_rows_of(unit, &nrows);
        const int gt = tid - kFirstGatherWarp * 32;
#pragma unroll 1
        for (int j = 0; j < 2; ++j) {
          const int u = g + qslots + j, s = u % kStages;
          if (u >= kStages && ok) ok = mbar_wait<true>(bar(kBarKvEmpty + s), ((u / kStages) + 1) & 1, p.status);
          if (ok) {
            const uint32_t stage = sBase + s * kStageBytes;
#pragma unroll
            for (int cj = 0; cj < 3; ++cj)
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int row = (gt >> 3) + 16 * i, unit16 = gt & 7;
                const bool v = row < nrows;
                cp_async16(stage + cj * kQChunk + sw128_offset(row, unit16),
                           v ? q0 + row * kRowBytes + (3 * j + cj) * 128 + unit16 * 16 : reinterpret_cast<const uint8_t*>(p.q), v ? 16u : 0u);
              }
            // ... and behind them half of the dims that stay in shared memory (384..), as pieces of [64 rows x 32 dims]: 64
            // bytes per row, the four 16-byte units of a row permuted by (row / 2) % 4, so that both these copies (64 bytes of
            // eight rows per instruction) and the row-per-lane reads of the exchange warps are free of bank conflicts
#pragma unroll
            for (int pc = 0; pc < kQPiecesPerSlot; ++pc)
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                const int row = (gt >> 2) + 32 * i, u16 = gt & 3;
                const bool v = row < nrows;
                cp_async16(stage + kQPieceOff + pc * kQPiece + row * 64 + ((u16 ^ ((row >> 1) & 3)) << 4),
                           v ? q0 + row * kRowBytes + 768 + (kQPiecesPerSlot * j + pc) * 64 + u16 * 16 : reinterpret_cast<const uint8_t*>(p.q),
                           v ? 16u : 0u);
              }
            cp_async_arrive_noinc(bar(kBarKvFull + s));
          }
        }
        qslots += 2;
      }
      for (int it = 0; it < nvt; ++it, ++g) {
        const int tile = tile_list[qp * kMaxTiles + it], s = (g + qslots) % kStages;
        // the row numbers are fetched before the wait for the stage, so their latency is hidden behind it: lane l looks up
        // key 8 pw + (l & 7) of this CTA's 32 keys
        const int slot = tile * kBK + static_cast<int>(rank) * kKeys + pw * 8 + (lane & 7);
        const int my_idx = slot < p.topk ? __ldg(ctx.idx_row + slot) : -1;
        // row number inside kv, -1 for a key that does not take part: it is fetched with a source size of zero, which fills
        // the destination with zeros
        const int my_row = index_valid(ctx, my_idx) ? static_cast<int>(kv_row(p, ctx.b, my_idx)) : -1;
        if (g + qslots >= kStages && ok) ok = mbar_wait<true>(bar(kBarKvEmpty + s), (((g + qslots) / kStages) + 1) & 1, p.status);
        if (!ok) continue;
        const uint32_t stage = sBase + s * kStageBytes;
        // one instruction copies one 64-dim chunk (128 bytes, 8 lanes) of four keys
#pragma unroll
        for (int gh = 0; gh < 2; ++gh) {
          const int kl = 4 * gh + (lane >> 3);  // key of the warp's eight
          const int row = __shfl_sync(0xffffffffu, my_row, kl);
          const uint32_t dst = stage + sw128_offset(pw * 8 + kl, lane & 7);
          const uint32_t nbytes = row < 0 ? 0u : 16u;
          {
            const size_t r0 = static_cast<size_t>(row < 0 ? 0 : row);
            const uint8_t* src = kv_bytes + r0 * row_stride + (lane & 7) * 16;
#pragma unroll
            for (int c = 0; c < 8; ++c) cp_async16(dst + c * kChunk, src + c * 128, nbytes);
            if (kRope) cp_async16(dst + 8 * kChunk, last_base + r0 * last_stride + (lane & 7) * 16, nbytes);
          }
        }
        cp_async_arrive_noinc(bar(kBarKvFull + s));
        if (pw == 0 && lane == 0) tr(0, g);
      }
    }
    cp_async_wait<0>();
  } else if (warp < kQkWarp) {
    // ================================ Q loader + swap of the value halves ===========================
    // Q of an item arrives in two slots of the stage ring; these warps move it on: row m of the CTA's 64 heads, dims 0..383 to
    // tensor memory (lane L holds row L % 64: the A operand of a 64-row half must be present in both lane halves), dims 384..
    // to the Q buffer in shared memory.  Then, per tile, the swap (see top).
    const int xw = warp - kFirstExchangeWarp;  // = lane quarter of the tensor-memory stores
    const int L = xw * 32 + lane, m = L & 63;
    const int xt = tid - kFirstExchangeWarp * 32;  // 0..127
    const uint32_t lane_base = static_cast<uint32_t>(xw * 32) << 16;
    const uint32_t src_off = 4u * peer * kChunk;   // own chunks [4 (1 - r), +4): the dims the PEER's half of P V covers ...
    const uint32_t dst_off = 4u * rank * kChunk;   // ... go where the peer keeps those dims of ITS keys that I need: its chunks [4 r, +4)
    const uint32_t peer_base = map_to_cta(sBase, peer);
    const uint32_t peer_bars = map_to_cta(sBars, peer);
    int g = 0, ne = 0, qslots = 0, qslot_reads = 0;
    for (int k = 0; run_all && ok; ++k) {
      const int unit = item_of(k);
      if (unit < 0) break;
      const int qp = k & 1;
      if (!__all_sync(0xffffffffu, mbar_wait<true>(bar(kBarInfoFull + qp), (k >> 1) & 1, p.status))) { ok = false; break; }
      const int nvt = info[qp * 2];
      if (nvt > 0) {
        // all Q K^T MMAs of the previous non-empty item are complete: the tensor-memory part of Q can be replaced
        if (ne > 0 && !__all_sync(0xffffffffu, mbar_wait<true>(bar(kBarQFree), (ne - 1) & 1, p.status))) { ok = false; break; }
        ++ne;
        if (xt == 0) tr(16, k);
        tc_fence_after();
        // Tensor-memory part: the gather warps sent the rows through two slots of the stage ring (see there).  Lane L moves
        // row L % 64: per 64-dim chunk eight 16-byte loads from the swizzled chunk (conflict-free) and one 32-column store.
#pragma unroll 1
        for (int j = 0; j < 2; ++j) {
          const int u = g + qslots + j, s = u % kStages;
          if (!__all_sync(0xffffffffu, mbar_wait(bar(kBarKvFull + s), (u / kStages) & 1, p.status))) { ok = false; break; }
          const uint32_t stage = sBase + s * kStageBytes;
#pragma unroll 1
          for (int cj = 0; cj < 3; ++cj) {
            uint32_t w[32];
#pragma unroll
            for (int uu = 0; uu < 8; ++uu) {
              const uint4 x = ld_shared_v4(stage + cj * kQChunk + sw128_offset(m, uu));
              w[4 * uu] = x.x; w[4 * uu + 1] = x.y; w[4 * uu + 2] = x.z; w[4 * uu + 3] = x.w;
            }
            tmem_st32(tQ + lane_base + (3 * j + cj) * 32, w);
          }
          // the pieces behind them go to the Q buffer in the layout of the MMA's A operand; the two threads of a row copy two
          // 16-byte units of every piece each
#pragma unroll
          for (int pc = 0; pc < kQPiecesPerSlot; ++pc) {
            const int piece = kQPiecesPerSlot * j + pc;   // 32-dim piece of dims 384..
#pragma unroll
            for (int uu = 2 * (xw >> 1); uu < 2 * (xw >> 1) + 2; ++uu) {
              const uint4 x = ld_shared_v4(stage + kQPieceOff + pc * kQPiece + m * 64 + ((uu ^ ((m >> 1) & 3)) << 4));
              st_shared_v4(sQ + (piece >> 1) * kQChunk + sw128_offset(m, 4 * (piece & 1) + uu), x.x, x.y, x.z, x.w);
            }
          }
          // The slot carried no tile: every barrier of the stage that a tile would have completed once is completed once here,
          // so that the phases of all of them keep in step with the slot number.
          __syncwarp();
          if (lane == 0) { mbar_arrive(bar(kBarPeerRead + s)); mbar_arrive(bar(kBarQRead)); }
          if (xt == 0) {
            // all four warps have read the stage (a bounded wait, not a named barrier: a warp that gave up never comes)
            if (!mbar_wait(bar(kBarQRead), qslot_reads & 1, p.status)) ok = false;
            mbar_arrive(bar(kBarVFull + s));
            if (rank == 0) { mbar_arrive(bar(kBarPeerKvFull + s)); mbar_arrive(bar(kBarPeerVFull + s)); }
            mbar_arrive(bar(kBarKvEmpty + s));   // the stage may be refilled (both arrivals that the two P V issuers
            mbar_arrive(bar(kBarKvEmpty + s));   // would have supplied for a tile)
          }
          ++qslot_reads;
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        qslots += 2;
        if (xt == 0) tr(22, k);
        fence_proxy_async_smem();  // the Q buffer is read by the tensor cores
        tmem_wait_st();
        if (xt == 0) tr(23, k);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_at(bar_addr(kBarQReady), 0, rank);
        if (xt == 0) tr(17, k);
      }
      for (int it = 0; it < nvt; ++it, ++g) {
        const int sb = g & 1, s = (g + qslots) % kStages;
        const uint32_t ph = ((g + qslots) / kStages) & 1;
        // the Q K^T of the tile is complete on both SMs: neither CTA reads the regions any more
        if (!__all_sync(0xffffffffu, mbar_wait<true>(bar(kBarSFull + sb), (g >> 1) & 1, p.status))) { ok = false; break; }
        // these warps do not read the scores, but the buffer's "full" barrier must not complete another phase (tile g + 2)
        // before every waiter has seen this one: they are counted among the readers that free the buffer
        if (lane == 0) mbar_arrive(bar(kBarSFree + sb));
        if (xt == 0) tr(5, g);
        const uint32_t region = sBase + s * kStageBytes + src_off;
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = ld_shared_v4(region + (xt + 128 * j) * 16);
        {
          // the "I have read my region" signal must not overtake the loads: a warp issues in order and a store cannot issue
          // before its source registers are filled, so a (dummy) store of a word derived from all loads holds it back
          uint32_t dep = 0;
#pragma unroll
          for (int j = 0; j < 8; ++j) dep ^= v[j].x;
          st_shared_u32_volatile(sBase + kOffInfo + 64 + (warp - kFirstExchangeWarp) * 4, dep);
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster_relaxed(peer_bars + (kBarPeerRead + s) * 8);
        }
        // this CTA's receive barrier: armed once per tile (its previous use, three tiles ago, completed before that tile's P V)
        if (xt == 0) mbar_arrive_expect_tx(bar(kBarVFull + s), kSwapBytes);
        // the peer holds its region in registers: it may be overwritten
        if (!__all_sync(0xffffffffu, mbar_wait_cluster(bar(kBarPeerRead + s), ph, p.status))) { ok = false; break; }
        if (xt == 0) tr(6, g);
        const uint32_t dst = peer_base + s * kStageBytes + dst_off, dst_bar = peer_bars + (kBarVFull + s) * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) st_async_v4_b32(dst + (xt + 128 * j) * 16, dst_bar, v[j]);
        if (xt == 0) tr(7, g);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarInfoEmpty + qp));
    }
  } else if (warp == kQkWarp || warp == kQkWarpB) {
    const int par = warp == kQkWarp ? 0 : 1;
    if (rank == 0) {
      // ================================ Q K^T issuers (even CTA) ====================================
      // S[128 heads x 64 keys] over 36 (32 without rope dims) steps of 16 dims: A = Q (tensor memory for dims < 384, shared
      // memory beyond), B = the 32 gathered rows of each CTA.  The WHOLE warp walks the loops and waits, converged, and one
      // elected lane issues through predicated instructions (see umma_pair_ss_if for why).  Two such warps, one for the even
      // tiles (score buffer 0) and one for the odd tiles (buffer 1), so that the next tile's MMAs are queued while this
      // tile's hand-overs are in flight.
      constexpr uint32_t idesc_qk = make_idesc_f16(kBF16, kM, kBK, 0, 0);
      const uint32_t go = elect_one_lane();
      auto wait_all = [&](int slot, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait(bar(slot), parity, p.status)); };
      auto wait_all_cluster = [&](int slot, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait_cluster(bar(slot), parity, p.status)); };
      int g = 0, ne = 0;
      for (int k = 0; run_all && ok; ++k) {
        const int item = item_of(k);
        if (item < 0) break;
        const int qp = k & 1;
        if (!wait_all(kBarInfoFull + qp, (k >> 1) & 1)) { ok = false; break; }
        const int nvt = info[qp * 2];
        const int first = (g & 1) == par ? 0 : 1;            // this warp's first tile of the item
        const int last = nvt - 1 - (((g + nvt - 1) & 1) == par ? 0 : 1);   // ... and its last one
        if (nvt > 0) {  // items without a key neither load Q nor touch O: their barriers are skipped on both sides
          // (waited for also when no tile of the item is mine: a warp that skipped a phase of this barrier would find its
          // next parity test satisfied by the phase before and run an item ahead of its Q)
          if (!wait_all_cluster(kBarQReady, ne & 1)) { ok = false; break; }
          ++ne;
          // No tile of this item is mine: I am done with its Q at once.  Said with a commit, not a plain arrive: a plain arrive
          // could overtake the commit that ended this warp's previous item and complete THAT item's phase while its MMAs
          // still read Q; a commit arrives only after everything this lane issued before.
          if (first >= nvt) umma_pair_commit_if(go, bar(kBarQFree), 3);
        }
        for (int it = first; it < nvt; it += 2) {
          const int gg = g + it, u = gg + 2 * ne;   // ring slot: two slots per non-empty item so far carried Q rows
          const int s = u % kStages, sb = par;
          const uint32_t stage = sBase + s * kStageBytes;
          if (!wait_all(kBarKvFull + s, (u / kStages) & 1)) { ok = false; break; }
          if (!wait_all_cluster(kBarPeerKvFull + s, (u / kStages) & 1)) { ok = false; break; }
          // the softmax warps of both CTAs must have read the scores of tile gg-2 out of this buffer
          if (gg >= 2 && !wait_all(kBarSFree + sb, ((gg >> 1) + 1) & 1)) { ok = false; break; }
          if (gg >= 2 && !wait_all_cluster(kBarPeerSFree + sb, ((gg >> 1) + 1) & 1)) { ok = false; break; }
          fence_proxy_async_smem();  // the gathered rows were written by cp.async of other threads
          tc_fence_after();
          if (go) tr(1, gg);
          const uint64_t db0 = make_smem_desc(stage, 16, 1024, kSwizzle128B);
          // (loops over the 64-dim chunks left rolled: the issue rate does not need the unrolling and the smaller loop
          // body measurably helps the other roles that share the SM's instruction caches)
#pragma unroll 1
          for (int c = 0; c < 6; ++c) {
#pragma unroll
            for (int kq = 0; kq < 4; ++kq)
              umma_pair_ts_if(go, tS + sb * 32, tQ + (c * 4 + kq) * 8, db0 + ((c * kChunk + kq * 32) >> 4), idesc_qk, (c | kq) != 0);
          }
          const uint64_t da0 = make_smem_desc(sQ, 16, 1024, kSwizzle128B);
#pragma unroll 1
          for (int c = 0; c < kQSmemChunks; ++c) {
#pragma unroll
            for (int kq = 0; kq < 4; ++kq)
              umma_pair_ss_if(go, tS + sb * 32, da0 + ((c * kQChunk + kq * 32) >> 4), db0 + (((6 + c) * kChunk + kq * 32) >> 4), idesc_qk, 1);
          }
          umma_pair_commit_if(go, bar(kBarSFull + sb), 3);
          if (go) tr(2, gg);
          if (it == last) umma_pair_commit_if(go, bar(kBarQFree), 3);  // this warp's share of "the item's Q may be replaced"
        }
        if (!ok) break;
        g += nvt;
        if (go) mbar_arrive(bar(kBarInfoEmpty + qp));
        __syncwarp();
      }
    } else if (lane == 0) {
      // ---- odd CTA: tell the even CTA when this CTA's rows of a tile have landed (warp 16) / when this CTA's softmax and
      // exchange warps are past a score buffer (warp 17) ----
      const uint32_t target = map_to_cta(sBars, 0);
      int g = 0, ne = 0;
      for (int k = 0; run_all && ok; ++k) {
        const int item = item_of(k);
        if (item < 0) break;
        const int qp = k & 1;
        if (!mbar_wait<true>(bar(kBarInfoFull + qp), (k >> 1) & 1, p.status)) { ok = false; break; }
        const int nvt = info[qp * 2];
        if (nvt > 0) ++ne;
        for (int it = 0; ok && it < nvt; ++it, ++g) {
          if (par == 0) {
            const int u = g + 2 * ne, s = u % kStages;
            if (!mbar_wait(bar(kBarKvFull + s), (u / kStages) & 1, p.status)) { ok = false; break; }
            fence_proxy_async_smem();  // written by cp.async, read by the tensor cores
            mbar_arrive_cluster_relaxed(target + (kBarPeerKvFull + s) * 8);
            tr(1, g);
          } else {
            const int sb = g & 1;
            if (!mbar_wait(bar(kBarSFree + sb), (g >> 1) & 1, p.status)) { ok = false; break; }
            mbar_arrive_cluster_relaxed(target + (kBarPeerSFree + sb) * 8);
          }
        }
        if (!ok) break;
        mbar_arrive(bar(kBarInfoEmpty + qp));
      }
    }
  } else if (warp == kPvWarp || warp == kRelayWarp) {
    if (rank == 0) {
      const int j = warp == kPvWarp ? 0 : 1;   // which of the two N = 256 MMAs per 16 keys this warp issues
      // ================================ P V issuers (even CTA) ======================================
      // O[128 heads x 512 dims] += P[128 x 64] . V[64 x 512] as two MMAs of N = 256 per 16 keys: P K-major in shared memory,
      // V MN-major: keys of half kh, dims of the CTA's half j at stage + (4 kh + 2 j) chunks (own rows or swapped-in rows).
      // Converged warps with one issuing lane, like the Q K^T issuers.
      constexpr uint32_t idesc_pv = make_idesc_f16(kBF16, kM, 256, 0, 1);
      const uint32_t go = elect_one_lane();
      auto wait_all = [&](int slot, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait(bar(slot), parity, p.status)); };
      auto wait_all_cluster = [&](int slot, uint32_t parity) { return __all_sync(0xffffffffu, mbar_wait_cluster(bar(slot), parity, p.status)); };
      int g = 0, ne = 0;
      for (int k = 0; run_all && ok; ++k) {
        const int item = item_of(k);
        if (item < 0) break;
        const int qp = k & 1;
        if (!wait_all(kBarInfoFull + qp, (k >> 1) & 1)) { ok = false; break; }
        const int nvt = info[qp * 2];
        for (int it = 0; it < nvt; ++it, ++g) {
          const int u = g + 2 * (ne + 1);   // ring slot (ne counts the non-empty items BEFORE this one)
          const int s = u % kStages, pb = g & 1;
          if (!wait_all(kBarPReady + pb, (g >> 1) & 1)) { ok = false; break; }
          if (!wait_all_cluster(kBarPeerPReady + pb, (g >> 1) & 1)) { ok = false; break; }
          if (go) tr(13, g);
          if (!wait_all_cluster(kBarVFull + s, (u / kStages) & 1)) { ok = false; break; }
          if (go) tr(8, g);
          if (!wait_all_cluster(kBarPeerVFull + s, (u / kStages) & 1)) { ok = false; break; }
          if (go) tr(9, g);
          // the first P V of an item overwrites O: the previous non-empty item's output must have been read out
          if (it == 0 && ne > 0 && !wait_all_cluster(kBarOFree, (ne - 1) & 1)) { ok = false; break; }
          fence_proxy_async_smem();
          tc_fence_after();
          const uint32_t stage = sBase + s * kStageBytes;
          const uint64_t dp0 = make_smem_desc(sBase + kOffP + pb * kPBytes, 16, 1024, kSwizzle128B);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint64_t dv = make_smem_desc(stage + (4 * (ks >> 1) + 2 * j) * kChunk + (ks & 1) * 2048, kChunk, 1024, kSwizzle128B);
            umma_pair_ss_if(go, tO + 128 * j, dp0 + ((ks * 32) >> 4), dv, idesc_pv, (it | ks) != 0);
          }
          umma_pair_commit_if(go, bar(kBarKvEmpty + s), 3);
          umma_pair_commit_if(go, bar(kBarPFree + pb), 3);
          if (go) tr(10, g);
        }
        if (!ok) break;
        if (nvt > 0) ++ne;
        if (go) mbar_arrive(bar(kBarInfoEmpty + qp));
        __syncwarp();
      }
    } else if (lane == 0) {
      // ---- odd CTA: tell the even CTA when the even CTA's half of the swap has landed here (warp 18) / when this CTA's
      // softmax warps have written P (warp 19) ----
      const bool fwd_v = warp == kPvWarp;
      const uint32_t target = map_to_cta(sBars, 0);
      int g = 0, ne = 0;
      for (int k = 0; run_all && ok; ++k) {
        const int item = item_of(k);
        if (item < 0) break;
        const int qp = k & 1;
        if (!mbar_wait<true>(bar(kBarInfoFull + qp), (k >> 1) & 1, p.status)) { ok = false; break; }
        const int nvt = info[qp * 2];
        if (nvt > 0) ++ne;
        for (int it = 0; ok && it < nvt; ++it, ++g) {
          if (fwd_v) {
            const int u = g + 2 * ne, s = u % kStages;
            if (!mbar_wait_cluster(bar(kBarVFull + s), (u / kStages) & 1, p.status)) { ok = false; break; }
            fence_proxy_async_smem();  // written by st.async (generic proxy), read by the tensor cores
            mbar_arrive_cluster_relaxed(target + (kBarPeerVFull + s) * 8);
            tr(8, g);
          } else {
            const int pb = g & 1;
            if (!mbar_wait(bar(kBarPReady + pb), (g >> 1) & 1, p.status)) { ok = false; break; }
            tr(14, g);
            fence_proxy_async_smem();  // the P stores of this CTA's softmax warps (generic proxy) are read by the tensor cores
            mbar_arrive_cluster_relaxed(target + (kBarPeerPReady + pb) * 8);
            tr(15, g);
          }
        }
        if (!ok) break;
        mbar_arrive(bar(kBarInfoEmpty + qp));
      }
    }
  }

  // ---- teardown: every thread of both CTAs comes here, also after a failed wait -----------------------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // no CTA frees tensor memory or leaves while its peer may still use it or write into its shared memory
  if (warp == kQkWarp) tmem_dealloc_pair(tmem_base, kTmemCols);
}

// -------------------------------------------------------------------------------------------------
// host side
// -------------------------------------------------------------------------------------------------
bool sparse_mla_fwd_pair_supported(const FwdParams& p) {
  // (row numbers inside kv are kept in 32 bits by the gather warps)
  return (p.D == pr::kD || p.D == pr::kDV) && p.DV == pr::kDV && p.topk <= pr::kMaxTiles * pr::kBK &&
         static_cast<long long>(p.B) * p.S_kv <= 0x7fffffffLL;
}

int launch_sparse_mla_fwd_pair(const FwdParams& p, bool bf16, cudaStream_t stream) {
  int dev = 0, sms = 0;
  cudaError_t e = current_device_sms(&dev, &sms);
  if (e != cudaSuccess) return static_cast<int>(e);
  const bool rope = p.D == pr::kD;
  auto kern = rope ? (bf16 ? sparse_mla_fwd_pair_kernel<true, true> : sparse_mla_fwd_pair_kernel<false, true>)
                   : (bf16 ? sparse_mla_fwd_pair_kernel<true, false> : sparse_mla_fwd_pair_kernel<false, false>);
  if ((e = ensure_dynamic_smem(kern, dev, static_cast<int>(pr::kSmemBytes))) != cudaSuccess) return static_cast<int>(e);
  // persistent: one 2-CTA cluster per SM pair, each walking its share of the (query, head block) items
  long long clusters = sms / 2 > 0 ? sms / 2 : 1;
  const long long hb = (p.H + pr::kM - 1) / pr::kM, rows = static_cast<long long>(p.B) * p.S;
  const long long split_rows = p.nsplit > 1 ? ((p.split_queries > 0 && p.split_queries < rows) ? p.split_queries : rows) : 0;
  const long long units = split_rows * hb * (p.nsplit > 1 ? p.nsplit : 1) + (rows - split_rows) * hb;
  if (clusters > units) clusters = units;
  kern<<<dim3(static_cast<unsigned>(2 * clusters)), pr::kThreads, pr::kSmemBytes, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace dsa
