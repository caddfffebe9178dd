// bf16 GEMM for sm_100a on tcgen05 tensor cores, optionally fused with a split-K reduction and a
// cross-GPU all-reduce over peer memory.
//
//   acc[m, n] = sum_k A[m, k] * B[n, k]            (both operands K-major, i.e. "x @ W^T")
//
// A rows fill the 128 TMEM lanes of a tile (UMMA M = 128), B rows fill BN accumulator columns.
// The host decides which logical operand plays A: for a large token count the activations are A
// ("normal"), for decode-sized token counts the weight matrix is A and the few tokens are B
// ("swapped"), so the tensor core still sees full 128-row tiles and weights stream through TMA once.
// In both cases results are stored as out[token, feature].
//
// Structure of one CTA (192 threads), persistent over work items (tile, k range; see WorkIter):
//   warp 0   : TMA producer  - cp.async.bulk.tensor loads of A/B k-blocks into a smem ring (no multicast)
//   warp 1   : MMA issuer    - one elected lane issues tcgen05.mma (K = 16 per instruction) into TMEM;
//                              tcgen05.commit releases smem stages and publishes finished accumulators
//   warps 2-5: epilogue      - tcgen05.ld the accumulator (two TMEM buffers, so the next tile's MMAs
//                              overlap this tile's epilogue), then
//                                (whole tile, one rank)   bias / activation / residual, bf16 store;
//                                (split-K / stream-K)     park the fp32 partial in a local slot; the LAST contributor of
//                                                         the tile to arrive sums the partials in slot order and carries
//                                                         on (nobody waits for another CTA);
//                                (several ranks)          push the tile's partial to every rank with plain peer stores
//                                                         and sum the ranks' partials in rank order (bit-identical
//                                                         everywhere).  Two exchange protocols:
//                                   flagged words     - few-token tiles, up to 4 ranks: every value travels inside a
//                                                       16-byte {value, epoch, value, epoch} word and the thread that owns
//                                                       the feature row polls the words in its own memory right away;
//                                                       no fence, no counter;
//                                   arrival counters  - one system-scope fence per tile, a relaxed add on every rank's
//                                                       per-tile counter, and a second phase (all warps, after the CTA
//                                                       has pushed all of its tiles) that waits (bounded) for the tiles
//                                                       it owns.  All of a CTA's pushes precede its first wait and the
//                                                       grid is never larger than what is co-resident, so ranks cannot
//                                                       deadlock each other.
//   Consecutive fused calls alternate between two workspace halves; a rank can run at most one call ahead of a peer
//   (its next call needs that peer's partial), so a half is never overwritten while a peer still reads it.
//
// Every wait is bounded; on expiry the CTA records a status code in params.status and drains.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "launch.cuh"
#include "ptx_sm100.cuh"
#include "tpb_api.h"

namespace tpb {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int MAX_STAGES = 12;
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;
constexpr int MAX_WORLD = 8;
constexpr int LL_FIRST_SLOT = 32;  // first fp32 slot of the flagged-word area (slots below hold plain partials)
constexpr int LL_TILE_WORDS = 128 * 16;  // 16-byte flagged words owned by one tile: 128 feature rows x up to 16 token quads

struct GemmParams {
  int m_extent;   // rows of A (lanes side)
  int n_extent;   // rows of B (columns side)
  int k_extent;
  int m_tiles, n_tiles, k_blocks, k_splits, kb_per_split;
  int stages;
  int swapped;        // 0: A rows are tokens, B rows are features; 1: A rows are features, B rows are tokens
  int ld_out;         // elements between consecutive tokens in out / residual
  int ld_slot;        // elements between consecutive tokens in the fp32 partial slots (= GEMM feature count)
  __nv_bfloat16* out;
  const __nv_bfloat16* bias;      // [features] or null
  float bias_scale;               // bias is multiplied by this before it is added (a row-parallel shard stores bias / world)
  const __nv_bfloat16* residual;  // [tokens, ld_out] or null
  int act;                        // 0 none, 1 relu, 2 gelu(erf), 3 gelu(tanh), 4 silu, 5 gated silu: the GEMM features come in
                                  // groups of [16 gate | 16 up] rows and out[t, 16 g + i] = silu(gate_i) * up_i (half as wide)
  // reduce mode (k_splits > 1 or world > 1)
  int reduce;
  int world, rank;
  float* slots[MAX_WORLD];        // per destination rank: slots [0, world) = one partial per source rank; on the local
                                  // rank slots [world, world + k_splits) additionally park this rank's split-K partials
  uint32_t* arrivals[MAX_WORLD];  // per destination rank: [tiles] arrival counters
  uint32_t* expected;             // local: [tiles] counter value reached after the previous call
  uint32_t* split_counters;       // local: [tiles] arrivals of split-K partials (self re-arming)
  size_t slot_stride;             // elements between consecutive slots
  uint32_t* status;               // local status word (0 = ok)
  // flagged-word exchange for the cross-rank sum of small (swapped) problems: every fp32 partial travels as one
  // 8-byte word {value, epoch}; the receiver spins on the word itself, so no fence and no arrival counter is needed
  int ll;
  uint32_t* ll_epochs;            // local: [tiles] epoch of the previous flagged call (device-resident: graph replays advance it)
  float* mc_slots;                // NVLink multicast alias of every rank's slot area (null: one peer store per rank instead)
  // fused all-gather of the token-side operand (ag_world > 1): every rank owns a column slice [rows, ag_cols] of x;
  // the kernel first pushes its slice into every rank's gathered buffer, then consumes k-blocks slice by slice
  // (own slice first) as the peers' pushes arrive
  int ag_world, ag_rank, ag_kb_per_rank, ag_rows, ag_cols;
  uint32_t ag_epoch;                          // flags of this call reach at least this value
  const __nv_bfloat16* ag_src;                // local slice
  long long ag_src_ld, ag_dst_ld;
  __nv_bfloat16* ag_dst[MAX_WORLD];           // every rank's gathered buffer [rows, ag_world * ag_cols]
  __nv_bfloat16* ag_mc_dst;                   // multicast view of the gathered buffers (null: one peer store per rank)
  uint32_t* ag_flags[MAX_WORLD];              // every rank's arrival words [ag_world], indexed by source rank
  uint32_t* ag_push_counter;                  // local: CTAs done pushing (self re-arming)
  int stream_k;                   // 1: every CTA owns one contiguous range of (tile, k-block) units (see WorkIter)
  uint64_t wait_ns;               // wall-time bound of every wait inside the kernel
  size_t out_elems;               // extent of `out` in elements (checked before every store in a -DTPB_BOUNDS build)
  // MN-major operands (normal orientation only): the operand is stored [K rows][MN columns] in memory, i.e. it is the
  // transpose of what the K-major path expects.  Lets the backward GEMMs (dX = dY W, dW = dY^T X) read W, dY and X as
  // they lie in memory, without a transpose kernel in front.
  int a_mn, b_mn;
  // normalisation of the token operand folded into the GEMM (swapped orientation only): the caller multiplies the norm
  // weight into the GEMM weight once (W'[f, k] = W[f, k] g[k]); the epilogue warps compute every token's statistics from
  // norm_x while the weights stream and the epilogue applies  out = rstd (acc - mean rowsum[f]) + bias.
  int norm_mode;                  // 0 none, 1 RMSNorm, 2 LayerNorm
  float norm_eps;
  const __nv_bfloat16* norm_x;    // [tokens, norm_k]: the rows the statistics are taken over (row pitch norm_ld); usually
                                  // the token operand itself, a superset of its columns when the GEMM contracts a slice
  long long norm_ld;
  int norm_k;
  const float* norm_rowsum;       // LayerNorm only: [features] sums of the rows of W'
#ifdef TPB_GEMM_TRACE
  int debug_skip_mma;             // measurement aid: stream the operands through the smem ring without issuing MMAs
  int trace_block;                // measurement aid: CTA (index + 1) that records %globaltimer stamps into g_gemm_trace; 0 = off
#endif
};

// %globaltimer stamps of one CTA of the most recent traced launch (see tpb_gemm_trace):
// 0 entry, 1 setup done, 2 first accumulator ready, 3 partial stored / pushed, 4 system fence + barrier passed,
// 5 arrival counters bumped, 6 reduce phase entered, 7 all arrivals seen, 8 reduced tile written; partial-tile path
// (last item of the CTA): 9 partial parked, 10 fence + barrier passed, 11 counter bumped, 12 last contributor starts
// the sum; 13 teardown; whole-tile path: 14 accumulators read, 15 tile written.
// Compiled in only with -DTPB_GEMM_TRACE: the product build carries neither the stamps nor their parameters.
#ifdef TPB_GEMM_TRACE
__device__ unsigned long long g_gemm_trace[32];
#define TPB_TRACE(i)                                                                         \
  do {                                                                                       \
    if (p.trace_block && int(blockIdx.x) == p.trace_block - 1) g_gemm_trace[i] = globaltimer_ns(); \
  } while (0)
#else
#define TPB_TRACE(i) do { } while (0)
#endif


__device__ __forceinline__ float apply_act(float x, int act) {
  switch (act) {
    case 1: return fmaxf(x, 0.f);
    case 2: return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case 3: {
      float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanhf(u));
    }
    case 4: return x / (1.f + __expf(-x));
    default: return x;
  }
}

// Out-of-line copy for the few-token epilogues.  Those run once per CTA, straight through code that is cold in the
// instruction cache; with the activation switch (erf, tanh, exp expansions) inlined into every one of the 16 unrolled
// iterations, each iteration started with an instruction-cache miss (~0.25 us apiece, measured with %globaltimer).
__device__ __noinline__ float apply_act_call(float x, int act) { return apply_act(x, act); }

// Retry loop of the flagged exchange (out of line: it is inlined 16 times otherwise).  Bounded by wall time.
__device__ __noinline__ uint4 poll_flagged_word(const uint4* ptr, uint32_t flag, uint64_t limit_ns, bool* ok) {
  const uint64_t start = globaltimer_ns();
  uint4 w;
  for (uint32_t i = 0;; ++i) {
    w = ld_relaxed_sys_v4(ptr);
    if (w.y == flag && w.w == flag) {
      *ok = true;
      return w;
    }
    if (i > 64) __nanosleep(20);
    if ((i & 63) == 63 && globaltimer_ns() - start > limit_ns) {
      *ok = false;
      return w;
    }
  }
}

// Work decomposition, walked identically by the producer, the MMA issuer and the epilogue warps of a CTA.
//  * uniform: item w = (split, tile) for w = blockIdx.x, blockIdx.x + gridDim.x, ...; every tile has k_splits
//    contributors of kb_per_split k-blocks each.
//  * stream-K: the tiles * k_blocks units (one unit = one pipeline stage of one tile) are dealt out as one contiguous
//    range per CTA, boundary(c) = c * units / gridDim.x, so every CTA streams the same number of bytes whatever the
//    tile count; a range is cut into items at tile boundaries.  A tile covered by several CTAs gets its partial sums
//    parked and added up by the last contributor to arrive, exactly like split-K.
struct WorkItem {
  int tile, kb0, kb1;
  int ordinal, contributors;  // this item's index among the contributors of its tile / their number
};

struct WorkIter {
  int w, tiles;              // uniform mode
  long long u, u_end, units; // stream-K mode
  __device__ __forceinline__ long long boundary(long long c) const { return c * units / (long long)gridDim.x; }
  __device__ __forceinline__ int owner(long long unit) const {  // CTA whose range holds `unit`
    long long c = unit * (long long)gridDim.x / units;
    while (boundary(c + 1) <= unit) ++c;
    return int(c);
  }
  __device__ __forceinline__ WorkIter(const GemmParams& p) {
    tiles = p.m_tiles * p.n_tiles;
    w = blockIdx.x;
    units = (long long)tiles * p.k_blocks;
    u = boundary(blockIdx.x);
    u_end = boundary(blockIdx.x + 1);
  }
  __device__ __forceinline__ bool next(const GemmParams& p, WorkItem& item) {
    if (!p.stream_k) {
      if (w >= tiles * p.k_splits) return false;
      const int split = w / tiles;
      item.tile = w - split * tiles;
      item.kb0 = split * p.kb_per_split;
      item.kb1 = min(p.k_blocks, item.kb0 + p.kb_per_split);
      item.ordinal = split;
      item.contributors = p.k_splits;
      w += gridDim.x;
      return true;
    }
    if (u >= u_end) return false;
    item.tile = int(u / p.k_blocks);
    item.kb0 = int(u - (long long)item.tile * p.k_blocks);
    const long long len = min((long long)(p.k_blocks - item.kb0), u_end - u);
    item.kb1 = item.kb0 + int(len);
    if (len == p.k_blocks) {
      item.ordinal = 0;
      item.contributors = 1;
    } else {
      const long long t0 = (long long)item.tile * p.k_blocks;
      const int first = owner(t0);
      item.ordinal = int(blockIdx.x) - first;
      item.contributors = owner(t0 + p.k_blocks - 1) - first + 1;
    }
    u += len;
    return true;
  }
};

// KBOX = number of consecutive 64-column k-blocks fetched per pipeline stage.  With KBOX > 1 a stage
// pulls KBOX * 128 contiguous bytes of every operand row in back-to-back TMA boxes.
// NACC = number of independent TMEM accumulators per tile.  Consecutive tcgen05.mma instructions that
// accumulate into the same TMEM columns serialise on the accumulator; at N = 16 / 32 one instruction is
// far shorter than that dependent latency, so the k-steps are dealt round-robin to NACC accumulators that
// the epilogue adds up.  (At N >= 64 one accumulator keeps the tensor pipe busy.)
// Register budget: the many-token instantiations (BN >= 128) are compiled as if two CTAs had to share an SM (at most 168
// registers per thread, although shared memory admits one CTA only): that leaves every SM sub-partition room for the
// warps of a small-footprint collective kernel, which is how the prefill pipeline runs an all-reduce BESIDE a GEMM.
template <int BN, int KBOX, int NACC>
__global__ void __launch_bounds__(NUM_THREADS, BN >= 128 ? 2 : 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const GemmParams p) {
  constexpr uint32_t A_BYTES = BM * BK * 2;
  constexpr uint32_t B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = KBOX * (A_BYTES + B_BYTES);
  constexpr uint32_t ACC_COLS = NACC * BN;                                  // columns of one accumulator set
  constexpr uint32_t TMEM_COLS = (2 * ACC_COLS < 32) ? 32 : 2 * ACC_COLS;   // two sets; power of two by construction
  static_assert(TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "TMEM allocation must be a power of two <= 512");
  constexpr uint32_t MN_BLOCK_BYTES = 64 * BK * 2;  // one [BK k-rows][64 MN elements] block of an MN-major operand
  constexpr bool MN_CAPABLE = BN >= 128;            // instantiations that may get MN-major operands (see tpb_gemm_plan_ex)
  constexpr bool FEW_TOKENS = BN <= 64;             // instantiations of the swapped orientation: norm folding, flagged words
  constexpr int MMAS_PER_STAGE = KBOX * (BK / UMMA_K);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + size_t(p.stages) * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + MAX_STAGES;
  uint64_t* acc_full = empty_bar + MAX_STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;            // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* epi_ok = tmem_slot + 2;
  volatile uint32_t* epi_last = tmem_slot + 3;
  float* norm_stats = reinterpret_cast<float*>(tmem_slot + 4);  // [64 tokens][rstd, mean * rstd]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    TPB_TRACE(0);
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], EPI_THREADS / 32);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();     // everything below reads what earlier kernels wrote
  pdl_trigger();  // the next kernel in the stream may be scheduled and run its own prologue (see launch.cuh)
  if (threadIdx.x == 0) TPB_TRACE(1);

  const int tiles = p.m_tiles * p.n_tiles;

  if (p.ag_world > 1) {
    // ---------------- all-gather push: local slice -> every rank's gathered buffer ----------------
    const int vec_per_row = p.ag_cols >> 3;
    const long long total = (long long)p.ag_rows * vec_per_row;
    for (long long i = blockIdx.x * (long long)NUM_THREADS + threadIdx.x; i < total; i += (long long)gridDim.x * NUM_THREADS) {
      const long long r = i / vec_per_row;
      const int c = int(i % vec_per_row) * 8;
      const uint4 val = *reinterpret_cast<const uint4*>(p.ag_src + r * p.ag_src_ld + c);
      if (p.ag_mc_dst) {
        // one store, replicated to every rank by the NVSwitch: this GPU sends its slice once instead of once per peer
        multimem_st(p.ag_mc_dst + r * p.ag_dst_ld + p.ag_rank * p.ag_cols + c, val);
      } else {
#pragma unroll
        for (int d = 0; d < MAX_WORLD; ++d)
          if (d < p.ag_world) *reinterpret_cast<uint4*>(p.ag_dst[d] + r * p.ag_dst_ld + p.ag_rank * p.ag_cols + c) = val;
      }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t old = atomicAdd(p.ag_push_counter, 1u);
      if (old == gridDim.x - 1) {  // the whole slice has left this GPU: tell every rank
        *p.ag_push_counter = 0;
        __threadfence_system();
        for (int d = 0; d < p.ag_world; ++d) red_add_relaxed_sys(p.ag_flags[d] + p.ag_rank, 1u);
      }
    }
  }

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      uint32_t it = 0;
      WorkIter work(p);
      WorkItem item;
      while (!*abort_flag && work.next(p, item)) {
        const int mt = item.tile % p.m_tiles;
        const int nt = item.tile / p.m_tiles;
        const int kb0 = item.kb0, kb1 = item.kb1;
        int ag_ready_src = -1;
        for (int kb_seq = kb0; kb_seq < kb1; ++kb_seq, ++it) {
          int kb = kb_seq;
          if (p.ag_world > 1) {
            // start with the k-blocks of the local slice, then walk the other ranks' slices as they arrive
            kb = (kb_seq + p.ag_rank * p.ag_kb_per_rank) % p.k_blocks;
            const int src = kb / p.ag_kb_per_rank;
            if (src != ag_ready_src) {
              if (!wait_flag_ge(p.ag_flags[p.ag_rank] + src, p.ag_epoch, p.wait_ns)) {
                atomicMax(p.status, STATUS_TIMEOUT_FLAG);
                *abort_flag = 1;
                break;
              }
              asm volatile("fence.proxy.async;" ::: "memory");  // peer-written rows must be visible to the TMA engine
              ag_ready_src = src;
            }
          }
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
            atomicMax(p.status, STATUS_TIMEOUT_MBAR);
            *abort_flag = 1;
            break;
          }
          uint8_t* a_dst = smem + size_t(s) * STAGE_BYTES;
          uint8_t* b_dst = a_dst + KBOX * A_BYTES;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          // (MN-major operands only exist in the many-token instantiations: the few-token kernels stay small)
          if (MN_CAPABLE && p.a_mn) {  // (KBOX == 1) 64-wide MN blocks of BK k-rows each, stacked along MN
#pragma unroll
            for (int b = 0; b < BM / 64; ++b)
              tma_load_2d(a_dst + b * MN_BLOCK_BYTES, &tmap_a, &full_bar[s], mt * BM + b * 64, kb * BK);
          } else {
#pragma unroll
            for (int j = 0; j < KBOX; ++j)  // columns past K are filled with zeros by TMA and cost no DRAM traffic
              tma_load_2d(a_dst + j * A_BYTES, &tmap_a, &full_bar[s], (kb * KBOX + j) * BK, mt * BM);
          }
          if (MN_CAPABLE && p.b_mn) {
#pragma unroll
            for (int b = 0; b < BN / 64; ++b)
              tma_load_2d(b_dst + b * MN_BLOCK_BYTES, &tmap_b, &full_bar[s], nt * BN + b * 64, kb * BK);
          } else {
#pragma unroll
            for (int j = 0; j < KBOX; ++j)
              tma_load_2d(b_dst + j * B_BYTES, &tmap_b, &full_bar[s], (kb * KBOX + j) * BK, nt * BN);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      uint32_t it = 0;
      uint32_t local = 0;
      const uint32_t idesc = make_idesc_bf16(BM, BN, p.a_mn != 0, p.b_mn != 0);
      const bool any_mn = MN_CAPABLE && (p.a_mn | p.b_mn) != 0;
      WorkIter work(p);
      WorkItem item;
      for (; !*abort_flag && work.next(p, item); ++local) {
        const int kb0 = item.kb0, kb1 = item.kb1;
        const int acc = local & 1;
        const uint32_t acc_ph = (local >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1)) {
          atomicMax(p.status, STATUS_TIMEOUT_MBAR);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        uint32_t issued = 0;  // MMAs issued for this work item; MMA i accumulates into accumulator i % NACC
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % p.stages;
          const uint32_t ph = (it / p.stages) & 1;
          if (!mbar_wait(&full_bar[s], ph)) {
            atomicMax(p.status, STATUS_TIMEOUT_MBAR);
            *abort_flag = 1;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + size_t(s) * STAGE_BYTES);
          const uint32_t b_addr = a_addr + KBOX * A_BYTES;
#ifdef TPB_GEMM_TRACE
          if (p.debug_skip_mma) {
            issued += MMAS_PER_STAGE;
            if (kb + 1 < kb1) { mbar_arrive(&empty_bar[s]); continue; }
          }
#endif
          if (!any_mn) {  // (the issue loop of the few-token shapes is latency-critical: no per-instruction branches)
#pragma unroll
            for (int j = 0; j < KBOX; ++j) {
#pragma unroll
              for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                // K-major: a k-step of 16 elements is 32 bytes further along the swizzled 128-byte rows
                const uint64_t adesc = make_desc_kmajor_sw128(a_addr + j * A_BYTES + kk * UMMA_K * 2);
                const uint64_t bdesc = make_desc_kmajor_sw128(b_addr + j * B_BYTES + kk * UMMA_K * 2);
                umma_bf16(d_tmem + (issued % NACC) * BN, adesc, bdesc, idesc, issued >= NACC ? 1u : 0u);
                ++issued;
              }
            }
          } else {
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              // MN-major (KBOX == 1): a k-step is 16 k-rows (two 8-row swizzle atoms) further down the block
              const uint64_t adesc = p.a_mn ? make_desc_mnmajor_sw128(a_addr + kk * UMMA_K * 128, MN_BLOCK_BYTES)
                                            : make_desc_kmajor_sw128(a_addr + kk * UMMA_K * 2);
              const uint64_t bdesc = p.b_mn ? make_desc_mnmajor_sw128(b_addr + kk * UMMA_K * 128, MN_BLOCK_BYTES)
                                            : make_desc_kmajor_sw128(b_addr + kk * UMMA_K * 2);
              umma_bf16(d_tmem + (issued % NACC) * BN, adesc, bdesc, idesc, issued >= NACC ? 1u : 0u);
              ++issued;
            }
          }
          umma_commit(&empty_bar[s]);  // frees the smem stage when these MMAs retire
        }
        umma_commit(&acc_full[acc]);  // accumulators complete
      }
    }
  } else {
    // ---------------- epilogue warps ----------------
    const int quarter = warp & 3;  // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;
    // The epilogue of a decode GEMM runs once per CTA, right on the critical path, and every kernel parameter it
    // touches for the first time is a constant-cache miss served from L2 (a good fraction of a microsecond each, one
    // after the other).  Read them into registers now, while the first tiles are still streaming in.
    __nv_bfloat16* hot_out = p.out;
    const __nv_bfloat16* hot_bias = p.bias;
    const __nv_bfloat16* hot_residual = p.residual;
    int hot_ld_out = p.ld_out, hot_act = p.act, hot_n_extent = p.n_extent, hot_m_extent = p.m_extent;
    float hot_bias_scale = p.bias_scale;
    asm volatile("" : "+l"(hot_out), "+l"(hot_bias), "+l"(hot_residual), "+r"(hot_ld_out), "+r"(hot_act), "+r"(hot_n_extent),
                 "+r"(hot_m_extent), "+f"(hot_bias_scale));
    if (FEW_TOKENS && p.norm_mode) {
      // statistics of every token row of the unnormalised operand (swapped orientation: at most 64 tokens, all of them
      // in this CTA's tile), computed by the otherwise idle epilogue warps while the weights stream in
      const int chunks = p.norm_k >> 3;
      const float inv_k = 1.f / float(p.norm_k);
      for (int t = warp - 2; t < p.n_extent; t += EPI_THREADS / 32) {
        const uint4* xrow = reinterpret_cast<const uint4*>(p.norm_x + size_t(t) * p.norm_ld);
        float s1 = 0.f, s2 = 0.f;
        for (int c = lane; c < chunks; c += 32) {
          const uint4 u = xrow[c];
          const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float lo = bf16_bits_to_float(w4[i] & 0xFFFF), hi = bf16_bits_to_float(w4[i] >> 16);
            s1 += lo + hi;
            s2 += lo * lo + hi * hi;
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          s1 += __shfl_xor_sync(0xffffffffu, s1, o);
          s2 += __shfl_xor_sync(0xffffffffu, s2, o);
        }
        if (lane == 0) {
          const float mean = p.norm_mode == 2 ? s1 * inv_k : 0.f;
          const float rstd = rsqrtf(fmaxf(s2 * inv_k - mean * mean, 0.f) + p.norm_eps);
          norm_stats[2 * t] = rstd;
          norm_stats[2 * t + 1] = mean * rstd;
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
    }
    const bool hot_norm = FEW_TOKENS && p.norm_mode != 0;
    const float* hot_rowsum = p.norm_rowsum;
    uint32_t local = 0;
    WorkIter work(p);
    WorkItem item;
    for (; work.next(p, item); ++local) {
      const int tile = item.tile;
      const int mt = tile % p.m_tiles;
      const int nt = tile / p.m_tiles;
      const int acc = local & 1;
      const uint32_t acc_ph = (local >> 1) & 1;
      const int m = mt * BM + row;
      const bool m_ok = m < p.m_extent;
      // Few-token tiles: fetch this row's residual values and bias NOW, while the weights are still streaming - loaded
      // after the accumulators are ready they would add a full memory round trip to the critical path of the kernel.
      float res_pre[16];
      float bias_pre = 0.f;
      bool prefetched = false;
      if constexpr (BN == 16) {
        if (p.swapped && hot_act != 5 && nt == 0) {
          prefetched = true;
          if (m_ok) {
            if (hot_bias) bias_pre = hot_bias_scale * __bfloat162float(hot_bias[m]);
#pragma unroll
            for (int j = 0; j < 16; ++j)
              res_pre[j] = (hot_residual && j < hot_n_extent) ? __bfloat162float(hot_residual[size_t(j) * hot_ld_out + m]) : 0.f;
          }
        }
      }
      // one thread waits, the group agrees on the outcome (so that nobody is left at a named barrier)
      if (threadIdx.x == 64) {
        bool ok = !*abort_flag && mbar_wait(&acc_full[acc], acc_ph);
        if (!ok) {
          atomicMax(p.status, STATUS_TIMEOUT_MBAR);
          *abort_flag = 1;
        }
        *epi_ok = ok ? 1u : 0u;
      }
      uint32_t ll_flag = 0;
      if (p.ll) {  // read before the barrier; thread 64 advances the word only after it
        ll_flag = __ldcg(p.ll_epochs + tile) + 1u;
        if (ll_flag == 0) ll_flag = 1u;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
      if (!*epi_ok) break;
      tc_fence_after();
      if (threadIdx.x == 64) TPB_TRACE(2);
      const uint32_t t_lane = tmem_base + (uint32_t(quarter * 32) << 16) + acc * ACC_COLS;
      const int n_mma = (item.kb1 - item.kb0) * MMAS_PER_STAGE;
      const int n_acc = n_mma < NACC ? n_mma : NACC;  // accumulators that were written for this item

      // A chunk is 16 accumulator columns of this thread's row: (token m, features n0..n0+15) in the normal
      // orientation, (feature m, tokens n0..n0+15) in the swapped one.  idx(j) addresses out[token, feature].
      auto chunk_valid = [&](int n0) { return m_ok && n0 < p.n_extent; };
      auto read_acc = [&](int c0, float (&v)[16]) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.f;
#pragma unroll 1  // (rolled on purpose: this runs once per tile from a cold instruction cache, small code wins)
        for (int a = 0; a < n_acc; ++a) {
          uint32_t r[16];
          tmem_ld_x16(t_lane + a * BN + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] += __uint_as_float(r[j]);
        }
      };
      auto store_partial = [&](float* slot, int n0, const float (&v)[16]) {
        if (!chunk_valid(n0)) return;
        // (largest index this call touches in the slot: checked in a -DTPB_BOUNDS build, where it skips the whole chunk)
        if (!TPB_IN_BOUNDS((p.swapped ? size_t(min(n0 + 15, p.n_extent - 1)) * p.ld_slot + m : size_t(m) * p.ld_slot + min(n0 + 15, p.n_extent - 1)) <
                               p.slot_stride, p.status))
          return;
        if (!p.swapped) {
          const size_t base = size_t(m) * p.ld_slot + n0;
          if (n0 + 16 <= p.n_extent && (p.ld_slot & 3) == 0) {
            float4* dst = reinterpret_cast<float4*>(slot + base);
#pragma unroll
            for (int q = 0; q < 4; ++q) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          } else {
            for (int j = 0; j < 16 && n0 + j < p.n_extent; ++j) slot[base + j] = v[j];
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (n0 + j < p.n_extent) slot[size_t(n0 + j) * p.ld_slot + m] = v[j];
        }
      };
      // v = sum over the parked partials [first_slot, first_slot + count) of this tile, added in slot order.  The loads of
      // four slots are issued before the first value is used: a load that is consumed right away costs one full memory
      // round trip (more than a microsecond while the GPU streams weights), and those round trips would add up.
      auto sum_partials = [&](int count, int n0, float (&v)[16]) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.f;
        if (!chunk_valid(n0)) return;
        const float* base = p.slots[p.rank] + size_t(p.world) * p.slot_stride;
        const bool vec = !p.swapped && n0 + 16 <= p.n_extent && (p.ld_slot & 3) == 0;
#pragma unroll 1
        for (int h = 0; h < 16; h += 8) {  // half a chunk at a time keeps the batch in registers
          if (n0 + h >= p.n_extent) break;
#pragma unroll 1
          for (int s0 = 0; s0 < count; s0 += 4) {
            float t[4][8];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float* slot = base + size_t(s0 + q) * p.slot_stride;
              const bool live = s0 + q < count;
              if (vec) {
                const float4* src = reinterpret_cast<const float4*>(slot + size_t(m) * p.ld_slot + n0 + h);
                const float4 f0 = live ? __ldcg(src) : make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 f1 = live ? __ldcg(src + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
                t[q][0] = f0.x; t[q][1] = f0.y; t[q][2] = f0.z; t[q][3] = f0.w;
                t[q][4] = f1.x; t[q][5] = f1.y; t[q][6] = f1.z; t[q][7] = f1.w;
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const size_t idx = p.swapped ? size_t(n0 + h + j) * p.ld_slot + m : size_t(m) * p.ld_slot + n0 + h + j;
                  t[q][j] = (live && n0 + h + j < p.n_extent) ? __ldcg(slot + idx) : 0.f;
                }
              }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (h == 0) v[j] += t[q][j];
                else v[8 + j] += t[q][j];
              }
          }
        }
      };
      // gated silu, normal orientation: vg = 16 gate columns, vu = the 16 up columns that follow them
      auto finalize_gated = [&](int n0_gate, float (&vg)[16], float (&vu)[16]) {
        if (!chunk_valid(n0_gate)) return;
        const size_t base = size_t(m) * p.ld_out + (n0_gate >> 1);
        float o[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float gte = vg[j] + (p.bias ? p.bias_scale * __bfloat162float(p.bias[n0_gate + j]) : 0.f);
          const float upv = vu[j] + (p.bias ? p.bias_scale * __bfloat162float(p.bias[n0_gate + 16 + j]) : 0.f);
          o[j] = gte / (1.f + __expf(-gte)) * upv;
        }
        if ((p.ld_out & 7) == 0) {
          uint4 o0, o1;
          o0.x = pack_bf16x2(o[0], o[1]);   o0.y = pack_bf16x2(o[2], o[3]);
          o0.z = pack_bf16x2(o[4], o[5]);   o0.w = pack_bf16x2(o[6], o[7]);
          o1.x = pack_bf16x2(o[8], o[9]);   o1.y = pack_bf16x2(o[10], o[11]);
          o1.z = pack_bf16x2(o[12], o[13]); o1.w = pack_bf16x2(o[14], o[15]);
          if (TPB_IN_BOUNDS(base + 16 <= p.out_elems, p.status)) {
            uint4* op = reinterpret_cast<uint4*>(p.out + base);
            op[0] = o0;
            op[1] = o1;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (TPB_IN_BOUNDS(base + j < p.out_elems, p.status)) p.out[base + j] = __float2bfloat16(o[j]);
        }
      };
      auto finalize = [&](int n0, float (&v)[16]) {  // bias, activation, residual, bf16 store
        if (n0 >= hot_n_extent) return;  // (uniform across the warp)
        if (p.swapped && hot_act != 5) {
          // tokens are the accumulator columns, a lane owns one feature: neighbouring lanes pair up so that every
          // store carries two features (4 bytes); rows past the feature count only take part in the shuffle
          const float b = prefetched ? bias_pre : ((m_ok && hot_bias) ? hot_bias_scale * __bfloat162float(hot_bias[m]) : 0.f);
          const float rowsum = (hot_norm && hot_rowsum && m_ok) ? hot_rowsum[m] : 0.f;
          const bool pitch_even = (hot_ld_out & 1) == 0 && (reinterpret_cast<uintptr_t>(hot_out) & 3) == 0;
          const bool writes_pair = pitch_even && !(lane & 1) && m + 1 < hot_m_extent;
          const bool covered = pitch_even && (lane & 1);  // the even neighbour stores this lane's value
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (n0 + j >= hot_n_extent) break;  // (uniform) the code of the remaining iterations is never fetched
            const size_t idx = size_t(n0 + j) * hot_ld_out + m;
            float x = v[j];
            if (hot_norm) x = x * norm_stats[2 * (n0 + j)] - norm_stats[2 * (n0 + j) + 1] * rowsum;
            x += b;
            if (hot_act) x = apply_act_call(x, hot_act);
            if (hot_residual && m_ok) x += prefetched ? res_pre[j] : __bfloat162float(hot_residual[idx]);
            const float up = __shfl_down_sync(0xffffffffu, x, 1);
            if (m_ok && TPB_IN_BOUNDS(idx + (writes_pair ? 1 : 0) < p.out_elems, p.status)) {
              if (writes_pair) *reinterpret_cast<uint32_t*>(hot_out + idx) = pack_bf16x2(x, up);
              else if (!covered) hot_out[idx] = __float2bfloat16(x);
            }
          }
          return;
        }
        if (!m_ok) return;
        if (p.act == 5) {
          // gated silu, swapped orientation: lanes 0-15 of a warp hold gate rows, lanes 16-31 the matching up rows
          const float b = p.bias ? p.bias_scale * __bfloat162float(p.bias[m]) : 0.f;
          const float rowsum = (hot_norm && hot_rowsum) ? hot_rowsum[m] : 0.f;
          const int f_out = (m >> 5) * 16 + (m & 15);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float x = v[j];
            if (hot_norm && n0 + j < p.n_extent) x = x * norm_stats[2 * (n0 + j)] - norm_stats[2 * (n0 + j) + 1] * rowsum;
            x += b;
            const float partner = __shfl_xor_sync(0xffffffffu, x, 16);
            if ((lane & 16) == 0 && n0 + j < p.n_extent && TPB_IN_BOUNDS(size_t(n0 + j) * p.ld_out + f_out < p.out_elems, p.status))
              p.out[size_t(n0 + j) * p.ld_out + f_out] = __float2bfloat16(x / (1.f + __expf(-x)) * partner);
          }
          return;
        }
        if (!p.swapped) {
          const size_t base = size_t(m) * p.ld_out + n0;
          if (n0 + 16 <= p.n_extent && (p.ld_out & 7) == 0) {
            if (p.bias) {
              const uint4* bp = reinterpret_cast<const uint4*>(p.bias + n0);
              const uint4 b0 = bp[0], b1 = bp[1];
              const uint32_t bw[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                v[2 * j] += p.bias_scale * bf16_bits_to_float(bw[j] & 0xFFFF);
                v[2 * j + 1] += p.bias_scale * bf16_bits_to_float(bw[j] >> 16);
              }
            }
            if (p.act) {
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = apply_act(v[j], p.act);
            }
            if (p.residual) {
              const uint4* rp = reinterpret_cast<const uint4*>(p.residual + base);
              const uint4 r0 = rp[0], r1 = rp[1];
              const uint32_t rw[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                v[2 * j] += bf16_bits_to_float(rw[j] & 0xFFFF);
                v[2 * j + 1] += bf16_bits_to_float(rw[j] >> 16);
              }
            }
            uint4 o0, o1;
            o0.x = pack_bf16x2(v[0], v[1]);   o0.y = pack_bf16x2(v[2], v[3]);
            o0.z = pack_bf16x2(v[4], v[5]);   o0.w = pack_bf16x2(v[6], v[7]);
            o1.x = pack_bf16x2(v[8], v[9]);   o1.y = pack_bf16x2(v[10], v[11]);
            o1.z = pack_bf16x2(v[12], v[13]); o1.w = pack_bf16x2(v[14], v[15]);
            if (TPB_IN_BOUNDS(base + 16 <= p.out_elems, p.status)) {
              uint4* op = reinterpret_cast<uint4*>(p.out + base);
              op[0] = o0;
              op[1] = o1;
            }
          } else {
            for (int j = 0; j < 16 && n0 + j < p.n_extent; ++j) {
              float x = v[j] + (p.bias ? p.bias_scale * __bfloat162float(p.bias[n0 + j]) : 0.f);
              if (p.act) x = apply_act_call(x, p.act);
              if (p.residual) x += __bfloat162float(p.residual[base + j]);
              if (TPB_IN_BOUNDS(base + j < p.out_elems, p.status)) p.out[base + j] = __float2bfloat16(x);
            }
          }
        }
      };
      // flagged-word variant (swapped orientation only: all tokens sit in one tile): slot k of rank d's flagged area
      // holds rank k's partial, rounded to bf16 (what an all-reduce of bf16 activations sums as well), as 16-byte words
      // {bf16x2(t, t+1), epoch, bf16x2(t+2, t+3), epoch} laid out [tile][token quad][feature row]: the 32 lanes of a warp
      // touch 512 contiguous bytes per access.  Each 8-byte half carries its own epoch, so only 8-byte single-copy
      // atomicity is relied upon.  A tile always owns the same LL_TILE_WORDS words whatever the shape of the call, and its
      // epoch only grows, so a word left behind by an earlier call (of any shape) can never carry the epoch a later call
      // waits for.  The area starts LL_FIRST_SLOT slots into the workspace and a flagged slot spans two fp32 slots.
      bool ll_gave_up = false;
      const size_t ll_row = size_t(tile) * LL_TILE_WORDS + size_t(row);  // this thread's word of token quad 0; quad q is 128 q words on
      auto push_ll = [&](int n0, const float (&v)[16]) {
        if (!chunk_valid(n0)) return;
        if (p.mc_slots) {
          // one multimem.st per word reaches this rank's slot in EVERY rank's workspace (the NVSwitch replicates it); each
          // 8-byte half of a word carries its own copy of the flag, so nothing depends on the 16 bytes landing together
          uint4* dst = reinterpret_cast<uint4*>(p.mc_slots + size_t(LL_FIRST_SLOT + 2 * p.rank) * p.slot_stride) + ll_row + size_t(n0 >> 2) * BM;
          if (!TPB_IN_BOUNDS(ll_row + size_t((n0 >> 2) + 3) * BM < (p.slot_stride >> 1), p.status)) return;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (n0 + 4 * q >= p.n_extent) break;
            multimem_st(dst + q * BM, make_uint4(pack_bf16x2(v[4 * q], v[4 * q + 1]), ll_flag, pack_bf16x2(v[4 * q + 2], v[4 * q + 3]), ll_flag));
          }
          return;
        }
#pragma unroll 1  // (rolled: small code, see read_acc)
        for (int d = 0; d < p.world; ++d) {
          uint4* dst = reinterpret_cast<uint4*>(p.slots[d] + size_t(LL_FIRST_SLOT + 2 * p.rank) * p.slot_stride) + ll_row + size_t(n0 >> 2) * BM;
          if (!TPB_IN_BOUNDS(ll_row + size_t((n0 >> 2) + 3) * BM < (p.slot_stride >> 1), p.status)) break;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (n0 + 4 * q >= p.n_extent) break;
            st_relaxed_sys_v4(dst + q * BM, pack_bf16x2(v[4 * q], v[4 * q + 1]), ll_flag, pack_bf16x2(v[4 * q + 2], v[4 * q + 3]), ll_flag);
          }
        }
      };
      auto wait_ll = [&](const uint4* ptr, uint4 first) -> uint4 {
        if ((first.y == ll_flag && first.w == ll_flag) || ll_gave_up) return first;
        bool ok;
        first = poll_flagged_word(ptr, ll_flag, p.wait_ns, &ok);
        if (!ok) {
          atomicMax(p.status, STATUS_TIMEOUT_FLAG);
          ll_gave_up = true;
        }
        return first;
      };
      // sum the ranks' partials in rank order (identical on every rank); the caller runs the usual epilogue on the sums
      auto reduce_ll = [&](int n0, float (&sum)[16]) {
#pragma unroll
        for (int j = 0; j < 16; ++j) sum[j] = 0.f;
        if (!chunk_valid(n0)) return;
        const uint4* area = reinterpret_cast<const uint4*>(p.slots[p.rank] + size_t(LL_FIRST_SLOT) * p.slot_stride);
        const size_t slot_words = p.slot_stride >> 1;  // 16-byte words per flagged slot (= 2 fp32 slots)
        constexpr int KH = 4;  // 4 token quads x KH ranks of flagged words are in flight before the first one is examined
#pragma unroll 1
        for (int k0 = 0; k0 < p.world; k0 += KH) {  // ranks in ascending order: the sum is bitwise identical on every rank
          uint4 a[4][KH];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int k = 0; k < KH; ++k)
              if (n0 + 4 * q < p.n_extent && k0 + k < p.world)
                a[q][k] = ld_relaxed_sys_v4(area + size_t(k0 + k) * slot_words + ll_row + size_t((n0 >> 2) + q) * BM);
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (n0 + 4 * q < p.n_extent) {
#pragma unroll
              for (int k = 0; k < KH; ++k) {
                if (k0 + k < p.world) {
                  const uint4 w4 = wait_ll(area + size_t(k0 + k) * slot_words + ll_row + size_t((n0 >> 2) + q) * BM, a[q][k]);
                  sum[4 * q] += bf16_bits_to_float(w4.x & 0xFFFF);
                  sum[4 * q + 1] += bf16_bits_to_float(w4.x >> 16);
                  sum[4 * q + 2] += bf16_bits_to_float(w4.z & 0xFFFF);
                  sum[4 * q + 3] += bf16_bits_to_float(w4.z >> 16);
                }
              }
            }
          }
        }
      };
      auto push_to_peers = [&](int n0, const float (&v)[16]) {  // this rank's (split-reduced) partial -> slot[rank] everywhere
#pragma unroll
        for (int d = 0; d < MAX_WORLD; ++d)
          if (d < p.world) store_partial(p.slots[d] + size_t(p.rank) * p.slot_stride, n0, v);
      };

      const bool split_k = item.contributors > 1;
      const bool gated_cols = p.act == 5 && !p.swapped;  // column chunks alternate gate / up
      if (!split_k) {
        if (gated_cols) {
          if constexpr (BN >= 32) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
              float vg[16], vu[16];
              read_acc(c0, vg);
              read_acc(c0 + 16, vu);
              finalize_gated(nt * BN + c0, vg, vu);
            }
          }
        } else {
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) {
            float v[16];
            read_acc(c0, v);
            if (threadIdx.x == 64) TPB_TRACE(14);
            if (p.ll) push_ll(nt * BN + c0, v);
            else if (p.world > 1) push_to_peers(nt * BN + c0, v);
            else finalize(nt * BN + c0, v);
          }
        }
        if (threadIdx.x == 64) TPB_TRACE(15);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);  // accumulators may be overwritten from here on
        if (p.ll) {
          if (threadIdx.x == 64) {
            p.ll_epochs[tile] = ll_flag;
            TPB_TRACE(3);
          }
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) {
            float v[16];
            reduce_ll(nt * BN + c0, v);
            finalize(nt * BN + c0, v);
          }
          if (threadIdx.x == 64) TPB_TRACE(8);
        }
      } else {
        // split-K: park the partial in a local slot; the LAST split to arrive for this tile adds them up in split
        // order (deterministic) and carries on - nobody ever waits for another CTA.
        float* my_slot = p.slots[p.rank] + size_t(p.world + item.ordinal) * p.slot_stride;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          float v[16];
          read_acc(c0, v);
          store_partial(my_slot, nt * BN + c0, v);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        if (threadIdx.x == 64) TPB_TRACE(9);
        __threadfence();
        asm volatile("bar.sync 2, %0;" ::"n"(EPI_THREADS) : "memory");
        if (threadIdx.x == 64) {
          TPB_TRACE(10);
          const uint32_t old = atomicAdd(p.split_counters + tile, 1u);
          TPB_TRACE(11);
          const bool last = old == uint32_t(item.contributors - 1);
          if (last) p.split_counters[tile] = 0;  // every other split has arrived: safe to re-arm for the next call
          *epi_last = last ? 1u : 0u;
        }
        asm volatile("bar.sync 2, %0;" ::"n"(EPI_THREADS) : "memory");
        if (*epi_last) {
          __threadfence();
          if (threadIdx.x == 64) TPB_TRACE(12);
          if (gated_cols) {
            if constexpr (BN >= 32) {
#pragma unroll 1
              for (int c0 = 0; c0 < BN; c0 += 32) {
                float vg[16], vu[16];
                sum_partials(item.contributors, nt * BN + c0, vg);
                sum_partials(item.contributors, nt * BN + c0 + 16, vu);
                finalize_gated(nt * BN + c0, vg, vu);
              }
            }
          } else {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
              float v[16];
              sum_partials(item.contributors, nt * BN + c0, v);
              if (p.ll) push_ll(nt * BN + c0, v);
              else if (p.world > 1) push_to_peers(nt * BN + c0, v);
              else finalize(nt * BN + c0, v);
            }
            if (p.ll) {
              if (threadIdx.x == 64) p.ll_epochs[tile] = ll_flag;
#pragma unroll 1
              for (int c0 = 0; c0 < BN; c0 += 16) {
                float v[16];
                reduce_ll(nt * BN + c0, v);
                finalize(nt * BN + c0, v);
              }
            }
          }
        }
      }
      if (p.world > 1 && !p.ll && (!split_k || *epi_last)) {
        // make this tile's partial visible system-wide, then count one arrival on every rank
        // (the barrier orders every epilogue thread's stores before thread 64's fence, which is cumulative: one
        // system-scope fence per tile instead of one per thread - each costs microseconds)
        if (threadIdx.x == 64) TPB_TRACE(3);
        asm volatile("bar.sync 2, %0;" ::"n"(EPI_THREADS) : "memory");
        if (threadIdx.x == 64) {
          TPB_TRACE(4);
          __threadfence_system();
          for (int d = 0; d < p.world; ++d) red_add_relaxed_sys(p.arrivals[d] + tile, 1u);
          TPB_TRACE(5);
        }
      }
    }
  }

  // ---------------- cross-rank reduce phase ----------------
  __syncthreads();
  if (p.world > 1 && !p.ll) {
    const uint32_t contributions = uint32_t(p.world);
    const float* base_slot = p.slots[p.rank];
    // token / feature extents of one tile in out[token, feature] coordinates
    const int tok_tile = p.swapped ? BN : BM;
    const int feat_tile = p.swapped ? BM : BN;
    const int tokens = p.swapped ? p.n_extent : p.m_extent;
    const int features = p.swapped ? p.m_extent : p.n_extent;
    __shared__ uint32_t wait_ok;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
      const int mt = tile % p.m_tiles;
      const int nt = tile / p.m_tiles;
      if (threadIdx.x == 0) {
        TPB_TRACE(6);
        const uint32_t target = p.expected[tile] + contributions;
        bool ok = !*abort_flag && wait_flag_ge(p.arrivals[p.rank] + tile, target, p.wait_ns);
        TPB_TRACE(7);
        if (!ok) atomicMax(p.status, STATUS_TIMEOUT_FLAG);
        p.expected[tile] = target;
        wait_ok = ok ? 1u : 0u;
      }
      __syncthreads();
      if (wait_ok) {
        const int tok0 = (p.swapped ? nt : mt) * tok_tile;
        const int feat0 = (p.swapped ? mt : nt) * feat_tile;
        const int tok_n = min(tok_tile, tokens - tok0);
        const int feat_n = min(feat_tile, features - feat0);
        const int feat_vec = (feat_n + 3) >> 2;
        const bool vec_ok = (p.ld_out & 3) == 0 && (feat_n & 3) == 0;
        for (int e = threadIdx.x; e < tok_n * feat_vec; e += NUM_THREADS) {
          const int t = tok0 + e / feat_vec;
          const int f = feat0 + (e % feat_vec) * 4;
          const size_t idx = size_t(t) * p.ld_out + f;
          float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
          if (vec_ok) {
            for (int k = 0; k < p.world; ++k) {
              const float4 v = __ldcg(reinterpret_cast<const float4*>(base_slot + size_t(k) * p.slot_stride + idx));
              s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
          } else {
            float* sp = &s.x;
            for (int k = 0; k < p.world; ++k)
              for (int j = 0; j < 4 && f + j < feat0 + feat_n; ++j) sp[j] += __ldcg(base_slot + size_t(k) * p.slot_stride + idx + j);
          }
          float o[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (f + j < feat0 + feat_n) {
              float x = o[j] + (p.bias ? p.bias_scale * __bfloat162float(p.bias[f + j]) : 0.f);
              if (p.act) x = apply_act_call(x, p.act);
              if (p.residual) x += __bfloat162float(p.residual[idx + j]);
              if (TPB_IN_BOUNDS(idx + j < p.out_elems, p.status)) p.out[idx + j] = __float2bfloat16(x);
            }
          }
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) TPB_TRACE(8);
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) TPB_TRACE(13);
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D bf16 row-major [rows, cols] (cols contiguous, row pitch ld elements), box = [box_rows, 64 cols], 128B swizzle.
static int make_tmap_2d(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return TPB_ERR_DRIVER;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "tpb: cuTensorMapEncodeTiled failed (%d): base %p, %llu rows x %llu cols, pitch %llu elements, box %u x %u\n", int(r), ptr,
            (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld, box_rows, unsigned(BK));
  return r == CUDA_SUCCESS ? TPB_OK : TPB_ERR_TMAP;
}

static int g_debug_stages = 0, g_disable_ll = 0, g_enable_stream_k = 0;  // measurement aids, see tpb_gemm_debug
#ifdef TPB_GEMM_TRACE
static int g_debug_skip_mma = 0, g_trace_block = 0;
#endif
// split-K of few-tile weight-streaming GEMMs (see tpb_gemm_plan): a tile is split when it streams at least
// g_split_min_kb KiB of weights, into pieces of about g_split_target_kb KiB
static int g_split_min_kb = 1024, g_split_target_kb = 256;
static uint64_t g_wait_ns = TPB_WAIT_LIMIT_NS;  // bound of the waits for peer GPUs, see tpb_set_wait_limit

template <int BN, int KBOX, int NACC>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, int grid, cudaStream_t stream) {
  constexpr size_t stage_bytes = size_t(KBOX) * size_t(BM * BK * 2 + BN * BK * 2);
  int stages = int((227 * 1024 - 2048) / stage_bytes);
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages < 2) stages = 2;
  if (stages > p.kb_per_split + 1 && (p.stream_k || p.m_tiles * p.n_tiles * p.k_splits <= grid)) stages = max(2, p.kb_per_split + 1);
  if (g_debug_stages > 0 && g_debug_stages < stages) stages = g_debug_stages;
  p.stages = stages;
#ifdef TPB_GEMM_TRACE
  p.debug_skip_mma = g_debug_skip_mma;
  p.trace_block = g_trace_block;
#endif
  size_t smem = stages * stage_bytes + 1024 /*align*/ + (2 * MAX_STAGES + 4) * 8 + 16 + 64 * 2 * sizeof(float) /*norm statistics*/;
  // opt in to large dynamic shared memory (per device); static + dynamic must stay within 227 KB
  static size_t configured[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && configured[dev] < smem) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<BN, KBOX, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return TPB_ERR_CUDA;
    configured[dev] = smem;
  }
  return launch_kernel(gemm_bf16_tcgen05_kernel<BN, KBOX, NACC>, dim3(grid), dim3(NUM_THREADS), smem, stream, ta, tb, p) == cudaSuccess
             ? TPB_OK
             : TPB_ERR_CUDA;
}

static int g_sm_count[16] = {0};
static int sm_count() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return 148;
  if (!g_sm_count[dev]) cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
  return g_sm_count[dev] ? g_sm_count[dev] : 148;
}

}  // namespace tpb

using namespace tpb;

// Measurement aids (0 restores the defaults): cap the smem ring depth, skip the MMAs.
extern "C" int tpb_gemm_debug(int stages, int skip_mma) {
  g_debug_stages = stages;
#ifdef TPB_GEMM_TRACE
  g_debug_skip_mma = skip_mma;
#else
  if (skip_mma) return TPB_ERR_ARG;  // compiled out of the product build
#endif
  return TPB_OK;
}
// Thresholds of the automatic split-K of few-tile weight-streaming GEMMs (KiB of weights per tile; <= 0 keeps a value).
extern "C" int tpb_bounds_checked(void) {
#ifdef TPB_BOUNDS
  return 1;
#else
  return 0;
#endif
}
extern "C" int tpb_gemm_tune_split(int min_tile_kb, int target_kb) {
  if (min_tile_kb > 0) g_split_min_kb = min_tile_kb;
  if (target_kb > 0) g_split_target_kb = target_kb;
  return TPB_OK;
}
// Bound, in seconds, of every wait for a peer GPU inside the GEMM kernels (a kernel that runs into it records a status
// code and returns).  Applies to launches made after the call.
extern "C" int tpb_set_wait_limit(double seconds) {
  if (!(seconds > 0)) return TPB_ERR_ARG;
  g_wait_ns = uint64_t(seconds * 1e9);
  return TPB_OK;
}

// Measurement aid: CTA `block` (>= 0) of every following GEMM launch records %globaltimer stamps of its phases
// (block < 0 switches it off).  tpb_gemm_trace_read copies the 32 stamps of the current device to the host
// (synchronous; call it after synchronising the stream).
// The cross-rank sum of few-token problems exchanges flagged words by default when there are at most 4 ranks.
// disable > 0: every following launch uses the arrival-counter protocol; disable < 0: flagged words at any rank count.
extern "C" int tpb_gemm_disable_flagged_exchange(int disable) {
  g_disable_ll = disable;
  return TPB_OK;
}
// Non-zero: tpb_gemm_plan deals the few-token shapes out as stream-K ranges (off by default, see tpb_gemm_plan).
extern "C" int tpb_gemm_enable_stream_k(int enable) {
  g_enable_stream_k = enable;
  return TPB_OK;
}
#ifdef TPB_GEMM_TRACE
extern "C" int tpb_gemm_trace(int block) {
  g_trace_block = block < 0 ? 0 : block + 1;
  return TPB_OK;
}
extern "C" int tpb_gemm_trace_read(unsigned long long* out32) {
  return cudaMemcpyFromSymbol(out32, g_gemm_trace, sizeof(unsigned long long) * 32) == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}
#else
extern "C" int tpb_gemm_trace(int) { return TPB_ERR_ARG; }
extern "C" int tpb_gemm_trace_read(unsigned long long*) { return TPB_ERR_ARG; }
#endif

// Loads every GEMM kernel on the current device.  With lazy module loading the first launch of a kernel may have to
// synchronise; host threads that each drive one GPU of a process call this before their kernels start waiting for
// one another.
extern "C" int tpb_gemm_preload(void) {
  cudaFuncAttributes attr;
  cudaError_t e = cudaSuccess;
#define LOAD(BN, KBOX, NACC) if (e == cudaSuccess) e = cudaFuncGetAttributes(&attr, gemm_bf16_tcgen05_kernel<BN, KBOX, NACC>)
  LOAD(16, 1, 8); LOAD(16, 2, 8); LOAD(16, 4, 8); LOAD(32, 1, 8); LOAD(32, 2, 8); LOAD(32, 4, 8);
  LOAD(64, 1, 2); LOAD(128, 1, 1); LOAD(256, 1, 1);
#undef LOAD
  return e == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

// Plan of a linear layer out[tokens, features] = x[tokens, K] @ w[features, K]^T.
// force_splits > 0 fixes the split-K factor; force_kbox > 0 fixes the k-blocks per stage (1, 2 or 4).
extern "C" int tpb_gemm_plan(int tokens, int features, int k, int world, int force_splits, int force_kbox,
                             tpb_gemm_plan_t* plan) {
  return tpb_gemm_plan_ex(tokens, features, k, world, force_splits, force_kbox, 0, plan);
}

// flags bit 0: keep the tokens on the tensor-core rows whatever their number (needed by MN-major operands).
extern "C" int tpb_gemm_plan_ex(int tokens, int features, int k, int world, int force_splits, int force_kbox, int flags,
                                tpb_gemm_plan_t* plan) {
  if (!plan || tokens <= 0 || features <= 0 || k <= 0) return TPB_ERR_ARG;
  const int sms = sm_count();
  plan->swapped = (tokens <= 64 && !(flags & 1)) ? 1 : 0;
  int bn;
  if (plan->swapped) {
    bn = tokens <= 16 ? 16 : (tokens <= 32 ? 32 : 64);
    plan->m_tiles = (features + BM - 1) / BM;
    plan->n_tiles = (tokens + bn - 1) / bn;
  } else {
    bn = features >= 256 ? 256 : ((features > 64 || (flags & 1)) ? 128 : 64);  // (MN-major operands: 128-wide tiles at least)
    // prefer 128-wide tiles when 256-wide ones would leave most SMs idle
    if (bn == 256 && ((tokens + BM - 1) / BM) * ((features + 255) / 256) < sms) bn = 128;
    plan->m_tiles = (tokens + BM - 1) / BM;
    plan->n_tiles = (features + bn - 1) / bn;
  }
  plan->bn = bn;
  int kbox = (bn <= 32) ? 4 : 1;  // decode-sized GEMMs are a pure weight stream: fetch 512 contiguous bytes per row
                                  // and stage (measured on B200: 4 boxes per stage stream ~15% faster than 1)
  if (force_kbox > 0) kbox = force_kbox;
  if (bn > 32 || (kbox != 1 && kbox != 2 && kbox != 4)) kbox = 1;
  const int tiles = plan->m_tiles * plan->n_tiles;
  const int kb64 = (k + BK - 1) / BK;
  plan->stream_k = 0;
  // Stream-K for the weight-streaming (swapped) shapes: the time of such a GEMM is bytes / (CTAs x per-CTA stream rate),
  // so what matters is that all SMs stream equal shares - whatever the number of 128-row tiles.  force_splits > 0
  // keeps the uniform decomposition (1 = no split at all).
  // OFF unless tpb_gemm_enable_stream_k(1): measured on B200 (CUDA-graph timing, 8 tokens) the streaming phase does
  // get shorter (4096 x 4096: accumulators complete after 7 us instead of 12 us), but the partial-tile exchange - park,
  // fence, counter, batched re-read - costs more than that on every shape tried (4096 x 4096: 18.9 vs 16.4 us,
  // 1536 x 4096: 16.6 vs 15.7 us, 4096 x 11008: 27.2 vs 28.1 us).
  if (plan->swapped && force_splits <= 0 && g_enable_stream_k) {
    if (force_kbox <= 0)
      while (kbox > 1 && (long long)tiles * ((kb64 + kbox - 1) / kbox) < 4LL * sms) kbox >>= 1;  // keep >= 4 units per CTA if possible
    const int kblocks = (kb64 + kbox - 1) / kbox;
    const long long units = (long long)tiles * kblocks;
    int grid = int(units / 2 < sms ? (units / 2 > 0 ? units / 2 : 1) : sms);
    if (!(tiles >= grid && tiles % grid == 0)) {  // (an exact multiple of the grid is balanced already)
      // a tile may not have more contributors than there are parking slots below the flagged-word area
      const int max_contrib = 8;  // two batches of the partial-tile sum; also bounds the parking slots (world + 8 <= 17)
      for (;;) {
        const long long per = units / grid;  // shortest range
        const int contrib = int((kblocks + per - 1) / per) + 1;
        if (contrib <= max_contrib || grid == 1) {
          plan->k_splits = contrib < 2 ? 2 : contrib;  // upper bound, sizes the workspace checks
          break;
        }
        --grid;
      }
      plan->stream_k = 1;
      plan->kbox = kbox;
      plan->k_blocks = kblocks;
      plan->kb_per_split = int((units + grid - 1) / grid);
      plan->reduce = 1;
      plan->grid = grid;
    }
  }
  if (!plan->stream_k) {
    plan->kbox = kbox;
    plan->k_blocks = (kb64 + kbox - 1) / kbox;  // in units of one pipeline stage (kbox * 64 columns)
    int splits = 1;
    const long long tile_kb = (long long)BM * k * 2 / 1024;  // weights one 128-row tile streams
    if (force_splits > 0) {
      splits = force_splits;
    } else if (plan->swapped && tiles * 4 <= sms && tile_kb >= g_split_min_kb) {
      // Few weight tiles (a tensor-parallel shard of a projection): the GEMM is a pure weight stream and takes
      // bytes / (CTAs x per-CTA stream rate) - one CTA pulls about 120 GB/s - so a handful of CTAs streaming 1 MB each
      // is slow however little data there is.  Split K so that most SMs stream a share of about g_split_target_kb; the
      // partials meet in the slot workspace and the last CTA of a tile to arrive sums them (one fence + one atomic,
      // nobody waits).  The exchange costs 3 to 4 us, which is why tiles under 1 MB and grids of more than a quarter of
      // the SMs are left whole (measured on B200 with the shard shapes of a Llama-2-7B layer at 1, 2, 4 and 8 ranks:
      // 8-way qkv 16.9 -> 13.7 us, gate|up 17.8 -> 15.7 us, head 17.0 -> 15.8 us; 2-way o_proj 13.1 -> 15.2 us if split).
      splits = sms / tiles;
      const int by_bytes = int((tile_kb + g_split_target_kb - 1) / g_split_target_kb);
      if (splits > by_bytes) splits = by_bytes;
      if (splits > 16) splits = 16;
      if (force_kbox <= 0)
        while (kbox > 1 && (kb64 + kbox - 1) / kbox < splits) kbox >>= 1;  // enough pipeline stages to deal out
      plan->kbox = kbox;
      plan->k_blocks = (kb64 + kbox - 1) / kbox;
      if (splits < 1) splits = 1;
    } else if (tiles * 2 <= sms && plan->k_blocks * kbox >= 128) {
      // few output tiles and a long K (>= 8192): split K so that more SMs work on the problem
      splits = sms / tiles;
      const int by_k = (plan->k_blocks * kbox) / 64;
      if (splits > by_k) splits = by_k;
      if (splits > 3) splits = 3;
      if (splits < 1) splits = 1;
    }
    if (splits > plan->k_blocks) splits = plan->k_blocks;
    int per = (plan->k_blocks + splits - 1) / splits;
    splits = (plan->k_blocks + per - 1) / per;  // no empty split
    plan->k_splits = splits;
    plan->kb_per_split = per;
    plan->reduce = (splits > 1 || world > 1) ? 1 : 0;
    const int work = tiles * splits;
    plan->grid = work < sms ? work : sms;
  }
  plan->tokens_pad = plan->swapped ? plan->n_tiles * bn : plan->m_tiles * BM;
  plan->slot_elems = size_t(tokens) * size_t(features);
  plan->tiles = tiles;
  return TPB_OK;
}

static int gemm_impl(const void* x, const void* w, void* out, const void* bias, const void* residual, int tokens,
                     int features, int k, int ldx, int ldw, int ld_out, int act, float bias_scale,
                     const tpb_gemm_plan_t* plan, const tpb_reduce_ctx_t* rc, const tpb_allgather_ctx_t* ag,
                     const tpb_gemm_opts_t* opts, void* stream_) {
  if (!x || !w || !out || !plan) return TPB_ERR_ARG;
  {
    // cuTensorMapEncodeTiled is a driver call and needs a context bound to THIS thread.  A thread that has made no
    // context-binding runtime call yet (an autograd worker whose first native call is this GEMM) has none:
    // cudaSetDevice binds the primary context of the device the runtime considers current.
    static thread_local int bound_device = -1;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return TPB_ERR_CUDA;
    if (bound_device != dev) {
      if (cudaSetDevice(dev) != cudaSuccess) return TPB_ERR_CUDA;
      bound_device = dev;
    }
  }
  const bool x_mn = opts && opts->x_mn, w_mn = opts && opts->w_mn;
  if ((x_mn || w_mn) && (plan->swapped || plan->kbox != 1 || plan->bn < 128 || ag)) return TPB_ERR_ARG;
  if (opts && opts->norm_mode) {
    if (!plan->swapped || !opts->norm_x || ((opts->norm_k > 0 ? opts->norm_k : k) & 7) || (opts->norm_ld & 7) || ((uintptr_t)opts->norm_x & 15) || tokens > 64 ||
        opts->norm_mode < 0 || opts->norm_mode > 2 || (rc && rc->world > 1 && plan->reduce) || ag)
      return TPB_ERR_ARG;
  }
  if (act == 5 && ((features & 31) || residual || (rc && rc->world > 1 && plan->reduce && rc->world != 1))) return TPB_ERR_ARG;
  if ((ldx & 7) || (ldw & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return TPB_ERR_ALIGN;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.swapped = plan->swapped;
  p.m_extent = plan->swapped ? features : tokens;
  p.n_extent = plan->swapped ? tokens : features;
  p.k_extent = k;
  p.m_tiles = plan->m_tiles;
  p.n_tiles = plan->n_tiles;
  p.k_blocks = plan->k_blocks;
  p.k_splits = plan->k_splits;
  p.kb_per_split = plan->kb_per_split;
  p.stream_k = plan->stream_k;
  p.wait_ns = (opts && opts->wait_seconds > 0) ? uint64_t(opts->wait_seconds * 1e9) : g_wait_ns;
  p.out_elems = (opts && opts->out_elems > 0) ? opts->out_elems : size_t(tokens - 1) * size_t(ld_out) + size_t(act == 5 ? features / 2 : features);
  p.a_mn = x_mn ? 1 : 0;  // (MN-major operands only exist in the normal orientation: A = tokens, B = features)
  p.b_mn = w_mn ? 1 : 0;
  if (opts && opts->norm_mode) {
    p.norm_mode = opts->norm_mode;
    p.norm_eps = opts->norm_eps;
    p.norm_x = static_cast<const __nv_bfloat16*>(opts->norm_x);
    p.norm_ld = opts->norm_ld;
    p.norm_k = opts->norm_k > 0 ? opts->norm_k : k;
    p.norm_rowsum = opts->norm_rowsum;
  }
  p.ld_out = ld_out;
  p.ld_slot = act == 5 ? features : ld_out;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.act = act;
  p.bias_scale = bias_scale;
  p.reduce = plan->reduce;
  p.world = 1;
  p.rank = 0;
  if (plan->reduce) {
    if (!rc || rc->world < 1 || rc->world > MAX_WORLD) return TPB_ERR_ARG;
    if (size_t(tokens) * size_t(act == 5 ? features : ld_out) > rc->slot_stride) return TPB_ERR_WORKSPACE;
    if (rc->world + plan->k_splits > rc->max_slots || plan->tiles > rc->max_tiles || !rc->split_counters) return TPB_ERR_WORKSPACE;
    p.world = rc->world;
    p.rank = rc->rank;
    for (int d = 0; d < rc->world; ++d) {
      p.slots[d] = static_cast<float*>(rc->slots[d]);
      p.arrivals[d] = static_cast<uint32_t*>(rc->arrivals[d]);
    }
    p.expected = static_cast<uint32_t*>(rc->expected);
    p.split_counters = static_cast<uint32_t*>(rc->split_counters);
    p.slot_stride = rc->slot_stride;
    p.status = static_cast<uint32_t*>(rc->status);
    // default: flagged words at every rank count for up to 16 tokens (with bf16 words, 8 ranks, 8 tokens, replayed from
    // a CUDA graph: 13.3 vs 16.1 us for the o_proj shard of a Llama-2-7B layer, 15.7 vs 20.8 us for down_proj); beyond
    // 16 tokens at more than 4 ranks a thread polls many words per row and the arrival counters stay the default.
    const bool ll_wanted = g_disable_ll < 0 || (g_disable_ll == 0 && (rc->world <= 4 || tokens <= 16));
    if (rc->world > 1 && plan->swapped && act != 5 && rc->ll_epochs && ll_wanted && rc->max_slots >= LL_FIRST_SLOT + 2 * rc->world &&
        rc->world + plan->k_splits <= LL_FIRST_SLOT && size_t(plan->tiles) * LL_TILE_WORDS <= rc->slot_stride / 2) {
      p.ll = 1;
      p.ll_epochs = static_cast<uint32_t*>(rc->ll_epochs);
      p.mc_slots = static_cast<float*>(rc->mc_slots);
    }
  } else {
    if (!rc || !rc->status) return TPB_ERR_ARG;
    p.status = static_cast<uint32_t*>(rc->status);
  }

  if (ag) {
    if (ag->world < 2 || ag->world > MAX_WORLD || plan->k_splits != 1 || ag->cols_local % (plan->kbox * BK) || (ag->cols_local & 7) ||
        ag->cols_local * ag->world != k || (ag->local_ld & 7) || ((uintptr_t)ag->local & 15))
      return TPB_ERR_ARG;
    p.ag_world = ag->world;
    p.ag_rank = ag->rank;
    p.ag_kb_per_rank = ag->cols_local / (plan->kbox * BK);
    p.ag_rows = tokens;
    p.ag_cols = ag->cols_local;
    p.ag_epoch = ag->epoch;
    p.ag_src = static_cast<const __nv_bfloat16*>(ag->local);
    p.ag_src_ld = ag->local_ld;
    p.ag_dst_ld = ldx;
    for (int d = 0; d < ag->world; ++d) {
      p.ag_dst[d] = static_cast<__nv_bfloat16*>(ag->gathered[d]);
      p.ag_flags[d] = static_cast<uint32_t*>(ag->flags[d]);
    }
    p.ag_push_counter = static_cast<uint32_t*>(ag->push_counter);
    p.ag_mc_dst = static_cast<__nv_bfloat16*>(ag->mc_gathered);
  }

  const void* a_ptr = plan->swapped ? w : x;
  const void* b_ptr = plan->swapped ? x : w;
  const int a_rows = p.m_extent, b_rows = p.n_extent;
  const int lda = plan->swapped ? ldw : ldx, ldb = plan->swapped ? ldx : ldw;
  CUtensorMap ta, tb;
  // K-major operand: [rows, k] with boxes of [box rows][64 k]; MN-major operand: [k, rows] with boxes of [64 k][64 rows]
  int rcode = p.a_mn ? make_tmap_2d(&ta, a_ptr, k, a_rows, lda, BK) : make_tmap_2d(&ta, a_ptr, a_rows, k, lda, BM);
  if (rcode != TPB_OK) return rcode;
  rcode = p.b_mn ? make_tmap_2d(&tb, b_ptr, k, b_rows, ldb, BK) : make_tmap_2d(&tb, b_ptr, b_rows, k, ldb, plan->bn);
  if (rcode != TPB_OK) return rcode;

  switch (plan->bn * 10 + plan->kbox) {
    case 161: return launch_gemm<16, 1, 8>(ta, tb, p, plan->grid, stream);
    case 162: return launch_gemm<16, 2, 8>(ta, tb, p, plan->grid, stream);
    case 164: return launch_gemm<16, 4, 8>(ta, tb, p, plan->grid, stream);
    case 321: return launch_gemm<32, 1, 8>(ta, tb, p, plan->grid, stream);
    case 322: return launch_gemm<32, 2, 8>(ta, tb, p, plan->grid, stream);
    case 324: return launch_gemm<32, 4, 8>(ta, tb, p, plan->grid, stream);
    case 641: return launch_gemm<64, 1, 2>(ta, tb, p, plan->grid, stream);
    case 1281: return launch_gemm<128, 1, 1>(ta, tb, p, plan->grid, stream);
    case 2561: return launch_gemm<256, 1, 1>(ta, tb, p, plan->grid, stream);
    default: return TPB_ERR_ARG;
  }
}

extern "C" int tpb_gemm_bf16(const void* x, const void* w, void* out, const void* bias, const void* residual, int tokens,
                             int features, int k, int ldx, int ldw, int ld_out, int act, float bias_scale,
                             const tpb_gemm_plan_t* plan, const tpb_reduce_ctx_t* rc, void* stream_) {
  return gemm_impl(x, w, out, bias, residual, tokens, features, k, ldx, ldw, ld_out, act, bias_scale, plan, rc, nullptr, nullptr, stream_);
}

// tpb_gemm_bf16 with options: operands given transposed in memory (x as [k, tokens], w as [k, features]: the backward
// GEMMs of a linear layer need no transpose kernel), a normalisation of x folded into the kernel, a wait bound.
extern "C" int tpb_gemm_bf16_ex(const void* x, const void* w, void* out, const void* bias, const void* residual, int tokens,
                                int features, int k, int ldx, int ldw, int ld_out, int act, float bias_scale,
                                const tpb_gemm_plan_t* plan, const tpb_reduce_ctx_t* rc, const tpb_gemm_opts_t* opts,
                                void* stream_) {
  return gemm_impl(x, w, out, bias, residual, tokens, features, k, ldx, ldw, ld_out, act, bias_scale, plan, rc, nullptr, opts, stream_);
}

// All-gather fused with the GEMM that consumes it: x is split by columns over the ranks; every rank passes its
// slice ag->local [tokens, ag->cols_local] and the kernel (1) pushes the slice into column block `rank` of every
// rank's gathered buffer ag->gathered[d] [tokens, k] (row pitch ld_gathered) with plain peer stores and signals,
// (2) multiplies gathered[rank] @ w^T, reading the k-blocks of the local slice first and each peer's slice as soon
// as its arrival word reaches ag->epoch.  TMA only ever reads this GPU's own memory.  The plan must come from
// tpb_gemm_plan(tokens, features, k, 1, 1, kbox) with cols_local % (kbox * 64) == 0.
extern "C" int tpb_gemm_allgather_bf16(const void* w, void* out, const void* bias, int tokens, int features, int k,
                                       int ld_gathered, int ldw, int ld_out, int act, const tpb_gemm_plan_t* plan,
                                       const tpb_reduce_ctx_t* rc, const tpb_allgather_ctx_t* ag, void* stream_) {
  if (!ag) return TPB_ERR_ARG;
  return gemm_impl(ag->gathered[ag->rank], w, out, bias, nullptr, tokens, features, k, ld_gathered, ldw, ld_out, act, 1.0f, plan, rc,
                   ag, nullptr, stream_);
}
