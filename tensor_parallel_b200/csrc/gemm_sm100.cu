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
// Structure of one CTA (192 threads), persistent over work items (m_tile, n_tile, k_split):
//   warp 0   : TMA producer  - cp.async.bulk.tensor loads of A/B k-blocks into a smem ring (no multicast)
//   warp 1   : MMA issuer    - one elected lane issues tcgen05.mma (K = 16 per instruction) into TMEM;
//                              tcgen05.commit releases smem stages and publishes finished accumulators
//   warps 2-5: epilogue      - tcgen05.ld the accumulator (two TMEM buffers, so the next tile's MMAs
//                              overlap this tile's epilogue), then either
//                                (direct)  add bias / residual, convert to bf16, store; or
//                                (reduce)  store the fp32 partial tile into slot [rank * k_splits + split]
//                                          of EVERY rank's workspace with plain peer stores, then bump
//                                          that tile's arrival counter on every rank (release, system scope).
//   Reduce mode, second phase (all warps): for each output tile this CTA owns, wait (bounded) until
//   world * k_splits partials have arrived, sum them in a fixed order (bit-identical on all ranks),
//   add bias / residual and store bf16.  All of a CTA's pushes precede its first wait, and the grid is
//   never larger than what is co-resident, so ranks cannot deadlock each other.
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
  // fused all-gather of the token-side operand (ag_world > 1): every rank owns a column slice [rows, ag_cols] of x;
  // the kernel first pushes its slice into every rank's gathered buffer, then consumes k-blocks slice by slice
  // (own slice first) as the peers' pushes arrive
  int ag_world, ag_rank, ag_kb_per_rank, ag_rows, ag_cols;
  uint32_t ag_epoch;                          // flags of this call reach at least this value
  const __nv_bfloat16* ag_src;                // local slice
  long long ag_src_ld, ag_dst_ld;
  __nv_bfloat16* ag_dst[MAX_WORLD];           // every rank's gathered buffer [rows, ag_world * ag_cols]
  uint32_t* ag_flags[MAX_WORLD];              // every rank's arrival words [ag_world], indexed by source rank
  uint32_t* ag_push_counter;                  // local: CTAs done pushing (self re-arming)
  int debug_skip_mma;             // measurement aid: stream the operands through the smem ring without issuing MMAs
  int trace_block;                // measurement aid: CTA (index + 1) that records %globaltimer stamps into g_gemm_trace; 0 = off
};

// %globaltimer stamps of one CTA of the most recent traced launch (see tpb_gemm_trace):
// 0 entry, 1 setup done, 2 first accumulator ready, 3 partial stored / pushed, 4 system fence + barrier passed,
// 5 arrival counters bumped, 6 reduce phase entered, 7 all arrivals seen, 8 reduced tile written.
__device__ unsigned long long g_gemm_trace[16];
#define TPB_TRACE(i)                                                                         \
  do {                                                                                       \
    if (p.trace_block && int(blockIdx.x) == p.trace_block - 1) g_gemm_trace[i] = globaltimer_ns(); \
  } while (0)


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

// KBOX = number of consecutive 64-column k-blocks fetched per pipeline stage.  With KBOX > 1 a stage
// pulls KBOX * 128 contiguous bytes of every operand row in back-to-back TMA boxes.
// NACC = number of independent TMEM accumulators per tile.  Consecutive tcgen05.mma instructions that
// accumulate into the same TMEM columns serialise on the accumulator; at N = 16 / 32 one instruction is
// far shorter than that dependent latency, so the k-steps are dealt round-robin to NACC accumulators that
// the epilogue adds up.  (At N >= 64 one accumulator keeps the tensor pipe busy.)
template <int BN, int KBOX, int NACC>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const GemmParams p) {
  constexpr uint32_t A_BYTES = BM * BK * 2;
  constexpr uint32_t B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = KBOX * (A_BYTES + B_BYTES);
  constexpr uint32_t ACC_COLS = NACC * BN;                                  // columns of one accumulator set
  constexpr uint32_t TMEM_COLS = (2 * ACC_COLS < 32) ? 32 : 2 * ACC_COLS;   // two sets; power of two by construction
  static_assert(TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "TMEM allocation must be a power of two <= 512");
  constexpr uint32_t IDESC = make_idesc_bf16(BM, BN);
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
  pdl_trigger();  // the next kernel in the stream may start its own prologue now
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();     // everything below reads what earlier kernels wrote
  if (threadIdx.x == 0) TPB_TRACE(1);

  const int tiles = p.m_tiles * p.n_tiles;
  const int work_items = tiles * p.k_splits;

  if (p.ag_world > 1) {
    // ---------------- all-gather push: local slice -> every rank's gathered buffer ----------------
    const int vec_per_row = p.ag_cols >> 3;
    const long long total = (long long)p.ag_rows * vec_per_row;
    for (long long i = blockIdx.x * (long long)NUM_THREADS + threadIdx.x; i < total; i += (long long)gridDim.x * NUM_THREADS) {
      const long long r = i / vec_per_row;
      const int c = int(i % vec_per_row) * 8;
      const uint4 val = *reinterpret_cast<const uint4*>(p.ag_src + r * p.ag_src_ld + c);
#pragma unroll
      for (int d = 0; d < MAX_WORLD; ++d)
        if (d < p.ag_world) *reinterpret_cast<uint4*>(p.ag_dst[d] + r * p.ag_dst_ld + p.ag_rank * p.ag_cols + c) = val;
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
      for (int w = blockIdx.x; w < work_items && !*abort_flag; w += gridDim.x) {
        const int split = w / tiles;
        const int tile = w - split * tiles;
        const int mt = tile % p.m_tiles;
        const int nt = tile / p.m_tiles;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
        int ag_ready_src = -1;
        for (int kb_seq = kb0; kb_seq < kb1; ++kb_seq, ++it) {
          int kb = kb_seq;
          if (p.ag_world > 1) {
            // start with the k-blocks of the local slice, then walk the other ranks' slices as they arrive
            kb = (kb_seq + p.ag_rank * p.ag_kb_per_rank) % p.k_blocks;
            const int src = kb / p.ag_kb_per_rank;
            if (src != ag_ready_src) {
              if (!wait_flag_ge(p.ag_flags[p.ag_rank] + src, p.ag_epoch)) {
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
#pragma unroll
          for (int j = 0; j < KBOX; ++j)  // columns past K are filled with zeros by TMA and cost no DRAM traffic
            tma_load_2d(a_dst + j * A_BYTES, &tmap_a, &full_bar[s], (kb * KBOX + j) * BK, mt * BM);
#pragma unroll
          for (int j = 0; j < KBOX; ++j)
            tma_load_2d(b_dst + j * B_BYTES, &tmap_b, &full_bar[s], (kb * KBOX + j) * BK, nt * BN);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      uint32_t it = 0;
      uint32_t local = 0;
      for (int w = blockIdx.x; w < work_items && !*abort_flag; w += gridDim.x, ++local) {
        const int split = w / tiles;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
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
          if (p.debug_skip_mma) {
            issued += MMAS_PER_STAGE;
            if (kb + 1 < kb1) { mbar_arrive(&empty_bar[s]); continue; }
          }
#pragma unroll
          for (int j = 0; j < KBOX; ++j) {
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              const uint64_t adesc = make_desc_kmajor_sw128(a_addr + j * A_BYTES + kk * UMMA_K * 2);
              const uint64_t bdesc = make_desc_kmajor_sw128(b_addr + j * B_BYTES + kk * UMMA_K * 2);
              umma_bf16(d_tmem + (issued % NACC) * BN, adesc, bdesc, IDESC, issued >= NACC ? 1u : 0u);
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
    uint32_t local = 0;
    for (int w = blockIdx.x; w < work_items; w += gridDim.x, ++local) {
      const int split = w / tiles;
      const int tile = w - split * tiles;
      const int mt = tile % p.m_tiles;
      const int nt = tile / p.m_tiles;
      const int acc = local & 1;
      const uint32_t acc_ph = (local >> 1) & 1;
      // one thread waits, the group agrees on the outcome (so that nobody is left at a named barrier)
      if (threadIdx.x == 64) {
        bool ok = !*abort_flag && mbar_wait(&acc_full[acc], acc_ph);
        if (!ok) {
          atomicMax(p.status, STATUS_TIMEOUT_MBAR);
          *abort_flag = 1;
        }
        *epi_ok = ok ? 1u : 0u;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
      if (!*epi_ok) break;
      tc_fence_after();
      if (threadIdx.x == 64) TPB_TRACE(2);
      const int m = mt * BM + row;
      const bool m_ok = m < p.m_extent;
      const uint32_t t_lane = tmem_base + (uint32_t(quarter * 32) << 16) + acc * ACC_COLS;
      const int kb0 = split * p.kb_per_split;
      const int n_mma = (min(p.k_blocks, kb0 + p.kb_per_split) - kb0) * MMAS_PER_STAGE;
      const int n_acc = n_mma < NACC ? n_mma : NACC;  // accumulators that were written for this item

      // A chunk is 16 accumulator columns of this thread's row: (token m, features n0..n0+15) in the normal
      // orientation, (feature m, tokens n0..n0+15) in the swapped one.  idx(j) addresses out[token, feature].
      auto chunk_valid = [&](int n0) { return m_ok && n0 < p.n_extent; };
      auto read_acc = [&](int c0, float (&v)[16]) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.f;
#pragma unroll
        for (int a = 0; a < NACC; ++a) {
          if (a < n_acc) {
            uint32_t r[16];
            tmem_ld_x16(t_lane + a * BN + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] += __uint_as_float(r[j]);
          }
        }
      };
      auto store_partial = [&](float* slot, int n0, const float (&v)[16]) {
        if (!chunk_valid(n0)) return;
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
      auto add_partial = [&](const float* slot, int n0, float (&v)[16]) {
        if (!chunk_valid(n0)) return;
        if (!p.swapped) {
          const size_t base = size_t(m) * p.ld_slot + n0;
          if (n0 + 16 <= p.n_extent && (p.ld_slot & 3) == 0) {
            const float4* src = reinterpret_cast<const float4*>(slot + base);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float4 t = __ldcg(src + q);
              v[4 * q] += t.x; v[4 * q + 1] += t.y; v[4 * q + 2] += t.z; v[4 * q + 3] += t.w;
            }
          } else {
            for (int j = 0; j < 16 && n0 + j < p.n_extent; ++j) v[j] += __ldcg(slot + base + j);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (n0 + j < p.n_extent) v[j] += __ldcg(slot + size_t(n0 + j) * p.ld_slot + m);
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
          uint4* op = reinterpret_cast<uint4*>(p.out + base);
          op[0] = o0;
          op[1] = o1;
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) p.out[base + j] = __float2bfloat16(o[j]);
        }
      };
      auto finalize = [&](int n0, float (&v)[16]) {  // bias, activation, residual, bf16 store
        if (!chunk_valid(n0)) return;
        if (p.act == 5) {
          // gated silu, swapped orientation: lanes 0-15 of a warp hold gate rows, lanes 16-31 the matching up rows
          const float b = p.bias ? p.bias_scale * __bfloat162float(p.bias[m]) : 0.f;
          const int f_out = (m >> 5) * 16 + (m & 15);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float x = v[j] + b;
            const float partner = __shfl_xor_sync(0xffffffffu, x, 16);
            if ((lane & 16) == 0 && n0 + j < p.n_extent)
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
            uint4* op = reinterpret_cast<uint4*>(p.out + base);
            op[0] = o0;
            op[1] = o1;
          } else {
            for (int j = 0; j < 16 && n0 + j < p.n_extent; ++j) {
              float x = v[j] + (p.bias ? p.bias_scale * __bfloat162float(p.bias[n0 + j]) : 0.f);
              x = apply_act(x, p.act);
              if (p.residual) x += __bfloat162float(p.residual[base + j]);
              p.out[base + j] = __float2bfloat16(x);
            }
          }
        } else {
          const float b = p.bias ? p.bias_scale * __bfloat162float(p.bias[m]) : 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (n0 + j < p.n_extent) {
              float x = apply_act(v[j] + b, p.act);
              const size_t idx = size_t(n0 + j) * p.ld_out + m;
              if (p.residual) x += __bfloat162float(p.residual[idx]);
              p.out[idx] = __float2bfloat16(x);
            }
          }
        }
      };
      auto push_to_peers = [&](int n0, const float (&v)[16]) {  // this rank's (split-reduced) partial -> slot[rank] everywhere
#pragma unroll
        for (int d = 0; d < MAX_WORLD; ++d)
          if (d < p.world) store_partial(p.slots[d] + size_t(p.rank) * p.slot_stride, n0, v);
      };

      const bool split_k = p.k_splits > 1;
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
            if (p.world > 1) push_to_peers(nt * BN + c0, v);
            else finalize(nt * BN + c0, v);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);  // accumulators may be overwritten from here on
      } else {
        // split-K: park the partial in a local slot; the LAST split to arrive for this tile adds them up in split
        // order (deterministic) and carries on - nobody ever waits for another CTA.
        float* my_slot = p.slots[p.rank] + size_t(p.world + split) * p.slot_stride;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          float v[16];
          read_acc(c0, v);
          store_partial(my_slot, nt * BN + c0, v);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        __threadfence();
        asm volatile("bar.sync 2, %0;" ::"n"(EPI_THREADS) : "memory");
        if (threadIdx.x == 64) {
          const uint32_t old = atomicAdd(p.split_counters + tile, 1u);
          const bool last = old == uint32_t(p.k_splits - 1);
          if (last) p.split_counters[tile] = 0;  // every other split has arrived: safe to re-arm for the next call
          *epi_last = last ? 1u : 0u;
        }
        asm volatile("bar.sync 2, %0;" ::"n"(EPI_THREADS) : "memory");
        if (*epi_last) {
          __threadfence();
          if (gated_cols) {
            if constexpr (BN >= 32) {
#pragma unroll 1
              for (int c0 = 0; c0 < BN; c0 += 32) {
                float vg[16], vu[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) { vg[j] = 0.f; vu[j] = 0.f; }
                for (int sp = 0; sp < p.k_splits; ++sp) {
                  add_partial(p.slots[p.rank] + size_t(p.world + sp) * p.slot_stride, nt * BN + c0, vg);
                  add_partial(p.slots[p.rank] + size_t(p.world + sp) * p.slot_stride, nt * BN + c0 + 16, vu);
                }
                finalize_gated(nt * BN + c0, vg, vu);
              }
            }
          } else {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
              float v[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = 0.f;
              for (int sp = 0; sp < p.k_splits; ++sp)
                add_partial(p.slots[p.rank] + size_t(p.world + sp) * p.slot_stride, nt * BN + c0, v);
              if (p.world > 1) push_to_peers(nt * BN + c0, v);
              else finalize(nt * BN + c0, v);
            }
          }
        }
      }
      if (p.world > 1 && (!split_k || *epi_last)) {
        // make this tile's partial visible system-wide, then count one arrival on every rank
        if (threadIdx.x == 64) TPB_TRACE(3);
        __threadfence_system();
        asm volatile("bar.sync 2, %0;" ::"n"(EPI_THREADS) : "memory");
        if (threadIdx.x == 64) {
          TPB_TRACE(4);
          __threadfence_system();  // one release fence for all peers (orders the partial tiles the barrier made visible)
          for (int d = 0; d < p.world; ++d) red_add_relaxed_sys(p.arrivals[d] + tile, 1u);
          TPB_TRACE(5);
        }
      }
    }
  }

  // ---------------- cross-rank reduce phase ----------------
  __syncthreads();
  if (p.world > 1) {
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
        bool ok = !*abort_flag && wait_flag_ge(p.arrivals[p.rank] + tile, target);
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
              x = apply_act(x, p.act);
              if (p.residual) x += __bfloat162float(p.residual[idx + j]);
              p.out[idx + j] = __float2bfloat16(x);
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
  return r == CUDA_SUCCESS ? TPB_OK : TPB_ERR_TMAP;
}

static int g_debug_stages = 0, g_debug_skip_mma = 0, g_trace_block = 0;  // measurement aids, see tpb_gemm_debug

template <int BN, int KBOX, int NACC>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, int grid, cudaStream_t stream) {
  constexpr size_t stage_bytes = size_t(KBOX) * size_t(BM * BK * 2 + BN * BK * 2);
  int stages = int((227 * 1024 - 2048) / stage_bytes);
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (stages < 2) stages = 2;
  if (stages > p.kb_per_split + 1 && p.m_tiles * p.n_tiles * p.k_splits <= grid) stages = max(2, p.kb_per_split + 1);
  if (g_debug_stages > 0 && g_debug_stages < stages) stages = g_debug_stages;
  p.stages = stages;
  p.debug_skip_mma = g_debug_skip_mma;
  p.trace_block = g_trace_block;
  size_t smem = stages * stage_bytes + 1024 /*align*/ + (2 * MAX_STAGES + 4) * 8 + 16;
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
  g_debug_skip_mma = skip_mma;
  return TPB_OK;
}

// Measurement aid: CTA `block` (>= 0) of every following GEMM launch records %globaltimer stamps of its phases
// (block < 0 switches it off).  tpb_gemm_trace_read copies the 16 stamps of the current device to the host
// (synchronous; call it after synchronising the stream).
extern "C" int tpb_gemm_trace(int block) {
  g_trace_block = block < 0 ? 0 : block + 1;
  return TPB_OK;
}
extern "C" int tpb_gemm_trace_read(unsigned long long* out16) {
  return cudaMemcpyFromSymbol(out16, g_gemm_trace, sizeof(unsigned long long) * 16) == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

// Plan of a linear layer out[tokens, features] = x[tokens, K] @ w[features, K]^T.
// force_splits > 0 fixes the split-K factor; force_kbox > 0 fixes the k-blocks per stage (1, 2 or 4).
extern "C" int tpb_gemm_plan(int tokens, int features, int k, int world, int force_splits, int force_kbox,
                             tpb_gemm_plan_t* plan) {
  if (!plan || tokens <= 0 || features <= 0 || k <= 0) return TPB_ERR_ARG;
  const int sms = sm_count();
  plan->swapped = tokens <= 64 ? 1 : 0;
  int bn;
  if (plan->swapped) {
    bn = tokens <= 16 ? 16 : (tokens <= 32 ? 32 : 64);
    plan->m_tiles = (features + BM - 1) / BM;
    plan->n_tiles = (tokens + bn - 1) / bn;
  } else {
    bn = features >= 256 ? 256 : (features > 64 ? 128 : 64);
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
  plan->kbox = kbox;
  plan->k_blocks = ((k + BK - 1) / BK + kbox - 1) / kbox;  // in units of one pipeline stage (kbox * 64 columns)
  const int tiles = plan->m_tiles * plan->n_tiles;
  int splits = 1;
  if (force_splits > 0) {
    splits = force_splits;
  } else if (tiles * 2 <= sms && plan->k_blocks * kbox >= 128) {
    // few output tiles and a long K (>= 8192): split K so that more SMs stream weights.  Measured on B200 (kernel
    // time inside a CUDA graph): for shorter K the extra partial-tile pass costs more than the added SMs bring.
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
  plan->tokens_pad = plan->swapped ? plan->n_tiles * bn : plan->m_tiles * BM;
  plan->slot_elems = size_t(tokens) * size_t(features);
  plan->tiles = tiles;
  return TPB_OK;
}

static int gemm_impl(const void* x, const void* w, void* out, const void* bias, const void* residual, int tokens,
                     int features, int k, int ldx, int ldw, int ld_out, int act, float bias_scale,
                     const tpb_gemm_plan_t* plan, const tpb_reduce_ctx_t* rc, const tpb_allgather_ctx_t* ag, void* stream_) {
  if (!x || !w || !out || !plan) return TPB_ERR_ARG;
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
  }

  const void* a_ptr = plan->swapped ? w : x;
  const void* b_ptr = plan->swapped ? x : w;
  const int a_rows = p.m_extent, b_rows = p.n_extent;
  const int lda = plan->swapped ? ldw : ldx, ldb = plan->swapped ? ldx : ldw;
  CUtensorMap ta, tb;
  int rcode = make_tmap_2d(&ta, a_ptr, a_rows, k, lda, BM);
  if (rcode != TPB_OK) return rcode;
  rcode = make_tmap_2d(&tb, b_ptr, b_rows, k, ldb, plan->bn);
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
  return gemm_impl(x, w, out, bias, residual, tokens, features, k, ldx, ldw, ld_out, act, bias_scale, plan, rc, nullptr, stream_);
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
                   ag, stream_);
}
