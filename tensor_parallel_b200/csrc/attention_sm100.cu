// Flash-style attention forward for sm_100a on tcgen05 tensor cores.  Two kernels:
//   attn_fwd_pingpong_kernel (further down): two query tiles per CTA, the default for more than 128 queries
//   attn_fwd_tcgen05_kernel  (first)       : one query tile per CTA, for short query sequences
//
// attn_fwd_tcgen05_kernel: one CTA per (batch, query head, 128-query tile); keys / values stream through in tiles of 128:
//
//   warp 0   : TMA producer  - Q once, then K / V tiles into a 2-deep shared-memory ring (4-D tensor maps over the
//                              caller's strided [batch, seq, head, head_dim] views; no multicast)
//   warp 1   : MMA issuer    - S = Q K^T  (tcgen05.mma, M = 128 queries, N = 128 keys, both operands K-major) into one of
//                              two TMEM score buffers, and O_tile = P V (A = P from shared memory, B = V read MN-major as it
//                              lies in memory) into a TMEM output tile; QK of tile j + 1 is issued BEFORE the wait for the
//                              probabilities of tile j, so the tensor core works on the next scores while the softmax
//                              warps are busy
//   warps 2-9: softmax       - two threads per query row (= TMEM lane), one per half of the tile's 128 keys and of the
//                              head dimension, so that every SM scheduler has two softmax warps to hide TMEM and MUFU
//                              latency with.  Pass 1 reads the scores from TMEM, applies scale / bias / masks (tiles that
//                              need them write the result back) and takes the row maximum, which the two halves exchange
//                              through shared memory; then the previous tile's P V product is folded into the fp32 output
//                              registers (o = o * alpha + O_tile: the running output never lives in TMEM, so nothing there
//                              is ever rescaled); pass 2 exponentiates, sums, and stores the bf16 probabilities into
//                              shared memory in the 128-byte-swizzled K-major layout the tensor core reads.
//
// TMEM: scores 2 x 128 columns, output tile head_dim columns (512 allocated).  Shared memory at head_dim 128:
// Q 32 KB + 2 x (K 32 KB + V 32 KB) + P 32 KB = 192 KB.  Every mbarrier wait is bounded; on expiry the CTA records a
// status code and drains.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>

#include "attention_sm100.cuh"
#include "ptx_sm100.cuh"
#include "tpb_api.h"

namespace tpb {

typedef __nv_bfloat16 bf16;

constexpr int FA_M = 128;        // queries per CTA
constexpr int FA_N = 128;        // keys per tile
constexpr int FA_SOFTMAX_WARPS = 8;
constexpr int FA_THREADS = 64 + 32 * FA_SOFTMAX_WARPS;  // producer warp, MMA warp, eight softmax warps

struct FaParams {
  int sq, sk, q_heads, kv_heads, causal;
  float scale_log2e;
  bf16* out;
  long long o_sb, o_ss, o_sh;
  float* lse;
  const void* bias;  // additive score bias in natural-log units, -inf masks a key; element strides, 0 broadcasts
  int bias_kind;     // 0 none, 1 fp32, 2 bf16
  long long bias_sb, bias_sh, bias_sq, bias_sk;
  uint32_t* status;
};

template <int D>
__global__ void __launch_bounds__(FA_THREADS, 1)
attn_fwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  constexpr int DB = D / 64;                          // 64-wide blocks of the head dimension
  constexpr uint32_t Q_BYTES = DB * FA_BLOCK_BYTES;   // Q tile = K tile = V tile
  constexpr uint32_t P_BYTES = 2 * FA_BLOCK_BYTES;    // 128 x 128 probabilities
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COLS = FA_N, O_COL0 = 2 * FA_N;
  constexpr uint32_t IDESC_QK = make_idesc_bf16(FA_M, FA_N, false, false);
  constexpr uint32_t IDESC_PV = make_idesc_bf16(FA_M, D, false, true);

  extern __shared__ uint8_t fa_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* k_s = q_s + Q_BYTES;          // [2 stages]
  uint8_t* v_s = k_s + 2 * Q_BYTES;      // [2 stages]
  uint8_t* p_s = v_s + 2 * Q_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;     // [2]
  uint64_t* p_full = bars + 7;
  uint64_t* o_full = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* row_stat = reinterpret_cast<float*>(tmem_slot + 2);  // [2 sets][2 halves][128 rows]: row maxima, at the end row sums

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qblk = gridDim.x - 1 - blockIdx.x;  // heavy (late) causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.q_heads / p.kv_heads);
  const int q0 = qblk * FA_M;
  const int shift = p.sk - p.sq;  // query i may see keys j <= i + shift when causal
  int kv_end = p.sk;
  if (p.causal) kv_end = min(p.sk, q0 + FA_M + shift);
  const int n_tiles = kv_end > 0 ? (kv_end + FA_N - 1) / FA_N : 0;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
      mbar_init(&s_full[s], 1);
    }
    mbar_init(p_full, FA_SOFTMAX_WARPS);  // one arrival per softmax warp
    mbar_init(o_full, 1);
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

  auto give_up = [&](uint32_t code) {
    atomicMax(p.status, code);
    *abort_flag = 1;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one() && n_tiles > 0) {
      mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int d = 0; d < DB; ++d) tma_load_4d(q_s + d * FA_BLOCK_BYTES, &tmap_q, q_full, d * 64, q0, h, b);
      for (int j = 0; j < n_tiles && !*abort_flag; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1)) { give_up(STATUS_TIMEOUT_MBAR); break; }
        mbar_expect_tx(&kv_full[s], 2 * Q_BYTES);
#pragma unroll
        for (int d = 0; d < DB; ++d) {
          tma_load_4d(k_s + s * Q_BYTES + d * FA_BLOCK_BYTES, &tmap_k, &kv_full[s], d * 64, j * FA_N, kvh, b);
          tma_load_4d(v_s + s * Q_BYTES + d * FA_BLOCK_BYTES, &tmap_v, &kv_full[s], d * 64, j * FA_N, kvh, b);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one() && n_tiles > 0) {
      const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s);
      auto issue_qk = [&](int j) {  // S[j & 1] = Q K(j)^T
        const uint32_t k_addr = smem_u32(k_s + (j & 1) * Q_BYTES);
        const uint32_t d_tmem = tmem_base + (j & 1) * S_COLS;
#pragma unroll
        for (int d = 0; d < DB; ++d) {
#pragma unroll
          for (int kk = 0; kk < 64 / 16; ++kk) {
            const uint64_t adesc = make_desc_kmajor_sw128(q_addr + d * FA_BLOCK_BYTES + kk * 32);
            const uint64_t bdesc = make_desc_kmajor_sw128(k_addr + d * FA_BLOCK_BYTES + kk * 32);
            umma_bf16(d_tmem, adesc, bdesc, IDESC_QK, (d | kk) ? 1u : 0u);
          }
        }
        umma_commit(&s_full[j & 1]);
      };
      bool ok = mbar_wait(q_full, 0) && mbar_wait(&kv_full[0], 0);
      if (!ok) give_up(STATUS_TIMEOUT_MBAR);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; ok && j < n_tiles && !*abort_flag; ++j) {
        if (j + 1 < n_tiles) {
          // scores of the next tile: the softmax warps finished with this TMEM buffer when they delivered P(j - 1),
          // which PV(j - 1) below waited for
          if (!mbar_wait(&kv_full[(j + 1) & 1], ((j + 1) >> 1) & 1)) { give_up(STATUS_TIMEOUT_MBAR); break; }
          tc_fence_after();
          issue_qk(j + 1);
        }
        if (!mbar_wait(p_full, j & 1)) { give_up(STATUS_TIMEOUT_MBAR); break; }
        tc_fence_after();
        // O_tile = P(j) V(j): V tile [128 keys][D] is the MN-major B operand (N = head_dim contiguous)
        const uint32_t v_addr = smem_u32(v_s + (j & 1) * Q_BYTES);
#pragma unroll
        for (int kk = 0; kk < FA_N / 16; ++kk) {
          const uint64_t adesc = make_desc_kmajor_sw128(p_addr + (kk >> 2) * FA_BLOCK_BYTES + (kk & 3) * 32);
          const uint64_t bdesc = make_desc_mnmajor_sw128(v_addr + kk * 16 * 128, FA_BLOCK_BYTES);
          umma_bf16(tmem_base + O_COL0, adesc, bdesc, IDESC_PV, kk ? 1u : 0u);
        }
        umma_commit(o_full);
        umma_commit(&kv_empty[j & 1]);  // K(j) and V(j) may be overwritten once these MMAs retire
      }
    }
  } else {
    // ---------------- softmax warps ----------------
    constexpr int HN = FA_N / 2;   // keys per thread and tile
    constexpr int HD = D / 2;      // output columns per thread
    const int quarter = warp & 3;  // TMEM lane quarter this warp may access
    const int half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int qi = q0 + row;
    const uint32_t t_lane = tmem_base + (uint32_t(quarter * 32) << 16);
    float o_reg[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o_reg[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 1.f;
    const float* bias_f = static_cast<const float*>(p.bias);
    const bf16* bias_h = static_cast<const bf16*>(p.bias);
    const long long bias_row = p.bias_kind ? (b * p.bias_sb + h * p.bias_sh + (long long)min(qi, p.sq - 1) * p.bias_sq) : 0;
    bool alive = true;

    // o = o * alpha + O_tile (this thread's half of the head dimension), two columns per instruction
    auto fold_output = [&](float alpha) {
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        uint32_t t[32];
        tmem_ld_x32(t_lane + O_COL0 + half * HD + c, t);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          ffma2(o_reg[c + i], o_reg[c + i + 1], o_reg[c + i], o_reg[c + i + 1], alpha, alpha, __uint_as_float(t[i]), __uint_as_float(t[i + 1]));
      }
    };
    // The two threads of a row meet at a barrier of their own two warps.  Every softmax thread takes part in every such
    // barrier, whatever happened before: a thread that gave up keeps arriving (with neutral values), so that nobody is
    // left waiting.
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory"); };

    for (int j = 0; j < n_tiles; ++j) {
      if (alive && (*abort_flag || !mbar_wait(&s_full[j & 1], (j >> 1) & 1))) {
        if (!*abort_flag) give_up(STATUS_TIMEOUT_MBAR);
        alive = false;
      }
      tc_fence_after();
      const uint32_t s_addr = t_lane + (j & 1) * S_COLS + half * HN;
      const int key0 = j * FA_N + half * HN;
      // only tiles that touch the diagonal, the end of the keys or a bias need per-element work
      const bool plain = !p.bias_kind && j * FA_N + FA_N <= p.sk && (!p.causal || j * FA_N + FA_N - 1 <= q0 + shift);
      // ---- pass 1: this half's scores come out of TMEM once and stay in registers; row maximum ----
      uint32_t r[HN];
      float m_half = -INFINITY;
      if (alive) {
#pragma unroll
        for (int c = 0; c < HN; c += 32) tmem_ld_x32(s_addr + c, *reinterpret_cast<uint32_t(*)[32]>(r + c));
        tmem_ld_wait();
        if (plain) {
#pragma unroll
          for (int i = 0; i < HN; i += 2) m_half = fmax3(m_half, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
          m_half *= p.scale_log2e;  // (the scale is positive: the maximum commutes with it)
        } else {
#pragma unroll
          for (int i = 0; i < HN; ++i) {
            const int key = key0 + i;
            const bool dead = key >= p.sk || (p.causal && key > qi + shift);
            float sv = dead ? -INFINITY : __uint_as_float(r[i]) * p.scale_log2e;
            if (p.bias_kind && !dead) {
              const long long bi = bias_row + (long long)key * p.bias_sk;
              const float bv = p.bias_kind == 1 ? __ldg(bias_f + bi) : __bfloat162float(bias_h[bi]);
              sv += bv * 1.4426950408889634f;
            }
            r[i] = __float_as_uint(sv);
            m_half = fmaxf(m_half, sv);
          }
        }
      }
      float* stat = row_stat + (j & 1) * 2 * FA_M;  // (two sets, so that one barrier per tile is enough)
      stat[half * FA_M + row] = m_half;
      pair_sync();
      const float m_new = fmax3(m_run, m_half, stat[(half ^ 1) * FA_M + row]);
      const float base = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = m_run == -INFINITY ? 0.f : ex2_approx(m_run - base);
      // ---- fold the previous tile's P V into the output registers (also: P(j - 1) has been consumed) ----
      if (alive && j > 0) {
        if (!mbar_wait(o_full, (j - 1) & 1)) {
          give_up(STATUS_TIMEOUT_MBAR);
          alive = false;
        } else {
          tc_fence_after();
          fold_output(alpha_prev);
        }
      }
      // ---- pass 2: probabilities -> shared memory (K-major, 128-byte swizzle: chunk c of row r sits at c ^ (r & 7)) ----
      if (alive) {
        float sum0 = 0.f, sum1 = 0.f;
        uint8_t* p_row = p_s + half * FA_BLOCK_BYTES + row * 128;  // this half's 64 keys are one swizzled block
        const float mul = plain ? p.scale_log2e : 1.f;
        const float nbase = -base;
#pragma unroll
        for (int c = 0; c < HN; c += 8) {  // one 16-byte chunk of eight keys
          uint32_t packed[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float t0, t1;
            ffma2(t0, t1, __uint_as_float(r[c + 2 * i]), __uint_as_float(r[c + 2 * i + 1]), mul, mul, nbase, nbase);
            const float p0 = ex2_approx(t0), p1 = ex2_approx(t1);
            fadd2(sum0, sum1, sum0, sum1, p0, p1);
            packed[i] = pack_bf16x2(p0, p1);
          }
          *reinterpret_cast<uint4*>(p_row + ((((c >> 3)) ^ (row & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
        l_run = l_run * alpha + (sum0 + sum1);
      }
      m_run = m_new;
      alpha_prev = alpha;
      tc_fence_before();
      fence_proxy_async_smem();  // the probabilities must be visible to the tensor core's shared-memory reads
      __syncwarp();
      if (lane == 0 && alive) mbar_arrive(p_full);
    }
    if (alive && n_tiles > 0) {
      if (mbar_wait(o_full, (n_tiles - 1) & 1)) {
        tc_fence_after();
        fold_output(alpha_prev);
      } else {
        give_up(STATUS_TIMEOUT_MBAR);
        alive = false;
      }
    }
    // the two halves of a row add up their sums
    float* stat = row_stat + (n_tiles & 1) * 2 * FA_M;
    stat[half * FA_M + row] = l_run;
    pair_sync();
    l_run += stat[(half ^ 1) * FA_M + row];
    if (alive && qi < p.sq) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      bf16* orow = p.out + b * p.o_sb + (long long)qi * p.o_ss + (long long)h * p.o_sh + half * HD;
      if ((reinterpret_cast<uintptr_t>(orow) & 15) == 0) {
#pragma unroll
        for (int c = 0; c < HD; c += 8) {
          uint4 v;
          v.x = pack_bf16x2(o_reg[c] * inv, o_reg[c + 1] * inv);
          v.y = pack_bf16x2(o_reg[c + 2] * inv, o_reg[c + 3] * inv);
          v.z = pack_bf16x2(o_reg[c + 4] * inv, o_reg[c + 5] * inv);
          v.w = pack_bf16x2(o_reg[c + 6] * inv, o_reg[c + 7] * inv);
          *reinterpret_cast<uint4*>(orow + c) = v;
        }
      } else {
#pragma unroll
        for (int c = 0; c < HD; c += 2)
          *reinterpret_cast<uint32_t*>(orow + c) = pack_bf16x2(o_reg[c] * inv, o_reg[c + 1] * inv);
      }
      if (p.lse && half == 0)
        p.lse[((long long)b * p.q_heads + h) * p.sq + qi] = l_run > 0.f ? (m_run * 0.6931471805599453f + logf(l_run)) : -INFINITY;
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------------------------------
// Two query tiles per CTA, ping-pong: while the softmax warps of one tile work, the tensor core multiplies for the other.
//
//   warp 0     : TMA producer  - Q (two tiles of 128 queries) once, then K and V tiles into two 2-deep rings
//   warp 1     : MMA issuer    - per tile t: S_t = Q_t K(j)^T; wait for P_t(j); O_t += P_t(j) V(j); S_t = Q_t K(j + 1)^T ...
//                                The probabilities are the A operand read from TENSOR MEMORY (they overwrite the first 64
//                                columns of their own scores), V is the MN-major B operand as it lies in memory, and O_t
//                                accumulates in tensor memory over all key tiles.
//   warps 2-3  : idle (they give their registers to the softmax warps)
//   warps 4-7  : softmax of tile 0, warps 8-11: softmax of tile 1 - thread r owns query row r: scores out of TMEM once
//                (128 registers), row maximum, exponentials, bf16 probabilities back into TMEM.  The running maximum is
//                LAZY: the accumulated output is rescaled (TMEM load, multiply, store) only when the maximum rose by more
//                than 2^8 since the last rescale, which after the first tiles of a row is rare; the stale maximum cancels
//                in O / l and in the log-sum-exp.
//
// TMEM (512 columns): S_0 | S_1 | O_0 | O_1, 128 columns each.  Shared memory at head_dim 128: Q 64 KB + K 64 KB + V 64 KB.
// Ordering: MMAs of one thread execute in issue order, so QK_t(j + 1), issued after PV_t(j), may overwrite the columns
// PV_t(j) reads; s_full_t(j) (a commit after QK_t(j)) therefore also says that PV_t(j - 1) is complete, which is what a
// rescale of O_t needs.  Every mbarrier wait is bounded; on expiry the CTA records a status code and drains.
constexpr int FA2_M = 256;
constexpr int FA2_THREADS = 384;
constexpr float FA2_RESCALE_LOG2 = 8.f;

template <int D, int POLY>  // POLY of every 4 pairs of exponentials run on the FMA pipe
__global__ void __launch_bounds__(FA2_THREADS, 1)
attn_fwd_pingpong_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, const FaParams p) {
  constexpr int DB = D / 64;
  constexpr uint32_t T_BYTES = DB * FA_BLOCK_BYTES;  // one 128-row tile of Q, K or V
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t O_COL0 = 256;
  constexpr uint32_t IDESC_QK = make_idesc_bf16(FA_M, FA_N, false, false);
  constexpr uint32_t IDESC_PV = make_idesc_bf16(FA_M, D, false, true);

  extern __shared__ uint8_t fa_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;                 // [2 tiles]
  uint8_t* k_s = q_s + 2 * T_BYTES;    // [2 stages]
  uint8_t* v_s = k_s + 2 * T_BYTES;    // [2 stages]
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + 2 * T_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2 tiles]
  uint64_t* p_full = bars + 11;   // [2 tiles]
  uint64_t* o_full = bars + 13;   // [2 tiles]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qblk = gridDim.x - 1 - blockIdx.x;  // heavy (late) causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.q_heads / p.kv_heads);
  const int q0 = qblk * FA2_M;
  const int shift = p.sk - p.sq;  // query i may see keys j <= i + shift when causal
  int n_tiles[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    int kv_end = p.sk;
    if (p.causal) kv_end = min(p.sk, q0 + t * FA_M + FA_M + shift);
    n_tiles[t] = (q0 + t * FA_M < p.sq && kv_end > 0) ? (kv_end + FA_N - 1) / FA_N : 0;
  }
  const int n_max = max(n_tiles[0], n_tiles[1]);

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 4);  // one arrival per softmax warp of the tile
      mbar_init(&o_full[s], 1);
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

  auto give_up = [&](uint32_t code) {
    atomicMax(p.status, code);
    *abort_flag = 1;
  };

  if (warp < 4) {
    setmaxnreg_dec<56>();
    if (warp == 0) {
      // ---------------- TMA producer ----------------
      if (elect_one() && n_max > 0) {
        mbar_expect_tx(q_full, 2 * T_BYTES);
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
          for (int d = 0; d < DB; ++d) tma_load_4d(q_s + t * T_BYTES + d * FA_BLOCK_BYTES, &tmap_q, q_full, d * 64, q0 + t * FA_M, h, b);
        for (int j = 0; j < n_max && !*abort_flag; ++j) {
          const int s = j & 1;
          const uint32_t par = ((j >> 1) & 1) ^ 1;
          if (!mbar_wait(&k_empty[s], par)) { give_up(STATUS_TIMEOUT_MBAR); break; }
          mbar_expect_tx(&k_full[s], T_BYTES);
#pragma unroll
          for (int d = 0; d < DB; ++d) tma_load_4d(k_s + s * T_BYTES + d * FA_BLOCK_BYTES, &tmap_k, &k_full[s], d * 64, j * FA_N, kvh, b);
          if (!mbar_wait(&v_empty[s], par)) { give_up(STATUS_TIMEOUT_MBAR); break; }
          mbar_expect_tx(&v_full[s], T_BYTES);
#pragma unroll
          for (int d = 0; d < DB; ++d) tma_load_4d(v_s + s * T_BYTES + d * FA_BLOCK_BYTES, &tmap_v, &v_full[s], d * 64, j * FA_N, kvh, b);
        }
      }
    } else if (warp == 1) {
      // ---------------- MMA issuer ----------------
      if (elect_one() && n_max > 0) {
        const uint32_t q_addr = smem_u32(q_s);
        auto issue_qk = [&](int t, int j) {  // S_t = Q_t K(j)^T
          const uint32_t k_addr = smem_u32(k_s + (j & 1) * T_BYTES);
          const uint32_t d_tmem = tmem_base + t * FA_N;
#pragma unroll
          for (int d = 0; d < DB; ++d) {
#pragma unroll
            for (int kk = 0; kk < 64 / 16; ++kk) {
              const uint64_t adesc = make_desc_kmajor_sw128(q_addr + t * T_BYTES + d * FA_BLOCK_BYTES + kk * 32);
              const uint64_t bdesc = make_desc_kmajor_sw128(k_addr + d * FA_BLOCK_BYTES + kk * 32);
              umma_bf16(d_tmem, adesc, bdesc, IDESC_QK, (d | kk) ? 1u : 0u);
            }
          }
          umma_commit(&s_full[t]);
        };
        auto issue_pv = [&](int t, int j) {  // O_t (+)= P_t(j) V(j): P from tensor memory, V tile [128 keys][D] MN-major
          const uint32_t v_addr = smem_u32(v_s + (j & 1) * T_BYTES);
#pragma unroll
          for (int kk = 0; kk < FA_N / 16; ++kk) {
            const uint64_t bdesc = make_desc_mnmajor_sw128(v_addr + kk * 16 * 128, FA_BLOCK_BYTES);
            umma_bf16_tmem_a(tmem_base + O_COL0 + t * FA_N, tmem_base + t * FA_N + kk * 8, bdesc, IDESC_PV, (j | kk) ? 1u : 0u);
          }
        };
        bool ok = mbar_wait(q_full, 0) && mbar_wait(&k_full[0], 0);
        if (!ok) give_up(STATUS_TIMEOUT_MBAR);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int t = 0; t < 2; ++t)
            if (n_tiles[t] > 0) issue_qk(t, 0);
          umma_commit(&k_empty[0]);
        }
        for (int j = 0; ok && j < n_max && !*abort_flag; ++j) {
          const bool next = j + 1 < n_max;
          if (next && !mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1)) { give_up(STATUS_TIMEOUT_MBAR); break; }
          if (!mbar_wait(&v_full[j & 1], (j >> 1) & 1)) { give_up(STATUS_TIMEOUT_MBAR); break; }
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (ok && j < n_tiles[t]) {
              if (!mbar_wait(&p_full[t], j & 1)) {
                give_up(STATUS_TIMEOUT_MBAR);
                ok = false;
              } else {
                tc_fence_after();
                issue_pv(t, j);
                if (j == n_tiles[t] - 1)
                  umma_commit(&o_full[t]);
                else
                  issue_qk(t, j + 1);
              }
            }
          }
          if (!ok) break;
          umma_commit(&v_empty[j & 1]);          // V(j) may be overwritten once these MMAs retire
          if (next) umma_commit(&k_empty[(j + 1) & 1]);  // and K(j + 1)
        }
      }
    }
  } else {
    // ---------------- softmax warps ----------------
    setmaxnreg_inc<224>();
    const int t = (warp - 4) >> 2;
    const int quarter = warp & 3;  // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;
    const int qi = q0 + t * FA_M + row;
    const int my_tiles = n_tiles[t];
    const uint32_t s_addr = tmem_base + (uint32_t(quarter * 32) << 16) + t * FA_N;  // scores, and in their first 64 columns P
    const uint32_t o_addr = tmem_base + (uint32_t(quarter * 32) << 16) + O_COL0 + t * FA_N;
    float m_run = -INFINITY, l_run = 0.f;
    const float* bias_f = static_cast<const float*>(p.bias);
    const bf16* bias_h = static_cast<const bf16*>(p.bias);
    const long long bias_row = p.bias_kind ? (b * p.bias_sb + h * p.bias_sh + (long long)min(qi, p.sq - 1) * p.bias_sq) : 0;
    bool alive = true;

    for (int j = 0; j < my_tiles; ++j) {
      if (*abort_flag || !mbar_wait(&s_full[t], j & 1)) {
        if (!*abort_flag) give_up(STATUS_TIMEOUT_MBAR);
        alive = false;
        break;
      }
      tc_fence_after();
      const int key0 = j * FA_N;
      // only tiles that touch the diagonal, the end of the keys or a bias need per-element work
      const bool plain = !p.bias_kind && key0 + FA_N <= p.sk && (!p.causal || key0 + FA_N - 1 <= q0 + t * FA_M + shift);
      uint32_t r[FA_N];
#pragma unroll
      for (int c = 0; c < FA_N; c += 32) tmem_ld_x32(s_addr + c, *reinterpret_cast<uint32_t(*)[32]>(r + c));
      tmem_ld_wait();
      float m_tile;
      if (!p.bias_kind) {
        if (!plain) {  // keys [0, visible) of this tile count, the others become -inf
          const int visible = min(p.sk, p.causal ? qi + shift + 1 : p.sk) - key0;
#pragma unroll
          for (int i = 0; i < FA_N; ++i)
            if (i >= visible) r[i] = 0xff800000u;
        }
        float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < FA_N; i += 4) {
          m0 = fmax3(m0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
          m1 = fmax3(m1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
        }
        m_tile = fmaxf(m0, m1) * p.scale_log2e;  // (the scale is positive: the maximum commutes with it)
      } else {
        m_tile = -INFINITY;
#pragma unroll
        for (int i = 0; i < FA_N; ++i) {
          const int key = key0 + i;
          const bool dead = key >= p.sk || (p.causal && key > qi + shift);
          float sv = dead ? -INFINITY : __uint_as_float(r[i]) * p.scale_log2e;
          if (!dead) {
            const long long bi = bias_row + (long long)key * p.bias_sk;
            const float bv = p.bias_kind == 1 ? __ldg(bias_f + bi) : __bfloat162float(bias_h[bi]);
            sv += bv * 1.4426950408889634f;
          }
          r[i] = __float_as_uint(sv);
          m_tile = fmaxf(m_tile, sv);
        }
      }
      // ---- lazy running maximum; rescale the accumulated output only after a large rise ----
      float factor = 1.f;
      bool rescale = false;
      if (m_run == -INFINITY) {
        m_run = m_tile;  // nothing accumulated for this row yet
      } else if (m_tile > m_run + FA2_RESCALE_LOG2) {
        factor = ex2_approx(m_run - m_tile);
        m_run = m_tile;
        rescale = true;
      }
      if (j > 0 && __any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_ld_x32(o_addr + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
          tmem_st_x32(o_addr + c, o);
        }
      }
      l_run *= factor;
      // ---- probabilities (bf16 pairs, key 2c and 2c + 1 in column c of this row) over the scores' first 64 columns ----
      const float mul = p.bias_kind ? 1.f : p.scale_log2e;
      const float nbase = m_run == -INFINITY ? 0.f : -m_run;
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int c = 0; c < FA_N / 2; c += 32) {
        uint32_t packed[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float t0, t1;
          ffma2(t0, t1, __uint_as_float(r[2 * (c + i)]), __uint_as_float(r[2 * (c + i) + 1]), mul, mul, nbase, nbase);
          float p0, p1;
          if ((i & 3) < POLY) {
            ex2_poly2(t0, t1);
            p0 = t0;
            p1 = t1;
          } else {
            p0 = ex2_approx(t0);
            p1 = ex2_approx(t1);
          }
          fadd2(sum0, sum1, sum0, sum1, p0, p1);
          packed[i] = pack_bf16x2(p0, p1);
        }
        tmem_st_x32(s_addr + c, packed);
      }
      l_run += sum0 + sum1;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
    }
    // ---- epilogue: O_t / l -> global memory ----
    if (alive && my_tiles > 0) {
      if (mbar_wait(&o_full[t], 0)) {
        tc_fence_after();
      } else {
        give_up(STATUS_TIMEOUT_MBAR);
        alive = false;
      }
    }
    if (alive && q0 + t * FA_M < p.sq) {  // (warp-uniform: the TMEM loads below are warp-wide)
      if (m_run == -INFINITY) l_run = 0.f;  // no visible key at all (the cubic turns a masked score into 2^-126, not 0)
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      bf16* orow = p.out + b * p.o_sb + (long long)min(qi, p.sq - 1) * p.o_ss + (long long)h * p.o_sh;
      const bool vec = (reinterpret_cast<uintptr_t>(orow) & 15) == 0;
#pragma unroll
      for (int c = 0; c < D; c += 32) {
        uint32_t o[32];
        if (my_tiles > 0) {
          tmem_ld_x32(o_addr + c, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (qi < p.sq) {
          if (vec) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
              v.y = pack_bf16x2(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
              v.z = pack_bf16x2(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
              v.w = pack_bf16x2(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c + i) = v;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 2)
              *reinterpret_cast<uint32_t*>(orow + c + i) = pack_bf16x2(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
          }
        }
      }
      if (p.lse && qi < p.sq)
        p.lse[((long long)b * p.q_heads + h) * p.sq + qi] = l_run > 0.f ? (m_run * 0.6931471805599453f + logf(l_run)) : -INFINITY;
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int D>
static int fa_launch(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaParams& p, dim3 grid, cudaStream_t stream) {
  constexpr size_t smem = size_t(D / 64) * FA_BLOCK_BYTES * 5 + 2 * FA_BLOCK_BYTES + 1024 + 128 + 4 * FA_M * sizeof(float);
  static std::atomic<bool> configured[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TPB_ERR_CUDA;
  if (!configured[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(attn_fwd_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return TPB_ERR_CUDA;
    configured[dev].store(true, std::memory_order_release);
  }
  attn_fwd_tcgen05_kernel<D><<<grid, FA_THREADS, smem, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

template <int D, int POLY>
static int fa2_launch(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaParams& p, dim3 grid, cudaStream_t stream) {
  constexpr size_t smem = size_t(D / 64) * FA_BLOCK_BYTES * 6 + 1024 + 256;
  static std::atomic<bool> configured[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TPB_ERR_CUDA;
  if (!configured[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(attn_fwd_pingpong_kernel<D, POLY>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return TPB_ERR_CUDA;
    configured[dev].store(true, std::memory_order_release);
  }
  attn_fwd_pingpong_kernel<D, POLY><<<grid, FA2_THREADS, smem, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

}  // namespace tpb

using namespace tpb;

// Same contract as tpb_attn_prefill_bias (strides in elements, head_dim contiguous, bias strides of 0 broadcast) plus:
// every stride of q / k / v must be a multiple of 8 elements and the bases 16-byte aligned (TMA), `status` is a device word
// that receives a non-zero code if a wait inside the kernel ran out of time.
extern "C" int tpb_attn_prefill_sm100(const void* q, const void* k, const void* v, void* out, float* lse, int batch, int sq, int sk,
                                      int q_heads, int kv_heads, int head_dim, long long q_sb, long long q_ss, long long q_sh,
                                      long long k_sb, long long k_ss, long long k_sh, long long v_sb, long long v_ss, long long v_sh,
                                      long long o_sb, long long o_ss, long long o_sh, int causal, float scale, const void* bias,
                                      int bias_dtype, long long bias_sb, long long bias_sh, long long bias_sq, long long bias_sk,
                                      void* status, void* stream_) {
  if (!q || !k || !v || !out || !status || batch <= 0 || sq <= 0 || sk <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads) return TPB_ERR_ARG;
  if (head_dim != 64 && head_dim != 128) return TPB_ERR_SIZE;
  if ((q_ss & 7) || (k_ss & 7) || (v_ss & 7) || (q_heads > 1 && (q_sh & 7)) || (kv_heads > 1 && ((k_sh & 7) || (v_sh & 7))) ||
      (batch > 1 && ((q_sb & 7) || (k_sb & 7) || (v_sb & 7))) || ((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15) ||
      (o_ss & 1) || (o_sh & 1) || (o_sb & 1) || ((uintptr_t)out & 3))
    return TPB_ERR_ALIGN;
  if (bias && bias_dtype != 0 && bias_dtype != 1) return TPB_ERR_ARG;
  if (fa_bind_thread() != TPB_OK) return TPB_ERR_CUDA;
  CUtensorMap tq, tk, tv;
  int rc = fa_tmap(&tq, q, head_dim, FA_N, sq, q_heads, batch, q_ss, q_sh, q_sb);
  if (rc == TPB_OK) rc = fa_tmap(&tk, k, head_dim, FA_N, sk, kv_heads, batch, k_ss, k_sh, k_sb);
  if (rc == TPB_OK) rc = fa_tmap(&tv, v, head_dim, FA_N, sk, kv_heads, batch, v_ss, v_sh, v_sb);
  if (rc != TPB_OK) return rc;
  FaParams p;
  memset(&p, 0, sizeof(p));
  p.sq = sq; p.sk = sk; p.q_heads = q_heads; p.kv_heads = kv_heads; p.causal = causal;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.out = static_cast<bf16*>(out);
  p.o_sb = o_sb; p.o_ss = o_ss; p.o_sh = o_sh;
  p.lse = lse;
  p.bias = bias;
  p.bias_kind = !bias ? 0 : (bias_dtype == 1 ? 1 : 2);
  p.bias_sb = bias_sb; p.bias_sh = bias_sh; p.bias_sq = bias_sq; p.bias_sk = bias_sk;
  p.status = static_cast<uint32_t*>(status);
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  static const bool one_tile = getenv("TPB_ATTN_ONE_TILE") != nullptr;  // (A/B switch: the kernel with one query tile per CTA)
  if (!one_tile && sq > FA_M) {
    dim3 grid((sq + FA2_M - 1) / FA2_M, q_heads, batch);
    // one pair of exponentials in four runs as a cubic on the FMA pipe (measured best of 0 / 1 / 2 / 3 in four:
    // 206 / 199 / 205 / 236 us at batch 4, 2048 tokens, 32 heads of 128, causal)
    return head_dim == 128 ? fa2_launch<128, 1>(tq, tk, tv, p, grid, s) : fa2_launch<64, 1>(tq, tk, tv, p, grid, s);
  }
  dim3 grid((sq + FA_M - 1) / FA_M, q_heads, batch);
  return head_dim == 128 ? fa_launch<128>(tq, tk, tv, p, grid, s) : fa_launch<64>(tq, tk, tv, p, grid, s);
}
