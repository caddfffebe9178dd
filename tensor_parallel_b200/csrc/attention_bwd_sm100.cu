// Attention backward for sm_100a on tcgen05 tensor cores, with an optional additive score bias (scores = S * scale + bias;
// d(bias) = P * (dP - delta), summed over whatever dimensions the bias broadcasts over, is added into an fp32 buffer by the
// dQ launch, which visits every (query, key) pair exactly once).
//
//   P  = exp(S * scale - lse)          S  = Q K^T
//   dV = P^T dO                        dP = dO V^T
//   dS = P * (dP - delta) * scale      delta[i] = sum_d out[i, d] * dout[i, d]
//   dQ = dS K                          dK = dS^T Q
//
// Two launches of ONE kernel template, both free of atomics and therefore deterministic (the optional bias gradient is the
// exception: fp32 atomic adds).  A CTA keeps 128 "resident"
// rows (the TMEM lanes) and streams the other sequence through in steps of 64 rows (TMEM columns):
//
//   dK / dV (DKV = true) : resident = 128 keys of one KV head (K and V tiles), streamed = queries (Q and dO, over all
//                          query heads of the group):  S^T = K Q^T and dP^T = V dO^T land in TMEM with a key per lane,
//                          the elementwise warps turn them into P^T and dS^T (bf16, written back over their own
//                          columns), and dV += P^T dO, dK += dS^T Q read them from TENSOR MEMORY as the A operand, the
//                          streamed tile being the MN-major B operand as it lies in memory.
//   dQ (DKV = false)     : resident = 128 queries of one head (Q and dO), streamed = keys (K and V): S = Q K^T,
//                          dP = dO V^T, dQ += dS K.
//
//   warp 0    : TMA producer (resident tiles once, streamed tiles into a 3-deep ring; for dK / dV also the streamed
//               queries' log-sum-exp and delta into shared memory)
//   warp 1    : MMA issuer; the two score products of step n + 1 are issued BEFORE the wait for the elementwise warps
//               of step n (two TMEM buffers), so the tensor core always has work
//   warps 2-9 : elementwise - two threads per TMEM lane, one per half of the step's 64 columns
//
// TMEM (512 columns): S 2 x 64 | dP 2 x 64 | accumulator 0 (dK or dQ) | accumulator 1 (dV).  Shared memory at head_dim
// 128: 2 x 32 KB resident + 3 x 2 x 16 KB streamed = 160 KB.  Every mbarrier wait is bounded; on expiry the CTA records
// a status code and drains.  No TMA load has a multicast qualifier.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <atomic>

#include "attention_sm100.cuh"
#include "ptx_sm100.cuh"
#include "tpb_api.h"

namespace tpb {

typedef __nv_bfloat16 bf16;

constexpr int BW_R = 128;      // resident rows = TMEM lanes
constexpr int BW_T = 64;       // streamed rows per step = TMEM columns of one score buffer
constexpr int BW_STAGES = 3;
constexpr int BW_THREADS = 320;
constexpr int BW_T_BLOCK_BYTES = BW_T * 128;  // one [64 rows][64 elements] swizzled block

struct BwParams {
  int sq, sk, q_heads, kv_heads, causal;
  float scale, scale_log2e;
  const float* lse;    // [batch][q_heads][sq], natural log
  const float* delta;  // [batch][q_heads][sq]
  bf16* out0;          // dK (DKV) or dQ
  long long o0_sb, o0_ss, o0_sh;
  bf16* out1;          // dV (DKV)
  long long o1_sb, o1_ss, o1_sh;
  const void* bias;    // additive score bias in natural-log units over (batch, head, query, key), element strides, 0 broadcasts
  int bias_kind;       // 0 none, 1 fp32, 2 bf16
  long long b_sb, b_sh, b_sq, b_sk;
  float* dbias;        // fp32, the bias' own strides, zero-initialised by the caller; written by the dQ launch only (or null)
  float inv_scale;
  uint32_t* status;
};

template <int D, bool DKV, bool BIAS>  // BIAS: the score-bias code exists only in the instantiations that need it
__global__ void __launch_bounds__(BW_THREADS, 1)
attn_bwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_r1, const __grid_constant__ CUtensorMap tmap_r2,
                        const __grid_constant__ CUtensorMap tmap_t1, const __grid_constant__ CUtensorMap tmap_t2, const BwParams p) {
  constexpr int DB = D / 64;
  constexpr uint32_t R_BYTES = DB * FA_BLOCK_BYTES;    // one resident tile (128 rows)
  constexpr uint32_t T_BYTES = DB * BW_T_BLOCK_BYTES;  // one streamed tile (64 rows)
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COL0 = 0, DP_COL0 = 2 * BW_T, ACC0_COL = 4 * BW_T, ACC1_COL = 4 * BW_T + D;
  constexpr uint32_t IDESC_S = make_idesc_bf16(BW_R, BW_T, false, false);
  constexpr uint32_t IDESC_ACC = make_idesc_bf16(BW_R, D, false, true);

  extern __shared__ uint8_t bw_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(bw_smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* r1_s = smem;
  uint8_t* r2_s = r1_s + R_BYTES;
  uint8_t* t1_s = r2_s + R_BYTES;              // [stages]
  uint8_t* t2_s = t1_s + BW_STAGES * T_BYTES;  // [stages]
  float* lse_s = reinterpret_cast<float*>(t2_s + BW_STAGES * T_BYTES);  // [stages][64]: lse * log2(e), +inf = no such query
  float* del_s = lse_s + BW_STAGES * BW_T;                              // [stages][64]: delta * scale
  uint64_t* bars = reinterpret_cast<uint64_t*>(del_s + BW_STAGES * BW_T);
  uint64_t* r_full = bars;
  uint64_t* t_full = bars + 1;                   // [stages]
  uint64_t* t_empty = bars + 1 + BW_STAGES;      // [stages]
  uint64_t* s_full = bars + 1 + 2 * BW_STAGES;   // [2]
  uint64_t* p_full = s_full + 2;                 // [2]
  uint64_t* acc_full = p_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z;
  const int shift = p.sk - p.sq;  // query i may see keys j <= i + shift when causal
  const int group = p.q_heads / p.kv_heads;
  // ---- what this CTA owns and which steps it walks (the same arithmetic in every role) ----
  int r0, head, kvh, step0, per_head, n_steps;
  if (DKV) {
    r0 = blockIdx.x * BW_R;  // first key; low key tiles see the most queries when causal, so they start first
    kvh = blockIdx.y;
    head = kvh * group;      // first query head of the group
    const int q_steps = (p.sq + BW_T - 1) / BW_T;
    step0 = p.causal ? max(0, r0 - shift) / BW_T : 0;  // first 64-query step with a query that sees key r0
    per_head = max(0, q_steps - step0);
    n_steps = per_head * group;
  } else {
    r0 = (gridDim.x - 1 - blockIdx.x) * BW_R;  // first query; late query tiles see the most keys when causal
    head = blockIdx.y;
    kvh = head / group;
    int kv_end = p.sk;
    if (p.causal) kv_end = min(p.sk, r0 + BW_R + shift);
    step0 = 0;
    per_head = kv_end > 0 ? (kv_end + BW_T - 1) / BW_T : 0;
    n_steps = per_head;
  }

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_r1);
    prefetch_tmap(&tmap_r2);
    prefetch_tmap(&tmap_t1);
    prefetch_tmap(&tmap_t2);
    mbar_init(r_full, 1);
    for (int s = 0; s < BW_STAGES; ++s) {
      mbar_init(&t_full[s], DKV ? 2 : 1);  // the TMA bytes, and for dK / dV the step's lse / delta written by the producer warp
      mbar_init(&t_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 8);  // one arrival per elementwise warp
    }
    mbar_init(acc_full, 1);
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
    // ---------------- TMA producer (the whole warp stays together: all lanes write lse / delta) ----------------
    if (n_steps > 0) {
      if (lane == 0) {
        mbar_expect_tx(r_full, 2 * R_BYTES);
#pragma unroll
        for (int d = 0; d < DB; ++d) {
          tma_load_4d(r1_s + d * FA_BLOCK_BYTES, &tmap_r1, r_full, d * 64, r0, DKV ? kvh : head, b);
          tma_load_4d(r2_s + d * FA_BLOCK_BYTES, &tmap_r2, r_full, d * 64, r0, DKV ? kvh : head, b);
        }
      }
      for (int n = 0; n < n_steps; ++n) {
        const int s = n % BW_STAGES;
        const uint32_t par = ((n / BW_STAGES) & 1) ^ 1;
        const bool ok = !*abort_flag && mbar_wait(&t_empty[s], par);
        if (!__all_sync(0xffffffffu, ok)) {
          if (lane == 0 && !*abort_flag) give_up(STATUS_TIMEOUT_MBAR);
          break;
        }
        const int g = DKV ? n / per_head : 0;
        const int row0 = (step0 + (DKV ? n - g * per_head : n)) * BW_T;  // first streamed row of the step
        const int t_head = DKV ? head + g : kvh;
        if (lane == 0) {
          mbar_expect_tx(&t_full[s], 2 * T_BYTES);
#pragma unroll
          for (int d = 0; d < DB; ++d) {
            tma_load_4d(t1_s + s * T_BYTES + d * BW_T_BLOCK_BYTES, &tmap_t1, &t_full[s], d * 64, row0, t_head, b);
            tma_load_4d(t2_s + s * T_BYTES + d * BW_T_BLOCK_BYTES, &tmap_t2, &t_full[s], d * 64, row0, t_head, b);
          }
        }
        if (DKV) {
#pragma unroll
          for (int c = lane; c < BW_T; c += 32) {
            const int qi = row0 + c;
            float l2 = INFINITY, dl = 0.f;
            if (qi < p.sq) {
              const long long idx = ((long long)b * p.q_heads + t_head) * p.sq + qi;
              const float l = __ldg(p.lse + idx);
              if (l != -INFINITY) l2 = l * 1.4426950408889634f;  // (a query without a visible key has P = 0 everywhere)
              dl = __ldg(p.delta + idx) * p.scale;
            }
            lse_s[s * BW_T + c] = l2;
            del_s[s * BW_T + c] = dl;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&t_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one() && n_steps > 0) {
      const uint32_t r1_addr = smem_u32(r1_s), r2_addr = smem_u32(r2_s);
      auto issue_scores = [&](int n) {  // S[n & 1] = R1 T1(n)^T, dP[n & 1] = R2 T2(n)^T
        const int s = n % BW_STAGES, buf = n & 1;
        const uint32_t t1_addr = smem_u32(t1_s + s * T_BYTES), t2_addr = smem_u32(t2_s + s * T_BYTES);
#pragma unroll
        for (int d = 0; d < DB; ++d) {
#pragma unroll
          for (int kk = 0; kk < 64 / 16; ++kk) {
            umma_bf16(tmem_base + S_COL0 + buf * BW_T, make_desc_kmajor_sw128(r1_addr + d * FA_BLOCK_BYTES + kk * 32),
                      make_desc_kmajor_sw128(t1_addr + d * BW_T_BLOCK_BYTES + kk * 32), IDESC_S, (d | kk) ? 1u : 0u);
          }
        }
#pragma unroll
        for (int d = 0; d < DB; ++d) {
#pragma unroll
          for (int kk = 0; kk < 64 / 16; ++kk) {
            umma_bf16(tmem_base + DP_COL0 + buf * BW_T, make_desc_kmajor_sw128(r2_addr + d * FA_BLOCK_BYTES + kk * 32),
                      make_desc_kmajor_sw128(t2_addr + d * BW_T_BLOCK_BYTES + kk * 32), IDESC_S, (d | kk) ? 1u : 0u);
          }
        }
        umma_commit(&s_full[buf]);
      };
      auto issue_accumulate = [&](int n) {
        const int s = n % BW_STAGES, buf = n & 1;
        const uint32_t t1_addr = smem_u32(t1_s + s * T_BYTES), t2_addr = smem_u32(t2_s + s * T_BYTES);
#pragma unroll
        for (int kk = 0; kk < BW_T / 16; ++kk) {
          // the bf16 operand of the 16 streamed rows kk: written by the thread that owns their column half, inside that half
          const uint32_t a_col = (kk >> 1) * 32 + (kk & 1) * 8;
          if (DKV)  // dV += P^T dO
            umma_bf16_tmem_a(tmem_base + ACC1_COL, tmem_base + S_COL0 + buf * BW_T + a_col,
                             make_desc_mnmajor_sw128(t2_addr + kk * 16 * 128, BW_T_BLOCK_BYTES), IDESC_ACC, (n | kk) ? 1u : 0u);
          // dK += dS^T Q   or   dQ += dS K
          umma_bf16_tmem_a(tmem_base + ACC0_COL, tmem_base + DP_COL0 + buf * BW_T + a_col,
                           make_desc_mnmajor_sw128(t1_addr + kk * 16 * 128, BW_T_BLOCK_BYTES), IDESC_ACC, (n | kk) ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(r_full, 0) && mbar_wait(&t_full[0], 0);
      if (!ok) give_up(STATUS_TIMEOUT_MBAR);
      if (ok) {
        tc_fence_after();
        issue_scores(0);
      }
      for (int n = 0; ok && n < n_steps && !*abort_flag; ++n) {
        if (n + 1 < n_steps) {
          // scores of the next step: their TMEM buffer was last read by the accumulate MMAs of step n - 1 (issued
          // before these) and by the elementwise warps of step n - 1 (who delivered before those were issued)
          if (!mbar_wait(&t_full[(n + 1) % BW_STAGES], ((n + 1) / BW_STAGES) & 1)) { give_up(STATUS_TIMEOUT_MBAR); break; }
          tc_fence_after();
          issue_scores(n + 1);
        }
        if (!mbar_wait(&p_full[n & 1], (n >> 1) & 1)) { give_up(STATUS_TIMEOUT_MBAR); break; }
        tc_fence_after();
        issue_accumulate(n);
        umma_commit(&t_empty[n % BW_STAGES]);  // the streamed tiles of step n may be overwritten once these MMAs retire
      }
      umma_commit(acc_full);
    }
  } else {
    // ---------------- elementwise warps ----------------
    constexpr int HC = BW_T / 2;   // columns per thread and step
    constexpr int HD = D / 2;      // accumulator columns per thread in the epilogue
    const int quarter = warp & 3;  // TMEM lane quarter this warp may access
    const int half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int ri = r0 + row;  // key (DKV) or query
    const uint32_t t_lane = tmem_base + (uint32_t(quarter * 32) << 16);
    float my_lse2 = INFINITY, my_del = 0.f;
    if (!DKV && ri < p.sq) {
      const long long idx = ((long long)b * p.q_heads + head) * p.sq + ri;
      const float l = __ldg(p.lse + idx);
      if (l != -INFINITY) my_lse2 = l * 1.4426950408889634f;
      my_del = __ldg(p.delta + idx) * p.scale;
    }
    bool alive = true;

    for (int n = 0; n < n_steps; ++n) {
      const int s = n % BW_STAGES, buf = n & 1;
      if (*abort_flag || (DKV && !mbar_wait(&t_full[s], (n / BW_STAGES) & 1)) || !mbar_wait(&s_full[buf], (n >> 1) & 1)) {
        if (!*abort_flag) give_up(STATUS_TIMEOUT_MBAR);
        alive = false;
        break;
      }
      tc_fence_after();
      const int g = DKV ? n / per_head : 0;
      const int col0 = (step0 + (DKV ? n - g * per_head : n)) * BW_T + half * HC;  // first query (DKV) or key of my columns
      uint32_t sv[HC], dv[HC];
      tmem_ld_x32(t_lane + S_COL0 + buf * BW_T + half * HC, sv);
      tmem_ld_x32(t_lane + DP_COL0 + buf * BW_T + half * HC, dv);
      tmem_ld_wait();
      // columns [lo, hi) of mine are visible pairs
      int lo = 0, hi = HC;
      if (DKV) {
        if (ri >= p.sk) hi = 0;
        if (p.causal) lo = max(0, ri - shift - col0);  // query >= key - shift
      } else {
        hi = min(HC, min(p.sk, p.causal ? ri + shift + 1 : p.sk) - col0);  // key <= query + shift
      }
      const bool masked = lo > 0 || hi < HC;
      // score bias: element (query, key) = (col0 + c, ri) for dK / dV and (ri, col0 + c) for dQ
      const float* bias_f = static_cast<const float*>(p.bias);
      const bf16* bias_h = static_cast<const bf16*>(p.bias);
      const int b_head = DKV ? head + g : head;
      const long long bias_base = BIAS ? (long long)b * p.b_sb + (long long)b_head * p.b_sh + (long long)ri * (DKV ? p.b_sk : p.b_sq) : 0;
      const long long bias_step = DKV ? p.b_sq : p.b_sk;  // per column
      const int col_limit = DKV ? p.sq : p.sk, row_limit = DKV ? p.sk : p.sq;
      uint32_t pp[HC / 2], ds[HC / 2];
#pragma unroll
      for (int c = 0; c < HC; c += 2) {
        float l0, l1, d0, d1;
        if (DKV) {
          const float2 l = *reinterpret_cast<const float2*>(lse_s + s * BW_T + half * HC + c);
          const float2 d = *reinterpret_cast<const float2*>(del_s + s * BW_T + half * HC + c);
          l0 = l.x; l1 = l.y; d0 = d.x; d1 = d.y;
        } else {
          l0 = l1 = my_lse2;
          d0 = d1 = my_del;
        }
        float x0, x1, p0, p1, g0, g1;
        ffma2(x0, x1, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]), p.scale_log2e, p.scale_log2e, -l0, -l1);
        long long bi0 = 0, bi1 = 0;
        if (BIAS) {
          bi0 = bias_base + (long long)(col0 + c) * bias_step;
          bi1 = bi0 + bias_step;
          const bool in0 = ri < row_limit && col0 + c < col_limit, in1 = ri < row_limit && col0 + c + 1 < col_limit;
          const float b0 = !in0 ? 0.f : (p.bias_kind == 1 ? __ldg(bias_f + bi0) : __bfloat162float(bias_h[bi0]));
          const float b1 = !in1 ? 0.f : (p.bias_kind == 1 ? __ldg(bias_f + bi1) : __bfloat162float(bias_h[bi1]));
          x0 += b0 * 1.4426950408889634f;
          x1 += b1 * 1.4426950408889634f;
        }
        p0 = ex2_approx(x0);
        p1 = ex2_approx(x1);
        if (masked) {
          if (c < lo || c >= hi) p0 = 0.f;
          if (c + 1 < lo || c + 1 >= hi) p1 = 0.f;
        }
        ffma2(g0, g1, __uint_as_float(dv[c]), __uint_as_float(dv[c + 1]), p.scale, p.scale, -d0, -d1);  // (dP - delta) * scale
        ffma2(g0, g1, g0, g1, p0, p1, 0.f, 0.f);
        if (BIAS && !DKV && p.dbias) {  // d(bias) = P (dP - delta) = dS / scale; pairs that are masked or out of range contribute nothing
          if (p0 != 0.f && ri < row_limit && col0 + c < col_limit) atomicAdd(p.dbias + bi0, g0 * p.inv_scale);
          if (p1 != 0.f && ri < row_limit && col0 + c + 1 < col_limit) atomicAdd(p.dbias + bi1, g1 * p.inv_scale);
        }
        if (DKV) pp[c >> 1] = pack_bf16x2(p0, p1);
        ds[c >> 1] = pack_bf16x2(g0, g1);
      }
      // bf16 pairs over the first 16 columns of this thread's own half (nobody else reads or writes those)
      if (DKV) tmem_st_x16(t_lane + S_COL0 + buf * BW_T + half * HC, pp);
      tmem_st_x16(t_lane + DP_COL0 + buf * BW_T + half * HC, ds);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[buf]);
    }
    // ---- epilogue: accumulators -> bf16 rows in global memory ----
    if (alive && n_steps > 0) {
      if (mbar_wait(acc_full, 0)) {
        tc_fence_after();
      } else {
        give_up(STATUS_TIMEOUT_MBAR);
        alive = false;
      }
    }
    if (alive) {
      const int limit = DKV ? p.sk : p.sq;
      const int o_head = DKV ? kvh : head;
#pragma unroll
      for (int a = 0; a < (DKV ? 2 : 1); ++a) {
        bf16* base = a == 0 ? p.out0 : p.out1;
        const long long sb = a == 0 ? p.o0_sb : p.o1_sb, ss = a == 0 ? p.o0_ss : p.o1_ss, sh = a == 0 ? p.o0_sh : p.o1_sh;
        bf16* orow = base + b * sb + (long long)min(ri, limit - 1) * ss + (long long)o_head * sh + half * HD;
        const bool vec = (reinterpret_cast<uintptr_t>(orow) & 15) == 0;
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          uint32_t o[32];
          if (n_steps > 0) {
            tmem_ld_x32(t_lane + (a == 0 ? ACC0_COL : ACC1_COL) + half * HD + c, o);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0u;
          }
          if (ri < limit) {
            if (vec) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(o[i]), __uint_as_float(o[i + 1]));
                v.y = pack_bf16x2(__uint_as_float(o[i + 2]), __uint_as_float(o[i + 3]));
                v.z = pack_bf16x2(__uint_as_float(o[i + 4]), __uint_as_float(o[i + 5]));
                v.w = pack_bf16x2(__uint_as_float(o[i + 6]), __uint_as_float(o[i + 7]));
                *reinterpret_cast<uint4*>(orow + c + i) = v;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; i += 2)
                *reinterpret_cast<uint32_t*>(orow + c + i) = pack_bf16x2(__uint_as_float(o[i]), __uint_as_float(o[i + 1]));
            }
          }
        }
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int D, bool DKV, bool BIAS>
static int bw_launch(const CUtensorMap& r1, const CUtensorMap& r2, const CUtensorMap& t1, const CUtensorMap& t2, const BwParams& p, dim3 grid,
                     cudaStream_t stream) {
  constexpr size_t smem = size_t(D / 64) * (2 * FA_BLOCK_BYTES + 2 * BW_STAGES * BW_T_BLOCK_BYTES) + 2 * BW_STAGES * BW_T * sizeof(float) + 1024 + 256;
  static std::atomic<bool> configured[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TPB_ERR_CUDA;
  if (!configured[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(attn_bwd_tcgen05_kernel<D, DKV, BIAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess)
      return TPB_ERR_CUDA;
    configured[dev].store(true, std::memory_order_release);
  }
  attn_bwd_tcgen05_kernel<D, DKV, BIAS><<<grid, BW_THREADS, smem, stream>>>(r1, r2, t1, t2, p);
  return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

}  // namespace tpb

using namespace tpb;

// Same contract as tpb_attn_backward_bias (strides in elements, head_dim contiguous; bias strides of 0 broadcast; dbias is fp32 with
// the bias' strides, zero-initialised; `delta` is a [batch][q_heads][sq] fp32
// scratch buffer this call fills) plus: every stride of q / k / v / dout must be a multiple of 8 elements and their bases
// 16-byte aligned (TMA); `status` is a device word that receives a non-zero code if a wait inside a kernel ran out of time.
extern "C" int tpb_attn_backward_sm100(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
                                       float* delta, void* dq, void* dk, void* dv, int batch, int sq, int sk, int q_heads, int kv_heads,
                                       int head_dim, long long q_sb, long long q_ss, long long q_sh, long long k_sb, long long k_ss,
                                       long long k_sh, long long v_sb, long long v_ss, long long v_sh, long long o_sb, long long o_ss,
                                       long long o_sh, long long do_sb, long long do_ss, long long do_sh, long long dq_sb, long long dq_ss,
                                       long long dq_sh, long long dk_sb, long long dk_ss, long long dk_sh, int causal, float scale,
                                       const void* bias, int bias_dtype, long long bias_sb, long long bias_sh, long long bias_sq,
                                       long long bias_sk, float* dbias, void* status, void* stream_) {
  if (!q || !k || !v || !out || !dout || !lse || !delta || !dq || !dk || !dv || !status || batch <= 0 || sq <= 0 || sk <= 0 || q_heads <= 0 ||
      kv_heads <= 0 || q_heads % kv_heads)
    return TPB_ERR_ARG;
  if (head_dim != 64 && head_dim != 128) return TPB_ERR_SIZE;
  if ((bias && bias_dtype != 0 && bias_dtype != 1) || (dbias && !bias) || (bias && !(scale > 0.f))) return TPB_ERR_ARG;
  const long long strides[] = {q_ss, k_ss, v_ss, do_ss, q_heads > 1 ? q_sh : 0, q_heads > 1 ? do_sh : 0, kv_heads > 1 ? k_sh : 0,
                               kv_heads > 1 ? v_sh : 0, batch > 1 ? q_sb : 0, batch > 1 ? k_sb : 0, batch > 1 ? v_sb : 0, batch > 1 ? do_sb : 0};
  for (long long s : strides)
    if (s & 7) return TPB_ERR_ALIGN;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)dout) & 15) return TPB_ERR_ALIGN;
  if ((dq_ss | dq_sh | dq_sb | dk_ss | dk_sh | dk_sb) & 1 || (((uintptr_t)dq | (uintptr_t)dk | (uintptr_t)dv) & 3)) return TPB_ERR_ALIGN;
  if (fa_bind_thread() != TPB_OK) return TPB_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  int rc = tpb_attn_bwd_delta(out, dout, delta, batch, sq, q_heads, head_dim, o_sb, o_ss, o_sh, do_sb, do_ss, do_sh, stream_);
  if (rc != TPB_OK) return rc;
  CUtensorMap q128, do128, k128, v128, q64, do64, k64, v64;
  rc = fa_tmap(&q128, q, head_dim, BW_R, sq, q_heads, batch, q_ss, q_sh, q_sb);
  if (rc == TPB_OK) rc = fa_tmap(&do128, dout, head_dim, BW_R, sq, q_heads, batch, do_ss, do_sh, do_sb);
  if (rc == TPB_OK) rc = fa_tmap(&k128, k, head_dim, BW_R, sk, kv_heads, batch, k_ss, k_sh, k_sb);
  if (rc == TPB_OK) rc = fa_tmap(&v128, v, head_dim, BW_R, sk, kv_heads, batch, v_ss, v_sh, v_sb);
  if (rc == TPB_OK) rc = fa_tmap(&q64, q, head_dim, BW_T, sq, q_heads, batch, q_ss, q_sh, q_sb);
  if (rc == TPB_OK) rc = fa_tmap(&do64, dout, head_dim, BW_T, sq, q_heads, batch, do_ss, do_sh, do_sb);
  if (rc == TPB_OK) rc = fa_tmap(&k64, k, head_dim, BW_T, sk, kv_heads, batch, k_ss, k_sh, k_sb);
  if (rc == TPB_OK) rc = fa_tmap(&v64, v, head_dim, BW_T, sk, kv_heads, batch, v_ss, v_sh, v_sb);
  if (rc != TPB_OK) return rc;
  BwParams p;
  memset(&p, 0, sizeof(p));
  p.sq = sq; p.sk = sk; p.q_heads = q_heads; p.kv_heads = kv_heads; p.causal = causal;
  p.scale = scale;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.lse = lse;
  p.delta = delta;
  p.status = static_cast<uint32_t*>(status);
  p.bias = bias;
  p.bias_kind = !bias ? 0 : (bias_dtype == 1 ? 1 : 2);
  p.b_sb = bias_sb; p.b_sh = bias_sh; p.b_sq = bias_sq; p.b_sk = bias_sk;
  p.dbias = nullptr;  // (the dK / dV launch leaves it alone)
  p.inv_scale = scale > 0.f ? 1.f / scale : 0.f;
  // dK / dV: the dk strides serve dv too (the existing contract)
  p.out0 = static_cast<bf16*>(dk); p.o0_sb = dk_sb; p.o0_ss = dk_ss; p.o0_sh = dk_sh;
  p.out1 = static_cast<bf16*>(dv); p.o1_sb = dk_sb; p.o1_ss = dk_ss; p.o1_sh = dk_sh;
  dim3 grid_kv((sk + BW_R - 1) / BW_R, kv_heads, batch);
  const bool with_bias = bias != nullptr;
  if (head_dim == 128)
    rc = with_bias ? bw_launch<128, true, true>(k128, v128, q64, do64, p, grid_kv, s) : bw_launch<128, true, false>(k128, v128, q64, do64, p, grid_kv, s);
  else
    rc = with_bias ? bw_launch<64, true, true>(k128, v128, q64, do64, p, grid_kv, s) : bw_launch<64, true, false>(k128, v128, q64, do64, p, grid_kv, s);
  if (rc != TPB_OK) return rc;
  p.out0 = static_cast<bf16*>(dq); p.o0_sb = dq_sb; p.o0_ss = dq_ss; p.o0_sh = dq_sh;
  p.out1 = nullptr;
  p.dbias = dbias;
  dim3 grid_q((sq + BW_R - 1) / BW_R, q_heads, batch);
  if (head_dim == 128)
    return with_bias ? bw_launch<128, false, true>(q128, do128, k64, v64, p, grid_q, s) : bw_launch<128, false, false>(q128, do128, k64, v64, p, grid_q, s);
  return with_bias ? bw_launch<64, false, true>(q128, do128, k64, v64, p, grid_q, s) : bw_launch<64, false, false>(q128, do128, k64, v64, p, grid_q, s);
}
