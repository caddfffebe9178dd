// Backward of the tiled attention (flash-style: scores are recomputed tile by tile, never stored).
//
//   delta[b,h,i] = sum_d out[b,i,h,d] * dout[b,i,h,d]                       (attn_bwd_delta_kernel)
//   P  = exp(S * scale - lse)          S = Q K^T
//   dV = P^T dO                        dP = dO V^T
//   dS = P * (dP - delta) * scale
//   dQ = dS K                          dK = dS^T Q
// With an additive score bias (relative positions, ALiBi, padding masks) the scores are S * scale + bias, and the gradient
// of the bias is d(bias) = P * (dP - delta), summed over whatever dimensions the bias broadcasts over: the dQ kernel,
// which visits every (query, key) pair exactly once, adds it into an fp32 buffer with the bias' own (broadcast) strides.
//
// Two kernels, both free of atomics and therefore deterministic:
//   attn_bwd_dq_kernel  : one CTA per 64 query rows of one head, loops over key tiles (like the forward)
//   attn_bwd_dkv_kernel : one CTA per 64 keys of one KV head, loops over the query heads of its group and
//                         over 32-row query tiles; works on transposed tiles (keys are the MMA rows), so dK / dV
//                         accumulate in registers
// GQA / MQA, causal masking with a cached prefix (sk >= sq) and arbitrary q / k / v strides are supported.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "attn_common.cuh"
#include "tpb_api.h"

namespace tpb {

constexpr float LOG2E = 1.4426950408889634f;

// Additive score bias in natural-log units (kind 0 none, 1 fp32, 2 bf16) addressed with element strides over
// (batch, head, query, key), a stride of 0 broadcasting; dbias (optional, fp32, zero-initialised) uses the same strides.
struct BiasArgs {
  const void* bias;
  int kind;
  long long sb, sh, sq, sk;
  float* dbias;
};

__device__ __forceinline__ float bias_at(const BiasArgs& ba, long long idx) {
  return ba.kind == 1 ? __ldg(static_cast<const float*>(ba.bias) + idx) : __bfloat162float(static_cast<const bf16*>(ba.bias)[idx]);
}

__global__ void attn_bwd_delta_kernel(const bf16* __restrict__ out, const bf16* __restrict__ dout, float* __restrict__ delta,
                                      int sq, int heads, int d, long long o_sb, long long o_ss, long long o_sh,
                                      long long do_sb, long long do_ss, long long do_sh, long long rows) {
  const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);  // (b, h, i)
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int i = int(row % sq);
  const int h = int((row / sq) % heads);
  const long long b = row / ((long long)sq * heads);
  const bf16* o = out + b * o_sb + (long long)i * o_ss + (long long)h * o_sh;
  const bf16* g = dout + b * do_sb + (long long)i * do_ss + (long long)h * do_sh;
  float acc = 0.f;
  for (int c = lane; c < d; c += 32) acc += __bfloat162float(o[c]) * __bfloat162float(g[c]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[row] = acc;
}

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ------------------------------------------------------------------------------------------------
// dQ: rows = queries
// ------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(PF_THREADS)
attn_bwd_dq_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                   const bf16* __restrict__ dout, const float* __restrict__ lse, const float* __restrict__ delta,
                   bf16* __restrict__ dq, int sq, int sk, int q_heads, int kv_heads, long long q_sb, long long q_ss,
                   long long q_sh, long long k_sb, long long k_ss, long long k_sh, long long v_sb, long long v_ss,
                   long long v_sh, long long do_sb, long long do_ss, long long do_sh, long long dq_sb, long long dq_ss,
                   long long dq_sh, int causal, float scale, const BiasArgs ba) {
  extern __shared__ __align__(128) uint8_t bw_smem[];
  bf16* q_s = reinterpret_cast<bf16*>(bw_smem);
  bf16* do_s = q_s + PF_M * D;
  bf16* k_s = do_s + PF_M * D;
  bf16* v_s = k_s + PF_N * D;

  const int mblk = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (q_heads / kv_heads);
  const int q0 = mblk * PF_M;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int id = lane >> 3, r8 = lane & 7;
  const int shift = sk - sq;
  const float scale_log2e = scale * LOG2E;

  const bf16* qg = q + b * q_sb + (long long)h * q_sh;
  const bf16* dog = dout + b * do_sb + (long long)h * do_sh;
  const bf16* kg = k + b * k_sb + (long long)kvh * k_sh;
  const bf16* vg = v + b * v_sb + (long long)kvh * v_sh;

  int kv_end = sk;
  if (causal) kv_end = min(sk, q0 + PF_M + shift);
  const int n_iters = kv_end > 0 ? (kv_end + PF_N - 1) / PF_N : 0;

  load_tile<D>(q_s, qg, q_ss, q0, sq);
  load_tile<D>(do_s, dog, do_ss, q0, sq);
  cp_async_commit();

  float lse2[2], dl[2];
#pragma unroll
  for (int r2 = 0; r2 < 2; ++r2) {
    const int qi = q0 + warp * 16 + g + r2 * 8;
    const long long idx = ((long long)b * q_heads + h) * sq + min(qi, sq - 1);
    lse2[r2] = lse[idx] * LOG2E;
    dl[r2] = delta[idx];
  }
  float dq_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) dq_acc[i][j] = 0.f;

  for (int it = 0; it < n_iters; ++it) {
    const int kv0 = it * PF_N;
    __syncthreads();  // every warp is done with the previous K / V tiles
    load_tile<D>(k_s, kg, k_ss, kv0, sk);
    load_tile<D>(v_s, vg, v_ss, kv0, sk);
    cp_async_commit();
    cp_async_wait_all();
    __syncthreads();

    float s_acc[PF_N / 8][4], dp_acc[PF_N / 8][4];
#pragma unroll
    for (int i = 0; i < PF_N / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) { s_acc[i][j] = 0.f; dp_acc[i][j] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t qf[4], gf[4];
      ldmatrix_x4(qf, tile_ptr<D>(q_s, warp * 16 + (id & 1) * 8 + r8, ks * 2 + (id >> 1)));
      ldmatrix_x4(gf, tile_ptr<D>(do_s, warp * 16 + (id & 1) * 8 + r8, ks * 2 + (id >> 1)));
#pragma unroll
      for (int np = 0; np < PF_N / 16; ++np) {
        uint32_t kb[4], vb[4];
        ldmatrix_x4(kb, tile_ptr<D>(k_s, np * 16 + (id >> 1) * 8 + r8, ks * 2 + (id & 1)));
        ldmatrix_x4(vb, tile_ptr<D>(v_s, np * 16 + (id >> 1) * 8 + r8, ks * 2 + (id & 1)));
        mma_bf16_16816(s_acc[2 * np], qf, kb[0], kb[1]);
        mma_bf16_16816(s_acc[2 * np + 1], qf, kb[2], kb[3]);
        mma_bf16_16816(dp_acc[2 * np], gf, vb[0], vb[1]);
        mma_bf16_16816(dp_acc[2 * np + 1], gf, vb[2], vb[3]);
      }
    }
    // dS = P * (dP - delta) * scale  -> A fragments
    uint32_t dsf[PF_N / 16][4];
    const int qi0 = q0 + warp * 16 + g;
#pragma unroll
    for (int nt = 0; nt < PF_N / 8; ++nt) {
      float ds[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = kv0 + nt * 8 + 2 * t4 + (j & 1);
        const int r2 = j >> 1;
        const int qi = qi0 + r2 * 8;
        const bool dead = key >= sk || qi >= sq || (causal && key > qi + shift) || lse2[r2] == -INFINITY;
        float sv = s_acc[nt][j] * scale_log2e;
        long long bi = 0;
        if (ba.kind && !dead) {
          bi = b * ba.sb + h * ba.sh + (long long)qi * ba.sq + (long long)key * ba.sk;
          sv += bias_at(ba, bi) * LOG2E;
        }
        const float p = dead ? 0.f : exp2f(sv - lse2[r2]);
        const float dscore = p * (dp_acc[nt][j] - dl[r2]);  // gradient of the biased score
        if (ba.dbias && !dead && dscore != 0.f) atomicAdd(ba.dbias + bi, dscore);
        ds[j] = dscore * scale;
      }
      dsf[nt >> 1][(nt & 1) * 2] = pack2(ds[0], ds[1]);
      dsf[nt >> 1][(nt & 1) * 2 + 1] = pack2(ds[2], ds[3]);
    }
    // dQ += dS K   (B operand: K tile read transposed, k = key, n = d)
#pragma unroll
    for (int ks = 0; ks < PF_N / 16; ++ks) {
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t kb[4];
        ldmatrix_x4_trans(kb, tile_ptr<D>(k_s, ks * 16 + (id & 1) * 8 + r8, dp * 2 + (id >> 1)));
        mma_bf16_16816(dq_acc[2 * dp], dsf[ks], kb[0], kb[1]);
        mma_bf16_16816(dq_acc[2 * dp + 1], dsf[ks], kb[2], kb[3]);
      }
    }
  }
  cp_async_wait_all();
#pragma unroll
  for (int r2 = 0; r2 < 2; ++r2) {
    const int qi = q0 + warp * 16 + g + r2 * 8;
    if (qi >= sq) continue;
    bf16* row = dq + b * dq_sb + (long long)qi * dq_ss + (long long)h * dq_sh;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt)
      *reinterpret_cast<uint32_t*>(row + dt * 8 + 2 * t4) = pack2(dq_acc[dt][r2 * 2], dq_acc[dt][r2 * 2 + 1]);
  }
}

// ------------------------------------------------------------------------------------------------
// dK, dV: rows = keys, query tiles of 32 rows
// ------------------------------------------------------------------------------------------------
constexpr int BQ = 32;

template <int D>
__global__ void __launch_bounds__(PF_THREADS)
attn_bwd_dkv_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                    const bf16* __restrict__ dout, const float* __restrict__ lse, const float* __restrict__ delta,
                    bf16* __restrict__ dk, bf16* __restrict__ dv, int sq, int sk, int q_heads, int kv_heads,
                    long long q_sb, long long q_ss, long long q_sh, long long k_sb, long long k_ss, long long k_sh,
                    long long v_sb, long long v_ss, long long v_sh, long long do_sb, long long do_ss, long long do_sh,
                    long long dk_sb, long long dk_ss, long long dk_sh, int causal, float scale, const BiasArgs ba) {
  extern __shared__ __align__(128) uint8_t bw_smem[];
  bf16* k_s = reinterpret_cast<bf16*>(bw_smem);
  bf16* v_s = k_s + PF_N * D;
  bf16* q_s = v_s + PF_N * D;
  bf16* do_s = q_s + BQ * D;
  float* lse_s = reinterpret_cast<float*>(do_s + BQ * D);
  float* dl_s = lse_s + BQ;

  const int kv0 = blockIdx.x * PF_N;
  const int kvh = blockIdx.y, b = blockIdx.z;
  const int group = q_heads / kv_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int id = lane >> 3, r8 = lane & 7;
  const int shift = sk - sq;
  const float scale_log2e = scale * LOG2E;

  load_tile<D>(k_s, k + b * k_sb + (long long)kvh * k_sh, k_ss, kv0, sk);
  load_tile<D>(v_s, v + b * v_sb + (long long)kvh * v_sh, v_ss, kv0, sk);
  cp_async_commit();

  float dk_acc[D / 8][4], dv_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) { dk_acc[i][j] = 0.f; dv_acc[i][j] = 0.f; }

  // first query row that can see any key of this tile
  int q_begin = 0;
  if (causal) q_begin = max(0, kv0 - shift);
  q_begin = (q_begin / BQ) * BQ;

  for (int hq = kvh * group; hq < (kvh + 1) * group; ++hq) {
    const bf16* qg = q + b * q_sb + (long long)hq * q_sh;
    const bf16* dog = dout + b * do_sb + (long long)hq * do_sh;
    const float* lse_row = lse + ((long long)b * q_heads + hq) * sq;
    const float* dl_row = delta + ((long long)b * q_heads + hq) * sq;
    for (int qs = q_begin; qs < sq; qs += BQ) {
      __syncthreads();  // previous Q / dO tiles fully consumed
      load_rows<D>(q_s, qg, q_ss, qs, sq, BQ);
      load_rows<D>(do_s, dog, do_ss, qs, sq, BQ);
      cp_async_commit();
      if (threadIdx.x < BQ) {
        const int qi = qs + threadIdx.x;
        lse_s[threadIdx.x] = qi < sq ? lse_row[qi] * LOG2E : -INFINITY;
        dl_s[threadIdx.x] = qi < sq ? dl_row[qi] : 0.f;
      }
      cp_async_wait_all();
      __syncthreads();

      // S^T = K Q^T and dP^T = V dO^T   (16 keys x 32 queries per warp)
      float st[BQ / 8][4], dpt[BQ / 8][4];
#pragma unroll
      for (int i = 0; i < BQ / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { st[i][j] = 0.f; dpt[i][j] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t kf[4], vf[4];
        ldmatrix_x4(kf, tile_ptr<D>(k_s, warp * 16 + (id & 1) * 8 + r8, ks * 2 + (id >> 1)));
        ldmatrix_x4(vf, tile_ptr<D>(v_s, warp * 16 + (id & 1) * 8 + r8, ks * 2 + (id >> 1)));
#pragma unroll
        for (int np = 0; np < BQ / 16; ++np) {
          uint32_t qb[4], gb[4];
          ldmatrix_x4(qb, tile_ptr<D>(q_s, np * 16 + (id >> 1) * 8 + r8, ks * 2 + (id & 1)));
          ldmatrix_x4(gb, tile_ptr<D>(do_s, np * 16 + (id >> 1) * 8 + r8, ks * 2 + (id & 1)));
          mma_bf16_16816(st[2 * np], kf, qb[0], qb[1]);
          mma_bf16_16816(st[2 * np + 1], kf, qb[2], qb[3]);
          mma_bf16_16816(dpt[2 * np], vf, gb[0], gb[1]);
          mma_bf16_16816(dpt[2 * np + 1], vf, gb[2], gb[3]);
        }
      }
      // P^T and dS^T as A fragments (rows = keys, k = queries)
      uint32_t pf[BQ / 16][4], dsf[BQ / 16][4];
      const int key0 = kv0 + warp * 16 + g;
#pragma unroll
      for (int nt = 0; nt < BQ / 8; ++nt) {
        float pv[4], ds[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int col = nt * 8 + 2 * t4 + (j & 1);
          const int qi = qs + col;
          const int key = key0 + (j >> 1) * 8;
          const float l2 = lse_s[col];
          const bool dead = key >= sk || qi >= sq || (causal && key > qi + shift) || l2 == -INFINITY;
          float sv = st[nt][j] * scale_log2e;
          if (ba.kind && !dead) sv += bias_at(ba, b * ba.sb + hq * ba.sh + (long long)qi * ba.sq + (long long)key * ba.sk) * LOG2E;
          pv[j] = dead ? 0.f : exp2f(sv - l2);
          ds[j] = pv[j] * (dpt[nt][j] - dl_s[col]) * scale;
        }
        pf[nt >> 1][(nt & 1) * 2] = pack2(pv[0], pv[1]);
        pf[nt >> 1][(nt & 1) * 2 + 1] = pack2(pv[2], pv[3]);
        dsf[nt >> 1][(nt & 1) * 2] = pack2(ds[0], ds[1]);
        dsf[nt >> 1][(nt & 1) * 2 + 1] = pack2(ds[2], ds[3]);
      }
      // dV += P^T dO ; dK += dS^T Q    (B operands read transposed: k = query, n = d)
#pragma unroll
      for (int ks = 0; ks < BQ / 16; ++ks) {
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
          uint32_t gb[4], qb[4];
          ldmatrix_x4_trans(gb, tile_ptr<D>(do_s, ks * 16 + (id & 1) * 8 + r8, dp * 2 + (id >> 1)));
          ldmatrix_x4_trans(qb, tile_ptr<D>(q_s, ks * 16 + (id & 1) * 8 + r8, dp * 2 + (id >> 1)));
          mma_bf16_16816(dv_acc[2 * dp], pf[ks], gb[0], gb[1]);
          mma_bf16_16816(dv_acc[2 * dp + 1], pf[ks], gb[2], gb[3]);
          mma_bf16_16816(dk_acc[2 * dp], dsf[ks], qb[0], qb[1]);
          mma_bf16_16816(dk_acc[2 * dp + 1], dsf[ks], qb[2], qb[3]);
        }
      }
    }
  }
  cp_async_wait_all();
#pragma unroll
  for (int r2 = 0; r2 < 2; ++r2) {
    const int key = kv0 + warp * 16 + g + r2 * 8;
    if (key >= sk) continue;
    bf16* krow = dk + b * dk_sb + (long long)key * dk_ss + (long long)kvh * dk_sh;
    bf16* vrow = dv + b * dk_sb + (long long)key * dk_ss + (long long)kvh * dk_sh;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      *reinterpret_cast<uint32_t*>(krow + dt * 8 + 2 * t4) = pack2(dk_acc[dt][r2 * 2], dk_acc[dt][r2 * 2 + 1]);
      *reinterpret_cast<uint32_t*>(vrow + dt * 8 + 2 * t4) = pack2(dv_acc[dt][r2 * 2], dv_acc[dt][r2 * 2 + 1]);
    }
  }
}

}  // namespace tpb

using namespace tpb;

// q, dout, out, dq: [batch, sq, q_heads, d]; k, v, dk, dv: [batch, sk, kv_heads, d]; strides in elements with a
// contiguous head_dim; dq uses its own strides, dk and dv share (dk_sb, dk_ss, dk_sh).  lse [batch, q_heads, sq]
// is the log-sum-exp written by tpb_attn_prefill; delta is a caller-provided fp32 scratch of the same shape.
//
// bias (may be null): the additive score bias the forward pass was given, dtype bias_dtype (0 bf16, 1 fp32), element strides
// over (batch, head, query, key) with 0 broadcasting.  dbias (may be null): fp32 buffer addressed with the same strides,
// zero-initialised by the caller; receives the gradient of the bias (added with atomics where the bias broadcasts).
// delta[b, h, i] = sum_d out[b, i, h, d] * dout[b, i, h, d] (fp32, [batch][heads][sq]); strides in elements.
extern "C" int tpb_attn_bwd_delta(const void* out, const void* dout, float* delta, int batch, int sq, int heads, int head_dim,
                                  long long o_sb, long long o_ss, long long o_sh, long long do_sb, long long do_ss, long long do_sh,
                                  void* stream_) {
  if (!out || !dout || !delta || batch <= 0 || sq <= 0 || heads <= 0 || head_dim <= 0) return TPB_ERR_ARG;
  const long long rows = (long long)batch * heads * sq;
  attn_bwd_delta_kernel<<<int((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      (const bf16*)out, (const bf16*)dout, delta, sq, heads, head_dim, o_sb, o_ss, o_sh, do_sb, do_ss, do_sh, rows);
  return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

extern "C" int tpb_attn_backward_bias(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                      const float* lse, float* delta, void* dq, void* dk, void* dv, int batch, int sq, int sk,
                                      int q_heads, int kv_heads, int head_dim, long long q_sb, long long q_ss, long long q_sh,
                                      long long k_sb, long long k_ss, long long k_sh, long long v_sb, long long v_ss,
                                      long long v_sh, long long o_sb, long long o_ss, long long o_sh, long long do_sb,
                                      long long do_ss, long long do_sh, long long dq_sb, long long dq_ss, long long dq_sh,
                                      long long dk_sb, long long dk_ss, long long dk_sh, int causal, float scale, const void* bias,
                                      int bias_dtype, long long bias_sb, long long bias_sh, long long bias_sq, long long bias_sk,
                                      float* dbias, void* stream_) {
  if (!q || !k || !v || !out || !dout || !lse || !delta || !dq || !dk || !dv || batch <= 0 || sq <= 0 || sk <= 0 || q_heads % kv_heads)
    return TPB_ERR_ARG;
  if ((bias && bias_dtype != 0 && bias_dtype != 1) || (dbias && !bias)) return TPB_ERR_ARG;
  BiasArgs ba;
  ba.bias = bias;
  ba.kind = !bias ? 0 : (bias_dtype == 1 ? 1 : 2);
  ba.sb = bias_sb; ba.sh = bias_sh; ba.sq = bias_sq; ba.sk = bias_sk;
  ba.dbias = dbias;
  if (head_dim != 64 && head_dim != 128) return TPB_ERR_SIZE;
  const long long strides[] = {q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh, do_sb, do_ss, do_sh};
  for (long long s : strides)
    if (s & 7) return TPB_ERR_ALIGN;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)dout) & 15) return TPB_ERR_ALIGN;
  if ((dq_ss | dq_sh | dq_sb | dk_ss | dk_sh | dk_sb) & 1) return TPB_ERR_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const long long rows = (long long)batch * q_heads * sq;
  attn_bwd_delta_kernel<<<int((rows + 7) / 8), 256, 0, s>>>((const bf16*)out, (const bf16*)dout, delta, sq, q_heads, head_dim, o_sb,
                                                            o_ss, o_sh, do_sb, do_ss, do_sh, rows);
  const size_t smem_dq = size_t(2 * PF_M + 2 * PF_N) * head_dim * 2;
  const size_t smem_dkv = size_t(2 * PF_N + 2 * BQ) * head_dim * 2 + 2 * BQ * sizeof(float);
  static bool cfg[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !cfg[dev]) {
    cudaFuncSetAttribute(attn_bwd_dq_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(size_t(2 * PF_M + 2 * PF_N) * 128 * 2));
    cudaFuncSetAttribute(attn_bwd_dkv_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         int(size_t(2 * PF_N + 2 * BQ) * 128 * 2 + 2 * BQ * sizeof(float)));
    cfg[dev] = true;
  }
  dim3 grid_q((sq + PF_M - 1) / PF_M, q_heads, batch), grid_kv((sk + PF_N - 1) / PF_N, kv_heads, batch);
#define ARGS_DQ (const bf16*)q, (const bf16*)k, (const bf16*)v, (const bf16*)dout, lse, delta, (bf16*)dq, sq, sk, q_heads, kv_heads, q_sb, \
                q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh, do_sb, do_ss, do_sh, dq_sb, dq_ss, dq_sh, causal, scale, ba
#define ARGS_DKV (const bf16*)q, (const bf16*)k, (const bf16*)v, (const bf16*)dout, lse, delta, (bf16*)dk, (bf16*)dv, sq, sk, q_heads,   \
                 kv_heads, q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh, do_sb, do_ss, do_sh, dk_sb, dk_ss, dk_sh, causal, scale, ba
  if (head_dim == 128) {
    attn_bwd_dq_kernel<128><<<grid_q, PF_THREADS, smem_dq, s>>>(ARGS_DQ);
    attn_bwd_dkv_kernel<128><<<grid_kv, PF_THREADS, smem_dkv, s>>>(ARGS_DKV);
  } else {
    attn_bwd_dq_kernel<64><<<grid_q, PF_THREADS, smem_dq, s>>>(ARGS_DQ);
    attn_bwd_dkv_kernel<64><<<grid_kv, PF_THREADS, smem_dkv, s>>>(ARGS_DKV);
  }
#undef ARGS_DQ
#undef ARGS_DKV
  return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

extern "C" int tpb_attn_backward(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                 const float* lse, float* delta, void* dq, void* dk, void* dv, int batch, int sq, int sk,
                                 int q_heads, int kv_heads, int head_dim, long long q_sb, long long q_ss, long long q_sh,
                                 long long k_sb, long long k_ss, long long k_sh, long long v_sb, long long v_ss,
                                 long long v_sh, long long o_sb, long long o_ss, long long o_sh, long long do_sb,
                                 long long do_ss, long long do_sh, long long dq_sb, long long dq_ss, long long dq_sh,
                                 long long dk_sb, long long dk_ss, long long dk_sh, int causal, float scale, void* stream_) {
  return tpb_attn_backward_bias(q, k, v, out, dout, lse, delta, dq, dk, dv, batch, sq, sk, q_heads, kv_heads, head_dim, q_sb, q_ss, q_sh,
                                k_sb, k_ss, k_sh, v_sb, v_ss, v_sh, o_sb, o_ss, o_sh, do_sb, do_ss, do_sh, dq_sb, dq_ss, dq_sh, dk_sb,
                                dk_ss, dk_sh, causal, scale, nullptr, 0, 0, 0, 0, 0, nullptr, stream_);
}
