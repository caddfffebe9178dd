// Attention kernels for a head-sharded KV cache.
//   tpb_qkv_rope_append : rotary embedding on q / k of new tokens + write k, v into the pre-allocated
//                         cache [batch, kv_heads, max_seq, head_dim] (position taken from a device scalar,
//                         so a captured decode step can be replayed for every token)
//   tpb_attn_decode     : one query token per sequence against the cache; split over the key range
//                         (flash-decoding) so that small batches still cover all SMs, fp32 online softmax
//   tpb_attn_prefill    : tiled flash-style attention for many query tokens (causal or not, MHA / GQA / MQA,
//                         arbitrary q / k / v strides), fp32 online softmax, optional log-sum-exp output
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <atomic>

#include "attn_common.cuh"
#include "launch.cuh"
#include "ptx_sm100.cuh"
#include "tpb_api.h"

namespace tpb {

// ------------------------------------------------------------------------------------------------
// rope + cache append
// ------------------------------------------------------------------------------------------------
__global__ void qkv_rope_append_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                                       bf16* __restrict__ q_out, bf16* __restrict__ kcache, bf16* __restrict__ vcache,
                                       const int* __restrict__ base_pos, int batch, int seq, int q_heads, int kv_heads,
                                       int head_dim, int rotary_dim, float log2_theta, int interleaved, int max_seq,
                                       long long q_ld, long long k_ld, long long v_ld) {
  const int half = rotary_dim >> 1;
  const int pairs = head_dim >> 1;  // work unit = 2 elements
  const int heads = q_heads + 2 * kv_heads;
  const long long total = (long long)batch * seq * heads * pairs;
  const int pos0 = base_pos ? base_pos[0] : 0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int p = int(i % pairs);
    const int h = int((i / pairs) % heads);
    const long long t = i / ((long long)pairs * heads);
    const int b = int(t / seq), s = int(t % seq);
    const int pos = pos0 + s;
    if (pos >= max_seq) continue;
    if (h >= q_heads + kv_heads) {  // v: plain copy of elements (2p, 2p+1)
      const int hv = h - q_heads - kv_heads;
      const bf16* src = v + t * v_ld + (long long)hv * head_dim + 2 * p;
      bf16* dst = vcache + (((long long)b * kv_heads + hv) * max_seq + pos) * head_dim + 2 * p;
      *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(src);
      continue;
    }
    const bool is_q = h < q_heads;
    const int hh = is_q ? h : h - q_heads;
    const bf16* src = (is_q ? q + t * q_ld : k + t * k_ld) + (long long)hh * head_dim;
    bf16* dst = is_q ? q_out + (t * q_heads + hh) * head_dim
                     : kcache + (((long long)b * kv_heads + hh) * max_seq + pos) * head_dim;
    if (p < half) {
      const int ia = interleaved ? 2 * p : p;
      const int ib = interleaved ? 2 * p + 1 : p + half;
      const float inv_freq = exp2f(-log2_theta * (2.f * float(p) / float(rotary_dim)));
      float sn, cs;
      sincosf(float(pos) * inv_freq, &sn, &cs);
      const float a = __bfloat162float(src[ia]), c = __bfloat162float(src[ib]);
      dst[ia] = __float2bfloat16(a * cs - c * sn);
      dst[ib] = __float2bfloat16(c * cs + a * sn);
    } else {
      // elements beyond the rotary span: pairs [half, pairs) map to elements rotary_dim + 2*(p-half) (+1)
      const int e = rotary_dim + 2 * (p - half);
      dst[e] = src[e];
      dst[e + 1] = src[e + 1];
    }
  }
}

// One thread moves 8 consecutive elements of the first rotary half together with their 8 partners of the second
// half (or, for the interleaved layout / the non-rotary tail / v, one 16-byte chunk), so every access is a 16-byte
// vector.  Requires head_dim, rotary_dim / 2 (non-interleaved) or rotary_dim (interleaved) to be multiples of 8.
__global__ void qkv_rope_append_vec_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                                           bf16* __restrict__ q_out, bf16* __restrict__ kcache, bf16* __restrict__ vcache,
                                           const int* __restrict__ base_pos, int batch, int seq, int q_heads, int kv_heads,
                                           int head_dim, int rotary_dim, float log2_theta, int interleaved, int max_seq,
                                           long long q_ld, long long k_ld, long long v_ld) {
  const int half = rotary_dim >> 1;
  // chunks per head: rotary part handled as (half / 8) pair-chunks when split, (rotary_dim / 8) chunks when interleaved
  const int rot_chunks = interleaved ? rotary_dim / 8 : half / 8;
  const int tail_chunks = (head_dim - rotary_dim) / 8;
  const int qk_chunks = rot_chunks + tail_chunks;
  const int v_chunks = head_dim / 8;
  const long long per_token = (long long)(q_heads + kv_heads) * qk_chunks + (long long)kv_heads * v_chunks;
  const long long total = (long long)batch * seq * per_token;
  const int pos0 = base_pos ? base_pos[0] : 0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / per_token;
    long long w = i % per_token;
    const int b = int(t / seq), sidx = int(t % seq);
    const int pos = pos0 + sidx;
    if (pos >= max_seq) continue;
    const long long qk_total = (long long)(q_heads + kv_heads) * qk_chunks;
    if (w >= qk_total) {  // v: straight 16-byte copy into the cache
      w -= qk_total;
      const int hv = int(w / v_chunks), c = int(w % v_chunks) * 8;
      const uint4 val = *reinterpret_cast<const uint4*>(v + t * v_ld + (long long)hv * head_dim + c);
      *reinterpret_cast<uint4*>(vcache + (((long long)b * kv_heads + hv) * max_seq + pos) * head_dim + c) = val;
      continue;
    }
    const int h = int(w / qk_chunks), c = int(w % qk_chunks);
    const bool is_q = h < q_heads;
    const int hh = is_q ? h : h - q_heads;
    const bf16* src = (is_q ? q + t * q_ld : k + t * k_ld) + (long long)hh * head_dim;
    bf16* dst = is_q ? q_out + (t * q_heads + hh) * head_dim
                     : kcache + (((long long)b * kv_heads + hh) * max_seq + pos) * head_dim;
    if (c >= rot_chunks) {  // non-rotary tail
      const int e = rotary_dim + (c - rot_chunks) * 8;
      *reinterpret_cast<uint4*>(dst + e) = *reinterpret_cast<const uint4*>(src + e);
      continue;
    }
    if (!interleaved) {
      const int e = c * 8;
      uint4 lo = *reinterpret_cast<const uint4*>(src + e), hi = *reinterpret_cast<const uint4*>(src + e + half);
      uint32_t* lw = &lo.x;
      uint32_t* hw = &hi.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float a[2] = {__uint_as_float(lw[j] << 16), __uint_as_float(lw[j] & 0xFFFF0000u)};
        float bb[2] = {__uint_as_float(hw[j] << 16), __uint_as_float(hw[j] & 0xFFFF0000u)};
        float ra[2], rb[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int p = e + 2 * j + u;
          const float inv_freq = exp2f(-log2_theta * (2.f * float(p) / float(rotary_dim)));
          float sn, cs;
          sincosf(float(pos) * inv_freq, &sn, &cs);
          ra[u] = a[u] * cs - bb[u] * sn;
          rb[u] = bb[u] * cs + a[u] * sn;
        }
        __nv_bfloat162 o1 = __floats2bfloat162_rn(ra[0], ra[1]), o2 = __floats2bfloat162_rn(rb[0], rb[1]);
        lw[j] = *reinterpret_cast<uint32_t*>(&o1);
        hw[j] = *reinterpret_cast<uint32_t*>(&o2);
      }
      *reinterpret_cast<uint4*>(dst + e) = lo;
      *reinterpret_cast<uint4*>(dst + e + half) = hi;
    } else {
      const int e = c * 8;  // pairs (e, e+1), (e+2, e+3), ...
      uint4 val = *reinterpret_cast<const uint4*>(src + e);
      uint32_t* vw = &val.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = __uint_as_float(vw[j] << 16), bb = __uint_as_float(vw[j] & 0xFFFF0000u);
        const int p = (e >> 1) + j;
        const float inv_freq = exp2f(-log2_theta * (2.f * float(p) / float(rotary_dim)));
        float sn, cs;
        sincosf(float(pos) * inv_freq, &sn, &cs);
        __nv_bfloat162 o = __floats2bfloat162_rn(a * cs - bb * sn, bb * cs + a * sn);
        vw[j] = *reinterpret_cast<uint32_t*>(&o);
      }
      *reinterpret_cast<uint4*>(dst + e) = val;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// decode attention
// ------------------------------------------------------------------------------------------------
constexpr int DEC_WARPS = 8;
constexpr int DEC_THREADS = DEC_WARPS * 32;
constexpr int DEC_STAGES = 4;  // depth of the per-thread K/V ring: DEC_STAGES - 1 key groups are in flight while one is consumed

// Dynamic shared memory of the decode kernels: DEC_STAGES x {K, V} x 16-byte chunks x one slot per thread.
template <int D> constexpr size_t dec_ring_bytes() { return size_t(DEC_STAGES) * 2 * (D / 64) * DEC_THREADS * 16; }

// Element of the head vector that lane slice `part` (0..7) holds in position e of its registers: 16-byte chunk c = e / 8
// of a lane sits at elements [64 c + 8 part, +8), so the 8 lanes of a key cover 128 contiguous bytes per copy instruction
// (whole 32-byte sectors, no sector is requested twice).
__device__ __forceinline__ int dec_elem(int part, int e) { return (e >> 3) * 64 + part * 8 + (e & 7); }

template <int N> __device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Streams keys [k_begin, k_end) of one (sequence, KV head) through `consume(kf, vf, valid)`.  A warp takes four keys
// per iteration (8 lanes per key, EPL elements of K and of V per lane).  Every lane copies its own slices with
// cp.async into its private slots of a DEC_STAGES-deep ring, so several groups are in flight per lane without holding
// them in registers, and nobody reads another thread's slot (no barrier).  kbase / vbase already point at this
// lane's first chunk (element 8 * part of key 0); see dec_elem for the slice layout.  The trip count is uniform across the warp
// (consume() shuffles); lanes whose key is out of range copy nothing and pass valid = false.
template <int D, typename Consume>
__device__ __forceinline__ void stream_keys(const bf16* kbase, const bf16* vbase, int k_begin, int k_end, int warp, int sub,
                                            uint4* ring, Consume&& consume) {
  constexpr int EPL = D / 8, C = EPL / 8, STEP = DEC_WARPS * 4;
  auto slot = [&](int stage, int kv, int c) { return ring + ((stage * 2 + kv) * C + c) * DEC_THREADS + threadIdx.x; };
  auto issue = [&](int stage, int group_base) {
    const int key = group_base + sub;
    if (key < k_end) {
      const bf16* kp = kbase + (long long)key * D;
      const bf16* vp = vbase + (long long)key * D;
#pragma unroll
      for (int c = 0; c < C; ++c) {
        cp_async16(slot(stage, 0, c), kp + c * 64, true);
        cp_async16(slot(stage, 1, c), vp + c * 64, true);
      }
    }
    cp_async_commit();  // committed even when empty: the group count per iteration stays fixed
  };
  int key_base = k_begin + warp * 4;
#pragma unroll
  for (int st = 0; st < DEC_STAGES - 1; ++st) issue(st, key_base + st * STEP);
  for (int it = 0; key_base < k_end; key_base += STEP, ++it) {
    issue((it + DEC_STAGES - 1) % DEC_STAGES, key_base + (DEC_STAGES - 1) * STEP);
    cp_async_wait_group<DEC_STAGES - 1>();
    const int stage = it % DEC_STAGES;
    float kf[EPL], vf[EPL];
#pragma unroll
    for (int c = 0; c < C; ++c) {
      const uint4 kr = *slot(stage, 0, c), vr = *slot(stage, 1, c);
      const uint32_t kw[4] = {kr.x, kr.y, kr.z, kr.w}, vw[4] = {vr.x, vr.y, vr.z, vr.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        kf[c * 8 + 2 * j] = __uint_as_float(kw[j] << 16);
        kf[c * 8 + 2 * j + 1] = __uint_as_float(kw[j] & 0xFFFF0000u);
        vf[c * 8 + 2 * j] = __uint_as_float(vw[j] << 16);
        vf[c * 8 + 2 * j + 1] = __uint_as_float(vw[j] & 0xFFFF0000u);
      }
    }
    consume(kf, vf, key_base + sub < k_end);
  }
  cp_async_wait_group<0>();
}

template <int D, int G>
__global__ void __launch_bounds__(DEC_THREADS)
attn_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                   bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                   const int* __restrict__ len_ptr, int len_add, int q_heads, int kv_heads, int g_total, int g_offset,
                   int max_seq, int splits, float scale_log2e) {
  constexpr int EPL = D / 8;  // elements per lane (8 lanes cooperate on one key)
  const int bh = blockIdx.x;  // b * kv_heads + kvh
  const int b = bh / kv_heads, kvh = bh % kv_heads;
  const int split = blockIdx.y;
  const int len = (len_ptr ? len_ptr[0] : 0) + len_add;
  const int chunk = (len + splits - 1) / splits;
  const int k0 = split * chunk, k1 = min(len, k0 + chunk);

  __shared__ float q_s[G][D];
  __shared__ float red_o[DEC_WARPS][G][D];
  __shared__ float red_m[DEC_WARPS][G], red_l[DEC_WARPS][G];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane >> 3;   // which of the 4 keys of this warp iteration
  const int part = lane & 7;   // which D/8 slice
  for (int i = threadIdx.x; i < G * D; i += DEC_THREADS) {
    const int g = i / D, d = i % D;
    const int qh = kvh * g_total + g_offset + g;
    q_s[g][d] = __bfloat162float(q[((long long)b * q_heads + qh) * D + d]) * scale_log2e;
  }
  __syncthreads();

  float m[G], l[G], acc[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.f;
  }
  const bf16* kbase = kcache + (long long)bh * max_seq * D + part * 8;
  const bf16* vbase = vcache + (long long)bh * max_seq * D + part * 8;

  extern __shared__ uint4 dec_ring[];
  stream_keys<D>(kbase, vbase, k0, k1, warp, sub, dec_ring, [&](const float (&kf)[EPL], const float (&vf)[EPL], bool valid) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) s += kf[e] * q_s[g][dec_elem(part, e)];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      if (valid) {
        const float m_new = fmaxf(m[g], s);
        const float corr = exp2f(m[g] - m_new);
        const float pexp = exp2f(s - m_new);
        l[g] = l[g] * corr + pexp;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] = acc[g][e] * corr + pexp * vf[e];
        m[g] = m_new;
      }
    }
  });

  // merge the 4 key sub-groups of a warp (lanes differing in bits 3,4), then the warps
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int off = 8; off <= 16; off <<= 1) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m[g], off);
      const float l_o = __shfl_xor_sync(0xffffffffu, l[g], off);
      const float m_new = fmaxf(m[g], m_o);
      const float c_me = m[g] == -INFINITY ? 0.f : exp2f(m[g] - m_new);
      const float c_o = m_o == -INFINITY ? 0.f : exp2f(m_o - m_new);
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float a_o = __shfl_xor_sync(0xffffffffu, acc[g][e], off);
        acc[g][e] = acc[g][e] * c_me + a_o * c_o;
      }
      l[g] = l[g] * c_me + l_o * c_o;
      m[g] = m_new;
    }
    if (sub == 0) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) red_o[warp][g][dec_elem(part, e)] = acc[g][e];
      if (part == 0) { red_m[warp][g] = m[g]; red_l[warp][g] = l[g]; }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += DEC_THREADS) {
    const int g = i / D, d = i % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, red_m[w][g]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float c = red_m[w][g] == -INFINITY ? 0.f : exp2f(red_m[w][g] - mm);
      ll += red_l[w][g] * c;
      oo += red_o[w][g][d] * c;
    }
    const int qh = kvh * g_total + g_offset + g;
    const long long row = (long long)b * q_heads + qh;
    if (splits == 1) {
      out[row * D + d] = __float2bfloat16(ll > 0.f ? oo / ll : 0.f);
    } else {
      part_o[(row * splits + split) * D + d] = oo;
      if (d == 0) { part_ml[(row * splits + split) * 2] = mm; part_ml[(row * splits + split) * 2 + 1] = ll; }
    }
  }
}

template <int D>
__global__ void attn_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                           bf16* __restrict__ out, int splits) {
  const long long row = blockIdx.x;
  const int d = threadIdx.x;
  float mm = -INFINITY, ll = 0.f, oo = 0.f;
  for (int s0 = 0; s0 < splits; s0 += 8) {  // loads of 8 splits in flight at once
    float ms[8], ls[8], os[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const bool live = s0 + q < splits;
      const long long pr = row * splits + s0 + q;
      ms[q] = live ? part_ml[pr * 2] : -INFINITY;
      ls[q] = live ? part_ml[pr * 2 + 1] : 0.f;
      os[q] = live ? part_o[pr * D + d] : 0.f;
    }
    float m_new = mm;
#pragma unroll
    for (int q = 0; q < 8; ++q) m_new = fmaxf(m_new, ms[q]);
    const float c_old = mm == -INFINITY ? 0.f : exp2f(mm - m_new);
    ll *= c_old;
    oo *= c_old;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float c = ms[q] == -INFINITY ? 0.f : exp2f(ms[q] - m_new);
      ll += ls[q] * c;
      oo += os[q] * c;
    }
    mm = m_new;
  }
  out[row * D + d] = __float2bfloat16(ll > 0.f ? oo / ll : 0.f);
}

// ------------------------------------------------------------------------------------------------
// fused decode step: RoPE on q / k, cache append, split-KV attention and the split combine in ONE kernel
// ------------------------------------------------------------------------------------------------
// q / k / v are rows of the fused projection output (one new token per sequence).  The CTA whose key range
// contains the new position takes that key / value from the projection (rotated on the fly) instead of the
// cache and also stores them into the cache for later steps.  With splits > 1 every CTA parks its partial
// result; the last CTA to arrive for a (sequence, KV head) merges the partials (no second launch).
// counters: uint32 [batch * kv_heads], zero-initialised once; they re-arm themselves.
template <int D, int G>
__global__ void __launch_bounds__(DEC_THREADS)
attn_decode_fused_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                         bf16* __restrict__ kcache, bf16* __restrict__ vcache, bf16* __restrict__ out,
                         float* __restrict__ part_o, float* __restrict__ part_ml, uint32_t* __restrict__ counters,
                         const int* __restrict__ pos_ptr, int q_heads, int kv_heads, int g_total, int g_offset, int max_seq,
                         int splits, float scale_log2e, int rotary_dim, float log2_theta, int interleaved, long long q_ld,
                         long long k_ld, long long v_ld, const float2* __restrict__ rope_table, long long out_ld) {
  constexpr int EPL = D / 8;
  pdl_wait();
  const int bh = blockIdx.x;
  const int b = bh / kv_heads, kvh = bh % kv_heads;
  const int split = blockIdx.y;
  // several groups of G query heads of the same KV head may share a launch (grid z): each has its own arrival counter
  g_offset += blockIdx.z * G;
  counters += (size_t)blockIdx.z * gridDim.x;
  const int pos = pos_ptr[0];
  const int len = min(pos + 1, max_seq);
  const int chunk = (len + splits - 1) / splits;
  const int k0 = split * chunk, k1 = min(len, k0 + chunk);
  const bool owns_new = pos < max_seq && pos >= k0 && pos < k1;
  const int k1_cache = owns_new ? pos : k1;  // keys taken from the cache

  __shared__ float q_s[G][D];
  __shared__ float knew_s[D], vnew_s[D];
  __shared__ float red_o[DEC_WARPS][G][D];
  __shared__ float red_m[DEC_WARPS][G], red_l[DEC_WARPS][G];
  __shared__ uint32_t is_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane >> 3, part = lane & 7;
  const int half = rotary_dim >> 1;

  // rotate q (G heads) and the new k into shared memory; one thread per element pair
  for (int i = threadIdx.x; i < (G + 1) * (D / 2); i += DEC_THREADS) {
    const int hsel = i / (D / 2), p = i % (D / 2);
    const bool is_k = hsel == G;
    const bf16* src = is_k ? k + b * k_ld + (long long)kvh * D : q + b * q_ld + (long long)(kvh * g_total + g_offset + hsel) * D;
    float* dst = is_k ? knew_s : q_s[hsel];
    const float mul = is_k ? 1.f : scale_log2e;
    if (p < half) {
      const int ia = interleaved ? 2 * p : p;
      const int ib = interleaved ? 2 * p + 1 : p + half;
      float sn, cs;
      if (rope_table) {  // (cos, sin) of every position, filled by rope_table_kernel with the formula below
        const float2 t = __ldg(rope_table + (long long)pos * half + p);
        cs = t.x;
        sn = t.y;
      } else {
        const float inv_freq = exp2f(-log2_theta * (2.f * float(p) / float(rotary_dim)));
        sincosf(float(pos) * inv_freq, &sn, &cs);
      }
      const float a = __bfloat162float(src[ia]), c = __bfloat162float(src[ib]);
      // round through bf16 like the stand-alone append kernel, so cached and in-flight keys agree bit for bit
      dst[ia] = __bfloat162float(__float2bfloat16(a * cs - c * sn)) * mul;
      dst[ib] = __bfloat162float(__float2bfloat16(c * cs + a * sn)) * mul;
    } else {
      const int e = rotary_dim + 2 * (p - half);
      dst[e] = __bfloat162float(src[e]) * mul;
      dst[e + 1] = __bfloat162float(src[e + 1]) * mul;
    }
  }
  for (int i = threadIdx.x; i < D; i += DEC_THREADS) vnew_s[i] = __bfloat162float(v[b * v_ld + (long long)kvh * D + i]);
  __syncthreads();
  if (owns_new) {  // persist the new key / value for later steps
    for (int i = threadIdx.x; i < D; i += DEC_THREADS) {
      kcache[((long long)bh * max_seq + pos) * D + i] = __float2bfloat16(knew_s[i]);
      vcache[((long long)bh * max_seq + pos) * D + i] = __float2bfloat16(vnew_s[i]);
    }
  }

  float m[G], l[G], acc[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.f;
  }
  const bf16* kbase = kcache + (long long)bh * max_seq * D + part * 8;
  const bf16* vbase = vcache + (long long)bh * max_seq * D + part * 8;

  auto consume = [&](const float (&kf)[EPL], const float (&vf)[EPL], bool valid) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float sc = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) sc += kf[e] * q_s[g][dec_elem(part, e)];
      sc += __shfl_xor_sync(0xffffffffu, sc, 1);
      sc += __shfl_xor_sync(0xffffffffu, sc, 2);
      sc += __shfl_xor_sync(0xffffffffu, sc, 4);
      if (valid) {
        const float m_new = fmaxf(m[g], sc);
        const float corr = exp2f(m[g] - m_new);
        const float pexp = exp2f(sc - m_new);
        l[g] = l[g] * corr + pexp;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] = acc[g][e] * corr + pexp * vf[e];
        m[g] = m_new;
      }
    }
  };

  extern __shared__ uint4 dec_ring[];
  stream_keys<D>(kbase, vbase, k0, k1_cache, warp, sub, dec_ring, consume);
  if (owns_new && warp == 0) {  // the new token's key / value come straight from shared memory (warp-uniform branch)
    float kf[EPL], vf[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      kf[e] = __bfloat162float(__float2bfloat16(knew_s[dec_elem(part, e)]));
      vf[e] = __bfloat162float(__float2bfloat16(vnew_s[dec_elem(part, e)]));
    }
    consume(kf, vf, sub == 0);
  }

#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int off = 8; off <= 16; off <<= 1) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m[g], off);
      const float l_o = __shfl_xor_sync(0xffffffffu, l[g], off);
      const float m_new = fmaxf(m[g], m_o);
      const float c_me = m[g] == -INFINITY ? 0.f : exp2f(m[g] - m_new);
      const float c_o = m_o == -INFINITY ? 0.f : exp2f(m_o - m_new);
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float a_o = __shfl_xor_sync(0xffffffffu, acc[g][e], off);
        acc[g][e] = acc[g][e] * c_me + a_o * c_o;
      }
      l[g] = l[g] * c_me + l_o * c_o;
      m[g] = m_new;
    }
    if (sub == 0) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) red_o[warp][g][dec_elem(part, e)] = acc[g][e];
      if (part == 0) { red_m[warp][g] = m[g]; red_l[warp][g] = l[g]; }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += DEC_THREADS) {
    const int g = i / D, d = i % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, red_m[w][g]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float c = red_m[w][g] == -INFINITY ? 0.f : exp2f(red_m[w][g] - mm);
      ll += red_l[w][g] * c;
      oo += red_o[w][g][d] * c;
    }
    const int qh = kvh * g_total + g_offset + g;
    const long long row = (long long)b * q_heads + qh;
    if (splits == 1) {
      out[(long long)b * out_ld + (long long)qh * D + d] = __float2bfloat16(ll > 0.f ? oo / ll : 0.f);
    } else {
      part_o[(row * splits + split) * D + d] = oo;
      if (d == 0) { part_ml[(row * splits + split) * 2] = mm; part_ml[(row * splits + split) * 2 + 1] = ll; }
    }
  }
  if (splits == 1) return;
  // last split to arrive merges the partial results of all splits
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t old = atomicAdd(counters + bh, 1u);
    const bool last = old == uint32_t(splits - 1);
    if (last) counters[bh] = 0;
    is_last = last ? 1u : 0u;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int i = threadIdx.x; i < G * D; i += DEC_THREADS) {
    const int g = i / D, d = i % D;
    const long long row = (long long)b * q_heads + kvh * g_total + g_offset + g;
    // all loads of a batch of 8 splits are issued before the first one is used (each dependent load would cost a
    // full memory round trip); batches are folded with the running (max, sum, output) like one more online-softmax step
    float mm = -INFINITY, ll = 0.f, oo = 0.f;
    for (int s0 = 0; s0 < splits; s0 += 8) {
      float ms[8], ls[8], os[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const bool live = s0 + q < splits;
        const long long pr = row * splits + s0 + q;
        ms[q] = live ? __ldcg(part_ml + pr * 2) : -INFINITY;
        ls[q] = live ? __ldcg(part_ml + pr * 2 + 1) : 0.f;
        os[q] = live ? __ldcg(part_o + pr * D + d) : 0.f;
      }
      float m_new = mm;
#pragma unroll
      for (int q = 0; q < 8; ++q) m_new = fmaxf(m_new, ms[q]);
      const float c_old = mm == -INFINITY ? 0.f : exp2f(mm - m_new);
      ll *= c_old;
      oo *= c_old;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float c = ms[q] == -INFINITY ? 0.f : exp2f(ms[q] - m_new);
        ll += ls[q] * c;
        oo += os[q] * c;
      }
      mm = m_new;
    }
    out[(long long)b * out_ld + (long long)(kvh * g_total + g_offset + g) * D + d] = __float2bfloat16(ll > 0.f ? oo / ll : 0.f);
  }
}

// table[pos * (rotary_dim / 2) + p] = (cos, sin)(pos * theta^(-2p / rotary_dim)), the angles of the rotary embedding
__global__ void rope_table_kernel(float2* __restrict__ table, int positions, int half, int rotary_dim, float log2_theta) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= (long long)positions * half) return;
  const int pos = int(i / half), p = int(i % half);
  const float inv_freq = exp2f(-log2_theta * (2.f * float(p) / float(rotary_dim)));
  float sn, cs;
  sincosf(float(pos) * inv_freq, &sn, &cs);
  table[i] = make_float2(cs, sn);
}

// ------------------------------------------------------------------------------------------------
// prefill attention (legacy mma.sync tensor path; 64 query rows x 64 keys per step, 4 warps)
// ------------------------------------------------------------------------------------------------
// BIAS: 0 none, 1 fp32, 2 bf16 additive score bias addressed as bias[b * bias_sb + h * bias_sh + i * bias_sq + j * bias_sk]
// (a stride of 0 broadcasts: relative-position biases are [1, H, Sq, Sk], padding masks [B, 1, 1, Sk], ALiBi [1, H, 1, Sk]).
// The bias is in natural-log units like the scores; -inf entries mask a key.
template <int D, int BIAS = 0>
__global__ void __launch_bounds__(PF_THREADS)
attn_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                    bf16* __restrict__ out, float* __restrict__ lse, int sq, int sk, int q_heads, int kv_heads,
                    long long q_sb, long long q_ss, long long q_sh, long long k_sb, long long k_ss, long long k_sh,
                    long long v_sb, long long v_ss, long long v_sh, long long o_sb, long long o_ss, long long o_sh,
                    int causal, float scale_log2e, const void* __restrict__ bias = nullptr, long long bias_sb = 0,
                    long long bias_sh = 0, long long bias_sq = 0, long long bias_sk = 0) {
  extern __shared__ __align__(128) uint8_t pf_smem[];
  bf16* q_s = reinterpret_cast<bf16*>(pf_smem);
  bf16* k_s = q_s + PF_M * D;
  bf16* v_s = k_s + PF_N * D;

  const int mblk = (gridDim.x - 1 - blockIdx.x);  // heavy (late) causal blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (q_heads / kv_heads);
  const int q0 = mblk * PF_M;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int shift = sk - sq;  // query i may see keys j <= i + shift when causal

  const bf16* qg = q + b * q_sb + (long long)h * q_sh;
  const bf16* kg = k + b * k_sb + (long long)kvh * k_sh;
  const bf16* vg = v + b * v_sb + (long long)kvh * v_sh;

  int kv_end = sk;
  if (causal) kv_end = min(sk, q0 + PF_M + shift);
  const int n_iters = kv_end > 0 ? (kv_end + PF_N - 1) / PF_N : 0;

  load_tile<D>(q_s, qg, q_ss, q0, sq);
  if (n_iters > 0) load_tile<D>(k_s, kg, k_ss, 0, sk);
  cp_async_commit();

  uint32_t qf[D / 16][4];
  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  for (int it = 0; it < n_iters; ++it) {
    const int kv0 = it * PF_N;
    cp_async_wait_all();
    __syncthreads();  // K(it) (and Q) landed; every warp is done with V(it-1)
    load_tile<D>(v_s, vg, v_ss, kv0, sk);
    cp_async_commit();
    if (it == 0) {
      const int id = lane >> 3, r = lane & 7;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks)
        ldmatrix_x4(qf[ks], tile_ptr<D>(q_s, warp * 16 + (id & 1) * 8 + r, ks * 2 + (id >> 1)));
    }
    // S = Q K^T  (16 x 64 per warp)
    float s_acc[PF_N / 8][4];
#pragma unroll
    for (int i = 0; i < PF_N / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s_acc[i][j] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int np = 0; np < PF_N / 16; ++np) {
        uint32_t kb[4];
        const int id = lane >> 3, r = lane & 7;
        ldmatrix_x4(kb, tile_ptr<D>(k_s, np * 16 + (id >> 1) * 8 + r, ks * 2 + (id & 1)));
        mma_bf16_16816(s_acc[2 * np], qf[ks], kb[0], kb[1]);
        mma_bf16_16816(s_acc[2 * np + 1], qf[ks], kb[2], kb[3]);
      }
    }
    // mask + online softmax (rows g and g+8 of this warp's 16 rows)
    const int qi0 = q0 + warp * 16 + g;
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int nt = 0; nt < PF_N / 8; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = kv0 + nt * 8 + 2 * t4 + (j & 1);
        const int qi = qi0 + (j >> 1) * 8;
        const bool dead = key >= sk || (causal && key > qi + shift);
        float sv = dead ? -INFINITY : s_acc[nt][j] * scale_log2e;
        if (BIAS != 0 && !dead && qi < sq) {
          const long long bi = b * bias_sb + h * bias_sh + (long long)qi * bias_sq + (long long)key * bias_sk;
          const float bv = BIAS == 1 ? __ldg(static_cast<const float*>(bias) + bi)
                                     : __bfloat162float(static_cast<const bf16*>(bias)[bi]);
          sv += bv * 1.4426950408889634f;
        }
        s_acc[nt][j] = sv;
        m_new[j >> 1] = fmaxf(m_new[j >> 1], sv);
      }
    }
#pragma unroll
    for (int r2 = 0; r2 < 2; ++r2) {
      m_new[r2] = fmaxf(m_new[r2], __shfl_xor_sync(0xffffffffu, m_new[r2], 1));
      m_new[r2] = fmaxf(m_new[r2], __shfl_xor_sync(0xffffffffu, m_new[r2], 2));
    }
    float corr[2], base[2], row_sum[2] = {0.f, 0.f};
#pragma unroll
    for (int r2 = 0; r2 < 2; ++r2) {
      base[r2] = m_new[r2] == -INFINITY ? 0.f : m_new[r2];
      corr[r2] = m_run[r2] == -INFINITY ? 0.f : exp2f(m_run[r2] - base[r2]);
      m_run[r2] = m_new[r2];
    }
    uint32_t pf[PF_N / 16][4];
#pragma unroll
    for (int nt = 0; nt < PF_N / 8; ++nt) {
      const float p0 = exp2f(s_acc[nt][0] - base[0]), p1 = exp2f(s_acc[nt][1] - base[0]);
      const float p2 = exp2f(s_acc[nt][2] - base[1]), p3 = exp2f(s_acc[nt][3] - base[1]);
      row_sum[0] += p0 + p1;
      row_sum[1] += p2 + p3;
      __nv_bfloat162 lo = __floats2bfloat162_rn(p0, p1), hi = __floats2bfloat162_rn(p2, p3);
      pf[nt >> 1][(nt & 1) * 2] = *reinterpret_cast<uint32_t*>(&lo);
      pf[nt >> 1][(nt & 1) * 2 + 1] = *reinterpret_cast<uint32_t*>(&hi);
    }
#pragma unroll
    for (int r2 = 0; r2 < 2; ++r2) l_run[r2] = l_run[r2] * corr[r2] + row_sum[r2];
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      o_acc[dt][0] *= corr[0]; o_acc[dt][1] *= corr[0];
      o_acc[dt][2] *= corr[1]; o_acc[dt][3] *= corr[1];
    }
    cp_async_wait_all();
    __syncthreads();  // V(it) landed; every warp is done with K(it)
    if (it + 1 < n_iters) {
      load_tile<D>(k_s, kg, k_ss, kv0 + PF_N, sk);
      cp_async_commit();
    }
    // O += P V
#pragma unroll
    for (int ks = 0; ks < PF_N / 16; ++ks) {
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t vb[4];
        const int id = lane >> 3, r = lane & 7;
        ldmatrix_x4_trans(vb, tile_ptr<D>(v_s, ks * 16 + (id & 1) * 8 + r, dp * 2 + (id >> 1)));
        mma_bf16_16816(o_acc[2 * dp], pf[ks], vb[0], vb[1]);
        mma_bf16_16816(o_acc[2 * dp + 1], pf[ks], vb[2], vb[3]);
      }
    }
  }
  cp_async_wait_all();

  // finalize: row sums live in quads
#pragma unroll
  for (int r2 = 0; r2 < 2; ++r2) {
    l_run[r2] += __shfl_xor_sync(0xffffffffu, l_run[r2], 1);
    l_run[r2] += __shfl_xor_sync(0xffffffffu, l_run[r2], 2);
  }
#pragma unroll
  for (int r2 = 0; r2 < 2; ++r2) {
    const int qi = q0 + warp * 16 + g + r2 * 8;
    if (qi >= sq) continue;
    const float inv = l_run[r2] > 0.f ? 1.f / l_run[r2] : 0.f;
    bf16* orow = out + b * o_sb + (long long)qi * o_ss + (long long)h * o_sh;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      __nv_bfloat162 o2 = __floats2bfloat162_rn(o_acc[dt][r2 * 2] * inv, o_acc[dt][r2 * 2 + 1] * inv);
      *reinterpret_cast<__nv_bfloat162*>(orow + dt * 8 + 2 * t4) = o2;
    }
    if (lse && t4 == 0)
      lse[((long long)b * q_heads + h) * sq + qi] =
          l_run[r2] > 0.f ? (m_run[r2] * 0.6931471805599453f + logf(l_run[r2])) : -INFINITY;
  }
}

}  // namespace tpb

using namespace tpb;

extern "C" int tpb_qkv_rope_append(const void* q, const void* k, const void* v, void* q_out, void* kcache, void* vcache,
                                   const int* base_pos, int batch, int seq, int q_heads, int kv_heads, int head_dim,
                                   int rotary_dim, float theta, int interleaved, int max_seq, long long q_ld,
                                   long long k_ld, long long v_ld, void* stream_) {
  if (!q || !k || !v || !q_out || !kcache || !vcache || batch <= 0 || seq <= 0) return TPB_ERR_ARG;
  if ((head_dim & 1) || (rotary_dim & 1) || rotary_dim > head_dim || (q_ld & 1) || (k_ld & 1) || (v_ld & 1)) return TPB_ERR_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const int half_ = rotary_dim / 2;
  const bool vec_ok = (head_dim % 8 == 0) && (interleaved ? rotary_dim % 8 == 0 : half_ % 8 == 0) && !(q_ld & 7) && !(k_ld & 7) &&
                      !(v_ld & 7) && !((uintptr_t)q & 15) && !((uintptr_t)k & 15) && !((uintptr_t)v & 15) && !((uintptr_t)q_out & 15) &&
                      !((uintptr_t)kcache & 15) && !((uintptr_t)vcache & 15);
  if (vec_ok) {
    const int rot_chunks = interleaved ? rotary_dim / 8 : half_ / 8;
    const long long per_token = (long long)(q_heads + kv_heads) * (rot_chunks + (head_dim - rotary_dim) / 8) + (long long)kv_heads * (head_dim / 8);
    const long long vwork = (long long)batch * seq * per_token;
    long long vgrid = (vwork + 255) / 256;
    if (vgrid > 148 * 32) vgrid = 148 * 32;
    qkv_rope_append_vec_kernel<<<int(vgrid), 256, 0, s>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, (bf16*)q_out, (bf16*)kcache,
                                                          (bf16*)vcache, base_pos, batch, seq, q_heads, kv_heads, head_dim, rotary_dim,
                                                          log2f(theta), interleaved, max_seq, q_ld, k_ld, v_ld);
    return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
  }
  const long long work = (long long)batch * seq * (q_heads + 2 * kv_heads) * (head_dim / 2);
  long long grid = (work + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  qkv_rope_append_kernel<<<int(grid), 256, 0, s>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, (bf16*)q_out, (bf16*)kcache,
                                                   (bf16*)vcache, base_pos, batch, seq, q_heads, kv_heads, head_dim, rotary_dim,
                                                   log2f(theta), interleaved, max_seq, q_ld, k_ld, v_ld);
  return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

// Kernels launched by the most recent tpb_attn_decode / tpb_attn_decode_fused call of this thread.
static thread_local int g_last_launches = 0;
extern "C" int tpb_last_launches(void) { return g_last_launches; }

// Opts a decode kernel instantiation in to its dynamic shared memory (once per kernel and device).
template <auto Kernel>
static bool dec_smem_ready(size_t bytes) {
  static std::atomic<bool> done[64];  // one array per kernel instantiation; rank threads of one process may race here
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  if (!done[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)) != cudaSuccess) return false;
    done[dev].store(true, std::memory_order_release);
  }
  return true;
}

// workspace: part_o fp32 [batch*q_heads*splits*head_dim], part_ml fp32 [batch*q_heads*splits*2]
extern "C" int tpb_attn_decode(const void* q, const void* kcache, const void* vcache, void* out, float* part_o,
                               float* part_ml, const int* len_ptr, int len_add, int batch, int q_heads, int kv_heads,
                               int head_dim, int max_seq, int splits, float scale, void* stream_) {
  if (!q || !kcache || !vcache || !out || batch <= 0 || splits < 1 || q_heads % kv_heads) return TPB_ERR_ARG;
  if (splits > 1 && (!part_o || !part_ml)) return TPB_ERR_ARG;
  if (head_dim != 64 && head_dim != 128) return TPB_ERR_SIZE;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const int g_total = q_heads / kv_heads;
  const float sl2 = scale * 1.4426950408889634f;
  dim3 grid(batch * kv_heads, splits);
  int done = 0, launches = 0;
  while (done < g_total) {
    const int left = g_total - done;
    const int gmax = head_dim == 128 ? 4 : 8;
    int gnow = 1;
    while (gnow * 2 <= left && gnow * 2 <= gmax) gnow *= 2;
#define DEC(D, G)                                                                                                      \
  if (!dec_smem_ready<attn_decode_kernel<D, G>>(dec_ring_bytes<D>())) return TPB_ERR_CUDA;                               \
  attn_decode_kernel<D, G><<<grid, DEC_THREADS, dec_ring_bytes<D>(), s>>>(                                                \
      (const bf16*)q, (const bf16*)kcache, (const bf16*)vcache, (bf16*)out, part_o, part_ml, len_ptr, len_add, q_heads,   \
      kv_heads, g_total, done, max_seq, splits, sl2)
    if (head_dim == 128) {
      if (gnow == 1) { DEC(128, 1); } else if (gnow == 2) { DEC(128, 2); } else { DEC(128, 4); }
    } else {
      if (gnow == 1) { DEC(64, 1); } else if (gnow == 2) { DEC(64, 2); } else if (gnow == 4) { DEC(64, 4); } else { DEC(64, 8); }
    }
#undef DEC
    done += gnow;
    ++launches;
  }
  if (splits > 1) {
    if (head_dim == 128)
      attn_decode_combine_kernel<128><<<batch * q_heads, 128, 0, s>>>(part_o, part_ml, (bf16*)out, splits);
    else
      attn_decode_combine_kernel<64><<<batch * q_heads, 64, 0, s>>>(part_o, part_ml, (bf16*)out, splits);
    ++launches;
  }
  g_last_launches = launches;
  return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

// Strides are in elements; head_dim must be contiguous (stride 1) in q, k, v and out.  bias (may be null) is an
// additive score bias of dtype bias_dtype (0 bf16, 1 fp32) with element strides bias_s* over (batch, head, query, key);
// a stride of 0 broadcasts that dimension.
extern "C" int tpb_attn_prefill_bias(const void* q, const void* k, const void* v, void* out, float* lse, int batch, int sq,
                                     int sk, int q_heads, int kv_heads, int head_dim, long long q_sb, long long q_ss,
                                     long long q_sh, long long k_sb, long long k_ss, long long k_sh, long long v_sb,
                                     long long v_ss, long long v_sh, long long o_sb, long long o_ss, long long o_sh,
                                     int causal, float scale, const void* bias, int bias_dtype, long long bias_sb,
                                     long long bias_sh, long long bias_sq, long long bias_sk, void* stream_) {
  if (!q || !k || !v || !out || batch <= 0 || sq <= 0 || sk <= 0 || q_heads % kv_heads) return TPB_ERR_ARG;
  if (head_dim != 64 && head_dim != 128) return TPB_ERR_SIZE;
  if ((q_ss & 7) || (q_sh & 7) || (q_sb & 7) || (k_ss & 7) || (k_sh & 7) || (k_sb & 7) || (v_ss & 7) || (v_sh & 7) ||
      (v_sb & 7) || (o_ss & 1) || (o_sh & 1) || (o_sb & 1) || ((uintptr_t)q & 15) || ((uintptr_t)k & 15) || ((uintptr_t)v & 15))
    return TPB_ERR_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  dim3 grid((sq + PF_M - 1) / PF_M, q_heads, batch);
  const float sl2 = scale * 1.4426950408889634f;
  const size_t smem = size_t(PF_M + 2 * PF_N) * head_dim * 2;
  if (bias && bias_dtype != 0 && bias_dtype != 1) return TPB_ERR_ARG;
#define PF_LAUNCH(D, B)                                                                                                   \
  do {                                                                                                                    \
    if (!dec_smem_ready<attn_prefill_kernel<D, B>>(smem)) return TPB_ERR_CUDA;                                            \
    attn_prefill_kernel<D, B><<<grid, PF_THREADS, smem, s>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, (bf16*)out, lse, sq, sk, \
                                                             q_heads, kv_heads, q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh,  \
                                                             o_sb, o_ss, o_sh, causal, sl2, bias, bias_sb, bias_sh, bias_sq, bias_sk); \
  } while (0)
  const int mode = !bias ? 0 : (bias_dtype == 1 ? 1 : 2);
  if (head_dim == 128) {
    if (mode == 0) PF_LAUNCH(128, 0); else if (mode == 1) PF_LAUNCH(128, 1); else PF_LAUNCH(128, 2);
  } else {
    if (mode == 0) PF_LAUNCH(64, 0); else if (mode == 1) PF_LAUNCH(64, 1); else PF_LAUNCH(64, 2);
  }
#undef PF_LAUNCH
  return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

extern "C" int tpb_attn_prefill(const void* q, const void* k, const void* v, void* out, float* lse, int batch, int sq,
                                int sk, int q_heads, int kv_heads, int head_dim, long long q_sb, long long q_ss,
                                long long q_sh, long long k_sb, long long k_ss, long long k_sh, long long v_sb,
                                long long v_ss, long long v_sh, long long o_sb, long long o_ss, long long o_sh,
                                int causal, float scale, void* stream_) {
  return tpb_attn_prefill_bias(q, k, v, out, lse, batch, sq, sk, q_heads, kv_heads, head_dim, q_sb, q_ss, q_sh, k_sb, k_ss,
                               k_sh, v_sb, v_ss, v_sh, o_sb, o_ss, o_sh, causal, scale, nullptr, 0, 0, 0, 0, 0, stream_);
}

// Fills table [positions][rotary_dim / 2] of (cos, sin) pairs (fp32) for tpb_attn_decode_fused's rope_table argument:
// the decode kernel then looks the angles of the new position up instead of evaluating sincosf in every CTA.
extern "C" int tpb_rope_table(void* table, int positions, int rotary_dim, float theta, void* stream_) {
  if (!table || positions <= 0 || rotary_dim <= 0 || (rotary_dim & 1)) return TPB_ERR_ARG;
  const long long n = (long long)positions * (rotary_dim / 2);
  rope_table_kernel<<<int((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<float2*>(table), positions, rotary_dim / 2, rotary_dim, log2f(theta));
  return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

// One launch per decode step and layer: RoPE(q, k) + cache append + attention over [0, pos] + split combine.
// q / k / v: rows of the projection output for ONE new token per sequence ([batch, heads * head_dim], row pitches
// q_ld / k_ld / v_ld); pos_ptr[0] = position of the new token = number of tokens already cached.
// part_o / part_ml as for tpb_attn_decode; counters: uint32 [counter_elems] >= batch * kv_heads, zeroed once by the caller;
// with batch * q_heads of them every group of query heads of a KV head fits into ONE launch (GQA / MQA with large groups).
// rope_table: optional output of tpb_rope_table covering every position < max_seq (null: angles are computed in place).
// out: [batch][q_heads * head_dim] with a row pitch of out_ld elements (<= 0: dense).
extern "C" int tpb_attn_decode_fused(const void* q, const void* k, const void* v, void* kcache, void* vcache, void* out,
                                     float* part_o, float* part_ml, void* counters, const int* pos_ptr, int batch, int q_heads,
                                     int kv_heads, int head_dim, int max_seq, int splits, float scale, int rotary_dim, float theta,
                                     int interleaved, long long q_ld, long long k_ld, long long v_ld, const void* rope_table,
                                     long long out_ld, int counter_elems, void* stream_) {
  if (!q || !k || !v || !kcache || !vcache || !out || !pos_ptr || batch <= 0 || splits < 1 || q_heads % kv_heads) return TPB_ERR_ARG;
  if (splits > 1 && (!part_o || !part_ml || !counters)) return TPB_ERR_ARG;
  if (head_dim != 64 && head_dim != 128) return TPB_ERR_SIZE;
  if ((rotary_dim & 1) || rotary_dim > head_dim) return TPB_ERR_ARG;
  if (out_ld <= 0) out_ld = (long long)q_heads * head_dim;  // (rows of `out` may be column slices of a wider buffer)
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const int g_total = q_heads / kv_heads;
  const float sl2 = scale * 1.4426950408889634f;
  const float l2t = log2f(theta);
  int done = 0, launches = 0;
  while (done < g_total) {
    const int left = g_total - done;
    const int gmax = head_dim == 128 ? 4 : 8;
    int gnow = 1;
    while (gnow * 2 <= left && gnow * 2 <= gmax) gnow *= 2;
    // equal groups share one launch (grid z) when the caller's counter array has a counter for each of them
    int reps = left / gnow;
    if (splits > 1 && (long long)batch * kv_heads * reps > counter_elems) reps = 1;
    dim3 grid(batch * kv_heads, splits, reps);
#define DECF(D, G)                                                                                                           \
  if (!dec_smem_ready<attn_decode_fused_kernel<D, G>>(dec_ring_bytes<D>())) return TPB_ERR_CUDA;                               \
  launch_kernel(attn_decode_fused_kernel<D, G>, grid, dim3(DEC_THREADS), dec_ring_bytes<D>(), s, (const bf16*)q, (const bf16*)k, (const bf16*)v, \
                (bf16*)kcache, (bf16*)vcache, (bf16*)out, part_o, part_ml, (uint32_t*)counters, pos_ptr, q_heads, kv_heads, g_total, \
                done, max_seq, splits, sl2, rotary_dim, l2t, interleaved, q_ld, k_ld, v_ld, (const float2*)rope_table, out_ld)
    if (head_dim == 128) {
      if (gnow == 1) { DECF(128, 1); } else if (gnow == 2) { DECF(128, 2); } else { DECF(128, 4); }
    } else {
      if (gnow == 1) { DECF(64, 1); } else if (gnow == 2) { DECF(64, 2); } else if (gnow == 4) { DECF(64, 4); } else { DECF(64, 8); }
    }
#undef DECF
    done += gnow * reps;
    ++launches;
  }
  g_last_launches = launches;
  return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of tpb_attn_decode (declared and documented in tpb_noalloc.h).
// ------------------------------------------------------------------------------------------------
#include <mutex>

#include "tpb_noalloc.h"

// Workspace of the split-KV partial results, owned by the library.  In host code this name is only a
// handle for cudaGetSymbolAddress, never a pointer that a kernel could use.
static __device__ __align__(256) float g_noalloc_decode_scratch[TPB_NOALLOC_SCRATCH_FLOATS];

namespace {
std::mutex g_noalloc_mutex;
float* g_noalloc_scratch_addr[64] = {nullptr};  // per device: device address of the array above

// Device address of the workspace on the current device; resolved once per device.
int noalloc_scratch(float** addr) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TPB_ERR_CUDA;
  std::lock_guard<std::mutex> guard(g_noalloc_mutex);
  if (!g_noalloc_scratch_addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_decode_scratch) != cudaSuccess || !p) return TPB_ERR_CUDA;
    g_noalloc_scratch_addr[dev] = static_cast<float*>(p);
  }
  *addr = g_noalloc_scratch_addr[dev];
  return TPB_OK;
}
}  // namespace

extern "C" int tpb_attn_decode_noalloc(const void* q, const void* kcache, const void* vcache, void* out,
                                       const int* len_ptr, int len_add, int batch, int q_heads, int kv_heads,
                                       int head_dim, int max_seq, int splits, float scale, void* stream_) {
  if (!q || !kcache || !vcache || !out || batch <= 0 || q_heads <= 0 || kv_heads <= 0 || splits < 1) return TPB_ERR_ARG;
  if (head_dim != 64 && head_dim != 128) return TPB_ERR_SIZE;
  const long long rows = (long long)batch * q_heads * splits;
  if (rows * (head_dim + 2) > (long long)TPB_NOALLOC_SCRATCH_FLOATS) return TPB_ERR_SIZE;
  float* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc != TPB_OK) return rc;
  // layout inside the workspace: [rows * head_dim] partial outputs, then [rows * 2] (max, sum) pairs
  float* part_o = scratch;
  float* part_ml = scratch + rows * head_dim;
  return tpb_attn_decode(q, kcache, vcache, out, part_o, part_ml, len_ptr, len_add, batch, q_heads, kv_heads, head_dim,
                         max_seq, splits, scale, stream_);
}
