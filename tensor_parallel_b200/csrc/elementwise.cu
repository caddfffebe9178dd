// Memory-bound operators: RMSNorm / LayerNorm (forward + backward, optional fused residual add),
// rotary embedding, gated / plain activations (forward + backward), embedding gather, fused AdamW,
// dtype casts.  All kernels move data with 16-byte vector accesses and keep a row resident in
// registers between the statistics pass and the normalisation pass, so every tensor is read once.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "launch.cuh"
#include "ptx_sm100.cuh"
#include "tpb_api.h"

namespace tpb {

typedef __nv_bfloat16 bf16;

template <typename T> struct Vec8 {};  // 8 elements of T <-> 8 floats
template <> struct Vec8<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float (&v)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
  static __device__ __forceinline__ void store(bf16* p, const float (&v)[8]) {
    uint4 u;
    uint32_t* w = &u.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
};

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<bf16>(bf16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ bf16 from_f<bf16>(float x) { return __float2bfloat16(x); }
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// block-wide sum of up to two values; blockDim.x <= 1024
__device__ __forceinline__ void block_sum2(float& a, float& b) {
  __shared__ float sa[32], sb[32];
  a = warp_sum(a);
  b = warp_sum(b);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) { sa[warp] = a; sb[warp] = b; }
  __syncthreads();
  a = lane < nw ? sa[lane] : 0.f;
  b = lane < nw ? sb[lane] : 0.f;
  a = warp_sum(a);
  b = warp_sum(b);
}

// ------------------------------------------------------------------------------------------------
// Norms.  One CTA per row; a thread holds up to MAXV vectors of 8 elements (cols <= blockDim*8*MAXV).
// mode 0 = RMSNorm (no mean, no bias), mode 1 = LayerNorm.
// If residual != null:  h = x + residual is normalised and also written to sum_out.
// ------------------------------------------------------------------------------------------------
constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV = 8;  // cols <= 16384

// MAXV = vectors of 8 elements a thread may hold (cols <= 256 * 8 * MAXV); small MAXV keeps the register count
// low so that more rows are in flight per SM.
template <typename T, int MODE, int MAXV>
__global__ void __launch_bounds__(NORM_THREADS)
norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ weight,
                const T* __restrict__ bias, T* __restrict__ out, T* __restrict__ sum_out, float* __restrict__ rstd_out,
                float* __restrict__ mean_out, int cols, float eps) {
  pdl_wait();
  const size_t row = blockIdx.x;
  const T* xr = x + row * cols;
  const int nvec = cols >> 3;
  float v[MAXV][8];
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = threadIdx.x + i * NORM_THREADS;
    if (vi < nvec) {
      Vec8<T>::load(xr + vi * 8, v[i]);
      if (residual) {
        float r[8];
        Vec8<T>::load(residual + row * cols + vi * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += r[j];
        if (sum_out) {
          // round to the storage type first so that the statistics match what later kernels will read
          Vec8<T>::store(sum_out + row * cols + vi * 8, v[i]);
          Vec8<T>::load(sum_out + row * cols + vi * 8, v[i]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { s1 += v[i][j]; s2 += v[i][j] * v[i][j]; }
    }
  }
  block_sum2(s1, s2);
  const float inv_n = 1.f / float(cols);
  const float mean = MODE == 1 ? s1 * inv_n : 0.f;
  const float var = MODE == 1 ? fmaxf(s2 * inv_n - mean * mean, 0.f) : s2 * inv_n;
  const float rstd = rsqrtf(var + eps);
  if (threadIdx.x == 0) {
    if (rstd_out) rstd_out[row] = rstd;
    if (mean_out) mean_out[row] = mean;
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int vi = threadIdx.x + i * NORM_THREADS;
    if (vi < nvec) {
      float w[8], b[8], o[8];
      if (weight) Vec8<T>::load(weight + vi * 8, w);
      if (MODE == 1 && bias) Vec8<T>::load(bias + vi * 8, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float y = (v[i][j] - mean) * rstd;
        if (weight) y *= w[j];
        if (MODE == 1 && bias) y += b[j];
        o[j] = y;
      }
      Vec8<T>::store(out + row * cols + vi * 8, o);
    }
  }
}

// Backward: dx per row; dweight / dbias accumulated with fp32 atomics into zero-initialised buffers.
// Each CTA handles ROWS_PER_CTA consecutive rows and keeps its column partial sums in registers.
constexpr int NORM_BWD_MAXV = 4;  // cols <= 8192 in the backward kernel (register limit)

template <typename T, int MODE>
__global__ void __launch_bounds__(NORM_THREADS)
norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ weight,
                const float* __restrict__ rstd_in, const float* __restrict__ mean_in, T* __restrict__ dx,
                float* __restrict__ dweight, float* __restrict__ dbias, int rows, int cols, int rows_per_cta) {
  const int nvec = cols >> 3;
  float dw_acc[NORM_BWD_MAXV][8], db_acc[NORM_BWD_MAXV][8];
#pragma unroll
  for (int i = 0; i < NORM_BWD_MAXV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { dw_acc[i][j] = 0.f; db_acc[i][j] = 0.f; }
  const int row0 = blockIdx.x * rows_per_cta;
  const int row1 = min(rows, row0 + rows_per_cta);
  for (int row = row0; row < row1; ++row) {
    const float rstd = rstd_in[row];
    const float mean = MODE == 1 ? mean_in[row] : 0.f;
    float xh[NORM_BWD_MAXV][8], g[NORM_BWD_MAXV][8];
    float s1 = 0.f, s2 = 0.f;  // sum(g), sum(g * xhat)
#pragma unroll
    for (int i = 0; i < NORM_BWD_MAXV; ++i) {
      const int vi = threadIdx.x + i * NORM_THREADS;
      if (vi < nvec) {
        float d[8], xv[8], w[8];
        Vec8<T>::load(dy + size_t(row) * cols + vi * 8, d);
        Vec8<T>::load(x + size_t(row) * cols + vi * 8, xv);
        if (weight) Vec8<T>::load(weight + vi * 8, w);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xv[j] - mean) * rstd;
          dw_acc[i][j] += d[j] * xh[i][j];
          db_acc[i][j] += d[j];
          g[i][j] = weight ? d[j] * w[j] : d[j];
          s1 += g[i][j];
          s2 += g[i][j] * xh[i][j];
        }
      }
    }
    block_sum2(s1, s2);
    const float inv_n = 1.f / float(cols);
    const float c1 = MODE == 1 ? s1 * inv_n : 0.f;
    const float c2 = s2 * inv_n;
#pragma unroll
    for (int i = 0; i < NORM_BWD_MAXV; ++i) {
      const int vi = threadIdx.x + i * NORM_THREADS;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (g[i][j] - c1 - xh[i][j] * c2) * rstd;
        Vec8<T>::store(dx + size_t(row) * cols + vi * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NORM_BWD_MAXV; ++i) {
    const int vi = threadIdx.x + i * NORM_THREADS;
    if (vi < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (dweight) atomicAdd(dweight + vi * 8 + j, dw_acc[i][j]);
        if (MODE == 1 && dbias) atomicAdd(dbias + vi * 8 + j, db_acc[i][j]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Rotary embedding on x[tokens, heads, head_dim] (in place allowed), positions[tokens] (int64) or a
// device scalar base position (for graph-replayed decode steps): pos = base[0] + token % seq.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, T* __restrict__ out, const int64_t* __restrict__ positions,
                            const int* __restrict__ base_pos, int seq, int tokens, int heads, int head_dim,
                            int rotary_dim, float log2_theta, int interleaved, int inverse, long long x_stride_tok,
                            long long out_stride_tok) {
  const int half = rotary_dim >> 1;
  const long long total = (long long)tokens * heads * half;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int p = int(i % half);
    const int h = int((i / half) % heads);
    const int t = int(i / ((long long)half * heads));
    const float pos = positions ? float(positions[t]) : float(base_pos[0] + (t % seq));
    const float inv_freq = exp2f(-log2_theta * (2.f * float(p) / float(rotary_dim)));
    float s, c;
    sincosf(pos * inv_freq, &s, &c);
    if (inverse) s = -s;
    const int ia = interleaved ? 2 * p : p;
    const int ib = interleaved ? 2 * p + 1 : p + half;
    const T* xp = x + t * x_stride_tok + (long long)h * head_dim;
    T* op = out + t * out_stride_tok + (long long)h * head_dim;
    const float a = to_f<T>(xp[ia]), b = to_f<T>(xp[ib]);
    op[ia] = from_f<T>(a * c - b * s);
    op[ib] = from_f<T>(b * c + a * s);
  }
}

// bf16 fast path: one thread rotates 8 consecutive elements of the first rotary half with their partners in the
// second half (split layout) or 4 adjacent pairs (interleaved layout) using 16-byte accesses.
__global__ void rope_vec_kernel(const bf16* __restrict__ x, bf16* __restrict__ out, const int64_t* __restrict__ positions,
                                const int* __restrict__ base_pos, int seq, int tokens, int heads, int head_dim, int rotary_dim,
                                float log2_theta, int interleaved, int inverse, long long x_stride_tok, long long out_stride_tok) {
  const int half = rotary_dim >> 1;
  const int chunks = interleaved ? rotary_dim / 8 : half / 8;
  const long long total = (long long)tokens * heads * chunks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = int(i % chunks);
    const int h = int((i / chunks) % heads);
    const int t = int(i / ((long long)chunks * heads));
    const float pos = positions ? float(positions[t]) : float(base_pos[0] + (t % seq));
    const bf16* xp = x + t * x_stride_tok + (long long)h * head_dim;
    bf16* op = out + t * out_stride_tok + (long long)h * head_dim;
    const int e = c * 8;
    if (!interleaved) {
      uint4 lo = *reinterpret_cast<const uint4*>(xp + e), hi = *reinterpret_cast<const uint4*>(xp + e + half);
      uint32_t* lw = &lo.x;
      uint32_t* hw = &hi.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a[2] = {__uint_as_float(lw[j] << 16), __uint_as_float(lw[j] & 0xFFFF0000u)};
        const float b[2] = {__uint_as_float(hw[j] << 16), __uint_as_float(hw[j] & 0xFFFF0000u)};
        float ra[2], rb[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const float inv_freq = exp2f(-log2_theta * (2.f * float(e + 2 * j + u) / float(rotary_dim)));
          float sn, cs;
          sincosf(pos * inv_freq, &sn, &cs);
          if (inverse) sn = -sn;
          ra[u] = a[u] * cs - b[u] * sn;
          rb[u] = b[u] * cs + a[u] * sn;
        }
        __nv_bfloat162 o1 = __floats2bfloat162_rn(ra[0], ra[1]), o2 = __floats2bfloat162_rn(rb[0], rb[1]);
        lw[j] = *reinterpret_cast<uint32_t*>(&o1);
        hw[j] = *reinterpret_cast<uint32_t*>(&o2);
      }
      *reinterpret_cast<uint4*>(op + e) = lo;
      *reinterpret_cast<uint4*>(op + e + half) = hi;
    } else {
      uint4 val = *reinterpret_cast<const uint4*>(xp + e);
      uint32_t* vw = &val.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = __uint_as_float(vw[j] << 16), b = __uint_as_float(vw[j] & 0xFFFF0000u);
        const float inv_freq = exp2f(-log2_theta * (2.f * float((e >> 1) + j) / float(rotary_dim)));
        float sn, cs;
        sincosf(pos * inv_freq, &sn, &cs);
        if (inverse) sn = -sn;
        __nv_bfloat162 o = __floats2bfloat162_rn(a * cs - b * sn, b * cs + a * sn);
        vw[j] = *reinterpret_cast<uint32_t*>(&o);
      }
      *reinterpret_cast<uint4*>(op + e) = val;
    }
  }
}

// pass-through of the non-rotary tail when out != x
template <typename T>
__global__ void rope_tail_kernel(const T* __restrict__ x, T* __restrict__ out, int tokens, int heads, int head_dim,
                                 int rotary_dim, long long x_stride_tok, long long out_stride_tok) {
  const int tail = head_dim - rotary_dim;
  const long long total = (long long)tokens * heads * tail;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int p = int(i % tail);
    const int h = int((i / tail) % heads);
    const int t = int(i / ((long long)tail * heads));
    out[t * out_stride_tok + (long long)h * head_dim + rotary_dim + p] = x[t * x_stride_tok + (long long)h * head_dim + rotary_dim + p];
  }
}

// ------------------------------------------------------------------------------------------------
// Activations.  kind: 1 relu, 2 gelu(erf), 3 gelu(tanh), 4 silu.  Gated variants compute act(gate) * up.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float act_fwd(float x, int kind) {
  switch (kind) {
    case 1: return fmaxf(x, 0.f);
    case 2: return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case 3: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanhf(u));
    }
    case 4: return x / (1.f + expf(-x));
    default: return x;
  }
}
__device__ __forceinline__ float act_grad(float x, int kind) {
  switch (kind) {
    case 1: return x > 0.f ? 1.f : 0.f;
    case 2: return 0.5f * (1.f + erff(x * 0.70710678118654752f)) + x * 0.3989422804014327f * expf(-0.5f * x * x);
    case 3: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      const float t = tanhf(u);
      return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
    }
    case 4: {
      const float s = 1.f / (1.f + expf(-x));
      return s * (1.f + x * (1.f - s));
    }
    default: return 1.f;
  }
}

template <typename T>
__global__ void act_fwd_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out, long long nvec,
                               int kind, int cols, long long gate_ld, long long up_ld) {
  // logical shape [rows, cols]; gate / up may be column slices of a wider fused projection (leading dims)
  const int vec_per_row = cols >> 3;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = int(i % vec_per_row) * 8;
    float g[8], u[8], o[8];
    Vec8<T>::load(gate + r * gate_ld + c, g);
    if (up) Vec8<T>::load(up + r * up_ld + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = act_fwd(g[j], kind) * (up ? u[j] : 1.f);
    Vec8<T>::store(out + r * cols + c, o);
  }
}

template <typename T>
__global__ void act_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ gate, const T* __restrict__ up,
                               T* __restrict__ dgate, T* __restrict__ dup, long long nvec, int kind) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float d[8], g[8], u[8], dg[8], du[8];
    Vec8<T>::load(dout + i * 8, d);
    Vec8<T>::load(gate + i * 8, g);
    if (up) Vec8<T>::load(up + i * 8, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dg[j] = d[j] * act_grad(g[j], kind) * (up ? u[j] : 1.f);
      du[j] = d[j] * act_fwd(g[j], kind);
    }
    Vec8<T>::store(dgate + i * 8, dg);
    if (up) Vec8<T>::store(dup + i * 8, du);
  }
}

// ------------------------------------------------------------------------------------------------
// Embedding gather: out[t, :] = table[ids[t], :]   (cols % 8 == 0)
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const int64_t* __restrict__ ids, const T* __restrict__ table, T* __restrict__ out,
                                 int tokens, int cols, long long table_ld, long long out_ld) {
  pdl_wait();
  const int vec_per_row = cols >> 3;
  const long long total = (long long)tokens * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = int(i / vec_per_row);
    const int c = int(i % vec_per_row) * 8;
    const int64_t id = ids[t];
    if constexpr (sizeof(T) == 2) {
      *reinterpret_cast<uint4*>(out + t * out_ld + c) = *reinterpret_cast<const uint4*>(table + id * table_ld + c);
    } else {
      reinterpret_cast<float4*>(out + t * out_ld + c)[0] = reinterpret_cast<const float4*>(table + id * table_ld + c)[0];
      reinterpret_cast<float4*>(out + t * out_ld + c)[1] = reinterpret_cast<const float4*>(table + id * table_ld + c)[1];
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Fused AdamW: one pass over (param, grad, exp_avg, exp_avg_sq [, fp32 master]).
// Bias corrections are passed pre-computed; grads may be bf16 or fp32 (grad_is_fp32).
// ------------------------------------------------------------------------------------------------
template <typename P>
__global__ void adamw_kernel(P* __restrict__ param, const void* __restrict__ grad, float* __restrict__ m,
                             float* __restrict__ v, float* __restrict__ master, long long n, float lr, float beta1,
                             float beta2, float eps, float weight_decay, float bc1, float bc2, float grad_scale,
                             int grad_is_fp32) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float g = grad_is_fp32 ? static_cast<const float*>(grad)[i] : __bfloat162float(static_cast<const bf16*>(grad)[i]);
    g *= grad_scale;
    float p = master ? master[i] : to_f<P>(param[i]);
    const float mi = beta1 * m[i] + (1.f - beta1) * g;
    const float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    p *= 1.f - lr * weight_decay;
    p -= lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    if (master) master[i] = p;
    param[i] = from_f<P>(p);
  }
}

template <typename A, typename B>
__global__ void cast_kernel(const A* __restrict__ in, B* __restrict__ out, long long n, float scale) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = from_f<B>(to_f<A>(in[i]) * scale);
}

static inline int grid_for(long long work, int threads) {
  long long g = (work + threads - 1) / threads;
  if (g > 148LL * 16) g = 148LL * 16;
  if (g < 1) g = 1;
  return int(g);
}

}  // namespace tpb

using namespace tpb;

#define TPB_CHECK_LAUNCH() return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA

// dtype: 0 = bf16, 1 = fp32.  mode: 0 = RMSNorm, 1 = LayerNorm.
extern "C" int tpb_norm_fwd(const void* x, const void* residual, const void* weight, const void* bias, void* out,
                            void* sum_out, float* rstd_out, float* mean_out, int rows, int cols, float eps, int mode,
                            int dtype, void* stream_) {
  if (!x || !out || rows <= 0 || cols <= 0) return TPB_ERR_ARG;
  if ((cols & 7) || cols > NORM_THREADS * 8 * NORM_MAXV) return TPB_ERR_SIZE;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
#define LAUNCH3(T, M, V)                                                                                              \
  launch_kernel(norm_fwd_kernel<T, M, V>, dim3(rows), dim3(NORM_THREADS), 0, s, (const T*)x, (const T*)residual, (const T*)weight, \
                (const T*)bias, (T*)out, (T*)sum_out, rstd_out, mean_out, cols, eps)
#define LAUNCH(T, M)                                                                     \
  do {                                                                                   \
    if (cols <= NORM_THREADS * 8) LAUNCH3(T, M, 1);                                      \
    else if (cols <= NORM_THREADS * 16) LAUNCH3(T, M, 2);                                \
    else if (cols <= NORM_THREADS * 32) LAUNCH3(T, M, 4);                                \
    else LAUNCH3(T, M, 8);                                                               \
  } while (0)
  if (dtype == 0) { if (mode) LAUNCH(bf16, 1); else LAUNCH(bf16, 0); }
  else            { if (mode) LAUNCH(float, 1); else LAUNCH(float, 0); }
#undef LAUNCH
#undef LAUNCH3
  TPB_CHECK_LAUNCH();
}

extern "C" int tpb_norm_bwd(const void* dy, const void* x, const void* weight, const float* rstd, const float* mean,
                            void* dx, float* dweight, float* dbias, int rows, int cols, int mode, int dtype,
                            void* stream_) {
  if (!dy || !x || !dx || !rstd || rows <= 0) return TPB_ERR_ARG;
  if ((cols & 7) || cols > NORM_THREADS * 8 * NORM_BWD_MAXV) return TPB_ERR_SIZE;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  int rows_per_cta = (rows + 148 * 4 - 1) / (148 * 4);
  if (rows_per_cta < 1) rows_per_cta = 1;
  const int grid = (rows + rows_per_cta - 1) / rows_per_cta;
#define LAUNCH(T, M)                                                                                                  \
  norm_bwd_kernel<T, M><<<grid, NORM_THREADS, 0, s>>>((const T*)dy, (const T*)x, (const T*)weight, rstd, mean, (T*)dx, \
                                                      dweight, dbias, rows, cols, rows_per_cta)
  if (dtype == 0) { if (mode) LAUNCH(bf16, 1); else LAUNCH(bf16, 0); }
  else            { if (mode) LAUNCH(float, 1); else LAUNCH(float, 0); }
#undef LAUNCH
  TPB_CHECK_LAUNCH();
}

extern "C" int tpb_rope(const void* x, void* out, const int64_t* positions, const int* base_pos, int seq, int tokens,
                        int heads, int head_dim, int rotary_dim, float theta, int interleaved, int inverse,
                        long long x_stride_tok, long long out_stride_tok, int dtype, void* stream_) {
  if (!x || !out || (!positions && !base_pos) || tokens <= 0 || (rotary_dim & 1) || rotary_dim > head_dim) return TPB_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const long long work = (long long)tokens * heads * (rotary_dim / 2);
  const float l2t = log2f(theta);
  const int half_ = rotary_dim / 2;
  const bool vec_ok = dtype == 0 && head_dim % 8 == 0 && (interleaved ? rotary_dim % 8 == 0 : half_ % 8 == 0) && rotary_dim > 0 &&
                      !(x_stride_tok & 7) && !(out_stride_tok & 7) && !((uintptr_t)x & 15) && !((uintptr_t)out & 15);
  if (vec_ok) {
    const long long vwork = (long long)tokens * heads * (interleaved ? rotary_dim / 8 : half_ / 8);
    rope_vec_kernel<<<grid_for(vwork, 256), 256, 0, s>>>((const bf16*)x, (bf16*)out, positions, base_pos, seq, tokens, heads, head_dim,
                                                         rotary_dim, l2t, interleaved, inverse, x_stride_tok, out_stride_tok);
  } else if (dtype == 0)
    rope_kernel<bf16><<<grid_for(work, 256), 256, 0, s>>>((const bf16*)x, (bf16*)out, positions, base_pos, seq, tokens, heads,
                                                          head_dim, rotary_dim, l2t, interleaved, inverse, x_stride_tok, out_stride_tok);
  else
    rope_kernel<float><<<grid_for(work, 256), 256, 0, s>>>((const float*)x, (float*)out, positions, base_pos, seq, tokens, heads,
                                                           head_dim, rotary_dim, l2t, interleaved, inverse, x_stride_tok, out_stride_tok);
  if (x != out && rotary_dim < head_dim) {
    const long long tw = (long long)tokens * heads * (head_dim - rotary_dim);
    if (dtype == 0)
      rope_tail_kernel<bf16><<<grid_for(tw, 256), 256, 0, s>>>((const bf16*)x, (bf16*)out, tokens, heads, head_dim, rotary_dim, x_stride_tok, out_stride_tok);
    else
      rope_tail_kernel<float><<<grid_for(tw, 256), 256, 0, s>>>((const float*)x, (float*)out, tokens, heads, head_dim, rotary_dim, x_stride_tok, out_stride_tok);
  }
  TPB_CHECK_LAUNCH();
}

extern "C" int tpb_act_fwd(const void* gate, const void* up, void* out, long long rows, int cols, long long gate_ld,
                           long long up_ld, int kind, int dtype, void* stream_) {
  if (!gate || !out || rows <= 0 || cols <= 0) return TPB_ERR_ARG;
  if ((cols & 7) || (gate_ld & 7) || (up_ld & 7)) return TPB_ERR_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const long long nvec = rows * (cols / 8);
  if (dtype == 0)
    act_fwd_kernel<bf16><<<grid_for(nvec, 256), 256, 0, s>>>((const bf16*)gate, (const bf16*)up, (bf16*)out, nvec, kind, cols, gate_ld, up_ld);
  else
    act_fwd_kernel<float><<<grid_for(nvec, 256), 256, 0, s>>>((const float*)gate, (const float*)up, (float*)out, nvec, kind, cols, gate_ld, up_ld);
  TPB_CHECK_LAUNCH();
}

extern "C" int tpb_act_bwd(const void* dout, const void* gate, const void* up, void* dgate, void* dup, long long n,
                           int kind, int dtype, void* stream_) {
  if (!dout || !gate || !dgate || n <= 0) return TPB_ERR_ARG;
  if (n & 7) return TPB_ERR_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const long long nvec = n / 8;
  if (dtype == 0)
    act_bwd_kernel<bf16><<<grid_for(nvec, 256), 256, 0, s>>>((const bf16*)dout, (const bf16*)gate, (const bf16*)up, (bf16*)dgate, (bf16*)dup, nvec, kind);
  else
    act_bwd_kernel<float><<<grid_for(nvec, 256), 256, 0, s>>>((const float*)dout, (const float*)gate, (const float*)up, (float*)dgate, (float*)dup, nvec, kind);
  TPB_CHECK_LAUNCH();
}

extern "C" int tpb_embedding(const int64_t* ids, const void* table, void* out, int tokens, int cols, long long table_ld,
                             long long out_ld, int dtype, void* stream_) {
  if (!ids || !table || !out || tokens <= 0) return TPB_ERR_ARG;
  if ((cols & 7) || (table_ld & 7) || (out_ld & 7)) return TPB_ERR_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const long long work = (long long)tokens * (cols / 8);
  if (dtype == 0)
    launch_kernel(embedding_kernel<bf16>, dim3(grid_for(work, 256)), dim3(256), 0, s, ids, (const bf16*)table, (bf16*)out, tokens, cols, table_ld, out_ld);
  else
    embedding_kernel<float><<<grid_for(work, 256), 256, 0, s>>>(ids, (const float*)table, (float*)out, tokens, cols, table_ld, out_ld);
  TPB_CHECK_LAUNCH();
}

extern "C" int tpb_adamw(void* param, const void* grad, float* m, float* v, float* master, long long n, float lr,
                         float beta1, float beta2, float eps, float weight_decay, int step, float grad_scale,
                         int param_dtype, int grad_is_fp32, void* stream_) {
  if (!param || !grad || !m || !v || n <= 0 || step < 1) return TPB_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const float bc1 = 1.f - powf(beta1, float(step));
  const float bc2 = 1.f - powf(beta2, float(step));
  if (param_dtype == 0)
    adamw_kernel<bf16><<<grid_for(n, 256), 256, 0, s>>>((bf16*)param, grad, m, v, master, n, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale, grad_is_fp32);
  else
    adamw_kernel<float><<<grid_for(n, 256), 256, 0, s>>>((float*)param, grad, m, v, master, n, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale, grad_is_fp32);
  TPB_CHECK_LAUNCH();
}

// direction: 0 = bf16 -> fp32, 1 = fp32 -> bf16
extern "C" int tpb_cast(const void* in, void* out, long long n, float scale, int direction, void* stream_) {
  if (!in || !out || n <= 0) return TPB_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  if (direction == 0)
    cast_kernel<bf16, float><<<grid_for(n, 256), 256, 0, s>>>((const bf16*)in, (float*)out, n, scale);
  else
    cast_kernel<float, bf16><<<grid_for(n, 256), 256, 0, s>>>((const float*)in, (bf16*)out, n, scale);
  TPB_CHECK_LAUNCH();
}

// ------------------------------------------------------------------------------------------------
// bf16 matrix transpose out[c, r] = in[r, c] through a padded 64x64 shared tile (both sides coalesced)
// ------------------------------------------------------------------------------------------------
namespace tpb {
__global__ void transpose_bf16_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int rows, int cols,
                                      long long in_ld, long long out_ld) {
  __shared__ bf16 tile[64][66];
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const int r = r0 + i;
    for (int j = threadIdx.x; j < 64; j += blockDim.x) {
      const int c = c0 + j;
      if (r < rows && c < cols) tile[i][j] = in[(long long)r * in_ld + c];
    }
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 64; i += blockDim.y) {
    const int c = c0 + i;
    for (int j = threadIdx.x; j < 64; j += blockDim.x) {
      const int r = r0 + j;
      if (r < rows && c < cols) out[(long long)c * out_ld + r] = tile[j][i];
    }
  }
}
}  // namespace tpb

extern "C" int tpb_transpose_bf16(const void* in, void* out, int rows, int cols, long long in_ld, long long out_ld,
                                  void* stream_) {
  if (!in || !out || rows <= 0 || cols <= 0) return TPB_ERR_ARG;
  dim3 grid((cols + 63) / 64, (rows + 63) / 64), block(64, 8);
  tpb::transpose_bf16_kernel<<<grid, block, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const tpb::bf16*>(in), static_cast<tpb::bf16*>(out), rows, cols, in_ld, out_ld);
  TPB_CHECK_LAUNCH();
}
