// Vocab-parallel cross-entropy: each rank holds logits for its slice of the vocabulary only.
//   tpb_ce_stats : per row -> (local max, local sum of exp(logit - local max), target logit or 0) + "target is mine" flag
//   tpb_ce_grad  : given the global log-sum-exp per row, overwrite the local logits with
//                  d loss / d logit = (softmax - onehot) * scale   (rows with an ignored label become 0)
// Only [rows, 4] floats per rank have to cross the interconnect; full logits never exist anywhere.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "tpb_api.h"

namespace tpb {

typedef __nv_bfloat16 bf16;
constexpr int CE_THREADS = 256;

__device__ __forceinline__ float ce_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float ce_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(CE_THREADS)
ce_stats_kernel(const bf16* __restrict__ logits, const int64_t* __restrict__ labels, float* __restrict__ stats, int cols,
                long long ld, int vocab_start, int ignore_index) {
  const long long row = blockIdx.x;
  const bf16* x = logits + row * ld;
  __shared__ float red[CE_THREADS / 32];
  __shared__ float bcast;
  float m = -INFINITY;
  for (int c = threadIdx.x; c < cols; c += CE_THREADS) m = fmaxf(m, __bfloat162float(x[c]));
  m = ce_warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < CE_THREADS / 32 ? red[threadIdx.x] : -INFINITY;
    t = ce_warp_max(t);
    if (threadIdx.x == 0) bcast = t;
  }
  __syncthreads();
  m = bcast;
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += CE_THREADS) s += expf(__bfloat162float(x[c]) - m);
  s = ce_warp_sum(s);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < CE_THREADS / 32; ++w) t += red[w];
    const long long label = labels[row];
    const long long local = label - vocab_start;
    const bool mine = label != ignore_index && local >= 0 && local < cols;
    stats[row * 4 + 0] = m;
    stats[row * 4 + 1] = t;
    stats[row * 4 + 2] = mine ? __bfloat162float(x[local]) : 0.f;
    stats[row * 4 + 3] = mine ? 1.f : 0.f;
  }
}

__global__ void __launch_bounds__(CE_THREADS)
ce_grad_kernel(bf16* __restrict__ logits, const int64_t* __restrict__ labels, const float* __restrict__ lse, int cols,
               long long ld, int vocab_start, int ignore_index, const float* __restrict__ scale_ptr) {
  const long long row = blockIdx.x;
  bf16* x = logits + row * ld;
  const long long label = labels[row];
  const float scale = scale_ptr[0];
  if (label == ignore_index) {
    for (int c = threadIdx.x; c < cols; c += CE_THREADS) x[c] = __float2bfloat16(0.f);
    return;
  }
  const float l = lse[row];
  const long long local = label - vocab_start;
  for (int c = threadIdx.x; c < cols; c += CE_THREADS) {
    float p = expf(__bfloat162float(x[c]) - l);
    if (c == local) p -= 1.f;
    x[c] = __float2bfloat16(p * scale);
  }
}

}  // namespace tpb

extern "C" int tpb_ce_stats(const void* logits, const int64_t* labels, float* stats, int rows, int cols, long long ld,
                            int vocab_start, int ignore_index, void* stream_) {
  if (!logits || !labels || !stats || rows <= 0 || cols <= 0) return TPB_ERR_ARG;
  tpb::ce_stats_kernel<<<rows, tpb::CE_THREADS, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const tpb::bf16*>(logits), labels, stats, cols, ld, vocab_start, ignore_index);
  return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

extern "C" int tpb_ce_grad(void* logits, const int64_t* labels, const float* lse, int rows, int cols, long long ld,
                           int vocab_start, int ignore_index, const float* scale_ptr, void* stream_) {
  if (!logits || !labels || !lse || !scale_ptr || rows <= 0 || cols <= 0) return TPB_ERR_ARG;
  tpb::ce_grad_kernel<<<rows, tpb::CE_THREADS, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<tpb::bf16*>(logits), labels, lse, cols, ld, vocab_start, ignore_index, scale_ptr);
  return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}
