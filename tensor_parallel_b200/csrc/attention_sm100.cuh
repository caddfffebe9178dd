// Shared by the tcgen05 attention kernels (forward and backward): packed fp32 arithmetic, exponentials, and the 4-D
// tensor maps over strided [batch, seq, head, head_dim] views.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "tpb_api.h"

// (defined in attention_bwd.cu) delta[b, h, i] = sum_d out[b, i, h, d] * dout[b, i, h, d], fp32 [batch][heads][sq]
extern "C" int tpb_attn_bwd_delta(const void* out, const void* dout, float* delta, int batch, int sq, int heads, int head_dim,
                                  long long o_sb, long long o_ss, long long o_sh, long long do_sb, long long do_ss, long long do_sh,
                                  void* stream);

namespace tpb {

constexpr int FA_BLOCK_BYTES = 128 * 128;  // one [128 rows][64 elements] swizzled block

__device__ __forceinline__ float ex2_approx(float x) {  // 2^x on the special-function unit; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Two fp32 lanes per instruction (fma.rn.f32x2 / add.f32x2): the softmax warps are bound by instruction issue.
__device__ __forceinline__ void ffma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void fadd2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}

// 2^x on the FMA pipe for a pair of values (the special-function unit, at 16 results per clock and SM, is what bounds the
// softmax of a 128 x 128 tile: as long as the tensor core needs for its two products).  x = n + f with n = round(x) taken
// from the low mantissa bits of x + 1.5 * 2^23, a cubic for 2^f on [-0.5, 0.5] (relative error 7.5e-5, far below the bf16
// rounding of the probabilities), n added into the exponent field.  x is clamped at -126: a masked score becomes 2^-126.
__device__ __forceinline__ void ex2_poly2(float& x0, float& x1) {
  constexpr float MAGIC = 12582912.f;
  x0 = fmaxf(x0, -126.f);
  x1 = fmaxf(x1, -126.f);
  float t0, t1, n0, n1, f0, f1, p0, p1;
  fadd2(t0, t1, x0, x1, MAGIC, MAGIC);
  fadd2(n0, n1, t0, t1, -MAGIC, -MAGIC);
  ffma2(f0, f1, n0, n1, -1.f, -1.f, x0, x1);
  ffma2(p0, p1, f0, f1, 0.0551716685f, 0.0551716685f, 0.2426111251f, 0.2426111251f);
  ffma2(p0, p1, p0, p1, f0, f1, 0.6932609677f, 0.6932609677f);
  ffma2(p0, p1, p0, p1, f0, f1, 0.9999280572f, 0.9999280572f);
  x0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
  x1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn fa_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// bf16 [batch][seq][heads][head_dim] view with element strides (head_dim contiguous); box = [64 head_dim][box_rows rows of seq].
static int fa_tmap(CUtensorMap* map, const void* ptr, int head_dim, int box_rows, long long seq, int heads, int batch, long long s_seq,
                   long long s_head, long long s_batch) {
  EncodeTiledFn fn = fa_encode_fn();
  if (!fn) return TPB_ERR_DRIVER;
  cuuint64_t dims[4] = {cuuint64_t(head_dim), cuuint64_t(seq), cuuint64_t(heads), cuuint64_t(batch)};
  // a dimension of extent 1 may come with any stride (even 0): give it a legal one
  cuuint64_t strides[3] = {cuuint64_t(s_seq) * 2, cuuint64_t(heads > 1 ? s_head : head_dim) * 2, cuuint64_t(batch > 1 ? s_batch : head_dim) * 2};
  if (seq == 1) strides[0] = cuuint64_t(head_dim) * 2;
  cuuint32_t box[4] = {64, cuuint32_t(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "tpb: attention tensor map rejected (%d): base %p, seq %lld, heads %d, batch %d, strides %lld / %lld / %lld\n", int(r), ptr,
            seq, heads, batch, s_seq, s_head, s_batch);
  return r == CUDA_SUCCESS ? TPB_OK : TPB_ERR_TMAP;
}

// The tensor-map encoder needs a context bound to the calling thread (autograd worker threads have none at first).
static int fa_bind_thread() {
  static thread_local int bound_device = -1;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return TPB_ERR_CUDA;
  if (bound_device != dev) {
    if (cudaSetDevice(dev) != cudaSuccess) return TPB_ERR_CUDA;
    bound_device = dev;
  }
  return TPB_OK;
}

}  // namespace tpb
