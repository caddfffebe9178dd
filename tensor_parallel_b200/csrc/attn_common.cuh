// Building blocks shared by the tiled attention kernels (forward and backward): 16-byte asynchronous copies
// into XOR-swizzled shared-memory tiles, ldmatrix fragment loads and the m16n8k16 bf16 tensor-core instruction.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tpb {

typedef __nv_bfloat16 bf16;

constexpr int PF_M = 64, PF_N = 64, PF_THREADS = 128;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// smem tile [rows][D] bf16, 16-byte chunks XOR-swizzled by (row & 7)
template <int D>
__device__ __forceinline__ bf16* tile_ptr(bf16* base, int row, int chunk) {
  return base + row * D + ((chunk ^ (row & 7)) << 3);
}

template <int D>
__device__ __forceinline__ void load_tile(bf16* smem, const bf16* gmem, long long row_stride, int row0, int rows_valid) {
  constexpr int CH = D / 8;
  for (int i = threadIdx.x; i < PF_N * CH; i += PF_THREADS) {
    const int r = i / CH, c = i % CH;
    const bool ok = row0 + r < rows_valid;
    const bf16* src = gmem + (long long)(ok ? row0 + r : 0) * row_stride + c * 8;
    cp_async16(tile_ptr<D>(smem, r, c), src, ok);
  }
}


// same as load_tile but for `rows` rows (a multiple of 8, at most 64)
template <int D>
__device__ __forceinline__ void load_rows(bf16* smem, const bf16* gmem, long long row_stride, int row0, int rows_valid, int rows) {
  constexpr int CH = D / 8;
  for (int i = threadIdx.x; i < rows * CH; i += PF_THREADS) {
    const int r = i / CH, c = i % CH;
    const bool ok = row0 + r < rows_valid;
    const bf16* src = gmem + (long long)(ok ? row0 + r : 0) * row_stride + c * 8;
    cp_async16(tile_ptr<D>(smem, r, c), src, ok);
  }
}

}  // namespace tpb
