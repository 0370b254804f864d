// Warp-level tensor-core helpers (mma.sync m16n8k16 bf16, ldmatrix, cp.async) shared
// by the attention kernels.
#pragma once
#include "common.cuh"

namespace sb200 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  // src-size 0 zero-fills the 16 destination bytes without touching gmem
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem),
               "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem)));
}

// d (16x8 fp32) += a (16x16 bf16, row) * b (16x8 bf16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Address helpers for a row-major smem tile with `ld` elements per row.
// A operand (16 rows x 16 k) at (r0, k0): lane -> row r0 + lane%16, col k0 + 8*(lane/16)
template <typename T>
__device__ __forceinline__ const T* lda_addr(const T* tile, int ld, int r0, int k0, int lane) {
  return tile + (r0 + (lane & 15)) * ld + k0 + ((lane >> 4) << 3);
}
// B operand from a [n][k] row-major tile (k contiguous), two n-tiles (16 n x 16 k) at (n0, k0):
// regs: {nt0.b0, nt0.b1, nt1.b0, nt1.b1}
template <typename T>
__device__ __forceinline__ const T* ldb_nk_addr(const T* tile, int ld, int n0, int k0, int lane) {
  return tile + (n0 + (lane & 7) + ((lane >> 4) << 3)) * ld + k0 + (((lane >> 3) & 1) << 3);
}
// B operand from a [k][n] row-major tile (n contiguous) with ldmatrix.trans, two n-tiles
// (16 k x 16 n) at (k0, n0): regs: {nt0.b0, nt0.b1, nt1.b0, nt1.b1}
template <typename T>
__device__ __forceinline__ const T* ldb_kn_addr(const T* tile, int ld, int k0, int n0, int lane) {
  return tile + (k0 + (lane & 7) + (((lane >> 3) & 1) << 3)) * ld + n0 + ((lane >> 4) << 3);
}

}  // namespace sb200
