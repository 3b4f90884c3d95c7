// Warp-level tensor-core helpers (mma.sync m16n8k16 bf16 -> fp32) and cp.async wrappers, used by the
// small in-kernel contractions (conv sequence, attention core) where a TMEM round trip is not worth it.
//
// Fragment layout of m16n8k16 (g = lane / 4, t = lane % 4):
//   A (16x16, row): a0=(g, 2t..2t+1)  a1=(g+8, 2t..)  a2=(g, 2t+8..)  a3=(g+8, 2t+8..)
//   B (16x8,  col): b0=(k=2t..2t+1, n=g)  b1=(k=2t+8.., n=g)
//   C (16x8):       c0,c1=(g, 2t..2t+1)   c2,c3=(g+8, 2t..2t+1)
#pragma once
#include <stdint.h>

namespace hb200 {

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem_dst)), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// Two 8x8 b16 matrices, transposed on load: with row addresses &V[k0 + (lane & 15)][n0] the result is
// the B fragment (b0, b1) of a [k][n]-stored operand.
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* smem_row_ptr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
               : "=r"(r0), "=r"(r1)
               : "r"(smem_u32(smem_row_ptr)));
}

}  // namespace hb200
