// Warp-level bf16 tensor-core primitives (mma.sync m16n8k16, fp32 accumulation) for kernels whose tiles are too
// ragged for the tcgen05 path: (token, head) query rows gathered from different sequences, expert segments of a few
// rows.  Fragment layout (g = lane / 4, t = lane % 4):
//   A (16 x 16, row-major): a0 = A[g][2t..2t+1], a1 = A[g+8][2t..], a2 = A[g][2t+8..], a3 = A[g+8][2t+8..]
//   B (16 x 8, "col"):      b0 = B[2t..2t+1][g], b1 = B[2t+8..2t+9][g]
//   C (16 x 8):             c0, c1 = C[g][2t..2t+1], c2, c3 = C[g+8][2t..2t+1]
#pragma once
#include "util.cuh"

namespace llmctl {

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// A fragment of the 16 x 16 block at (row0, k0) of a row-major bf16 matrix in shared memory: one ldmatrix.x4 (rows
// must start on 16-byte boundaries: ld % 8 == 0, k0 % 8 == 0, 16-byte aligned base).
__device__ __forceinline__ void load_a_frag(uint32_t (&a)[4], const __nv_bfloat16* m, int ld, int row0, int k0, int lane) {
  const __nv_bfloat16* p = m + (row0 + (lane & 15)) * ld + k0 + ((lane >> 4) << 3);
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
               : "r"(addr));
}

// B fragment when B[k][n] = m[n0 + n][k0 + k], i.e. the operand is stored [n][k] row-major (weights [out, in],
// keys [key][dim]): one ldmatrix.x2 without transposition (same alignment rule).
__device__ __forceinline__ void load_b_frag_nk(uint32_t (&b)[2], const __nv_bfloat16* m, int ld, int n0, int k0, int lane) {
  const __nv_bfloat16* p = m + (n0 + (lane & 7)) * ld + k0 + (((lane >> 3) & 1) << 3);
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(b[0]), "=r"(b[1]) : "r"(addr));
}

// B fragment when the operand is stored [k][n] row-major (values [key][dim]): ldmatrix with transposition.  Rows must
// start on 16-byte boundaries (ld % 8 == 0, n0 % 8 == 0).
__device__ __forceinline__ void load_b_frag_kn(uint32_t (&b)[2], const __nv_bfloat16* m, int ld, int k0, int n0, int lane) {
  const __nv_bfloat16* p = m + (k0 + (lane & 15)) * ld + n0;     // lanes 0-7: rows k0..k0+7, lanes 8-15: k0+8..k0+15
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(b[0]), "=r"(b[1]) : "r"(addr));
}

// 16-byte asynchronous global -> shared copies (both addresses 16-byte aligned), grouped and awaited per thread.
__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }
// All but the most recently committed group have landed.
__device__ __forceinline__ void cp_async_wait_prior() { asm volatile("cp.async.wait_group 1;\n" ::: "memory"); }

}  // namespace llmctl
