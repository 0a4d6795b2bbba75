// Warp-level tensor-core helpers shared by the attention kernels.
#pragma once

#include "common.cuh"

namespace air {

// D (16x8, f32) += A (16x16, bf16, row) * B (16x8, bf16, col).  With g = lane / 4, t = lane % 4:
//   a0 = A[g][2t..2t+1], a1 = A[g+8][2t..2t+1], a2 = A[g][2t+8..2t+9], a3 = A[g+8][2t+8..2t+9]
//   b0 = B[2t..2t+1][g], b1 = B[2t+8..2t+9][g];  c0,c1 = D[g][2t..2t+1], c2,c3 = D[g+8][2t..2t+1]
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint4 ldg16(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// Address of the 16-byte chunk `chunk` (0..7) of row `row` in a [64][128 B] tile with 128-byte swizzle.
__device__ __forceinline__ uint32_t swizzled(uint32_t tile, int row, int chunk) {
    return tile + row * 128 + ((chunk ^ (row & 7)) << 4);
}

}  // namespace air
