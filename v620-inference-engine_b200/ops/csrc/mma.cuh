// Warp-level tensor-core helpers for the skinny (M <= 16 rows) decode products: ldmatrix loads from
// padded shared-memory rows and the m16n8k16 bf16 MMA with fp32 accumulation.  The decode products
// are memory-bound; the tensor core is used to cut the instruction count per weight byte by an
// order of magnitude so that eight warps per SM keep up with the bulk-copy stream from HBM.
//
// Operand roles: A = 16 weight rows x 16 k (row-major in shared memory), B = 8 activation rows x 16 k
// (activation rows are B's columns), D[weight row][activation row] fp32.
#pragma once
#include "stream.cuh"

namespace qw {

// Row stride padding: 16 bytes more than the row keeps the 8 row addresses of an ldmatrix in
// different bank groups when the row length is a multiple of 128 bytes.
constexpr unsigned ROW_PAD = 16;

__device__ __forceinline__ void ldmatrix_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(saddr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t &r0, uint32_t &r1, uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(saddr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Address operand of ldmatrix.x4 for a 16 x 16 A tile: lane l supplies row (l & 15), k offset (l >> 4) * 8.
__device__ __forceinline__ uint32_t a_tile_addr(uint32_t tile_base, unsigned row_stride, int k0, int lane) {
    return tile_base + (unsigned)(lane & 15) * row_stride + (unsigned)(k0 + ((lane >> 4) << 3)) * 2u;
}
// Address operand of ldmatrix.x2 for an 8 x 16 B tile (8 activation rows): lanes 0-7 rows at k0, lanes 8-15 rows at k0+8.
// Rows >= nrows read the zero row `zero_row`.
__device__ __forceinline__ uint32_t b_tile_addr(uint32_t x_base, unsigned row_stride, int row0, int nrows, int zero_row,
                                                int k0, int lane) {
    const int r = row0 + (lane & 7);
    const int rr = r < nrows ? r : zero_row;
    return x_base + (unsigned)rr * row_stride + (unsigned)(k0 + (((lane >> 3) & 1) << 3)) * 2u;
}

// Fragment coordinates of the accumulator: c[0],c[1] -> (row = lane/4, n = 2*(lane%4) + {0,1}); c[2],c[3] -> row + 8.

}  // namespace qw
