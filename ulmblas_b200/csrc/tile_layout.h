// Shared-memory tile layout of the FP64 GEMM kernels and the lane -> element
// maps of the FP64 tensor-core instruction, as plain integer functions usable
// from both host and device code (the host copy feeds a CPU model of the
// kernel's index arithmetic in the tests).
//
// One pipeline stage holds 16 consecutive k of an operand tile: 16 doubles
// are 128 bytes, the span of the TMA 128-byte swizzle.  An operand whose
// K dimension is contiguous in global memory ("K-major": op(A) = A^T, or
// op(B) = B) is staged as rows of 16 k, one row per m (or n).  An operand
// whose M/N dimension is contiguous ("MN-major": op(A) = A, op(B) = B^T) is
// staged as 16x16 boxes: 16 rows (one per k) of 16 consecutive m (or n).
// In both cases the 16-byte chunk index inside a 128-byte row is XOR-ed with
// (row index mod 8) -- what CU_TENSOR_MAP_SWIZZLE_128B does on a 1024-byte
// aligned destination.
//
// mma.sync.aligned.m16n8k8.row.col.f64 fragments (g = lane/4, t = lane%4):
//   A: a0 (g,t)  a1 (g+8,t)  a2 (g,t+4)  a3 (g+8,t+4)
//   B: b0 (k=t, n=g)  b1 (k=t+4, n=g)
//   C: c0 (g,2t) c1 (g,2t+1) c2 (g+8,2t) c3 (g+8,2t+1)
// The kernels do not feed tile row r to MMA row r: any permutation of the
// rows of A (carried into C's rows), of the columns of B (into C's columns)
// and of k (same for A and B) leaves the product intact, and the permutations
// below make every fragment a single conflict-free 16-byte shared load.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define ULMB_HD __host__ __device__ __forceinline__
#else
#define ULMB_HD inline
#endif

namespace ulmb200 {

constexpr int kBK = 16;                    // k per stage
enum Major : int { MN_MAJOR = 0, K_MAJOR = 1 };

// K-major operands: MMA row/col index g (0..7) <-> tile row perm8(g) inside an
// aligned group of 8.  Lanes g = 2q, 2q+1 of a quarter-warp land on rows that
// differ in bit 2, so their swizzled chunks never collide.
ULMB_HD int perm8(int g) { return (g >> 1) + ((g & 1) << 2); }

// Byte offset of element (r, k) of an operand tile inside its stage buffer:
// r = m (or n) index within the CTA tile, k in [0,16).
template <int MAJOR>
ULMB_HD uint32_t elem_off(int r, int k)
{
    if (MAJOR == K_MAJOR)
        return (uint32_t)(r * 128 + ((((k >> 1) ^ (r & 7))) << 4) + (k & 1) * 8);
    return (uint32_t)((r >> 4) * 2048 + k * 128 + (((((r & 15) >> 1) ^ (k & 7))) << 4) + (r & 1) * 8);
}

// k index (0..15 within the stage) fed to MMA k-slot `slot` (0..7) of k8-step h
// (0..1): slots t and t+4 of lane group t read the two doubles of chunk t+4h.
ULMB_HD int k_of_slot(int h, int slot) { return 2 * ((slot & 3) + 4 * h) + (slot >> 2); }

// Per-lane base offsets of the fragment loads.  Tile/step selection adds
// compile-time constants:
//   A, K-major : base[h]; m16 tile i, half hf (rows g / g+8): + i*2048 + hf*1024
//                16 bytes at that address = (a[hf], a[hf+2])
//   A, MN-major: base[s]; m16 tile i, step h:               + i*2048 + h*1024
//                16 bytes = (a[2s], a[2s+1])
//   B, K-major : base[h]; n8 tile j:                         + j*1024
//                16 bytes = (b0, b1)
//   B, MN-major: base[s]; n16 group jj, step h:              + jj*2048 + h*1024
//                16 bytes = (b[s] of tile 2jj, b[s] of tile 2jj+1)
// w0 = first tile row (col) of the warp inside the CTA tile, a multiple of 16.
template <int MAJOR>
ULMB_HD void frag_base(int w0, int lane, uint32_t base[2])
{
    const int g = lane >> 2, t = lane & 3;
    if (MAJOR == K_MAJOR) {
        const int p = perm8(g);
        base[0] = (uint32_t)((w0 + p) * 128 + (((t) ^ p) << 4));
        base[1] = (uint32_t)((w0 + p) * 128 + (((t + 4) ^ p) << 4));
    } else {
        base[0] = (uint32_t)((w0 >> 4) * 2048 + (2 * t) * 128 + ((g ^ ((2 * t) & 7)) << 4));
        base[1] = (uint32_t)((w0 >> 4) * 2048 + (2 * t + 1) * 128 + ((g ^ ((2 * t + 1) & 7)) << 4));
    }
}

// Tile row of MMA row (g + 8*half) for the m16 tile starting at tile row rb.
template <int MAJOR_A>
ULMB_HD int c_row(int rb, int lane, int half)
{
    const int g = lane >> 2;
    return (MAJOR_A == K_MAJOR) ? rb + perm8(g) + 8 * half : rb + 2 * g + half;
}

// Tile column of MMA column (2t + which) for the n8 tile starting at column cb
// (a multiple of 8; for MN-major B the tiles of a 16-column group interleave).
template <int MAJOR_B>
ULMB_HD int c_col(int cb, int lane, int which)
{
    const int cc = 2 * (lane & 3) + which;
    return (MAJOR_B == K_MAJOR) ? cb + perm8(cc) : (cb & ~15) + 2 * cc + ((cb >> 3) & 1);
}

}  // namespace ulmb200
