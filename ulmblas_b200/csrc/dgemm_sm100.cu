// FP64 GEMM for sm_100a:  C <- alpha * op(A) * op(B) + beta * C, column-major.
//
// Replaces the reference's cache-blocking driver, panel packing, macro-kernel
// and SSE micro-kernel (ulmblas/level3/gemm.tcc:16-87, pack/gepack.tcc,
// mkernel/mgemm.tcc, ukernel/sse/ugemm.tcc).  Where the reference packs A and B
// into contiguous panels so its 4x4 register kernel streams them, this kernel
// has TMA drop 128-byte-swizzled operand tiles straight into shared memory
// (no packed copy in global memory) and feeds them to the FP64 tensor-core
// instruction (mma.sync m16n8k8 .f64 -- tcgen05 has no FP64 kind).  The
// transposes are absorbed by the tile layout, alpha/beta by the epilogue.
//
// Two kernels share the fragment code:
//   dgemm_tma_kernel  persistent, warp-specialised: one producer warp issues
//                     TMA loads into a ring of stages guarded by mbarriers,
//                     the consumer warps run DMMA out of shared memory.
//                     Needs 16-byte aligned A/B and even leading dimensions.
//   dgemm_ldg_kernel  same tile and fragment layout filled with predicated
//                     8-byte global loads; any alignment, any ld.
#include "common.h"
#include "tile_layout.h"
#include "dgemm_schedule.h"

#include <atomic>

namespace ulmb200 {

struct GemmParams {
    int64_t m, n, k;
    double alpha, beta;
    const double *A, *B;      // used by the ldg kernel only
    int64_t lda, ldb;
    double *C;
    int64_t ldc;
    int tiles_m, tiles_n;
    int tri;                  // 0 full, 1 upper triangle only (row<=col), 2 lower (row>=col)
    int *err;                 // device error word
    // Scheduler words of this launch's stream, all zero between launches (the kernel puts them
    // back): [0] hands out work units beyond the first wave, [1] counts CTAs that are done,
    // [2 + r] is the fold flag of shared tile r.  nullptr: units go round-robin by CTA index.
    int *sched;
    int dynamic;              // 1: units beyond the CTA's own index come from sched[0]
    // Work units.  u < split_first: tile u, all of K.  u >= split_first: stream unit
    // j = u - split_first of nsu.  The region_tiles tiles that do work among the tile ids
    // >= split_first form, stage by stage, one sequence of region_tiles * kt pipeline stages,
    // and stream unit j takes the j-th of nsu equal shares of it -- so the tiles beyond the
    // last full wave are shared evenly by all CTAs instead of idling most of them.
    int split_first, nsu, region_tiles;
    unsigned short rtile[kRegionMax];   // tri != 0: tile id - split_first of region tile r
    // In-place product with a triangular first or second operand (the leaf of the triangular solver
    // and multiply: C is the very block of B that is being read).  The triangular operand spans T
    // tiles; the other dimension is cut into strips of one tile.  The tile at place d of a strip
    // meets only d + 1 (low) or T - d (high) blocks of 128 k, and the rows (columns) it writes are
    // what the longer tiles of its strip still read.  So the units go out longest first, each tile
    // counts, per block of k, the loads it has seen land, and a tile stores only when every longer
    // tile of its strip has counted its block (word [2 + strip * T + d] of the scheduler words; the
    // storing tile puts it back to zero).  A tile waits only for units handed out before its own.
    //   1: left,  op(T) lower: tile row d multiplies blocks 0..d, units by falling d
    //   2: left,  op(T) upper: blocks d..T-1, units by rising d, blocks taken from the last down
    //   3: right, op(T) upper: tile column d multiplies blocks 0..d
    //   4: right, op(T) lower: blocks d..T-1
    int leaf;
    // Many products of one shape in one launch: product b = hi * bat_nlo + lo of nbatch shifts the tile
    // coordinates of op(A) by lo * bat_am[0] + hi * bat_am[1] rows and ..ak.. columns (of k), those of
    // op(B) likewise, and C by bat_c elements.  Whole tiles only; k is a multiple of the stage depth.
    int nbatch, bat_nlo;
    int bat_am[2], bat_ak[2], bat_bn[2], bat_bk[2];
    int64_t bat_c[2];
    int bat_cr[2], bat_cc[2];     // the same shift of C as rows and columns
    int c_tma;                    // the tensor maps of C are valid: whole tiles leave through shared memory
    int64_t c_m, c_n;             // rows and columns of the stored C those maps describe
    // host side only: extents of the stored operands when they differ from the product's (batches)
    int64_t ext_a_mn, ext_a_k, ext_b_mn, ext_b_k, ext_c_m, ext_c_n;
};

// What the output thread needs to know about a tile that will leave through the buffer.
struct StashInfo {
    int row, col;            // first row and column of the tile in C (batch shift included)
    int load;                // beta != 0: the old tile is fetched into the buffer first
    int unit;                // -1: no more tiles
    int wait_idx, expect;    // leaf mode: the counter that must reach expect before C may be written, -1 = none
    // piece of a shared tile: fold flag (-1 = none), the value it must show before this piece may be folded
    // (0: the head, which waits for nothing), the value to leave there afterwards, and whether the piece is
    // added to C (every piece but the head) instead of stored
    int flag_idx, flag_wait, flag_pub, add;
};

// batch mode: coordinate shifts of product b
struct BatchShift {
    int am, ak, bn, bk, cr, cc;
    int64_t c;
};
__device__ __forceinline__ BatchShift batch_shift(const GemmParams &p, int b)
{
    const int hi = b / p.bat_nlo, lo = b - hi * p.bat_nlo;
    BatchShift s;
    s.am = lo * p.bat_am[0] + hi * p.bat_am[1];
    s.ak = lo * p.bat_ak[0] + hi * p.bat_ak[1];
    s.bn = lo * p.bat_bn[0] + hi * p.bat_bn[1];
    s.bk = lo * p.bat_bk[0] + hi * p.bat_bk[1];
    s.c = lo * p.bat_c[0] + hi * p.bat_c[1];
    s.cr = lo * p.bat_cr[0] + hi * p.bat_cr[1];
    s.cc = lo * p.bat_cc[0] + hi * p.bat_cc[1];
    return s;
}


// tile id of region tile r
__device__ __forceinline__ int region_tile(const GemmParams &p, int r)
{
    return p.split_first + (p.tri ? (int)p.rtile[r] : r);
}

__device__ __forceinline__ void dmma_16x8x8(double (&c)[4], const double (&a)[4], const double (&b)[2])
{
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+d"(c[0]), "+d"(c[1]), "+d"(c[2]), "+d"(c[3])
        : "d"(a[0]), "d"(a[1]), "d"(a[2]), "d"(a[3]), "d"(b[0]), "d"(b[1]));
}

__device__ __forceinline__ double2 lds128(uint32_t addr)
{
    double2 v;
    asm volatile("ld.shared.v2.f64 {%0,%1}, [%2];" : "=d"(v.x), "=d"(v.y) : "r"(addr));
    return v;
}

// Releases a stage the warp has finished reading.  The tensor-core instructions that consume the
// fragments may be scheduled after a plain arrive, and then nothing makes the arrive wait for the stage's
// last shared loads: a TMA refill was seen to overtake a load still in flight (wrong values of one to four
// k in one 16-row block of a tile, about once in 10^2 launches of a product whose CTAs take a second piece
// of work).  So every lane reads one more word of the stage after the stage's tensor-core instructions --
// shared loads of a warp return in the order they were issued -- and lane 0 stores that word before it
// arrives: the store cannot issue before the load has returned, and the arrive, a release, follows the store.
// (The same load issued right behind the fragment loads, ahead of the tensor-core instructions, did not
// close the window: measured.)
__device__ __forceinline__ void release_stage(uint64_t *empty_bar, uint32_t stage_addr, volatile uint32_t *sink, int lane)
{
    uint32_t last;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(last) : "r"(stage_addr + 4u * (uint32_t)lane) : "memory");
    __syncwarp();
    if (lane == 0) mbar_arrive_after(empty_bar, last, sink);
}

// One pipeline stage (16 k) of a warp's MT x NT grid of m16n8 tiles.
template <int MAJOR_A, int MAJOR_B, int MT, int NT>
__device__ __forceinline__ void mma_stage(uint32_t sA, uint32_t sB, const uint32_t (&ba)[2],
                                              const uint32_t (&bb)[2], double (&acc)[MT][NT][4])
{
    static_assert(NT % 2 == 0, "n8 tiles come in pairs");
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        double a[MT][4];
        double b[NT][2];
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            if (MAJOR_A == K_MAJOR) {
                double2 lo = lds128(sA + ba[h] + i * 2048);
                double2 hi = lds128(sA + ba[h] + i * 2048 + 1024);
                a[i][0] = lo.x; a[i][2] = lo.y; a[i][1] = hi.x; a[i][3] = hi.y;
            } else {
                double2 s0 = lds128(sA + ba[0] + i * 2048 + h * 1024);
                double2 s1 = lds128(sA + ba[1] + i * 2048 + h * 1024);
                a[i][0] = s0.x; a[i][1] = s0.y; a[i][2] = s1.x; a[i][3] = s1.y;
            }
        }
        if (MAJOR_B == K_MAJOR) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                double2 v = lds128(sB + bb[h] + j * 1024);
                b[j][0] = v.x; b[j][1] = v.y;
            }
        } else {
#pragma unroll
            for (int jj = 0; jj < NT / 2; ++jj) {
                double2 s0 = lds128(sB + bb[0] + jj * 2048 + h * 1024);
                double2 s1 = lds128(sB + bb[1] + jj * 2048 + h * 1024);
                b[2 * jj][0] = s0.x; b[2 * jj + 1][0] = s0.y;
                b[2 * jj][1] = s1.x; b[2 * jj + 1][1] = s1.y;
            }
        }
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < NT; ++j) dmma_16x8x8(acc[i][j], a[i], b[j]);
    }
}

// C(row, col) <- alpha*acc + beta*C for the warp's accumulators; rows/cols
// outside m x n (and outside the requested triangle) are skipped.  The old values are read past
// L1 (ld.global.cg): the pieces of a shared tile hand their partial sums on through C, and a CTA
// that works on two tiles may hold a line in L1 that straddles both -- when the columns of C do not
// start on 128-byte boundaries the last rows of one tile share a line with the first of the next --
// from before the other tile's previous piece was written.  The old values of C
// of G m16 tiles are fetched first (independent loads in flight together), then combined
// and stored: the epilogue costs G times fewer memory round trips.  With M-contiguous A the
// two rows a lane holds are adjacent (2g, 2g+1), so a 16-byte aligned C moves them as one
// 16-byte access.
template <int MAJOR_A, int MAJOR_B, int MT, int NT, int G>
__device__ __forceinline__ void epilogue(const GemmParams &p, double *__restrict__ C, double beta, int64_t m0, int64_t n0,
                                         int wm0, int wn0, int lane, double (&acc)[MT][NT][4])
{
    static_assert(MT % G == 0, "m16 tiles are taken G at a time");
    const double alpha = p.alpha;
    const bool use_c = beta != 0.0;
    const bool vec = MAJOR_A == MN_MAJOR && p.tri == 0 &&
                     ((reinterpret_cast<uintptr_t>(C) & 15) == 0) && (p.ldc % 2 == 0);
#pragma unroll
    for (int i0 = 0; i0 < MT; i0 += G) {
        double old[G][NT][4];
        bool ok[G][NT][4];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const int i = i0 + g;
            const int64_t r0 = m0 + c_row<MAJOR_A>(wm0 + 16 * i, lane, 0);
            const int64_t r1 = m0 + c_row<MAJOR_A>(wm0 + 16 * i, lane, 1);
            if (vec && r1 < p.m) {
                // rows r0 (even) and r1 = r0 + 1: registers {0,2} of column 2t, {1,3} of column 2t+1
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int w = 0; w < 2; ++w) {
                        const int64_t col = n0 + c_col<MAJOR_B>(wn0 + 8 * j, lane, w);
                        const bool v = col < p.n;
                        ok[g][j][w] = ok[g][j][2 + w] = v;
                        double2 o = make_double2(0.0, 0.0);
                        if (use_c && v) o = __ldcg(reinterpret_cast<const double2 *>(C + r0 + col * p.ldc));
                        old[g][j][w] = o.x; old[g][j][2 + w] = o.y;
                    }
            } else {
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int64_t row = (e >> 1) ? r1 : r0;
                        const int64_t col = n0 + c_col<MAJOR_B>(wn0 + 8 * j, lane, e & 1);
                        bool v = row < p.m && col < p.n;
                        if (p.tri == 1) v = v && row <= col;
                        if (p.tri == 2) v = v && row >= col;
                        ok[g][j][e] = v;
                        old[g][j][e] = (v && use_c) ? __ldcg(C + row + col * p.ldc) : 0.0;
                    }
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const int i = i0 + g;
            const int64_t r0 = m0 + c_row<MAJOR_A>(wm0 + 16 * i, lane, 0);
            const int64_t r1 = m0 + c_row<MAJOR_A>(wm0 + 16 * i, lane, 1);
            if (vec && r1 < p.m) {
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int w = 0; w < 2; ++w) {
                        const int64_t col = n0 + c_col<MAJOR_B>(wn0 + 8 * j, lane, w);
                        if (ok[g][j][w]) {
                            double2 o;
                            o.x = alpha * acc[i][j][w];
                            o.y = alpha * acc[i][j][2 + w];
                            if (use_c) { o.x = fma(beta, old[g][j][w], o.x); o.y = fma(beta, old[g][j][2 + w], o.y); }
                            *reinterpret_cast<double2 *>(C + r0 + col * p.ldc) = o;
                        }
                    }
            } else {
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (ok[g][j][e]) {
                            const int64_t row = (e >> 1) ? r1 : r0;
                            const int64_t col = n0 + c_col<MAJOR_B>(wn0 + 8 * j, lane, e & 1);
                            double v = alpha * acc[i][j][e];
                            if (use_c) v = fma(beta, old[g][j][e], v);
                            C[row + col * p.ldc] = v;
                        }
                    }
            }
        }
    }
}

// Asks L2 for the lines of C this lane's epilogue will read, long before it reads them (issued
// when the tile's main loop starts; rows and columns outside the matrix are left alone).
template <int MAJOR_A, int MAJOR_B, int MT, int NT>
__device__ __forceinline__ void prefetch_c(const GemmParams &p, int64_t m0, int64_t n0, int wm0, int wn0, int lane)
{
#pragma unroll
    for (int i = 0; i < MT; ++i) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int64_t row = m0 + c_row<MAJOR_A>(wm0 + 16 * i, lane, h);
            // with M-contiguous A the two rows of a lane share a line: one request does
            if (MAJOR_A == MN_MAJOR && h == 1) continue;
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    const int64_t col = n0 + c_col<MAJOR_B>(wn0 + 8 * j, lane, w);
                    if (row < p.m && col < p.n)
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.C + row + col * p.ldc));
                }
        }
    }
}

// Persistent tile order: groups of 8 tile-rows swept column by column, so the
// CTAs running together share a handful of A and B panels in L2.
__host__ __device__ __forceinline__ void tile_coord(int id, int tiles_m, int tiles_n, int &tm, int &tn)
{
    constexpr int GM = 8;
    const int per_group = GM * tiles_n;
    const int group = id / per_group;
    const int first = group * GM;
    const int gsz = GM < tiles_m - first ? GM : tiles_m - first;
    const int r = id - group * per_group;
    tm = first + r % gsz;
    tn = r / gsz;
}

// true if the whole tile lies outside the requested triangle
__host__ __device__ __forceinline__ bool tile_skipped(int tri, int64_t m0, int64_t n0, int bm, int bn)
{
    if (tri == 1) return m0 > n0 + bn - 1;      // all rows below the diagonal
    if (tri == 2) return m0 + bm - 1 < n0;      // all rows above the diagonal
    return false;
}

// Thread layout: WARPS_M*WARPS_N consumer warps (whole warpgroups) followed by one
// producer warpgroup of which a single lane issues the TMA loads.  Registers are
// budgeted per 4-warp group, so with 8 consumer warps the kernel launches at the
// 168-register cap of 384 threads and then moves registers from the producer
// group to the consumers (setmaxnreg), which hold 64 accumulators plus fragments.
template <int BM, int BN, int WARPS_M, int WARPS_N, int MAJOR_A, int MAJOR_B, int STAGES, int MIN_CTAS>
__global__ void __launch_bounds__((WARPS_M *WARPS_N + 4) * 32, MIN_CTAS)
dgemm_tma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmCs, const GemmParams p)
{
    constexpr int NCW = WARPS_M * WARPS_N;          // consumer warps
    constexpr int WM = BM / WARPS_M, WN = BN / WARPS_N;
    constexpr int MT = WM / 16, NT = WN / 8;
    constexpr uint32_t A_BYTES = BM * 128, B_BYTES = BN * 128;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static_assert(WM % 16 == 0 && WN % 16 == 0, "warp tile must be a multiple of 16x16");

    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: the swizzle pattern is a function of the address
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                ~uintptr_t(1023));
    // The one-CTA-per-SM shape sends finished tiles out through a tile-sized buffer in shared memory when a
    // tensor map covers C.  One thread of the producer group fetches the old tile into the buffer by TMA while
    // the tile is being multiplied (beta != 0), the consumers fold alpha * acc into it and go on with the next
    // tile, and the same thread stores the buffer by TMA while the tensor pipe is busy again: no consumer
    // waits for global memory.  Tiles the map cannot serve (a tile across the diagonal of a triangular
    // update, pieces of shared tiles) are written by the consumers themselves.
    constexpr bool STASH = (MIN_CTAS == 1);
    constexpr uint32_t STASH_BYTES = STASH ? BM * BN * 8 : 0;
    constexpr int CBOX = 32;                                                        // columns per TMA box of C
    double *stash = reinterpret_cast<double *>(smem + STAGES * STAGE_BYTES);      // column-major BM x BN
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + STAGES * STAGE_BYTES + STASH_BYTES);
    uint64_t *empty = full + STAGES;
    uint64_t *tile_started = empty + STAGES;       // consumers -> output thread: a tile's place is in info[]
    uint64_t *stash_ready = tile_started + 1;      // output thread -> consumers: buffer free / old tile landed
    uint64_t *stash_full = stash_ready + 1;        // consumers -> output thread: the new tile is in the buffer
    StashInfo *info = reinterpret_cast<StashInfo *>(stash_full + 1);               // [2], tiles alternate
    volatile int *abort_flag = reinterpret_cast<volatile int *>(info + 2);
    volatile int *tile_slot = abort_flag + 1;      // tile id carried by each stage, -1 = no more work
    volatile uint32_t *release_sink = reinterpret_cast<volatile uint32_t *>(tile_slot + STAGES);     // one word per consumer warp

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], NCW);
        }
        mbar_init(tile_started, 1);
        mbar_init(stash_ready, 1);
        mbar_init(stash_full, NCW);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
        if (STASH && p.c_tma) { prefetch_tmap(&tmC); prefetch_tmap(&tmCs); }
    }
    __syncthreads();

    const int num_units = p.split_first + p.nsu;
    const int kt = (int)((p.k + kBK - 1) / kBK);

    constexpr bool REBALANCE = (NCW == 8 && MIN_CTAS == 1);
    constexpr bool SHARE = (MIN_CTAS == 1);          // only the one-CTA-per-SM shape shares tiles
    constexpr int EG = 1;   // m16 tiles whose old C values are fetched together (2 makes the 128 x 128 kernels spill)
    if (warp >= NCW) {
        // ---------------- producer warpgroup ----------------
        if (REBALANCE) asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp == NCW && lane == 0) {
            // Units are handed out dynamically: the first one is the CTA's own index, the rest come
            // from a global counter.  A CTA that starts late (its SM was busy with another
            // kernel, e.g. a collective) then simply takes fewer units instead of holding up the
            // whole grid with a fixed share.
            uint32_t it = 0;
            bool live = true;
            // loads the stages [kc0, kc1) of the tile at (m0, n0), from the last down if rev; ak and bk
            // shift the k coordinate of either operand (batches); false once the kernel has given up
            auto load_piece = [&](int unit, int64_t m0, int64_t n0, int kc0, int kc1, bool rev = false, int ak = 0,
                                  int bk = 0) -> bool {
                for (int kc = kc0; kc < kc1; ++kc, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                    if (*abort_flag || !mbar_wait(&empty[s], ph ^ 1)) {
                        *abort_flag = 1;
                        atomicExch(p.err, 101);
                        return false;
                    }
                    tile_slot[s] = unit;
                    uint8_t *sa = smem + s * STAGE_BYTES, *sb = sa + A_BYTES;
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    const int k0 = (rev ? kc0 + kc1 - 1 - kc : kc) * kBK;
                    if (MAJOR_A == K_MAJOR) {
                        tma_load_2d(sa, &tmA, k0 + ak, (int)m0, &full[s]);
                    } else {
#pragma unroll
                        for (int b = 0; b < BM / 16; ++b)
                            tma_load_2d(sa + b * 2048, &tmA, (int)m0 + 16 * b, k0 + ak, &full[s]);
                    }
                    if (MAJOR_B == K_MAJOR) {
                        tma_load_2d(sb, &tmB, k0 + bk, (int)n0, &full[s]);
                    } else {
#pragma unroll
                        for (int b = 0; b < BN / 16; ++b)
                            tma_load_2d(sb + b * 2048, &tmB, (int)n0 + 16 * b, k0 + bk, &full[s]);
                    }
                }
                return true;
            };
            int unit = blockIdx.x;
            while (live && unit < num_units) {
                if (SHARE && p.leaf) {
                    const LeafUnit u = leaf_decode(p.leaf, p.tiles_m, p.tiles_n, unit, kt);
                    live = load_piece(unit, (int64_t)u.tm * BM, (int64_t)u.tn * BN, u.kc0, u.kc1, u.rev != 0);
                } else if (SHARE && p.nbatch > 1) {
                    const int per = p.tiles_m * p.tiles_n, b = unit / per;
                    int tm, tn;
                    tile_coord(unit - b * per, p.tiles_m, p.tiles_n, tm, tn);
                    const BatchShift sh = batch_shift(p, b);
                    live = load_piece(unit, (int64_t)tm * BM + sh.am, (int64_t)tn * BN + sh.bn, 0, kt, false, sh.ak, sh.bk);
                } else if (!SHARE || unit < p.split_first) {
                    int tm, tn;
                    tile_coord(unit, p.tiles_m, p.tiles_n, tm, tn);
                    const int64_t m0 = (int64_t)tm * BM, n0 = (int64_t)tn * BN;
                    if (!tile_skipped(p.tri, m0, n0, BM, BN)) live = load_piece(unit, m0, n0, 0, kt);
                } else {
                    StreamWalk walk(p.region_tiles, p.nsu, unit - p.split_first, kt);
                    Piece pc;
                    while (live && walk.next(pc)) {
                        int tm, tn;
                        tile_coord(region_tile(p, pc.r), p.tiles_m, p.tiles_n, tm, tn);
                        live = load_piece(unit, (int64_t)tm * BM, (int64_t)tn * BN, pc.kc0, pc.kc1);
                    }
                }
                if (live) unit = p.dynamic ? (int)gridDim.x + atomicAdd(p.sched, 1) : unit + (int)gridDim.x;
            }
            if (live) {
                // one empty stage carries the end mark to the consumers
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (*abort_flag || !mbar_wait(&empty[s], ph ^ 1)) {
                    *abort_flag = 1;
                    atomicExch(p.err, 101);
                    live = false;
                } else {
                    tile_slot[s] = -1;
                    mbar_arrive(&full[s]);
                }
            }
            if (p.dynamic) {
                // every CTA has taken its last number by the time it counts itself done; the last one
                // to do so puts both words back to zero for the next launch on this stream
                __threadfence();
                if (atomicAdd(p.sched + 1, 1) == (int)gridDim.x - 1) {
                    atomicExch(p.sched, 0);
                    atomicExch(p.sched + 1, 0);
                }
            }
            live = live && (*abort_flag == 0);
            if (!live) {
                // give loads already in flight a bounded time to land before the CTA retires
                for (int s = 0; s < STAGES; ++s)
                    for (int i = 0; i < 1024 && !mbar_try_wait(&full[s], 0) && !mbar_try_wait(&full[s], 1); ++i)
                        __nanosleep(256);
            }
        }
        if (STASH && warp == NCW + 1 && p.c_tma) {
            // ---------------- output warp ----------------
            // Lane 0 (the output thread) does all the waiting and issues the bulk copies; the other lanes only
            // help with the one row a store map cannot reach (below).
            for (uint32_t nt = 0;; ++nt) {
                int row = 0, col = 0, flag_idx = -1, flag_pub = 0, add = 0;
                int go = 0;
                if (lane == 0) go = [&]() -> int {
                    const StashInfo *I = info + (nt & 1);
                    if (*abort_flag) return 0;
                    if (!mbar_wait(tile_started, nt & 1)) {
                        if (!*abort_flag) {                    // not merely left behind by consumers that gave up
                            *abort_flag = 1;
                            atomicExch(p.err, 105);
                        }
                        return 0;
                    }
                    if (I->unit < 0) return 0;
                    row = I->row; col = I->col;
                    const int wait_idx = I->wait_idx, expect = I->expect, flag_wait = I->flag_wait;
                    flag_idx = I->flag_idx; flag_pub = I->flag_pub; add = I->add;
                    // the buffer is free: the stores of the tile before this one have read it (end of the loop body)
                    if (I->load) {
                        mbar_expect_tx(stash_ready, BM * BN * 8);
#pragma unroll
                        for (int b = 0; b < BN / CBOX; ++b)
                            tma_load_2d(stash + b * CBOX * BM, &tmC, row, col + CBOX * b, stash_ready);
                    } else {
                        mbar_arrive(stash_ready);
                    }
                    if (!mbar_wait(stash_full, nt & 1)) {
                        if (!*abort_flag) {
                            *abort_flag = 1;
                            atomicExch(p.err, 105);
                        }
                        return 0;
                    }
                    if (wait_idx >= 0) {
                        // in-place leaf: the longer tiles of the strip must have read these rows (columns) first
                        int *cnt = p.sched + 2 + wait_idx;
                        bool ok = false;
                        for (uint32_t spin = 0; spin < (1u << 22) && !ok; ++spin) {
                            ok = *reinterpret_cast<volatile int *>(cnt) == expect;
                            if (!ok) __nanosleep(64);
                        }
                        if (!ok) { *abort_flag = 1; atomicExch(p.err, 104); return 0; }
                        atomicExch(cnt, 0);                    // back to zero for the next launch on this stream
                        __threadfence();
                    }
                    if (flag_idx >= 0 && flag_wait > 0) {
                        // piece of a shared tile: the piece before it in k must be in C, completely
                        int *flag = p.sched + 2 + flag_idx;
                        bool ok = false;
                        for (uint32_t spin = 0; spin < (1u << 22) && !ok; ++spin) {
                            ok = *reinterpret_cast<volatile int *>(flag) == flag_wait;
                            if (!ok) __nanosleep(32);
                        }
                        if (!ok) { *abort_flag = 1; atomicExch(p.err, 103); return 0; }
                        __threadfence();
                        fence_proxy_async();                   // the bulk copies below come after what was just seen
                    }
                    if (add) {
#pragma unroll
                        for (int b = 0; b < BN / CBOX; ++b)
                            tma_reduce_add_2d(&tmCs, row, col + CBOX * b, stash + b * CBOX * BM);
                    } else {
#pragma unroll
                        for (int b = 0; b < BN / CBOX; ++b)
                            tma_store_2d(&tmCs, row, col + CBOX * b, stash + b * CBOX * BM);
                    }
                    bulk_commit_group();
                    return 1;
                }();
                go = __shfl_sync(0xffffffffu, go, 0);
                if (!go) break;
                // A TMA store clips the rows of a tile in units of 16 bytes: with an odd number of rows it would
                // write the element below the last one as well.  The store map therefore ends at the last even
                // row, and the one row it leaves out is written (or added to, in the memory system as well) by
                // the lanes of this warp, a few columns each.
                if (p.c_m & 1) {
                    row = __shfl_sync(0xffffffffu, row, 0);
                    if ((int64_t)row + BM >= p.c_m) {
                        col = __shfl_sync(0xffffffffu, col, 0);
                        add = __shfl_sync(0xffffffffu, add, 0);
                        __syncwarp();
                        const int r = (int)(p.c_m - 1 - row);
                        double *last = p.C + (p.c_m - 1) + (int64_t)col * p.ldc;
                        for (int c = lane; c < BN && col + c < p.c_n; c += 32) {
                            double *at = last + (int64_t)c * p.ldc;
                            if (add) atomicAdd(at, stash[c * BM + r]);
                            else *at = stash[c * BM + r];
                        }
                        __threadfence();
                        __syncwarp();
                    }
                }
                if (lane == 0) {
                    if (flag_idx >= 0) {
                        // the next piece of the tile may follow once this one is in C, not merely read from the buffer
                        bulk_wait_all();
                        __threadfence();
                        atomicExch(p.sched + 2 + flag_idx, flag_pub);
                    } else {
                        bulk_wait_read_all();
                    }
                }
                __syncwarp();           // the buffer is not handed back before every lane has read its row of it
            }
            if (lane == 0) bulk_wait_all();
        }
        return;
    }

    // ---------------- consumers ----------------
    if (REBALANCE) asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int wm0 = (warp % WARPS_M) * WM;
    const int wn0 = (warp / WARPS_M) * WN;
    uint32_t ba[2], bb[2];
    frag_base<MAJOR_A>(wm0, lane, ba);
    frag_base<MAJOR_B>(wn0, lane, bb);
    const uint32_t smem_base = smem_u32(smem);

    uint32_t it = 0;
    double acc[MT][NT][4];
    // multiplies the stages [kc0, kc1) of one tile into acc (zeroed first); false once the kernel has given up
    auto run_piece = [&](int kc0, int kc1, bool first_stage_ready) -> bool {
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.0;
        for (int kc = kc0; kc < kc1; ++kc, ++it) {
            const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
            if (!(first_stage_ready && kc == kc0) && (*abort_flag || !mbar_wait(&full[s], ph))) {
                *abort_flag = 1;
                atomicExch(p.err, 102);
                return false;
            }
            const uint32_t sA = smem_base + s * STAGE_BYTES;
            mma_stage<MAJOR_A, MAJOR_B, MT, NT>(sA, sA + A_BYTES, ba, bb, acc);
            release_stage(&empty[s], sA, release_sink + warp, lane);
        }
        return true;
    };

    // A tile leaves through the buffer if the tensor map of C can serve it: not a tile across the diagonal
    // of a triangular update, whose other half must stay untouched.
    auto through_stash = [&](int m0, int n0) -> bool {
        if (!STASH || !p.c_tma) return false;
        if (p.tri == 1) return m0 + BM - 1 <= n0;
        if (p.tri == 2) return m0 >= n0 + BN - 1;
        return true;
    };
    // Tells the output thread where the tile that is about to be multiplied goes (unit < 0: no more tiles).
    uint32_t nstash = 0;
    auto announce_tile = [&](int unit, int row, int col, bool load, int wait_idx, int expect) {
        if (threadIdx.x == 0) {
            StashInfo *I = info + (nstash & 1);
            I->row = row; I->col = col; I->load = load ? 1 : 0;
            I->unit = unit; I->wait_idx = wait_idx; I->expect = expect;
            I->flag_idx = -1; I->flag_wait = 0; I->flag_pub = 0; I->add = 0;
            mbar_arrive(tile_started);
        }
    };
    // The same for the piece [kc0, kc1) of shared tile r: the head is stored (beta applied), later pieces are
    // added, each once the tile's flag shows that the piece before it is in C.
    auto announce_piece = [&](int unit, int row, int col, int r, int kc0, int kc1) {
        if (threadIdx.x == 0) {
            StashInfo *I = info + (nstash & 1);
            I->row = row; I->col = col; I->load = (kc0 == 0 && p.beta != 0.0) ? 1 : 0;
            I->unit = unit; I->wait_idx = -1; I->expect = 0;
            I->flag_idx = r; I->flag_wait = kc0; I->flag_pub = kc1 == kt ? 0 : kc1; I->add = kc0 > 0 ? 1 : 0;
            mbar_arrive(tile_started);
        }
    };
    // Folds the finished tile into the buffer (alpha * acc + beta * old) and hands it to the output thread;
    // false once the kernel has given up.
    auto stash_tile = [&](double beta) -> bool {
        if (*abort_flag || !mbar_wait(stash_ready, nstash & 1)) {
            *abort_flag = 1;
            atomicExch(p.err, 106);
            return false;
        }
        ++nstash;
        const double alpha = p.alpha;
        const bool use_c = beta != 0.0;
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                if (MAJOR_A == MN_MAJOR) {
                    // the two rows a lane holds are adjacent: one 16-byte access per column
                    const int r0 = c_row<MAJOR_A>(wm0 + 16 * i, lane, 0);
#pragma unroll
                    for (int w = 0; w < 2; ++w) {
                        const int col = c_col<MAJOR_B>(wn0 + 8 * j, lane, w);
                        double2 *at = reinterpret_cast<double2 *>(stash + col * BM + r0);
                        double2 v = make_double2(alpha * acc[i][j][w], alpha * acc[i][j][2 + w]);
                        if (use_c) {
                            const double2 o = *at;
                            v.x = fma(beta, o.x, v.x);
                            v.y = fma(beta, o.y, v.y);
                        }
                        *at = v;
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int row = c_row<MAJOR_A>(wm0 + 16 * i, lane, e >> 1);
                        const int col = c_col<MAJOR_B>(wn0 + 8 * j, lane, e & 1);
                        double v = alpha * acc[i][j][e];
                        if (use_c) v = fma(beta, stash[col * BM + row], v);
                        stash[col * BM + row] = v;
                    }
                }
            }
        fence_proxy_async();                 // the TMA store reads what this thread has just written
        __syncwarp();
        if (lane == 0) mbar_arrive(stash_full);
        return true;
    };

    for (;;) {
        // the first stage of a unit tells which unit it is
        {
            const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
            if (*abort_flag || !mbar_wait(&full[s], ph)) {
                *abort_flag = 1;
                atomicExch(p.err, 102);
                return;
            }
        }
        const int unit = tile_slot[it % STAGES];
        if (unit < 0) {
            if (STASH && p.c_tma) announce_tile(-1, 0, 0, false, -1, 0);      // the output thread leaves after the last tile
            return;
        }
        if (SHARE && p.leaf) {
            static_assert(kLeafBlockStages * kBK == 128, "a block of k is one tile of the triangular operand");
            const LeafUnit u = leaf_decode(p.leaf, p.tiles_m, p.tiles_n, unit, kt);
            int *cnt = p.sched + 2 + u.strip * u.T;
            // the output thread stores once every longer tile of the strip has counted block d
            announce_tile(unit, u.tm * BM, u.tn * BN, false, u.expect > 0 ? u.strip * u.T + u.d : -1, u.expect);
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.0;
            for (int kc = u.kc0; kc < u.kc1; ++kc, ++it) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (kc != u.kc0 && (*abort_flag || !mbar_wait(&full[s], ph))) {
                    *abort_flag = 1;
                    atomicExch(p.err, 102);
                    return;
                }
                // the last stage of a block of k has landed: the tile that will overwrite those rows
                // (columns) of the strip has one reader less to wait for
                if (threadIdx.x == 0) {
                    bool last_of_block;
                    const int blk = leaf_block_of(u, kc - u.kc0, last_of_block);
                    if (last_of_block && blk != u.d) atomicAdd(cnt + blk, 1);
                }
                const uint32_t sA = smem_base + s * STAGE_BYTES;
                mma_stage<MAJOR_A, MAJOR_B, MT, NT>(sA, sA + A_BYTES, ba, bb, acc);
                release_stage(&empty[s], sA, release_sink + warp, lane);
            }
            if (!stash_tile(0.0)) return;
            continue;
        }
        if (SHARE && p.nbatch > 1) {
            const int per = p.tiles_m * p.tiles_n, b = unit / per;
            int tm, tn;
            tile_coord(unit - b * per, p.tiles_m, p.tiles_n, tm, tn);
            const BatchShift sh = batch_shift(p, b);
            announce_tile(unit, tm * BM + sh.cr, tn * BN + sh.cc, false, -1, 0);
            if (!run_piece(0, kt, true)) return;
            if (!stash_tile(0.0)) return;
            continue;
        }
        if (!SHARE || unit < p.split_first) {
            int tm, tn;
            tile_coord(unit, p.tiles_m, p.tiles_n, tm, tn);
            if (through_stash(tm * BM, tn * BN)) {
                announce_tile(unit, tm * BM, tn * BN, p.beta != 0.0, -1, 0);
                if (!run_piece(0, kt, true)) return;
                if (!stash_tile(p.beta)) return;
                continue;
            }
            if (SHARE && p.beta != 0.0) prefetch_c<MAJOR_A, MAJOR_B, MT, NT>(p, (int64_t)tm * BM, (int64_t)tn * BN, wm0, wn0, lane);
            if (!run_piece(0, kt, true)) return;
            epilogue<MAJOR_A, MAJOR_B, MT, NT, EG>(p, p.C, p.beta, (int64_t)tm * BM, (int64_t)tn * BN, wm0, wn0, lane, acc);
            continue;
        }
        StreamWalk walk(p.region_tiles, p.nsu, unit - p.split_first, kt);
        Piece pc;
        bool first = true;
        while (walk.next(pc)) {
            int tm, tn;
            tile_coord(region_tile(p, pc.r), p.tiles_m, p.tiles_n, tm, tn);
            const int64_t m0 = (int64_t)tm * BM, n0 = (int64_t)tn * BN;
            const bool whole = pc.kc0 == 0 && pc.kc1 == kt;
            if (whole && through_stash((int)m0, (int)n0)) {
                announce_tile(unit, (int)m0, (int)n0, p.beta != 0.0, -1, 0);
                if (!run_piece(pc.kc0, pc.kc1, first)) return;
                first = false;
                if (!stash_tile(p.beta)) return;
                continue;
            }
            if (!whole && through_stash((int)m0, (int)n0)) {
                // A piece of a shared tile leaves through the buffer as well: the consumers go on with their
                // next piece while the output thread waits for the tile's turn (same order of k as below)
                announce_piece(unit, (int)m0, (int)n0, pc.r, pc.kc0, pc.kc1);
                if (!run_piece(pc.kc0, pc.kc1, first)) return;
                first = false;
                if (!stash_tile(pc.kc0 == 0 ? p.beta : 0.0)) return;
                continue;
            }
            if (pc.kc0 > 0 || p.beta != 0.0) prefetch_c<MAJOR_A, MAJOR_B, MT, NT>(p, m0, n0, wm0, wn0, lane);
            if (!run_piece(pc.kc0, pc.kc1, first)) return;
            first = false;
            if (whole) {
                epilogue<MAJOR_A, MAJOR_B, MT, NT, EG>(p, p.C, p.beta, m0, n0, wm0, wn0, lane, acc);
                continue;
            }
            // A shared tile.  Its pieces fold into C in order of k: the head [0, x) applies beta and
            // leaves x in the tile's flag; the piece that starts at x waits (bounded) for that value,
            // adds its share and leaves its own end; the piece that ends at kt puts the flag back to
            // zero.  The order is fixed, so the result does not depend on timing.
            int *flag = p.sched + 2 + pc.r;
            if (pc.kc0 > 0) {
                if (threadIdx.x == 0) {
                    bool ok = false;
                    for (uint32_t spin = 0; spin < (1u << 22) && !ok; ++spin) {
                        ok = *reinterpret_cast<volatile int *>(flag) == pc.kc0;
                        if (!ok) __nanosleep(64);
                    }
                    if (!ok) { *abort_flag = 1; atomicExch(p.err, 103); }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
                if (*abort_flag) return;
                __threadfence();
            }
            epilogue<MAJOR_A, MAJOR_B, MT, NT, EG>(p, p.C, pc.kc0 > 0 ? 1.0 : p.beta, m0, n0, wm0, wn0, lane, acc);
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
            if (threadIdx.x == 0) atomicExch(flag, pc.kc1 == kt ? 0 : pc.kc1);
        }
    }
}

// ---------------------------------------------------------------------------
// Same tiles, filled by ordinary loads: any base alignment, any ld.
// ---------------------------------------------------------------------------
template <int BMN, int MAJOR, int NTHREADS>
__device__ __forceinline__ void ldg_tile(double (&r)[BMN * kBK / NTHREADS], const double *base,
                                         int64_t ld, int64_t mn0, int64_t mn_ext, int64_t k0,
                                         int64_t k_ext)
{
    // MN-major storage: element (mn, k) at base[mn + k*ld]; K-major: base[k + mn*ld]
    constexpr int PER = BMN * kBK / NTHREADS;
#pragma unroll
    for (int q = 0; q < PER; ++q) {
        const int e = threadIdx.x + q * NTHREADS;
        int rr, kk;
        if (MAJOR == MN_MAJOR) { rr = e % BMN; kk = e / BMN; }
        else                   { kk = e % kBK; rr = e / kBK; }
        const int64_t gmn = mn0 + rr, gk = k0 + kk;
        double v = 0.0;
        if (gmn < mn_ext && gk < k_ext)
            v = (MAJOR == MN_MAJOR) ? __ldg(base + gmn + gk * ld) : __ldg(base + gk + gmn * ld);
        r[q] = v;
    }
}

template <int BMN, int MAJOR, int NTHREADS>
__device__ __forceinline__ void sts_tile(uint8_t *s, const double (&r)[BMN * kBK / NTHREADS])
{
    constexpr int PER = BMN * kBK / NTHREADS;
#pragma unroll
    for (int q = 0; q < PER; ++q) {
        const int e = threadIdx.x + q * NTHREADS;
        int rr, kk;
        if (MAJOR == MN_MAJOR) { rr = e % BMN; kk = e / BMN; }
        else                   { kk = e % kBK; rr = e / kBK; }
        *reinterpret_cast<double *>(s + elem_off<MAJOR>(rr, kk)) = r[q];
    }
}

template <int BM, int BN, int WARPS_M, int WARPS_N, int MAJOR_A, int MAJOR_B>
__global__ void __launch_bounds__(WARPS_M *WARPS_N * 32)
dgemm_ldg_kernel(const GemmParams p)
{
    constexpr int NTHREADS = WARPS_M * WARPS_N * 32;
    constexpr int WM = BM / WARPS_M, WN = BN / WARPS_N;
    constexpr int MT = WM / 16, NT = WN / 8;
    constexpr uint32_t A_BYTES = BM * 128, B_BYTES = BN * 128;
    constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                                ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm0 = (warp % WARPS_M) * WM;
    const int wn0 = (warp / WARPS_M) * WN;
    uint32_t ba[2], bb[2];
    frag_base<MAJOR_A>(wm0, lane, ba);
    frag_base<MAJOR_B>(wn0, lane, bb);
    const uint32_t smem_base = smem_u32(smem);

    const int tile = blockIdx.x;
    int tm, tn;
    tile_coord(tile, p.tiles_m, p.tiles_n, tm, tn);
    const int64_t m0 = (int64_t)tm * BM, n0 = (int64_t)tn * BN;
    if (tile_skipped(p.tri, m0, n0, BM, BN)) return;
    const int kt = (int)((p.k + kBK - 1) / kBK);

    double acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.0;

    double ra[BM * kBK / NTHREADS], rb[BN * kBK / NTHREADS];
    ldg_tile<BM, MAJOR_A, NTHREADS>(ra, p.A, p.lda, m0, p.m, 0, p.k);
    ldg_tile<BN, MAJOR_B, NTHREADS>(rb, p.B, p.ldb, n0, p.n, 0, p.k);
    sts_tile<BM, MAJOR_A, NTHREADS>(smem, ra);
    sts_tile<BN, MAJOR_B, NTHREADS>(smem + A_BYTES, rb);
    __syncthreads();

    for (int kc = 0; kc < kt; ++kc) {
        const int cur = kc & 1;
        if (kc + 1 < kt) {
            ldg_tile<BM, MAJOR_A, NTHREADS>(ra, p.A, p.lda, m0, p.m, (int64_t)(kc + 1) * kBK, p.k);
            ldg_tile<BN, MAJOR_B, NTHREADS>(rb, p.B, p.ldb, n0, p.n, (int64_t)(kc + 1) * kBK, p.k);
        }
        const uint32_t sA = smem_base + cur * STAGE_BYTES;
        mma_stage<MAJOR_A, MAJOR_B, MT, NT>(sA, sA + A_BYTES, ba, bb, acc);
        if (kc + 1 < kt) {
            uint8_t *nxt = smem + (cur ^ 1) * STAGE_BYTES;
            sts_tile<BM, MAJOR_A, NTHREADS>(nxt, ra);
            sts_tile<BN, MAJOR_B, NTHREADS>(nxt + A_BYTES, rb);
        }
        __syncthreads();
    }
    epilogue<MAJOR_A, MAJOR_B, MT, NT, 1>(p, p.C, p.beta, m0, n0, wm0, wn0, lane, acc);
}

// C <- beta*C (beta == 0 assigns zeros), the alpha == 0 / k == 0 quick path
// (ulmblas/level3/gemm.tcc:52-55 -> level1extensions/gescal.tcc:11-39).
__global__ void dscal_matrix_kernel(double *C, int64_t ldc, int64_t m, int64_t n, double beta, int tri)
{
    const int64_t total = m * n;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = e % m, j = e / m;
        if (tri == 1 && i > j) continue;
        if (tri == 2 && i < j) continue;
        double *c = C + i + j * ldc;
        *c = (beta == 0.0) ? 0.0 : *c * beta;
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
// SMs the persistent grid leaves free (for a collective's kernels running beside it)
static std::atomic<int> g_sm_reserve{0};

int scale_matrix_device(cudaStream_t st, double *C, int64_t ldc, int64_t m, int64_t n, double beta, int tri)
{
    if (beta == 1.0 || m <= 0 || n <= 0) return ULMB200_OK;
    int64_t blocks = (m * n + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    dscal_matrix_kernel<<<(int)blocks, 256, 0, st>>>(C, ldc, m, n, beta, tri);
    count_launch();
    return check_cuda(cudaGetLastError(), "dscal_matrix_kernel", __FILE__, __LINE__);
}


template <int BM, int BN, int WARPS_M, int WARPS_N, int MAJOR_A, int MAJOR_B, int STAGES, int CTAS_PER_SM>
static int launch_tma(cudaStream_t st, const GemmParams &p, const double *A, const double *B, bool may_share)
{
    constexpr int ctas_per_sm = CTAS_PER_SM;
    CUtensorMap tmA, tmB;
    bool ok;
    // K-major: dim0 = k (contiguous), dim1 = m|n, box 16 x BM|BN.  MN-major: dim0 = m|n, dim1 = k, box 16 x 16.
    const int64_t am = p.ext_a_mn ? p.ext_a_mn : p.m, ak = p.ext_a_k ? p.ext_a_k : p.k;
    const int64_t bn = p.ext_b_mn ? p.ext_b_mn : p.n, bk = p.ext_b_k ? p.ext_b_k : p.k;
    if (MAJOR_A == K_MAJOR)
        ok = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, A, ak, am, p.lda, kBK, BM);
    else
        ok = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, A, am, ak, p.lda, 16, kBK);
    if (MAJOR_B == K_MAJOR)
        ok = ok && make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, B, bk, bn, p.ldb, kBK, BN);
    else
        ok = ok && make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, B, bn, bk, p.ldb, 16, kBK);
    if (!ok) return -1;   // caller falls back to the ldg kernel
    // C for the one-CTA-per-SM shape: boxes of BM rows x 32 columns, no swizzle.  Without a map (odd ldc,
    // unaligned C) the consumers write C themselves.
    GemmParams q = p;
    CUtensorMap tmC = tmA, tmCs = tmA;
    q.c_tma = 0;
    q.c_m = p.ext_c_m ? p.ext_c_m : p.m;
    q.c_n = p.ext_c_n ? p.ext_c_n : p.n;
    if (ctas_per_sm == 1 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0 && p.ldc % 2 == 0 && p.ldc < (1ll << 36)) {
        // one map to fetch old tiles, one to store new ones that ends at the last even row (see the output thread)
        const int64_t even_rows = q.c_m & ~1ll;
        q.c_tma = make_tmap_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, p.C, q.c_m, q.c_n, p.ldc, BM, 32,
                               CU_TENSOR_MAP_SWIZZLE_NONE) &&
                  (even_rows == 0 || make_tmap_2d(&tmCs, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, p.C, even_rows, q.c_n, p.ldc, BM, 32,
                                                  CU_TENSOR_MAP_SWIZZLE_NONE)) ? 1 : 0;
        if (even_rows == 0) q.c_tma = 0;              // a single row: the consumers write it themselves
    }
    if ((p.leaf || p.nbatch > 1) && !q.c_tma) return -1;     // those tiles only leave through the buffer

    constexpr size_t SMEM = (size_t)STAGES * (BM + BN) * 128 + (CTAS_PER_SM == 1 ? (size_t)BM * BN * 8 : 0) +
                            (2 * STAGES + 3) * 8 + 2 * sizeof(StashInfo) + 16 + 4 * STAGES + 4 * 16 + 1024;
    auto kern = dgemm_tma_kernel<BM, BN, WARPS_M, WARPS_N, MAJOR_A, MAJOR_B, STAGES, CTAS_PER_SM>;
    static bool attr_done[kMaxDevices] = {};
    const int dev = current_device();
    if (!attr_done[dev]) {
        ULMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
        attr_done[dev] = true;
    }
    const int tiles = p.tiles_m * p.tiles_n * (p.nbatch > 1 ? p.nbatch : 1);
    int sms = sm_count() - g_sm_reserve.load(std::memory_order_relaxed);
    if (sms < 1) sms = 1;
    const int slots = sms * ctas_per_sm;
    q.split_first = tiles; q.nsu = 0; q.region_tiles = 0;
    const int kt = (int)((p.k + kBK - 1) / kBK);
    const int mode = settings().dgemm_split;
    // Sharing the last tiles.  With one CTA per SM the tiles beyond the last full wave leave most
    // SMs idle for a whole tile time (a SYRK of order 8192: 2080 tiles = 14 waves + 8 tiles; a
    // 1024^3 product: 64 tiles on 148 SMs).  Those tiles' pipeline stages are dealt out evenly to
    // all CTAs instead, whenever that is cheaper than one more wave of whole tiles.
    if (p.leaf || p.nbatch > 1) {
        // in-place leaf, batch: one unit per tile, no sharing
        q.split_first = tiles;
    } else if (mode != 0 && may_share && p.sched && ctas_per_sm == 1 && tiles < (1 << 30)) {
        auto real = [&](int id) {
            int tm, tn;
            tile_coord(id, p.tiles_m, p.tiles_n, tm, tn);
            return !tile_skipped(p.tri, (int64_t)tm * BM, (int64_t)tn * BN, BM, BN);
        };
        int64_t nreal = tiles;
        if (p.tri != 0) {
            nreal = 0;
            for (int tn = 0; tn < p.tiles_n; ++tn)
                for (int tm = 0; tm < p.tiles_m; ++tm)
                    nreal += !tile_skipped(p.tri, (int64_t)tm * BM, (int64_t)tn * BN, BM, BN);
        }
        const int epi = settings().dgemm_epi > 0 ? settings().dgemm_epi : (q.c_tma && p.tri == 0 ? kBufferedEpilogueStages : kEpilogueStages);
        const SharePlan sp = plan_shared_tiles(nreal, kt, slots, mode == 2, epi);
        if (sp.nsu > 0) {
            int first = tiles, found = 0;
            while (first > 0 && found < sp.region_tiles) { --first; found += real(first); }
            if (tiles - first <= 65535) {
                if (p.tri != 0) {
                    int r = 0;
                    for (int id = first; id < tiles; ++id)
                        if (real(id)) q.rtile[r++] = (unsigned short)(id - first);
                }
                q.split_first = first; q.nsu = sp.nsu; q.region_tiles = sp.region_tiles;
            }
        }
    }
    const int64_t units = (int64_t)q.split_first + q.nsu;
    const int grid = (int)(units < slots ? units : slots);
    // More units than CTAs: they are handed out through the stream's counter word.  Without
    // scheduler words (none left for this stream) the CTAs stride through the units instead.
    q.dynamic = (units > grid && p.sched) ? 1 : 0;
    trace("dgemm kernel tile %dx%d %s grid %d units %lld (whole %d, shared tiles %d over %d CTAs) kt %d",
          BM, BN, q.dynamic ? "dynamic" : "static", grid, (long long)units, q.split_first, q.region_tiles, q.nsu, kt);
    kern<<<grid, (WARPS_M * WARPS_N + 4) * 32, SMEM, st>>>(tmA, tmB, tmC, tmCs, q);
    count_launch();
    ULMB_CUDA(cudaGetLastError());
    return ULMB200_OK;
}

template <int BM, int BN, int WARPS_M, int WARPS_N, int MAJOR_A, int MAJOR_B>
static int launch_ldg(cudaStream_t st, const GemmParams &p)
{
    constexpr size_t SMEM = (size_t)2 * (BM + BN) * 128 + 1024;
    auto kern = dgemm_ldg_kernel<BM, BN, WARPS_M, WARPS_N, MAJOR_A, MAJOR_B>;
    static bool attr_done[kMaxDevices] = {};
    const int dev = current_device();
    if (!attr_done[dev]) {
        ULMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
        attr_done[dev] = true;
    }
    kern<<<p.tiles_m * p.tiles_n, WARPS_M * WARPS_N * 32, SMEM, st>>>(p);
    count_launch();
    ULMB_CUDA(cudaGetLastError());
    return ULMB200_OK;
}

template <int MAJOR_A, int MAJOR_B>
static int dispatch(cudaStream_t st, GemmParams p, bool tma_ok, bool may_share)
{
    const Settings &cfg = settings();
    // Tile shape by estimated time.  Large tiles (128 x 128, one CTA per SM) run the tensor pipe best and
    // can share the last tiles' stages among all CTAs; half tiles (128 x 64, one CTA per SM) put a product of
    // few large tiles on twice as many SMs; small tiles (64 x 64, two CTAs per SM) waste least on padding
    // and fill the machine with the fewest rows and columns.  Per-SM times in microseconds, measured on
    // this part: one 16-k stage of a large tile 2.09, of a half tile 1.2, of a small tile 1.2 when two CTAs
    // share the SM (their operand traffic from L2 is twice the large tiles') and 0.85 when one has it
    // alone; an epilogue 1 (large and half tiles leave through shared memory beside the next tile's
    // main loop) / 2.
    const int64_t t128 = ((p.m + 127) / 128) * ((p.n + 127) / 128);
    const int64_t thalf = ((p.m + 127) / 128) * ((p.n + 63) / 64);
    const int64_t t64 = ((p.m + 63) / 64) * ((p.n + 63) / 64);
    const int kt = (int)((p.k + kBK - 1) / kBK);
    const int sms = sm_count();
    constexpr double kStage128 = 2.09, kStageHalf = 1.2, kStage64Pair = 1.2, kStage64Alone = 0.85, kEpi128 = 1.0,
                     kEpi64 = 2.0;
    const bool sharing = tma_ok && may_share && p.sched && cfg.dgemm_split != 0 && p.tri == 0;
    // pieces of shared tiles leave through the tile buffer when C can have a tensor map (as launch_tma decides)
    const bool c_map = (reinterpret_cast<uintptr_t>(p.C) & 15) == 0 && p.ldc % 2 == 0 && p.m > 1;
    const int epi = cfg.dgemm_epi > 0 ? cfg.dgemm_epi : (c_map ? kBufferedEpilogueStages : kEpilogueStages);
    // one CTA per SM: whole waves, the last one shared among all CTAs where that is cheaper
    auto one_per_sm = [&](int64_t tiles, double stage) {
        double t = (double)((tiles + sms - 1) / sms) * (kt * stage + kEpi128);
        if (sharing) {
            const SharePlan sp = plan_shared_tiles(tiles, kt, sms, false, epi);
            if (sp.nsu > 0)
                t = (double)(tiles / sms) * (kt * stage + kEpi128) + (double)shared_cost(sp.region_tiles, kt, sp.nsu, epi) * stage;
        }
        return t;
    };
    const double time128 = one_per_sm(t128, kStage128);
    const double time_half = one_per_sm(thalf, kStageHalf);
    const int64_t waves64 = (t64 + 2 * sms - 1) / (2 * sms);
    const double stage64 = t64 <= sms ? kStage64Alone : kStage64Pair;
    const double time64 = (double)waves64 * (kt * stage64 + kEpi64);
    int shape = time128 <= time64 ? 128 : 64;
    if (tma_ok && p.tri == 0 && time_half < (shape == 128 ? time128 : time64)) shape = 12864;
    if (cfg.dgemm_tile == 128 || cfg.dgemm_tile == 64 || (cfg.dgemm_tile == 12864 && tma_ok)) shape = cfg.dgemm_tile;
    if (cfg.dgemm_ldg) { tma_ok = false; if (shape == 12864) shape = 128; }
    if (shape == 128) {
        p.tiles_m = (int)((p.m + 127) / 128);
        p.tiles_n = (int)((p.n + 127) / 128);
        if (tma_ok) {
            // Three stages of 32 KB, not four: with both operands K-major (op(A) = A^T, op(B) = B)
            // a four-deep ring measured 6% slower (33.3 against 35.6 TFLOP/s at 8192^3); the other
            // three modes are within 1% either way.
            int r = launch_tma<128, 128, 2, 4, MAJOR_A, MAJOR_B, 3, 1>(st, p, p.A, p.B, may_share);
            if (r >= 0) return r;
        }
        return launch_ldg<128, 128, 2, 4, MAJOR_A, MAJOR_B>(st, p);
    }
    if (shape == 12864) {
        p.tiles_m = (int)((p.m + 127) / 128);
        p.tiles_n = (int)((p.n + 63) / 64);
        int r = launch_tma<128, 64, 2, 4, MAJOR_A, MAJOR_B, 4, 1>(st, p, p.A, p.B, may_share);
        if (r >= 0) return r;
    }
    p.tiles_m = (int)((p.m + 63) / 64);
    p.tiles_n = (int)((p.n + 63) / 64);
    if (tma_ok) {
        int r = launch_tma<64, 64, 2, 2, MAJOR_A, MAJOR_B, 4, 2>(st, p, p.A, p.B, false);
        if (r >= 0) return r;
    }
    return launch_ldg<64, 64, 2, 2, MAJOR_A, MAJOR_B>(st, p);
}

int dgemm_device(cudaStream_t st, int tri, int transA, int transB, int64_t m, int64_t n,
                 int64_t k, double alpha, const double *A, int64_t lda, const double *B,
                 int64_t ldb, double beta, double *C, int64_t ldc, int *err_word)
{
    if (m < 0 || n < 0 || k < 0) return set_status(ULMB200_BAD_ARGUMENT);
    const int64_t rowsA = transA ? k : m, rowsB = transB ? n : k;
    if (lda < (rowsA > 1 ? rowsA : 1) || ldb < (rowsB > 1 ? rowsB : 1) || ldc < (m > 1 ? m : 1))
        return set_status(ULMB200_BAD_ARGUMENT);
    if (m == 0 || n == 0) return set_status(ULMB200_OK);
    if (int st0 = ensure_device()) return set_status(st0);

    if (alpha == 0.0 || k == 0) return set_status(scale_matrix_device(st, C, ldc, m, n, beta, tri));

    GemmParams p = {};
    p.m = m; p.n = n; p.k = k; p.alpha = alpha; p.beta = beta;
    p.A = A; p.B = B; p.lda = lda; p.ldb = ldb; p.C = C; p.ldc = ldc;
    p.tiles_m = p.tiles_n = 0; p.tri = tri;
    p.split_first = 0; p.nsu = 0; p.region_tiles = 0; p.dynamic = 0;
    p.leaf = 0; p.nbatch = 0; p.bat_nlo = 1;
    p.ext_a_mn = p.ext_a_k = p.ext_b_mn = p.ext_b_k = p.ext_c_m = p.ext_c_n = 0;
    // A caller that brings its own error word must not allocate device memory: its launches take the
    // two words after the error word as tile counter and never share tiles (no fold flags there).
    // Such callers keep their calls on one device from overlapping, so the words are theirs alone.
    const bool may_share = err_word == nullptr;
    p.err = err_word ? err_word : device_error_word();
    if (!p.err) return set_status(ULMB200_CUDA_ERROR);
    p.sched = err_word ? err_word + 1 : sched_words(st);

    // TMA needs 16-byte aligned bases and row pitches, and 32-bit coordinates.
    const bool tma_ok = ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) == 0 &&
                        (lda % 2 == 0) && (ldb % 2 == 0) && m < (1ll << 31) - 256 &&
                        n < (1ll << 31) - 256 && k < (1ll << 31) - 256 &&
                        lda < (1ll << 36) && ldb < (1ll << 36);
    int r;
    if (!transA && !transB)      r = dispatch<MN_MAJOR, K_MAJOR>(st, p, tma_ok, may_share);
    else if (!transA && transB)  r = dispatch<MN_MAJOR, MN_MAJOR>(st, p, tma_ok, may_share);
    else if (transA && !transB)  r = dispatch<K_MAJOR, K_MAJOR>(st, p, tma_ok, may_share);
    else                         r = dispatch<K_MAJOR, MN_MAJOR>(st, p, tma_ok, may_share);
    return set_status(r);
}

// X <- op(T) * X (left) or X * op(T) (right) in place, T a triangular matrix of order dim whose 128 x 128
// diagonal blocks hold zeros in the other triangle (the inverted or zero-filled diagonal blocks of the
// triangular solver and multiply): the leaf of ulmBLAS's trlsm / trusm / trlmm / trumm recursion
// (ulmblas/level3/trlsm.tcc:61-74), without their packed copy of the block row.  lower_op: op(T) is
// lower triangular.  Blocks of T beyond the diagonal ones in the other triangle are never read.
// Returns -1 when the operands do not qualify (not TMA-addressable, no scheduler words, more tiles
// than counters); the caller then multiplies into a work tile and copies back.
int dgemm_leaf_inplace(cudaStream_t st, int left, int lower_op, int transT, int64_t dim, int64_t other, double alpha,
                       const double *T, int64_t ldt, double *X, int64_t ldx, int *err_word)
{
    if (dim <= 0 || other <= 0) return ULMB200_OK;
    if (err_word) return -1;
    const int64_t m = left ? dim : other, n = left ? other : dim, k = dim;
    const bool tma_ok = ((reinterpret_cast<uintptr_t>(T) | reinterpret_cast<uintptr_t>(X)) & 15) == 0 &&
                        (ldt % 2 == 0) && (ldx % 2 == 0) && other < (1ll << 31) - 256 && dim < (1ll << 31) - 256 &&
                        ldx < (1ll << 36) && ldt < (1ll << 36);
    if (!tma_ok) return -1;
    GemmParams p = {};
    p.m = m; p.n = n; p.k = k; p.alpha = alpha; p.beta = 0.0;
    p.A = left ? T : X; p.lda = left ? ldt : ldx;
    p.B = left ? X : T; p.ldb = left ? ldx : ldt;
    p.C = X; p.ldc = ldx;
    p.tiles_m = (int)((m + 127) / 128); p.tiles_n = (int)((n + 127) / 128);
    p.tri = 0; p.split_first = 0; p.nsu = 0; p.region_tiles = 0; p.dynamic = 0;
    p.nbatch = 0; p.bat_nlo = 1;
    p.ext_a_mn = p.ext_a_k = p.ext_b_mn = p.ext_b_k = p.ext_c_m = p.ext_c_n = 0;
    p.err = device_error_word();
    p.sched = sched_words(st);
    if (!p.err || !p.sched) return -1;
    if ((int64_t)p.tiles_m * p.tiles_n > kSchedFlags) return -1;
    // left: X_i = sum_j op(T)_ij X_j, a lower op(T) meets blocks j <= i; right: X_j = sum_i X_i op(T)_ij, an
    // upper op(T) meets blocks i <= j
    p.leaf = left ? (lower_op ? 1 : 2) : (lower_op ? 4 : 3);
    const int ta = left ? transT : 0, tb = left ? 0 : transT;
    int r;
    if (!ta && !tb)      r = launch_tma<128, 128, 2, 4, MN_MAJOR, K_MAJOR, 3, 1>(st, p, p.A, p.B, false);
    else if (!ta && tb)  r = launch_tma<128, 128, 2, 4, MN_MAJOR, MN_MAJOR, 3, 1>(st, p, p.A, p.B, false);
    else if (ta && !tb)  r = launch_tma<128, 128, 2, 4, K_MAJOR, K_MAJOR, 3, 1>(st, p, p.A, p.B, false);
    else                 r = launch_tma<128, 128, 2, 4, K_MAJOR, MN_MAJOR, 3, 1>(st, p, p.A, p.B, false);
    return r;
}

// nbatch products C_b <- alpha * A_b * B_b (no transposes, beta = 0) of one shape m x n x k in one launch.
// A_b, B_b, C_b are blocks of three stored matrices; block b = hi * nlo + lo starts lo * s[0] + hi * s[1]
// rows / columns further on, s being the pair given for that coordinate.  m and n are multiples of 128,
// k of 16; the blocks of different products do not overlap; a_rows .. c_cols are the extents of the stored
// matrices.  Returns -1 when TMA cannot address the operands.
int dgemm_batched(cudaStream_t st, int64_t m, int64_t n, int64_t k, double alpha, const double *A, int64_t lda,
                  int64_t a_rows, int64_t a_cols, const double *B, int64_t ldb, int64_t b_rows, int64_t b_cols,
                  double *C, int64_t ldc, int64_t c_rows, int64_t c_cols, const BatchShape &bs)
{
    if (m <= 0 || n <= 0 || k <= 0 || bs.count <= 0) return ULMB200_OK;
    if (m % 128 || n % 128 || k % kBK) return -1;
    const bool tma_ok = ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) == 0 &&
                        (lda % 2 == 0) && (ldb % 2 == 0) && a_rows < (1ll << 31) - 256 && a_cols < (1ll << 31) - 256 &&
                        b_rows < (1ll << 31) - 256 && b_cols < (1ll << 31) - 256 && lda < (1ll << 36) && ldb < (1ll << 36);
    if (!tma_ok) return -1;
    GemmParams p = {};
    p.m = m; p.n = n; p.k = k; p.alpha = alpha; p.beta = 0.0;
    p.A = A; p.lda = lda; p.B = B; p.ldb = ldb; p.C = C; p.ldc = ldc;
    p.tiles_m = (int)(m / 128); p.tiles_n = (int)(n / 128);
    p.tri = 0; p.split_first = 0; p.nsu = 0; p.region_tiles = 0; p.dynamic = 0; p.leaf = 0;
    p.nbatch = bs.count > 1 ? bs.count : 0; p.bat_nlo = bs.nlo > 0 ? bs.nlo : 1;
    for (int i = 0; i < 2; ++i) {
        p.bat_am[i] = bs.a_row[i]; p.bat_ak[i] = bs.a_col[i];
        p.bat_bk[i] = bs.b_row[i]; p.bat_bn[i] = bs.b_col[i];
        p.bat_c[i] = bs.c_row[i] + bs.c_col[i] * ldc;
        p.bat_cr[i] = (int)bs.c_row[i]; p.bat_cc[i] = (int)bs.c_col[i];
    }
    p.ext_a_mn = a_rows; p.ext_a_k = a_cols; p.ext_b_mn = b_cols; p.ext_b_k = b_rows;
    p.ext_c_m = c_rows; p.ext_c_n = c_cols;
    if (c_rows >= (1ll << 31) - 256 || c_cols >= (1ll << 31) - 256) return -1;
    p.err = device_error_word();
    p.sched = sched_words(st);
    if (!p.err) return -1;
    if (bs.count == 1) {
        // one product: the shifts of block (0, 0) are zero, a plain launch with the stored extents
        p.nbatch = 0;
    }
    return launch_tma<128, 128, 2, 4, MN_MAJOR, K_MAJOR, 3, 1>(st, p, p.A, p.B, false);
}

int sm_reserve_swap(int sms)
{
    return g_sm_reserve.exchange(sms < 0 ? 0 : sms, std::memory_order_relaxed);
}

}  // namespace ulmb200

extern "C" void ulmb200_set_sm_reserve(int sms)
{
    ulmb200::g_sm_reserve.store(sms < 0 ? 0 : sms, std::memory_order_relaxed);
}

extern "C" int ulmb200_dgemm(void *stream, int transA, int transB, int64_t m, int64_t n, int64_t k,
                             double alpha, const double *dA, int64_t ldA, const double *dB,
                             int64_t ldB, double beta, double *dC, int64_t ldC)
{
    return ulmb200::dgemm_device(static_cast<cudaStream_t>(stream), 0, transA, transB, m, n, k,
                                 alpha, dA, ldA, dB, ldB, beta, dC, ldC);
}
