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
    // In-place product with a block-triangular first or second operand (the leaf of the triangular
    // solver and multiply: C is the very block of B that is being read).  pair = 1: two tile rows over
    // each tile column, pair = 2: two tile columns over each tile row.  Unit 2q is the tile of pair q
    // that needs all of K; unit 2q+1 is tile number pair_half of the pair, which only meets its own
    // diagonal block of the triangular operand (stages [8*pair_half, ...)) and whose output region
    // the other tile still reads: it stores only after the other tile's loads have all landed
    // (flag q of the scheduler words).  0: off.
    int pair, pair_half;
};

// pair mode: unit -> tile coordinates and the range of pipeline stages it multiplies
__device__ __forceinline__ void pair_decode(const GemmParams &p, int unit, int kt, int &tm, int &tn, int &kc0, int &kc1)
{
    const int q = unit >> 1, late = unit & 1;
    const int which = late ? p.pair_half : 1 - p.pair_half;
    if (p.pair == 1) { tm = which; tn = q; } else { tm = q; tn = which; }
    constexpr int HB = 128 / kBK;                    // stages per 128 k = one tile's worth of the triangular operand
    kc0 = 0; kc1 = kt;
    if (late) {
        if (p.pair_half == 0) kc1 = kt < HB ? kt : HB;
        else kc0 = HB < kt ? HB : kt;
    }
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
// outside m x n (and outside the requested triangle) are skipped.  The old values of C
// of G m16 tiles are fetched first (independent loads in flight together), then combined
// and stored: the epilogue costs G times fewer memory round trips.  With M-contiguous A the
// two rows a lane holds are adjacent (2g, 2g+1), so a 16-byte aligned C moves them as one
// 16-byte access.
template <int MAJOR_A, int MAJOR_B, int MT, int NT, int G>
__device__ __forceinline__ void epilogue(const GemmParams &p, double beta, int64_t m0, int64_t n0, int wm0,
                                         int wn0, int lane, double (&acc)[MT][NT][4])
{
    static_assert(MT % G == 0, "m16 tiles are taken G at a time");
    const double alpha = p.alpha;
    const bool use_c = beta != 0.0;
    const bool vec = MAJOR_A == MN_MAJOR && p.tri == 0 &&
                     ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) && (p.ldc % 2 == 0);
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
                        if (use_c && v) o = *reinterpret_cast<const double2 *>(p.C + r0 + col * p.ldc);
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
                        old[g][j][e] = (v && use_c) ? p.C[row + col * p.ldc] : 0.0;
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
                            *reinterpret_cast<double2 *>(p.C + r0 + col * p.ldc) = o;
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
                            p.C[row + col * p.ldc] = v;
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
                 const GemmParams p)
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
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + STAGES * STAGE_BYTES);
    uint64_t *empty = full + STAGES;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + STAGES);
    volatile int *tile_slot = abort_flag + 1;      // tile id carried by each stage, -1 = no more work

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], NCW);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
    }
    __syncthreads();

    const int num_units = p.split_first + p.nsu;
    const int kt = (int)((p.k + kBK - 1) / kBK);

    constexpr bool REBALANCE = (NCW == 8 && MIN_CTAS == 1);
    constexpr bool SHARE = (MIN_CTAS == 1);          // only the one-CTA-per-SM shape shares tiles
    constexpr int EG = 1;   // m16 tiles per round of the epilogue (2 would need more registers than the 168 the kernel is built with)
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
            // loads the stages [kc0, kc1) of the tile at (m0, n0); false once the kernel has given up
            auto load_piece = [&](int unit, int64_t m0, int64_t n0, int kc0, int kc1) -> bool {
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
                    const int k0 = kc * kBK;
                    if (MAJOR_A == K_MAJOR) {
                        tma_load_2d(sa, &tmA, k0, (int)m0, &full[s]);
                    } else {
#pragma unroll
                        for (int b = 0; b < BM / 16; ++b)
                            tma_load_2d(sa + b * 2048, &tmA, (int)m0 + 16 * b, k0, &full[s]);
                    }
                    if (MAJOR_B == K_MAJOR) {
                        tma_load_2d(sb, &tmB, k0, (int)n0, &full[s]);
                    } else {
#pragma unroll
                        for (int b = 0; b < BN / 16; ++b)
                            tma_load_2d(sb + b * 2048, &tmB, (int)n0 + 16 * b, k0, &full[s]);
                    }
                }
                return true;
            };
            int unit = blockIdx.x;
            while (live && unit < num_units) {
                if (SHARE && p.pair) {
                    int tm, tn, kc0, kc1;
                    pair_decode(p, unit, kt, tm, tn, kc0, kc1);
                    live = load_piece(unit, (int64_t)tm * BM, (int64_t)tn * BN, kc0, kc1);
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
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
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
        if (unit < 0) return;
        if (SHARE && p.pair) {
            int tm, tn, kc0, kc1;
            pair_decode(p, unit, kt, tm, tn, kc0, kc1);
            if (!run_piece(kc0, kc1, true)) return;
            int *flag = p.sched + 2 + (unit >> 1);
            if ((unit & 1) == 0) {
                // every load of this tile has landed (each stage was waited for): its partner may store
                if (threadIdx.x == 0) { __threadfence(); atomicExch(flag, 1); }
            } else {
                if (threadIdx.x == 0) {
                    bool ok = false;
                    for (uint32_t spin = 0; spin < (1u << 22) && !ok; ++spin) {
                        ok = *reinterpret_cast<volatile int *>(flag) == 1;
                        if (!ok) __nanosleep(64);
                    }
                    if (!ok) { *abort_flag = 1; atomicExch(p.err, 104); }
                    else atomicExch(flag, 0);              // back to zero for the next launch on this stream
                }
                asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
                if (*abort_flag) return;
                __threadfence();
            }
            epilogue<MAJOR_A, MAJOR_B, MT, NT, EG>(p, p.beta, (int64_t)tm * BM, (int64_t)tn * BN, wm0, wn0, lane, acc);
            continue;
        }
        if (!SHARE || unit < p.split_first) {
            int tm, tn;
            tile_coord(unit, p.tiles_m, p.tiles_n, tm, tn);
            if (SHARE && p.beta != 0.0) prefetch_c<MAJOR_A, MAJOR_B, MT, NT>(p, (int64_t)tm * BM, (int64_t)tn * BN, wm0, wn0, lane);
            if (!run_piece(0, kt, true)) return;
            epilogue<MAJOR_A, MAJOR_B, MT, NT, EG>(p, p.beta, (int64_t)tm * BM, (int64_t)tn * BN, wm0, wn0, lane, acc);
            continue;
        }
        StreamWalk walk(p.region_tiles, p.nsu, unit - p.split_first, kt);
        Piece pc;
        bool first = true;
        while (walk.next(pc)) {
            int tm, tn;
            tile_coord(region_tile(p, pc.r), p.tiles_m, p.tiles_n, tm, tn);
            const int64_t m0 = (int64_t)tm * BM, n0 = (int64_t)tn * BN;
            if (pc.kc0 > 0 || p.beta != 0.0) prefetch_c<MAJOR_A, MAJOR_B, MT, NT>(p, m0, n0, wm0, wn0, lane);
            if (!run_piece(pc.kc0, pc.kc1, first)) return;
            first = false;
            if (pc.kc0 == 0 && pc.kc1 == kt) {
                epilogue<MAJOR_A, MAJOR_B, MT, NT, EG>(p, p.beta, m0, n0, wm0, wn0, lane, acc);
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
            epilogue<MAJOR_A, MAJOR_B, MT, NT, EG>(p, pc.kc0 > 0 ? 1.0 : p.beta, m0, n0, wm0, wn0, lane, acc);
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
    epilogue<MAJOR_A, MAJOR_B, MT, NT, 1>(p, p.beta, m0, n0, wm0, wn0, lane, acc);
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
    if (MAJOR_A == K_MAJOR)
        ok = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, A, p.k, p.m, p.lda, kBK, BM);
    else
        ok = make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, A, p.m, p.k, p.lda, 16, kBK);
    if (MAJOR_B == K_MAJOR)
        ok = ok && make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, B, p.k, p.n, p.ldb, kBK, BN);
    else
        ok = ok && make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, B, p.n, p.k, p.ldb, 16, kBK);
    if (!ok) return -1;   // caller falls back to the ldg kernel

    constexpr size_t SMEM = (size_t)STAGES * (BM + BN) * 128 + 2 * STAGES * 8 + 16 + 4 * STAGES + 1024;
    auto kern = dgemm_tma_kernel<BM, BN, WARPS_M, WARPS_N, MAJOR_A, MAJOR_B, STAGES, CTAS_PER_SM>;
    static bool attr_done[kMaxDevices] = {};
    const int dev = current_device();
    if (!attr_done[dev]) {
        ULMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
        attr_done[dev] = true;
    }
    const int tiles = p.tiles_m * p.tiles_n;
    int sms = sm_count() - g_sm_reserve.load(std::memory_order_relaxed);
    if (sms < 1) sms = 1;
    const int slots = sms * ctas_per_sm;
    GemmParams q = p;
    q.split_first = tiles; q.nsu = 0; q.region_tiles = 0;
    const int kt = (int)((p.k + kBK - 1) / kBK);
    const int mode = settings().dgemm_split;
    // Sharing the last tiles.  With one CTA per SM the tiles beyond the last full wave leave most
    // SMs idle for a whole tile time (a SYRK of order 8192: 2080 tiles = 14 waves + 8 tiles; a
    // 1024^3 product: 64 tiles on 148 SMs).  Those tiles' pipeline stages are dealt out evenly to
    // all CTAs instead, whenever that is cheaper than one more wave of whole tiles.
    if (p.pair) {
        // in-place leaf: two units per pair of tiles, no sharing
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
        const SharePlan sp = plan_shared_tiles(nreal, kt, slots, mode == 2);
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
    const int64_t units = p.pair ? (int64_t)tiles : (int64_t)q.split_first + q.nsu;
    const int grid = (int)(units < slots ? units : slots);
    // More units than CTAs: they are handed out through the stream's counter word.  Without
    // scheduler words (none left for this stream) the CTAs stride through the units instead.
    q.dynamic = (units > grid && p.sched) ? 1 : 0;
    trace("dgemm kernel tile %dx%d %s grid %d units %lld (whole %d, shared tiles %d over %d CTAs) kt %d",
          BM, BN, q.dynamic ? "dynamic" : "static", grid, (long long)units, q.split_first, q.region_tiles, q.nsu, kt);
    kern<<<grid, (WARPS_M * WARPS_N + 4) * 32, SMEM, st>>>(tmA, tmB, q);
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
    // can share the last tiles' stages among all CTAs; small tiles (64 x 64, two CTAs per SM) waste less
    // on padding and fill the machine with fewer rows and columns.  Per-SM times in microseconds,
    // measured on this part: one 16-k stage of a large tile 2.09, of a small tile 1.05 when two CTAs
    // share the SM and 0.70 when one has it alone; an epilogue 3 / 2.
    const int64_t t128 = ((p.m + 127) / 128) * ((p.n + 127) / 128);
    const int64_t t64 = ((p.m + 63) / 64) * ((p.n + 63) / 64);
    const int kt = (int)((p.k + kBK - 1) / kBK);
    const int sms = sm_count();
    constexpr double kStage128 = 2.09, kStage64Pair = 1.05, kStage64Alone = 0.70, kEpi128 = 3.0, kEpi64 = 2.0;
    double time128 = (double)((t128 + sms - 1) / sms) * (kt * kStage128 + kEpi128);
    if (tma_ok && may_share && p.sched && cfg.dgemm_split != 0 && p.tri == 0) {
        const SharePlan sp = plan_shared_tiles(t128, kt, sms, false);
        if (sp.nsu > 0)
            time128 = (double)(t128 / sms) * (kt * kStage128 + kEpi128) +
                      (double)shared_cost(sp.region_tiles, kt, sp.nsu) * kStage128;
    }
    const int64_t waves64 = (t64 + 2 * sms - 1) / (2 * sms);
    const double stage64 = t64 <= sms ? kStage64Alone : kStage64Pair;
    const double time64 = (double)waves64 * (kt * stage64 + kEpi64);
    bool big = time128 <= time64;
    if (cfg.dgemm_tile == 128) big = true;
    if (cfg.dgemm_tile == 64) big = false;
    if (cfg.dgemm_ldg) tma_ok = false;
    if (big) {
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

    GemmParams p;
    p.m = m; p.n = n; p.k = k; p.alpha = alpha; p.beta = beta;
    p.A = A; p.B = B; p.lda = lda; p.ldb = ldb; p.C = C; p.ldc = ldc;
    p.tiles_m = p.tiles_n = 0; p.tri = tri;
    p.split_first = 0; p.nsu = 0; p.region_tiles = 0; p.dynamic = 0;
    p.pair = 0; p.pair_half = 0;
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

// X <- op(T) * X (left) or X * op(T) (right) in place, T a block-triangular matrix of order dim <= 256
// whose off-diagonal zero block is really zero (the inverted or zero-filled diagonal blocks of the
// triangular solver and multiply): the leaf of ulmBLAS's trlsm / trusm / trlmm / trumm recursion
// (ulmblas/level3/trlsm.tcc:61-74), without their packed copy of the block row.  lower_op: op(T) is
// lower triangular.  Returns -1 when the operands do not qualify (not TMA-addressable, no scheduler
// words, too many tiles); the caller then multiplies into a work tile and copies back.
int dgemm_leaf_inplace(cudaStream_t st, int left, int lower_op, int transT, int64_t dim, int64_t other, double alpha,
                       const double *T, int64_t ldt, double *X, int64_t ldx, int *err_word)
{
    if (dim <= 0 || other <= 0) return ULMB200_OK;
    if (dim > 256 || err_word) return -1;
    const int64_t m = left ? dim : other, n = left ? other : dim, k = dim;
    const bool tma_ok = ((reinterpret_cast<uintptr_t>(T) | reinterpret_cast<uintptr_t>(X)) & 15) == 0 &&
                        (ldt % 2 == 0) && (ldx % 2 == 0) && other < (1ll << 31) - 256 && ldx < (1ll << 36);
    if (!tma_ok) return -1;
    GemmParams p;
    p.m = m; p.n = n; p.k = k; p.alpha = alpha; p.beta = 0.0;
    p.A = left ? T : X; p.lda = left ? ldt : ldx;
    p.B = left ? X : T; p.ldb = left ? ldx : ldt;
    p.C = X; p.ldc = ldx;
    p.tiles_m = (int)((m + 127) / 128); p.tiles_n = (int)((n + 127) / 128);
    p.tri = 0; p.split_first = 0; p.nsu = 0; p.region_tiles = 0; p.dynamic = 0;
    p.err = device_error_word();
    p.sched = sched_words(st);
    if (!p.err || !p.sched) return -1;
    const int pair_tiles = left ? p.tiles_m : p.tiles_n, pairs = left ? p.tiles_n : p.tiles_m;
    p.pair = 0; p.pair_half = 0;
    if (pair_tiles == 2) {
        if (pairs > kSchedFlags) return -1;
        p.pair = left ? 1 : 2;
        // the tile that only meets its own diagonal block: left, X_i = sum_j op(T)_ij X_j -> row block 0 for a lower
        // op(T); right, X_j = sum_i X_i op(T)_ij -> column block 1 for a lower op(T)
        p.pair_half = left ? (lower_op ? 0 : 1) : (lower_op ? 1 : 0);
    }
    // one tile along the triangular dimension: the tile's loads are all done before its epilogue stores, and no
    // other tile touches its rows (columns), so plain in-place is safe as long as the tiles are the large ones
    const int ta = left ? transT : 0, tb = left ? 0 : transT;
    int r;
    if (!ta && !tb)      r = launch_tma<128, 128, 2, 4, MN_MAJOR, K_MAJOR, 3, 1>(st, p, p.A, p.B, false);
    else if (!ta && tb)  r = launch_tma<128, 128, 2, 4, MN_MAJOR, MN_MAJOR, 3, 1>(st, p, p.A, p.B, false);
    else if (ta && !tb)  r = launch_tma<128, 128, 2, 4, K_MAJOR, K_MAJOR, 3, 1>(st, p, p.A, p.B, false);
    else                 r = launch_tma<128, 128, 2, 4, K_MAJOR, MN_MAJOR, 3, 1>(st, p, p.A, p.B, false);
    return r;
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
