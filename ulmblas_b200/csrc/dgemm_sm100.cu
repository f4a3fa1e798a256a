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

#include <atomic>

namespace ulmb200 {

constexpr int kSplitSpan = 512;           // most tile ids a tail split may span (flag words per launch)

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
    int *tile_counter;        // zeroed before the launch; hands out tiles beyond the first wave
    // Tail split (whole tiles keep ksplit = 1): tiles with id >= split_first are each worked on by
    // ksplit CTAs, one range of kchunk pipeline stages per CTA.  Work units are numbered
    //   u < split_first:  tile u, all of K
    //   u >= split_first: tile split_first + (u - split_first) / ksplit, part (u - split_first) % ksplit
    int split_first, ksplit, kchunk;
    int *flags;               // one word per split tile, zeroed beforehand: parts add into C in order
};

// work unit -> tile, part and the range of pipeline stages [kc0, kc1)
__device__ __forceinline__ void unit_decode(const GemmParams &p, int unit, int kt, int &tile, int &part,
                                            int &kc0, int &kc1)
{
    if (unit < p.split_first) { tile = unit; part = 0; kc0 = 0; kc1 = kt; return; }
    const int r = unit - p.split_first;
    tile = p.split_first + r / p.ksplit;
    part = r % p.ksplit;
    kc0 = part * p.kchunk;
    kc1 = min(kt, kc0 + p.kchunk);
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
// outside m x n (and outside the requested triangle) are skipped.  Per m16 tile
// all old values of C are fetched first (independent loads in flight together),
// then combined and stored.  With M-contiguous A the two rows a lane holds are
// adjacent (2g, 2g+1), so a 16-byte aligned C moves them as one 16-byte access.
template <int MAJOR_A, int MAJOR_B, int MT, int NT>
__device__ __forceinline__ void epilogue(const GemmParams &p, double beta, int64_t m0, int64_t n0, int wm0,
                                         int wn0, int lane, double (&acc)[MT][NT][4])
{
    const double alpha = p.alpha;
    const bool use_c = beta != 0.0;
    const bool vec = MAJOR_A == MN_MAJOR && p.tri == 0 &&
                     ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) && (p.ldc % 2 == 0);
#pragma unroll
    for (int i = 0; i < MT; ++i) {
        const int64_t r0 = m0 + c_row<MAJOR_A>(wm0 + 16 * i, lane, 0);
        const int64_t r1 = m0 + c_row<MAJOR_A>(wm0 + 16 * i, lane, 1);
        if (vec && r1 < p.m) {
            // rows r0 (even) and r1 = r0 + 1: registers {0,2} of column 2t, {1,3} of column 2t+1
            double2 old[NT][2];
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    const int64_t col = n0 + c_col<MAJOR_B>(wn0 + 8 * j, lane, w);
                    old[j][w] = (use_c && col < p.n)
                                    ? *reinterpret_cast<const double2 *>(p.C + r0 + col * p.ldc)
                                    : make_double2(0.0, 0.0);
                }
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    const int64_t col = n0 + c_col<MAJOR_B>(wn0 + 8 * j, lane, w);
                    if (col < p.n) {
                        double2 o;
                        o.x = alpha * acc[i][j][w];
                        o.y = alpha * acc[i][j][2 + w];
                        if (use_c) { o.x = fma(beta, old[j][w].x, o.x); o.y = fma(beta, old[j][w].y, o.y); }
                        *reinterpret_cast<double2 *>(p.C + r0 + col * p.ldc) = o;
                    }
                }
            continue;
        }
        double old[NT][4];
        bool ok[NT][4];
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int64_t row = (e >> 1) ? r1 : r0;
                const int64_t col = n0 + c_col<MAJOR_B>(wn0 + 8 * j, lane, e & 1);
                bool v = row < p.m && col < p.n;
                if (p.tri == 1) v = v && row <= col;
                if (p.tri == 2) v = v && row >= col;
                ok[j][e] = v;
                old[j][e] = (v && use_c) ? p.C[row + col * p.ldc] : 0.0;
            }
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (ok[j][e]) {
                    const int64_t row = (e >> 1) ? r1 : r0;
                    const int64_t col = n0 + c_col<MAJOR_B>(wn0 + 8 * j, lane, e & 1);
                    double v = alpha * acc[i][j][e];
                    if (use_c) v = fma(beta, old[j][e], v);
                    p.C[row + col * p.ldc] = v;
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

    const int num_tiles = p.tiles_m * p.tiles_n;
    const int num_units = p.split_first + (num_tiles - p.split_first) * p.ksplit;
    const int kt = (int)((p.k + kBK - 1) / kBK);

    constexpr bool REBALANCE = (NCW == 8 && MIN_CTAS == 1);
    if (warp >= NCW) {
        // ---------------- producer warpgroup ----------------
        if (REBALANCE) asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
        if (warp == NCW && lane == 0) {
            // Tiles are handed out dynamically: the first one is the CTA's own index, the rest come
            // from a global counter.  A CTA that starts late (its SM was busy with another
            // kernel, e.g. a collective) then simply takes fewer tiles instead of holding up the
            // whole grid with a fixed share.
            uint32_t it = 0;
            bool live = true;
            int unit = blockIdx.x;
            while (live) {
                bool skip = false;
                int64_t m0 = 0, n0 = 0;
                int kc0 = 0, kc1 = 1;                                // one empty stage carries the end mark
                if (unit < num_units) {
                    int tile, part, tm, tn;
                    unit_decode(p, unit, kt, tile, part, kc0, kc1);
                    tile_coord(tile, p.tiles_m, p.tiles_n, tm, tn);
                    m0 = (int64_t)tm * BM; n0 = (int64_t)tn * BN;
                    skip = tile_skipped(p.tri, m0, n0, BM, BN);
                }
                if (!skip) {
                    for (int kc = kc0; kc < kc1; ++kc, ++it) {
                        const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                        if (*abort_flag || !mbar_wait(&empty[s], ph ^ 1)) {
                            *abort_flag = 1;
                            atomicExch(p.err, 101);
                            live = false;
                            break;
                        }
                        if (unit >= num_units) {
                            tile_slot[s] = -1;
                            mbar_arrive(&full[s]);
                            live = false;
                            break;
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
                }
                if (live) unit = (int)gridDim.x + atomicAdd(p.tile_counter, 1);
            }
            live = (*abort_flag == 0);
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
    for (;;) {
        // the first stage of a tile tells which tile it is
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
        int tile, part, kc0, kc1, tm, tn;
        unit_decode(p, unit, kt, tile, part, kc0, kc1);
        tile_coord(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int64_t m0 = (int64_t)tm * BM, n0 = (int64_t)tn * BN;

        double acc[MT][NT][4];
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.0;

        for (int kc = kc0; kc < kc1; ++kc, ++it) {
            const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
            if (kc > kc0 && (*abort_flag || !mbar_wait(&full[s], ph))) {
                *abort_flag = 1;
                atomicExch(p.err, 102);
                return;
            }
            const uint32_t sA = smem_base + s * STAGE_BYTES;
            mma_stage<MAJOR_A, MAJOR_B, MT, NT>(sA, sA + A_BYTES, ba, bb, acc);
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        if (unit < p.split_first) {
            epilogue<MAJOR_A, MAJOR_B, MT, NT>(p, p.beta, m0, n0, wm0, wn0, lane, acc);
            continue;
        }
        // A split tile: part 0 applies beta; part i > 0 waits (bounded) until part i-1 has stored its
        // share, then adds its own.  The order is fixed, so the result does not depend on timing.  A
        // unit is only ever picked up by a running CTA after all units before it, so the part waited
        // for is already being worked on.
        int *flag = p.flags + (tile - p.split_first);
        if (part > 0) {
            if (threadIdx.x == 0) {
                bool ok = false;
                for (uint32_t spin = 0; spin < (1u << 22) && !ok; ++spin) {
                    ok = *reinterpret_cast<volatile int *>(flag) >= part;
                    if (!ok) __nanosleep(128);
                }
                if (!ok) { *abort_flag = 1; atomicExch(p.err, 103); }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
            if (*abort_flag) return;
            __threadfence();
        }
        epilogue<MAJOR_A, MAJOR_B, MT, NT>(p, part > 0 ? 1.0 : p.beta, m0, n0, wm0, wn0, lane, acc);
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
        if (threadIdx.x == 0) atomicExch(flag, part + 1);
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
    epilogue<MAJOR_A, MAJOR_B, MT, NT>(p, p.beta, m0, n0, wm0, wn0, lane, acc);
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


// ULMB200_DGEMM_SPLITK=0 switches the K splits off (test hook)
static int split_allowed()
{
    static const int v = [] { const char *e = getenv("ULMB200_DGEMM_SPLITK"); return e ? atoi(e) : 1; }();
    return v;
}

template <int BM, int BN, int WARPS_M, int WARPS_N, int MAJOR_A, int MAJOR_B, int STAGES, int CTAS_PER_SM>
static int launch_tma(cudaStream_t st, const GemmParams &p, const double *A, const double *B)
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
    GemmParams q = p;
    const bool may_alloc = p.ksplit != 0;
    q.split_first = tiles; q.ksplit = 1; q.kchunk = 0; q.flags = nullptr;
    // Tail split.  With one CTA per SM the tiles beyond the last full wave leave most SMs idle for a
    // whole tile time (a SYRK of order 8192: 2080 tiles = 14 waves + 8 tiles).  When that remainder
    // is at most half a wave, each of its tiles is shared by 2-8 CTAs, one K range each.
    const int allow_split = split_allowed();
    const int kt = (int)((p.k + kBK - 1) / kBK);
    if (allow_split && may_alloc && ctas_per_sm == 1 && tiles > sms && tiles <= 64 * sms && kt >= 32) {
        // tiles that do work (a triangular update skips those outside its triangle)
        auto real = [&](int id) {
            int tm, tn;
            tile_coord(id, p.tiles_m, p.tiles_n, tm, tn);
            return !tile_skipped(p.tri, (int64_t)tm * BM, (int64_t)tn * BN, BM, BN);
        };
        int64_t nreal = tiles;
        if (p.tri != 0) {
            // count per tile row/column analytically: tile (tm, tn) is real unless wholly outside
            nreal = 0;
            for (int tn = 0; tn < p.tiles_n; ++tn)
                for (int tm = 0; tm < p.tiles_m; ++tm)
                    nreal += !tile_skipped(p.tri, (int64_t)tm * BM, (int64_t)tn * BN, BM, BN);
        }
        const int rem = (int)(nreal % sms);
        if (nreal > sms && rem > 0) {
            // cut s ways (all parts resident at once: rem * s <= SMs), the last wave costs 1/s of a tile
            // time plus a chain of s short epilogues: take the cheapest s with at least 16 stages per part
            int ks = 1;
            double best = 0.8;
            for (int cand = 2; cand <= 8 && kt / cand >= 16 && rem * cand <= sms; ++cand) {
                const double cost = (double)((rem * cand + sms - 1) / sms) / cand + 0.01 * cand;
                if (cost < best) { best = cost; ks = cand; }
            }
            if (ks > 1) {
                const int kchunk = (kt + ks - 1) / ks;
                ks = (kt + kchunk - 1) / kchunk;                 // no empty part
                int first = tiles, found = 0;
                while (first > 0 && found < rem) { --first; found += real(first); }
                if (ks > 1 && tiles - first <= kSplitSpan) {
                    static std::atomic<unsigned> turn{0};
                    int *flags = static_cast<int *>(device_scratch(15, sizeof(int) * kSplitSpan * 8));
                    if (flags) {
                        flags += kSplitSpan * (turn.fetch_add(1, std::memory_order_relaxed) % 8);
                        ULMB_CUDA(cudaMemsetAsync(flags, 0, sizeof(int) * (size_t)(tiles - first), st));
                        q.split_first = first; q.ksplit = ks; q.kchunk = kchunk; q.flags = flags;
                    }
                }
            }
        }
    }
    // Few tiles and a long inner dimension (a product of tall, narrow operands): every tile is cut,
    // so that all SMs work on it.  Same mechanism, split_first = 0.
    if (allow_split && may_alloc && ctas_per_sm == 1 && p.tri == 0 && q.ksplit == 1 && tiles * 2 <= sms && kt >= 128) {
        int ks = sms / tiles;
        if (ks > 8) ks = 8;
        while (ks > 1 && kt / ks < 64) --ks;                     // at least 64 stages (1024 k) per part
        if (ks > 1) {
            const int kchunk = (kt + ks - 1) / ks;
            ks = (kt + kchunk - 1) / kchunk;
            static std::atomic<unsigned> turn_all{0};
            int *flags = ks > 1 ? static_cast<int *>(device_scratch(15, sizeof(int) * kSplitSpan * 8)) : nullptr;
            if (flags) {
                flags += kSplitSpan * (turn_all.fetch_add(1, std::memory_order_relaxed) % 8);
                ULMB_CUDA(cudaMemsetAsync(flags, 0, sizeof(int) * (size_t)tiles, st));
                q.split_first = 0; q.ksplit = ks; q.kchunk = kchunk; q.flags = flags;
            }
        }
    }
    const int64_t units = (int64_t)q.split_first + (int64_t)(tiles - q.split_first) * q.ksplit;
    const int grid = (int)(units < (int64_t)sms * ctas_per_sm ? units : (int64_t)sms * ctas_per_sm);
    // tile counter: one of 60 words next to the error word, taken round-robin so that launches
    // in flight on different streams do not share one
    static std::atomic<unsigned> rr{0};
    const unsigned turn = rr.fetch_add(1, std::memory_order_relaxed);
    q.tile_counter = p.err + 1 + (turn % 60);
    // The counter only matters when there is more work than CTAs.  Otherwise every CTA just learns
    // from it that nothing is left, which any non-negative value tells it -- so small products skip
    // the memset launch (except now and then, to keep the word from creeping towards overflow).
    if (units > grid || (turn & 1023u) < 60u) ULMB_CUDA(cudaMemsetAsync(q.tile_counter, 0, sizeof(int), st));
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
static int dispatch(cudaStream_t st, GemmParams p, bool tma_ok, int force_tile, int force_path)
{
    // Large tiles once they fill the machine; small tiles for small problems.
    const int64_t t128 = ((p.m + 127) / 128) * ((p.n + 127) / 128);
    bool big = t128 >= (int64_t)sm_count() * 3 / 4;
    // few tiles but a long inner dimension: large tiles cut along K fill the machine better than
    // small tiles do (768 x 768 x 8192: 30.2 TFLOP/s against 24.9 with 64 x 64 tiles); parts shorter
    // than 1024 k do not pay (1024^3 is faster on small tiles)
    if (p.tri == 0 && tma_ok && p.ksplit != 0 && split_allowed() && t128 * 2 <= sm_count() && p.k >= 128 * kBK &&
        t128 * (p.k / (64 * kBK)) >= sm_count() / 2)
        big = true;
    if (force_tile == 128) big = true;
    if (force_tile == 64) big = false;
    if (force_path == 1) tma_ok = false;
    if (big) {
        p.tiles_m = (int)((p.m + 127) / 128);
        p.tiles_n = (int)((p.n + 127) / 128);
        if (tma_ok) {
            // Three stages of 32 KB, not four: with both operands K-major (op(A) = A^T, op(B) = B)
            // a four-deep ring measured 6% slower (33.3 against 35.6 TFLOP/s at 8192^3); the other
            // three modes are within 1% either way.
            int r = launch_tma<128, 128, 2, 4, MAJOR_A, MAJOR_B, 3, 1>(st, p, p.A, p.B);
            if (r >= 0) return r;
        }
        return launch_ldg<128, 128, 2, 4, MAJOR_A, MAJOR_B>(st, p);
    }
    p.tiles_m = (int)((p.m + 63) / 64);
    p.tiles_n = (int)((p.n + 63) / 64);
    if (tma_ok) {
        int r = launch_tma<64, 64, 2, 2, MAJOR_A, MAJOR_B, 4, 2>(st, p, p.A, p.B);
        if (r >= 0) return r;
    }
    return launch_ldg<64, 64, 2, 2, MAJOR_A, MAJOR_B>(st, p);
}

// Test hooks (environment, read per call so tests can flip them):
//   ULMB200_DGEMM_TILE = 64 | 128   force a tile shape
//   ULMB200_DGEMM_PATH = ldg        force the non-TMA kernel
static void read_overrides(int &tile, int &path)
{
    tile = 0; path = 0;
    if (const char *t = getenv("ULMB200_DGEMM_TILE")) tile = atoi(t);
    if (const char *s = getenv("ULMB200_DGEMM_PATH")) path = (s[0] == 'l') ? 1 : 0;
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
    p.tiles_m = p.tiles_n = 0; p.tri = tri; p.tile_counter = nullptr;
    // ksplit = 0 on the way in: the caller brought its own error word because it must not allocate
    // device memory, so the tail split (which takes flag words from the scratch cache) stays off
    p.split_first = 0; p.ksplit = err_word ? 0 : 1; p.kchunk = 0; p.flags = nullptr;
    p.err = err_word ? err_word : device_error_word();
    if (!p.err) return set_status(ULMB200_CUDA_ERROR);

    // TMA needs 16-byte aligned bases and row pitches, and 32-bit coordinates.
    const bool tma_ok = ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) == 0 &&
                        (lda % 2 == 0) && (ldb % 2 == 0) && m < (1ll << 31) - 256 &&
                        n < (1ll << 31) - 256 && k < (1ll << 31) - 256 &&
                        lda < (1ll << 36) && ldb < (1ll << 36);
    int ftile, fpath;
    read_overrides(ftile, fpath);
    int r;
    if (!transA && !transB)      r = dispatch<MN_MAJOR, K_MAJOR>(st, p, tma_ok, ftile, fpath);
    else if (!transA && transB)  r = dispatch<MN_MAJOR, MN_MAJOR>(st, p, tma_ok, ftile, fpath);
    else if (transA && !transB)  r = dispatch<K_MAJOR, K_MAJOR>(st, p, tma_ok, ftile, fpath);
    else                         r = dispatch<K_MAJOR, MN_MAJOR>(st, p, tma_ok, ftile, fpath);
    return set_status(r);
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
