// FP32 GEMM on the FP32 FMA pipes, persistent and warp-specialised:
//     C <- alpha*op(A)*op(B) + beta*C,  FP32 accumulation.
//
// Replaces the float instantiation of the reference's gemm path (ulmblas/level3/gemm.tcc with
// pack/gepack.tcc and ukernel/ref/ugemm.tcc, MR = 8, NR = 4): where the reference packs panels so
// that its register kernel streams them, eight consumer warps here do nothing but shared-memory
// fragment loads and packed FMAs (fma.rn.f32x2, 16 x 8 outputs per thread of a 256 x 128 CTA
// tile) out of a ring of 16-k stages, and a producer warpgroup keeps the ring full:
//
//   * an operand whose M (or N) dimension is contiguous in memory (op(A) = A, op(B) = B^T) arrives
//     by TMA, one 32 x 16 box per 32 rows, straight into the [k][m] layout the consumers read;
//   * an operand whose K dimension is contiguous (op(A) = A^T, op(B) = B) is transposed on the way
//     in by the producer warps: 16-byte global loads along k, 4-byte shared stores with
//     consecutive lanes on consecutive m -- the reference's gepack_A / gepack_B with the transpose
//     strides (interfaces/blas/F77/gemm.cc:98-103), done per tile and without a packed copy.
//
// Registers follow the roles (setmaxnreg): 208 per consumer thread, 88 per producer thread
// (a producer thread keeps a whole stage's worth of its loads in flight: 12 x 16 bytes).
// Tiles are handed out dynamically, and the tiles beyond the last full wave are shared out stage
// by stage among all CTAs, exactly as in the FP64 kernel (dgemm_schedule.h).
//
// Needs 16-byte aligned A and B with leading dimensions that are multiples of 4; anything else
// takes the plain-load kernel in sgemm_sm100.cu.
#include "common.h"
#include "dgemm_schedule.h"

#include <string.h>

namespace ulmb200 {

namespace sw {
constexpr int BM = 256, BN = 128, BK = 16;
constexpr int CONSUMERS = 256, PRODUCERS = 128, THREADS = CONSUMERS + PRODUCERS;
constexpr int STAGES = 6;
static_assert(BN == PRODUCERS && BM == 2 * PRODUCERS, "a producer thread transposes two rows of A and one of B per stage");
constexpr uint32_t BOX_BYTES = BK * 32 * 4;                  // one 32 (m) x 16 (k) box: 16 rows of 128 bytes
constexpr uint32_t A_BYTES = (BM / 32) * BOX_BYTES, B_BYTES = (BN / 32) * BOX_BYTES;
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;          // 24 KB
constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 2 * STAGES * 8 + 128 + 1024;
}  // namespace sw

struct SgemmWsParams {
    int64_t m, n, k;
    float alpha, beta;
    const float *A, *B;
    int64_t lda, ldb;
    float *C;
    int64_t ldc;
    int tiles_m, tiles_n;
    int *err;
    int *sched;               // scheduler words of the launch's stream (common.h), nullptr: static round-robin
    int dynamic;
    int split_first, nsu, region_tiles;
};

__device__ __forceinline__ void sw_tile_coord(int id, int tiles_m, int tiles_n, int &tm, int &tn)
{
    constexpr int GM = 8;       // groups of 8 tile-rows swept column by column (L2 reuse)
    const int per_group = GM * tiles_n, group = id / per_group, first = group * GM;
    const int gsz = GM < tiles_m - first ? GM : tiles_m - first, r = id - group * per_group;
    tm = first + r % gsz;
    tn = r / gsz;
}

__device__ __forceinline__ void sw_ffma2(uint64_t &d, uint64_t a, uint64_t b)
{
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}

// One 32 x 16 box of an M/N-contiguous operand: x = first m (or n), y = first k.
__device__ __forceinline__ void sw_tma_box(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar)
{
    tma_load_2d(dst, map, x, y, bar);
}

// The K-contiguous operand's share of one stage is transposed on the way in by the producer
// threads: a thread takes one row (one m or n) of the tile -- four 16-byte loads along k -- and
// scatters it with sixteen 4-byte stores into the [k][row] boxes.  Lanes sit on consecutive
// rows, so the stores of a warp fall into 32 consecutive words.
__device__ __forceinline__ void sw_load_row(float4 (&v)[4], const float *base, int64_t ld, int64_t gr, int64_t r_ext,
                                            int64_t k0, int64_t k_ext)
{
    const float *p = base + k0 + gr * ld;
    if (gr < r_ext && k0 + 16 <= k_ext) {
#pragma unroll
        for (int q = 0; q < 4; ++q) v[q] = __ldg(reinterpret_cast<const float4 *>(p) + q);
    } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float e[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) e[j] = (gr < r_ext && k0 + 4 * q + j < k_ext) ? __ldg(p + 4 * q + j) : 0.0f;
            v[q] = make_float4(e[0], e[1], e[2], e[3]);
        }
    }
}

__device__ __forceinline__ void sw_store_row(uint8_t *tile, int r, const float4 (&v)[4])
{
    float *dst = reinterpret_cast<float *>(tile + (r >> 5) * sw::BOX_BYTES) + (r & 31);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        dst[(4 * q + 0) * 32] = v[q].x;
        dst[(4 * q + 1) * 32] = v[q].y;
        dst[(4 * q + 2) * 32] = v[q].z;
        dst[(4 * q + 3) * 32] = v[q].w;
    }
}

// A producer's wait for a free stage: the ring holds several microseconds of work, so the waiter
// can sleep between polls and leave the issue slots to the consumers.  Bounded like every wait.
__device__ __forceinline__ bool mbar_wait_idle(uint64_t *bar, uint32_t parity)
{
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 4) __nanosleep(256);
    }
    return false;
}

__device__ __forceinline__ void mbar_expect_tx_only(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// TA: op(A) = A^T (K contiguous).  TB: op(B) = B^T (N contiguous).
template <bool TA, bool TB>
__global__ void __launch_bounds__(sw::THREADS, 1)
sgemm_ws_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const SgemmWsParams p)
{
    using namespace sw;
    constexpr bool A_TMA = !TA, B_TMA = TB;
    constexpr uint32_t TX_BYTES = (A_TMA ? A_BYTES : 0u) + (B_TMA ? B_BYTES : 0u);
    // producer threads that have work: all of them when an operand is transposed on the way in, one
    // (the TMA issuer) when both operands arrive by TMA -- the others leave at once instead of polling
    constexpr int NPROD = (A_TMA && B_TMA) ? 1 : PRODUCERS;

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + STAGES * STAGE_BYTES);
    uint64_t *empty = full + STAGES;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + STAGES);
    volatile int *unit_seq = abort_flag + 1;                  // how many units producer thread 0 has drawn so far
    volatile int *unit_ring = abort_flag + 2;                 // [8]: the units drawn, for the other producer threads
    volatile int *unit_of_stage = abort_flag + 10;            // [STAGES]: unit a stage belongs to, -1 = end
    volatile uint32_t *release_sink = reinterpret_cast<volatile uint32_t *>(abort_flag + 16);      // one word per consumer warp

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            // every working producer thread arrives once per stage
            mbar_init(&full[s], NPROD);
            mbar_init(&empty[s], CONSUMERS / 32);
        }
        *abort_flag = 0;
        *unit_seq = 0;
        fence_barrier_init();
        if (A_TMA) prefetch_tmap(&tmA);
        if (B_TMA) prefetch_tmap(&tmB);
    }
    __syncthreads();

    const int num_units = p.split_first + p.nsu;
    const int kt = (int)((p.k + BK - 1) / BK);

    if (warp >= CONSUMERS / 32) {
        // ------------------------------ producers ------------------------------
        asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
        const int t = threadIdx.x - CONSUMERS;
        if (t >= NPROD) return;
        uint32_t it = 0;
        bool live = true;
        auto load_piece = [&](int unit, int64_t m0, int64_t n0, int kc0, int kc1) -> bool {
            for (int kc = kc0; kc < kc1; ++kc, ++it) {
                const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                if (*abort_flag || !mbar_wait_idle(&empty[s], ph ^ 1)) {
                    *abort_flag = 1;
                    atomicExch(p.err, 211);
                    return false;
                }
                uint8_t *sa = smem + s * STAGE_BYTES, *sb = sa + A_BYTES;
                const int k0 = kc * BK;
                if (t == 0) {
                    unit_of_stage[s] = unit;
                    if (TX_BYTES) mbar_expect_tx_only(&full[s], TX_BYTES);
                    if (A_TMA) {
#pragma unroll
                        for (int b = 0; b < BM / 32; ++b) sw_tma_box(sa + b * BOX_BYTES, &tmA, (int)m0 + 32 * b, k0, &full[s]);
                    }
                    if (B_TMA) {
#pragma unroll
                        for (int b = 0; b < BN / 32; ++b) sw_tma_box(sb + b * BOX_BYTES, &tmB, (int)n0 + 32 * b, k0, &full[s]);
                    }
                }
                // all loads of the stage are issued before anything is stored: one memory latency per stage
                float4 va[2][4], vb[4];
                if (!A_TMA) {
                    sw_load_row(va[0], p.A, p.lda, m0 + t, p.m, k0, p.k);
                    sw_load_row(va[1], p.A, p.lda, m0 + t + PRODUCERS, p.m, k0, p.k);
                }
                if (!B_TMA) sw_load_row(vb, p.B, p.ldb, n0 + t, p.n, k0, p.k);
                if (!A_TMA) {
                    sw_store_row(sa, t, va[0]);
                    sw_store_row(sa, t + PRODUCERS, va[1]);
                }
                if (!B_TMA) sw_store_row(sb, t, vb);
                mbar_arrive(&full[s]);                                    // releases this thread's stores
            }
            return true;
        };
        int unit = blockIdx.x;
        int drawn = 0;
        while (live && unit < num_units) {
            if (unit < p.split_first) {
                int tm, tn;
                sw_tile_coord(unit, p.tiles_m, p.tiles_n, tm, tn);
                live = load_piece(unit, (int64_t)tm * BM, (int64_t)tn * BN, 0, kt);
            } else {
                StreamWalk walk(p.region_tiles, p.nsu, unit - p.split_first, kt);
                Piece pc;
                while (live && walk.next(pc)) {
                    int tm, tn;
                    sw_tile_coord(p.split_first + pc.r, p.tiles_m, p.tiles_n, tm, tn);
                    live = load_piece(unit, (int64_t)tm * BM, (int64_t)tn * BN, pc.kc0, pc.kc1);
                }
            }
            if (!live) break;
            if (p.dynamic && NPROD == 1) {
                unit = (int)gridDim.x + atomicAdd(p.sched, 1);
            } else if (p.dynamic) {
                // Thread 0 draws the next unit and publishes it; the others pick it up with a bounded
                // wait (no block barrier: a thread that has given up must not strand the rest).  Thread 0
                // is never more than STAGES units ahead of any other producer thread, so 8 slots do.
                ++drawn;
                if (t == 0) {
                    unit_ring[drawn & 7] = (int)gridDim.x + atomicAdd(p.sched, 1);
                    __threadfence_block();
                    *unit_seq = drawn;
                } else {
                    bool ok = false;
                    for (uint32_t spin = 0; spin < (1u << 22) && !ok; ++spin) {
                        ok = *unit_seq >= drawn;
                        if (!ok) {
                            if (*abort_flag) break;
                            __nanosleep(32);
                        }
                    }
                    if (!ok) {
                        *abort_flag = 1;
                        atomicExch(p.err, 214);
                        live = false;
                        break;
                    }
                    __threadfence_block();
                }
                unit = unit_ring[drawn & 7];
            } else {
                unit += (int)gridDim.x;
            }
        }
        if (live) {
            // one empty stage carries the end mark
            const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
            if (*abort_flag || !mbar_wait_idle(&empty[s], ph ^ 1)) {
                *abort_flag = 1;
                atomicExch(p.err, 211);
            } else {
                if (t == 0) unit_of_stage[s] = -1;
                mbar_arrive(&full[s]);
            }
        }
        if (t == 0 && p.dynamic) {
            __threadfence();
            if (atomicAdd(p.sched + 1, 1) == (int)gridDim.x - 1) {
                atomicExch(p.sched, 0);
                atomicExch(p.sched + 1, 0);
            }
        }
        if (t == 0 && *abort_flag && TX_BYTES) {
            // give loads already in flight a bounded time to land before the CTA retires
            for (int s = 0; s < STAGES; ++s)
                for (int i = 0; i < 1024 && !mbar_try_wait(&full[s], 0) && !mbar_try_wait(&full[s], 1); ++i) __nanosleep(256);
        }
        return;
    }

    // ------------------------------ consumers ------------------------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const int wm0 = (warp & 1) * 128, wn0 = (warp >> 1) * 32;
    const int ly = lane >> 2, lx = lane & 3;
    const int am = wm0 + ly * 4;            // rows am + 32r + {0..3}, r = 0..3
    const int bn = wn0 + lx * 4;            // cols bn + 16c + {0..3}, c = 0..1
    // byte offsets of this thread's fragments inside a stage, k = 0
    const uint32_t a_off = (uint32_t)((warp & 1) * 4) * BOX_BYTES + ly * 16;
    const uint32_t b_off = A_BYTES + (uint32_t)(warp >> 1) * BOX_BYTES + lx * 16;
    const uint32_t smem_base = smem_u32(smem);

    uint64_t acc[8][8];                     // [row pair][column]
    uint32_t it = 0;

    auto lds_a = [&](uint32_t addr, uint64_t (&a2)[8]) {
#pragma unroll
        for (int r = 0; r < 4; ++r)
            asm volatile("ld.shared.v2.u64 {%0,%1}, [%2];" : "=l"(a2[2 * r]), "=l"(a2[2 * r + 1]) : "r"(addr + r * BOX_BYTES));
    };
    auto lds_b = [&](uint32_t addr, float4 (&bf)[2]) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
            asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                         : "=f"(bf[c].x), "=f"(bf[c].y), "=f"(bf[c].z), "=f"(bf[c].w) : "r"(addr + c * 64));
    };

    auto run_piece = [&](int kc0, int kc1, bool first_stage_ready) -> bool {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] = 0ull;
        for (int kc = kc0; kc < kc1; ++kc, ++it) {
            const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
            if (!(first_stage_ready && kc == kc0) && (*abort_flag || !mbar_wait(&full[s], ph))) {
                *abort_flag = 1;
                atomicExch(p.err, 212);
                return false;
            }
            const uint32_t sa = smem_base + s * STAGE_BYTES + a_off, sb = smem_base + s * STAGE_BYTES + b_off;
            // fragments of step kk+1 are fetched while step kk multiplies
            uint64_t a2[2][8];
            float4 bf[2][2];
            lds_a(sa, a2[0]);
            lds_b(sb, bf[0]);
#pragma unroll
            for (int kk = 0; kk < BK; ++kk) {
                const int cb = kk & 1, nb = cb ^ 1;
                if (kk + 1 < BK) {
                    lds_a(sa + (kk + 1) * 128, a2[nb]);
                    lds_b(sb + (kk + 1) * 128, bf[nb]);
                }
                uint64_t b2[8];
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    asm("mov.b64 %0, {%1,%1};" : "=l"(b2[4 * c + 0]) : "f"(bf[cb][c].x));
                    asm("mov.b64 %0, {%1,%1};" : "=l"(b2[4 * c + 1]) : "f"(bf[cb][c].y));
                    asm("mov.b64 %0, {%1,%1};" : "=l"(b2[4 * c + 2]) : "f"(bf[cb][c].z));
                    asm("mov.b64 %0, {%1,%1};" : "=l"(b2[4 * c + 3]) : "f"(bf[cb][c].w));
                }
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int i = 0; i < 8; ++i) sw_ffma2(acc[i][j], a2[cb][i], b2[j]);
            }
            // Release through one more load of the stage and a store of what it returned (shared loads of a warp
            // return in issue order; the store cannot issue before the load is back; the arrive follows the
            // store): a plain arrive may overtake fragment loads whose packed FMAs were scheduled after it, and
            // the TMA refill then changes the stage under them.
            {
                uint32_t last;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(last) : "r"(sa + 4u * (uint32_t)lane) : "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_after(&empty[s], last, release_sink + warp);
            }
        }
        return true;
    };

    // Old values of C are read past L1 (ld.global.cg): the pieces of a shared tile hand their partial sums on
    // through C, and a line that straddles two tiles (columns of C not on 128-byte boundaries) may sit in this
    // SM's L1 from before the other tile's previous piece was written.
    // C(row, col) <- alpha*acc + beta*C for this thread's 16 x 8 outputs, 4 consecutive rows per
    // 16-byte access where C allows it
    auto epilogue = [&](float beta, int64_t m0, int64_t n0) {
        const float alpha = p.alpha;
        const bool vec = ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) && (p.ldc % 4 == 0);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int64_t col = n0 + bn + (j & 3) + (j >> 2) * 16;
            if (col >= p.n) continue;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int64_t row = m0 + am + 32 * r;
                float v[4];
                asm("mov.b64 {%0,%1}, %2;" : "=f"(v[0]), "=f"(v[1]) : "l"(acc[2 * r][j]));
                asm("mov.b64 {%0,%1}, %2;" : "=f"(v[2]), "=f"(v[3]) : "l"(acc[2 * r + 1][j]));
                float *c = p.C + row + col * p.ldc;
                if (vec && row + 3 < p.m) {
                    float4 o = make_float4(alpha * v[0], alpha * v[1], alpha * v[2], alpha * v[3]);
                    if (beta != 0.0f) {
                        const float4 old = __ldcg(reinterpret_cast<const float4 *>(c));      // past L1: see below
                        o.x = fmaf(beta, old.x, o.x); o.y = fmaf(beta, old.y, o.y);
                        o.z = fmaf(beta, old.z, o.z); o.w = fmaf(beta, old.w, o.w);
                    }
                    *reinterpret_cast<float4 *>(c) = o;
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (row + e < p.m) {
                            float o = alpha * v[e];
                            if (beta != 0.0f) o = fmaf(beta, __ldcg(c + e), o);
                            c[e] = o;
                        }
                    }
                }
            }
        }
    };

    for (;;) {
        {
            const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
            if (*abort_flag || !mbar_wait(&full[s], ph)) {
                *abort_flag = 1;
                atomicExch(p.err, 212);
                return;
            }
        }
        const int unit = unit_of_stage[it % STAGES];
        if (unit < 0) return;
        if (unit < p.split_first) {
            int tm, tn;
            sw_tile_coord(unit, p.tiles_m, p.tiles_n, tm, tn);
            if (!run_piece(0, kt, true)) return;
            epilogue(p.beta, (int64_t)tm * BM, (int64_t)tn * BN);
            continue;
        }
        StreamWalk walk(p.region_tiles, p.nsu, unit - p.split_first, kt);
        Piece pc;
        bool first = true;
        while (walk.next(pc)) {
            int tm, tn;
            sw_tile_coord(p.split_first + pc.r, p.tiles_m, p.tiles_n, tm, tn);
            const int64_t m0 = (int64_t)tm * BM, n0 = (int64_t)tn * BN;
            if (!run_piece(pc.kc0, pc.kc1, first)) return;
            first = false;
            if (pc.kc0 == 0 && pc.kc1 == kt) {
                epilogue(p.beta, m0, n0);
                continue;
            }
            // a shared tile: its pieces fold into C in order of k (see dgemm_schedule.h)
            int *flag = p.sched + 2 + pc.r;
            if (pc.kc0 > 0) {
                if (threadIdx.x == 0) {
                    bool ok = false;
                    for (uint32_t spin = 0; spin < (1u << 22) && !ok; ++spin) {
                        ok = *reinterpret_cast<volatile int *>(flag) == pc.kc0;
                        if (!ok) __nanosleep(64);
                    }
                    if (!ok) { *abort_flag = 1; atomicExch(p.err, 213); }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS) : "memory");
                if (*abort_flag) return;
                __threadfence();
            }
            epilogue(pc.kc0 > 0 ? 1.0f : p.beta, m0, n0);
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS) : "memory");
            if (threadIdx.x == 0) atomicExch(flag, pc.kc1 == kt ? 0 : pc.kc1);
        }
    }
}

template <bool TA, bool TB>
static int launch_ws(cudaStream_t st, SgemmWsParams p)
{
    using namespace sw;
    CUtensorMap tmA, tmB;
    memset(&tmA, 0, sizeof tmA);
    memset(&tmB, 0, sizeof tmB);
    // M/N-contiguous operands: dim0 = m|n (contiguous), dim1 = k, box 32 x 16, no swizzle
    if (!TA && !make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.A, p.m, p.k, p.lda, 32, BK, CU_TENSOR_MAP_SWIZZLE_NONE))
        return -1;
    if (TB && !make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.B, p.n, p.k, p.ldb, 32, BK, CU_TENSOR_MAP_SWIZZLE_NONE))
        return -1;
    auto kern = sgemm_ws_kernel<TA, TB>;
    static bool attr_done[kMaxDevices] = {};
    const int dev = current_device();
    if (!attr_done[dev]) {
        ULMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
        attr_done[dev] = true;
    }
    const int tiles = p.tiles_m * p.tiles_n;
    const int slots = sm_count();
    const int kt = (int)((p.k + BK - 1) / BK);
    p.split_first = tiles; p.nsu = 0; p.region_tiles = 0;
    if (p.sched && settings().dgemm_split != 0) {
        const SharePlan sp = plan_shared_tiles(tiles, kt, slots, settings().dgemm_split == 2);
        if (sp.nsu > 0) { p.split_first = tiles - sp.region_tiles; p.nsu = sp.nsu; p.region_tiles = sp.region_tiles; }
    }
    const int64_t units = (int64_t)p.split_first + p.nsu;
    const int grid = (int)(units < slots ? units : slots);
    p.dynamic = (units > grid && p.sched) ? 1 : 0;
    trace("sgemm kernel 256x128 %s grid %d units %lld (whole %d, shared tiles %d over %d CTAs) kt %d",
          p.dynamic ? "dynamic" : "static", grid, (long long)units, p.split_first, p.region_tiles, p.nsu, kt);
    kern<<<grid, THREADS, SMEM, st>>>(tmA, tmB, p);
    count_launch();
    ULMB_CUDA(cudaGetLastError());
    return ULMB200_OK;
}

// Returns -1 when the operands do not qualify (the caller then takes the plain-load kernel).
int sgemm_ws_device(cudaStream_t st, int transA, int transB, int64_t m, int64_t n, int64_t k, float alpha, const float *A,
                    int64_t lda, const float *B, int64_t ldb, float beta, float *C, int64_t ldc)
{
    const bool ok = ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) == 0 && lda % 4 == 0 &&
                    ldb % 4 == 0 && m < (1ll << 31) - 512 && n < (1ll << 31) - 512 && k < (1ll << 31) - 512 &&
                    lda < (1ll << 36) && ldb < (1ll << 36);
    if (!ok) return -1;
    SgemmWsParams p;
    p.m = m; p.n = n; p.k = k; p.alpha = alpha; p.beta = beta;
    p.A = A; p.B = B; p.lda = lda; p.ldb = ldb; p.C = C; p.ldc = ldc;
    p.tiles_m = (int)((m + sw::BM - 1) / sw::BM);
    p.tiles_n = (int)((n + sw::BN - 1) / sw::BN);
    if ((int64_t)p.tiles_m * p.tiles_n >= (1 << 30)) return -1;
    p.err = device_error_word();
    if (!p.err) return ULMB200_CUDA_ERROR;
    p.sched = sched_words(st);
    p.dynamic = 0; p.split_first = 0; p.nsu = 0; p.region_tiles = 0;
    if (!transA && !transB) return launch_ws<false, false>(st, p);
    if (!transA && transB)  return launch_ws<false, true>(st, p);
    if (transA && !transB)  return launch_ws<true, false>(st, p);
    return launch_ws<true, true>(st, p);
}

}  // namespace ulmb200
