// Opt-in SGEMM on the 5th-generation tensor cores: 3xTF32 with FP32 accumulation
// in tensor memory.
//
// Every FP32 operand value x is split as  x = hi + lo  with hi = tf32(x) and
// lo = tf32(x - hi); the product keeps the three leading terms
//     a*b ~ lo_a*hi_b + hi_a*lo_b + hi_a*hi_b
// (the dropped lo*lo term is below 2^-22 |a||b|), each term a tcgen05.mma
// kind::tf32 into the same TMEM accumulator.  This replaces the float
// instantiation of the reference's micro-kernel (ulmblas/level3/ukernel/ref/
// ugemm.tcc, MR=8 NR=4) for callers who select ULMB200_SGEMM_3XTF32.
//
// Two steps per call:
//   1. split_tf32_kernel writes hi/lo copies of op(A) and op(B) into scratch,
//      both with K contiguous (transposing on the way when the caller's layout
//      has M or N contiguous), so the GEMM kernel only ever sees K-major tiles.
//   2. sgemm_3xtf32_kernel, persistent, one CTA per SM, 128x256 tile:
//        warp 0    TMA producer (4 tile loads per 32-deep k-block, 128-byte swizzle)
//        warp 1    owns tensor memory (512 columns = two 128x256 accumulators) and
//                  issues the MMAs: 4 k-steps x 3 terms per k-block, then commits
//                  the stage back to the producer / the accumulator to the epilogue
//        warps 2-5 epilogue: tcgen05.ld the accumulator (lane = row), apply
//                  alpha/beta, store column-major C (a warp writes 32 consecutive rows)
//      so the epilogue of tile i overlaps the MMAs of tile i+1.
#include "common.h"

namespace ulmb200 {

namespace tf {
constexpr int BM = 128, BN = 256, BK = 32, STAGES = 2;
constexpr uint32_t A_BYTES = BM * BK * 4;            // 16 KB  (hi or lo)
constexpr uint32_t B_BYTES = BN * BK * 4;            // 32 KB
constexpr uint32_t STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
constexpr uint32_t TMEM_COLS = 512;                  // 2 accumulators x 256 columns
constexpr int NTHREADS = 192;
// instruction descriptor: D = F32, A = B = TF32, both K-major, N = 256, M = 128
constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) |
                           ((uint32_t)(BM >> 4) << 24);
}  // namespace tf

struct Tf32Params {
    int64_t m, n, k;
    float alpha, beta;
    float *C;
    int64_t ldc;
    int tiles_m, tiles_n;
    int *err;
};

// ---- tcgen05 wrappers -------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// arrives on `bar` once every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}

// 32 lanes x 32 consecutive columns of 32-bit accumulators: thread = TMEM lane, v[j] = column j
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes with the
// 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte offset), the leading
// byte offset is unused for swizzled K-major layouts (encoded 1), descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t saddr)
{
    return (uint64_t)((saddr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}

// ---- step 1: hi/lo split (and transposition to K-major) ---------------------
__device__ __forceinline__ float to_tf32(float x)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

// X is column-major.  TRANSPOSE == false: X is K x MN (K contiguous), out[c*kpad + r].
// TRANSPOSE == true : X is MN x K (MN contiguous),  out[r*kpad + c]  through a 32x33 tile.
template <bool TRANSPOSE>
__global__ void __launch_bounds__(256) split_tf32_kernel(const float *X, int64_t ld, int64_t rows,
                                                         int64_t cols, float *hi, float *lo, int64_t kpad)
{
    __shared__ float tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;         // 32 x 8
    const int64_t r0 = (int64_t)blockIdx.x * 32, c0 = (int64_t)blockIdx.y * 32;
    if (!TRANSPOSE) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int64_t r = r0 + tx, c = c0 + ty + 8 * q;
            if (r < rows && c < cols) {
                const float x = X[r + c * ld];
                const float h = to_tf32(x);
                hi[c * kpad + r] = h;
                lo[c * kpad + r] = to_tf32(x - h);
            }
        }
    } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int64_t r = r0 + tx, c = c0 + ty + 8 * q;
            tile[ty + 8 * q][tx] = (r < rows && c < cols) ? X[r + c * ld] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int64_t r = r0 + ty + 8 * q, c = c0 + tx;         // c (= k) is now the fast index
            if (r < rows && c < cols) {
                const float x = tile[tx][ty + 8 * q];
                const float h = to_tf32(x);
                hi[r * kpad + c] = h;
                lo[r * kpad + c] = to_tf32(x - h);
            }
        }
    }
}

// ---- step 2: the GEMM ----------------------------------------------------------
__global__ void __launch_bounds__(tf::NTHREADS, 1)
sgemm_3xtf32_kernel(const __grid_constant__ CUtensorMap tmAh, const __grid_constant__ CUtensorMap tmAl,
                    const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmBl,
                    const Tf32Params p)
{
    using namespace tf;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + STAGES * STAGE_BYTES);
    uint64_t *empty = full + STAGES;
    uint64_t *tfull = empty + STAGES;          // accumulator ready for the epilogue
    uint64_t *tempty = tfull + 2;              // accumulator drained, MMA may overwrite
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tempty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 4); }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmAh); prefetch_tmap(&tmAl); prefetch_tmap(&tmBh); prefetch_tmap(&tmBl);
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_tiles = p.tiles_m * p.tiles_n;
    const int kt = (int)((p.k + BK - 1) / BK);
    constexpr int GM = 8;

    auto tile_mn = [&](int id, int64_t &m0, int64_t &n0) {
        const int per_group = GM * p.tiles_n, group = id / per_group, first = group * GM;
        const int gsz = min(GM, p.tiles_m - first), r = id - group * per_group;
        m0 = (int64_t)(first + r % gsz) * BM;
        n0 = (int64_t)(r / gsz) * BN;
    };

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            bool live = true;
            for (int tile = blockIdx.x; tile < num_tiles && live; tile += gridDim.x) {
                int64_t m0, n0;
                tile_mn(tile, m0, n0);
                for (int kc = 0; kc < kt; ++kc, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                    if (*abort_flag || !mbar_wait(&empty[s], ph ^ 1)) {
                        *abort_flag = 1; atomicExch(p.err, 201); live = false; break;
                    }
                    uint8_t *st = smem + s * STAGE_BYTES;
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    const int k0 = kc * BK;
                    tma_load_2d(st, &tmAh, k0, (int)m0, &full[s]);
                    tma_load_2d(st + A_BYTES, &tmAl, k0, (int)m0, &full[s]);
                    tma_load_2d(st + 2 * A_BYTES, &tmBh, k0, (int)n0, &full[s]);
                    tma_load_2d(st + 2 * A_BYTES + B_BYTES, &tmBl, k0, (int)n0, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            uint32_t it = 0, tcount = 0;
            bool live = true;
            for (int tile = blockIdx.x; tile < num_tiles && live; tile += gridDim.x, ++tcount) {
                const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
                if (*abort_flag || !mbar_wait(&tempty[acc], aph ^ 1)) {
                    *abort_flag = 1; atomicExch(p.err, 202); break;
                }
                tc_fence_after();
                const uint32_t d = tmem_base + acc * BN;
                for (int kc = 0; kc < kt; ++kc, ++it) {
                    const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
                    if (*abort_flag || !mbar_wait(&full[s], ph)) {
                        *abort_flag = 1; atomicExch(p.err, 203); live = false; break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                    const uint64_t dAh = smem_desc_k_sw128(sa), dAl = smem_desc_k_sw128(sa + A_BYTES);
                    const uint64_t dBh = smem_desc_k_sw128(sa + 2 * A_BYTES);
                    const uint64_t dBl = smem_desc_k_sw128(sa + 2 * A_BYTES + B_BYTES);
#pragma unroll
                    for (int kk = 0; kk < BK / 8; ++kk) {
                        const uint64_t adv = (uint64_t)(kk * 32 >> 4);      // 8 tf32 = 32 bytes along K
                        umma_tf32(d, dAl + adv, dBh + adv, IDESC, (kc | kk) ? 1u : 0u);   // small terms first
                        umma_tf32(d, dAh + adv, dBl + adv, IDESC, 1u);
                        umma_tf32(d, dAh + adv, dBh + adv, IDESC, 1u);
                    }
                    umma_commit(&empty[s]);          // stage reusable once these MMAs have read it
                }
                if (live) umma_commit(&tfull[acc]);  // accumulator complete
            }
        }
    } else {
        // ------------------------------ epilogue (warps 2..5) ------------------------------
        const int q = warp & 3;                      // TMEM lanes 32q .. 32q+31 belong to this warp
        uint32_t tcount = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
            const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
            int64_t m0, n0;
            tile_mn(tile, m0, n0);
            if (*abort_flag || !mbar_wait(&tfull[acc], aph)) {
                *abort_flag = 1; atomicExch(p.err, 204); break;
            }
            tc_fence_after();
            const int64_t row = m0 + q * 32 + lane;
            const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                tmem_ld_32x32(tbase + c0, v);
                if (row < p.m) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int64_t col = n0 + c0 + j;
                        if (col < p.n) {
                            float *c = p.C + row + col * p.ldc;
                            float o = p.alpha * __uint_as_float(v[j]);
                            if (p.beta != 0.0f) o = fmaf(p.beta, *c, o);
                            *c = o;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[acc]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- host side -------------------------------------------------------------------
// Scratch layout handed in by the caller (floats):
//   Ahi[m*kpad] Alo[m*kpad] Bhi[n*kpad] Blo[n*kpad],  kpad = k rounded up to 4.
size_t sgemm_3xtf32_scratch_floats(int64_t m, int64_t n, int64_t k)
{
    const int64_t kpad = (k + 3) / 4 * 4;
    return (size_t)(2 * (m + n) * kpad);
}

int sgemm_3xtf32_with_scratch(cudaStream_t st, int transA, int transB, int64_t m, int64_t n, int64_t k,
                              float alpha, const float *A, int64_t lda, const float *B, int64_t ldb,
                              float beta, float *C, int64_t ldc, float *scratch)
{
    const int64_t kpad = (k + 3) / 4 * 4;
    float *Ah = scratch, *Al = Ah + m * kpad, *Bh = Al + m * kpad, *Bl = Bh + n * kpad;

    // op(A) is m x k.  Stored k x m (K contiguous) when transposed, m x k otherwise.
    {
        const int64_t rows = transA ? k : m, cols = transA ? m : k;
        dim3 grid((unsigned)((rows + 31) / 32), (unsigned)((cols + 31) / 32));
        if (transA) split_tf32_kernel<false><<<grid, 256, 0, st>>>(A, lda, rows, cols, Ah, Al, kpad);
        else        split_tf32_kernel<true><<<grid, 256, 0, st>>>(A, lda, rows, cols, Ah, Al, kpad);
        count_launch();
    }
    // op(B) is k x n.  Stored k x n (K contiguous) when not transposed, n x k otherwise.
    {
        const int64_t rows = transB ? n : k, cols = transB ? k : n;
        dim3 grid((unsigned)((rows + 31) / 32), (unsigned)((cols + 31) / 32));
        if (!transB) split_tf32_kernel<false><<<grid, 256, 0, st>>>(B, ldb, rows, cols, Bh, Bl, kpad);
        else         split_tf32_kernel<true><<<grid, 256, 0, st>>>(B, ldb, rows, cols, Bh, Bl, kpad);
        count_launch();
    }
    ULMB_CUDA(cudaGetLastError());

    CUtensorMap tAh, tAl, tBh, tBl;
    const bool ok =
        make_tmap_2d(&tAh, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, Ah, k, m, kpad, tf::BK, tf::BM) &&
        make_tmap_2d(&tAl, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, Al, k, m, kpad, tf::BK, tf::BM) &&
        make_tmap_2d(&tBh, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, Bh, k, n, kpad, tf::BK, tf::BN) &&
        make_tmap_2d(&tBl, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, Bl, k, n, kpad, tf::BK, tf::BN);
    if (!ok) {
        fprintf(stderr, "ulmblas_b200: tensor map encoding failed for the 3xTF32 SGEMM\n");
        return ULMB200_CUDA_ERROR;
    }

    Tf32Params p;
    p.m = m; p.n = n; p.k = k; p.alpha = alpha; p.beta = beta; p.C = C; p.ldc = ldc;
    p.tiles_m = (int)((m + tf::BM - 1) / tf::BM);
    p.tiles_n = (int)((n + tf::BN - 1) / tf::BN);
    p.err = device_error_word();
    if (!p.err) return ULMB200_CUDA_ERROR;

    constexpr int SMEM = tf::STAGES * tf::STAGE_BYTES + 8 * (2 * tf::STAGES + 4) + 16 + 1024;
    static bool attr_done[kMaxDevices] = {};
    const int dev = current_device();
    if (!attr_done[dev]) {
        ULMB_CUDA(cudaFuncSetAttribute(sgemm_3xtf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        attr_done[dev] = true;
    }
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < sm_count() ? tiles : sm_count();
    sgemm_3xtf32_kernel<<<grid, tf::NTHREADS, SMEM, st>>>(tAh, tAl, tBh, tBl, p);
    count_launch();
    ULMB_CUDA(cudaGetLastError());
    return ULMB200_OK;
}

int sgemm_3xtf32_device(cudaStream_t st, int transA, int transB, int64_t m, int64_t n, int64_t k,
                        float alpha, const float *A, int64_t lda, const float *B, int64_t ldb,
                        float beta, float *C, int64_t ldc)
{
    if (m >= (1ll << 31) - 512 || n >= (1ll << 31) - 512 || k >= (1ll << 31) - 512) return ULMB200_TOO_LARGE;
    float *scratch = static_cast<float *>(device_scratch(5, sizeof(float) * sgemm_3xtf32_scratch_floats(m, n, k)));
    if (!scratch) return ULMB200_CUDA_ERROR;
    return sgemm_3xtf32_with_scratch(st, transA, transB, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, scratch);
}

}  // namespace ulmb200
