// FP32 GEMM on the FP32 FMA pipes:  C <- alpha*op(A)*op(B) + beta*C -- the entry point and the
// plain-load kernel.  Operands that TMA can address (16-byte aligned, leading dimensions that are
// multiples of 4) take the persistent warp-specialised kernel in sgemm_ws_sm100.cu; this file's
// kernel, filled by ordinary predicated loads, serves every other alignment and leading dimension.
//
// Replaces the float instantiation of the reference's gemm path
// (ulmblas/level3/gemm.tcc with ukernel/ref/ugemm.tcc, MR=8 NR=4).  The
// reference's sgemm_ widens to double internally (interfaces/blas/F77/gemm.cc:33,36);
// this kernel accumulates in FP32, which stays inside the 2*k*eps32 componentwise
// bound the results are held to.
//
// 256x128x16 CTA tile, 256 threads, 16x8 outputs per thread, one CTA per SM.
// Operand tiles are kept in shared memory as [k][m] / [k][n] whatever the global
// layout (the transposition happens on the way in).  Measured on this part, a
// 16-byte shared load costs 2 cycles when each aligned group of 4 lanes reads one
// address and 4 cycles otherwise, so the long side of the thread tile (16 rows of
// A, 4 loads) is indexed by lane/4 and the short side (8 columns of B, 2 loads)
// by lane%4: 16 shared-memory cycles per 128 FMAs.  The FMAs are issued as packed
// fma.rn.f32x2 on row pairs, which halves the issue slots they need.
#include "common.h"

namespace ulmb200 {

namespace sg {
constexpr int BM = 256, BN = 128, BK = 16, NT = 256;
constexpr int LDA_ = BM + 4, LDB_ = BN + 4;      // padded rows of the [k][m] / [k][n] tiles, floats
constexpr int A_TILE = BK * LDA_, B_TILE = BK * LDB_;
}  // namespace sg

struct SgemmParams {
    int64_t m, n, k;
    float alpha, beta;
    const float *A, *B;
    int64_t lda, ldb;
    float *C;
    int64_t ldc;
    int tiles_m, tiles_n;
    int *err;                 // device error word
};

// Global -> registers for one BMN x 16 operand tile, BMN*16/4/256 float4 per thread.
//   MN-contiguous storage (element (r,kk) at base[r + kk*ld]): runs of 4 consecutive r.
//   K-contiguous storage (base[kk + r*ld]): runs of 4 consecutive kk for one r.
//   VEC: 16-byte loads are legal (aligned base and ld).
template <int BMN, bool K_CONTIG, bool VEC>
__device__ __forceinline__ void sg_load(float (&v)[BMN * sg::BK / sg::NT], const float *base, int64_t ld,
                                        int64_t r0, int64_t r_ext, int64_t k0, int64_t k_ext)
{
    using namespace sg;
    constexpr int NQ = BMN * BK / 4 / NT;
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
        const int f = threadIdx.x + q * NT;            // which float4 of the tile
        int r, kk;
        if (!K_CONTIG) { r = (f % (BMN / 4)) * 4; kk = f / (BMN / 4); }
        else           { r = f % BMN;             kk = (f / BMN) * 4; }
        const int64_t gr = r0 + r, gk = k0 + kk;
        const float *p = K_CONTIG ? base + gk + gr * ld : base + gr + gk * ld;
        const bool inner_full = K_CONTIG ? (gk + 3 < k_ext) : (gr + 3 < r_ext);
        const bool outer_ok = K_CONTIG ? (gr < r_ext) : (gk < k_ext);
        if (VEC && inner_full && outer_ok) {
            const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
            v[4 * q + 0] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const bool ok = outer_ok && (K_CONTIG ? (gk + e < k_ext) : (gr + e < r_ext));
                v[4 * q + e] = ok ? __ldg(p + e) : 0.0f;
            }
        }
    }
}

// Registers -> shared [k][r] tile with row pitch LD floats.
template <int BMN, int LD, bool K_CONTIG>
__device__ __forceinline__ void sg_store(float *tile, const float (&v)[BMN * sg::BK / sg::NT])
{
    using namespace sg;
    constexpr int NQ = BMN * BK / 4 / NT;
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
        const int f = threadIdx.x + q * NT;
        if (!K_CONTIG) {
            const int r = (f % (BMN / 4)) * 4, kk = f / (BMN / 4);
            *reinterpret_cast<float4 *>(tile + kk * LD + r) =
                make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        } else {
            const int r = f % BMN, kk = (f / BMN) * 4;
#pragma unroll
            for (int e = 0; e < 4; ++e) tile[(kk + e) * LD + r] = v[4 * q + e];
        }
    }
}

__device__ __forceinline__ void ffma2(uint64_t &d, uint64_t a, uint64_t b)
{
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}

template <bool TA, bool TB, bool VEC>
__global__ void __launch_bounds__(sg::NT, 1) sgemm_fp32_kernel(const SgemmParams p)
{
    using namespace sg;
    extern __shared__ float smem_f[];
    float *As = smem_f;                       // [2][A_TILE]
    float *Bs = smem_f + 2 * A_TILE;          // [2][B_TILE]

    // tile order: groups of 8 tile-rows swept column by column (L2 reuse)
    int tm, tn;
    {
        constexpr int GM = 8;
        const int id = (int)blockIdx.x, per_group = GM * p.tiles_n, group = id / per_group;
        const int first = group * GM, gsz = min(GM, p.tiles_m - first), r = id - group * per_group;
        tm = first + r % gsz;
        tn = r / gsz;
    }
    const int64_t m0 = (int64_t)tm * BM, n0 = (int64_t)tn * BN;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm0 = (warp & 1) * 128, wn0 = (warp >> 1) * 32;
    const int ly = lane >> 2, lx = lane & 3;
    const int am = wm0 + ly * 4;            // rows am + 32r + {0..3}, r = 0..3
    const int bn = wn0 + lx * 4;            // cols bn + 16c + {0..3}, c = 0..1

    uint64_t acc[8][8];                     // [row pair][column]: rows (am + 32(p/2) + 2(p%2)) + {0,1}
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0ull;

    const int64_t kbeg = 0, kend = p.k;
    const int kt = (int)((kend - kbeg + BK - 1) / BK);
    float ra[BM * BK / NT], rb[BN * BK / NT];
    // op(A) is m x k: stored MN-contiguous when not transposed, K-contiguous when transposed.
    // op(B) is k x n: stored K-contiguous when not transposed, N-contiguous when transposed.
    sg_load<BM, TA, VEC>(ra, p.A, p.lda, m0, p.m, kbeg, kend);
    sg_load<BN, !TB, VEC>(rb, p.B, p.ldb, n0, p.n, kbeg, kend);
    sg_store<BM, LDA_, TA>(As, ra);
    sg_store<BN, LDB_, !TB>(Bs, rb);
    __syncthreads();

    for (int kc = 0; kc < kt; ++kc) {
        const int cur = kc & 1;
        if (kc + 1 < kt) {
            sg_load<BM, TA, VEC>(ra, p.A, p.lda, m0, p.m, kbeg + (int64_t)(kc + 1) * BK, kend);
            sg_load<BN, !TB, VEC>(rb, p.B, p.ldb, n0, p.n, kbeg + (int64_t)(kc + 1) * BK, kend);
        }
        const float *a_t = As + cur * A_TILE + am;
        const float *b_t = Bs + cur * B_TILE + bn;
        // fragments of step kk+1 are fetched while step kk multiplies
        uint64_t a2[2][8];
        float4 bf[2][2];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const ulonglong2 v = *reinterpret_cast<const ulonglong2 *>(a_t + 32 * r);
            a2[0][2 * r] = v.x; a2[0][2 * r + 1] = v.y;
        }
        bf[0][0] = *reinterpret_cast<const float4 *>(b_t);
        bf[0][1] = *reinterpret_cast<const float4 *>(b_t + 16);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const int cb = kk & 1, nb = cb ^ 1;
            if (kk + 1 < BK) {
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const ulonglong2 v = *reinterpret_cast<const ulonglong2 *>(a_t + (kk + 1) * LDA_ + 32 * r);
                    a2[nb][2 * r] = v.x; a2[nb][2 * r + 1] = v.y;
                }
                bf[nb][0] = *reinterpret_cast<const float4 *>(b_t + (kk + 1) * LDB_);
                bf[nb][1] = *reinterpret_cast<const float4 *>(b_t + (kk + 1) * LDB_ + 16);
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
                for (int i = 0; i < 8; ++i) ffma2(acc[i][j], a2[cb][i], b2[j]);
        }
        if (kc + 1 < kt) {
            sg_store<BM, LDA_, TA>(As + (cur ^ 1) * A_TILE, ra);
            sg_store<BN, LDB_, !TB>(Bs + (cur ^ 1) * B_TILE, rb);
        }
        __syncthreads();
    }

    // epilogue: column-major C, 4 consecutive rows per 16-byte store when legal
    const float alpha = p.alpha;
    const float beta = p.beta;
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
            if (VEC && row + 3 < p.m && ((reinterpret_cast<uintptr_t>(c) & 15) == 0)) {
                float4 o = make_float4(alpha * v[0], alpha * v[1], alpha * v[2], alpha * v[3]);
                if (beta != 0.0f) {
                    const float4 old = *reinterpret_cast<const float4 *>(c);
                    o.x = fmaf(beta, old.x, o.x); o.y = fmaf(beta, old.y, o.y);
                    o.z = fmaf(beta, old.z, o.z); o.w = fmaf(beta, old.w, o.w);
                }
                *reinterpret_cast<float4 *>(c) = o;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (row + e < p.m) {
                        float o = alpha * v[e];
                        if (beta != 0.0f) o = fmaf(beta, c[e], o);
                        c[e] = o;
                    }
                }
            }
        }
    }
}

__global__ void sscal_matrix_kernel(float *C, int64_t ldc, int64_t m, int64_t n, float beta)
{
    const int64_t total = m * n;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        float *c = C + e % m + (e / m) * ldc;
        *c = (beta == 0.0f) ? 0.0f : *c * beta;
    }
}

template <bool TA, bool TB, bool VEC>
static int launch_fp32(cudaStream_t st, const SgemmParams &p, int grid)
{
    constexpr int SMEM = 2 * (sg::A_TILE + sg::B_TILE) * (int)sizeof(float);
    auto kern = sgemm_fp32_kernel<TA, TB, VEC>;
    static bool attr_done[kMaxDevices] = {};
    const int dev = current_device();
    if (!attr_done[dev]) {
        ULMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        attr_done[dev] = true;
    }
    kern<<<grid, sg::NT, SMEM, st>>>(p);
    count_launch();
    ULMB_CUDA(cudaGetLastError());
    return ULMB200_OK;
}

// out(i, p) = in(p, i): in is rows x cols with the rows contiguous (element (p, i) at in[p + i * ldi]), out is
// cols x rows with ITS rows contiguous (element (i, p) at out[i + p * ldo]).  32 x 32 tiles through shared
// memory, both sides coalesced; any alignment.
__global__ void __launch_bounds__(256) transpose_f32_kernel(const float *in, int64_t ldi, int64_t rows, int64_t cols,
                                                            float *out, int64_t ldo, int64_t tiles_r)
{
    __shared__ float tile[32][33];
    const int64_t tr = blockIdx.x % tiles_r, tc = blockIdx.x / tiles_r;
    const int x = threadIdx.x & 31, y = threadIdx.x >> 5;               // 32 x 8 threads
    const int64_t p0 = tr * 32, i0 = tc * 32;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int64_t p = p0 + x, i = i0 + y + 8 * q;
        tile[y + 8 * q][x] = (p < rows && i < cols) ? in[p + i * ldi] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int64_t i = i0 + x, p = p0 + y + 8 * q;
        if (i < cols && p < rows) out[i + p * ldo] = tile[x][y + 8 * q];
    }
}

static int transpose_f32(cudaStream_t st, const float *in, int64_t ldi, int64_t rows, int64_t cols, float *out, int64_t ldo)
{
    const int64_t tiles_r = (rows + 31) / 32, tiles_c = (cols + 31) / 32;
    if (tiles_r * tiles_c >= (1ll << 31)) return -1;
    transpose_f32_kernel<<<(unsigned)(tiles_r * tiles_c), 256, 0, st>>>(in, ldi, rows, cols, out, ldo, tiles_r);
    count_launch();
    return check_cuda(cudaGetLastError(), "transpose_f32_kernel", __FILE__, __LINE__);
}

int sgemm_3xtf32_device(cudaStream_t st, int transA, int transB, int64_t m, int64_t n, int64_t k,
                        float alpha, const float *A, int64_t lda, const float *B, int64_t ldb,
                        float beta, float *C, int64_t ldc);
// the persistent TMA kernel (sgemm_ws_sm100.cu); -1 when the operands do not qualify for it
int sgemm_ws_device(cudaStream_t st, int transA, int transB, int64_t m, int64_t n, int64_t k, float alpha,
                    const float *A, int64_t lda, const float *B, int64_t ldb, float beta, float *C, int64_t ldc);

int sgemm_device(cudaStream_t st, int mode, int transA, int transB, int64_t m, int64_t n,
                 int64_t k, float alpha, const float *A, int64_t lda, const float *B, int64_t ldb,
                 float beta, float *C, int64_t ldc)
{
    if (m < 0 || n < 0 || k < 0) return set_status(ULMB200_BAD_ARGUMENT);
    const int64_t rowsA = transA ? k : m, rowsB = transB ? n : k;
    if (lda < (rowsA > 1 ? rowsA : 1) || ldb < (rowsB > 1 ? rowsB : 1) || ldc < (m > 1 ? m : 1))
        return set_status(ULMB200_BAD_ARGUMENT);
    if (mode != ULMB200_SGEMM_FP32 && mode != ULMB200_SGEMM_3XTF32) return set_status(ULMB200_BAD_ARGUMENT);
    if (m == 0 || n == 0) return set_status(ULMB200_OK);
    if (int s0 = ensure_device()) return set_status(s0);

    if (alpha == 0.0f || k == 0) {
        if (beta == 1.0f) return set_status(ULMB200_OK);
        int64_t blocks = (m * n + 255) / 256;
        const int64_t cap = (int64_t)sm_count() * 16;
        if (blocks > cap) blocks = cap;
        sscal_matrix_kernel<<<(int)blocks, 256, 0, st>>>(C, ldc, m, n, beta);
        count_launch();
        return set_status(check_cuda(cudaGetLastError(), "sscal_matrix_kernel", __FILE__, __LINE__));
    }
    if (mode == ULMB200_SGEMM_3XTF32)
        return set_status(sgemm_3xtf32_device(st, transA, transB, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc));

    if (!settings().sgemm_path) {
        // A K-contiguous operand (op(A) = A^T, op(B) = B) is transposed by the producer threads inside the
        // kernel, tile by tile (global loads along k, 4-byte shared stores), and that traffic through the
        // load/store pipe costs the consumers: 55 TFLOP/s with both operands K-contiguous against 62 with
        // both arriving by TMA.  For large products it is cheaper to write the M/N-contiguous copy once --
        // the reference's pack_A / pack_B done for the whole operand -- at 8 bytes of traffic per element
        // (2 % of the product's time at 4096^3) and to let TMA feed every tile.  An operand is copied when
        // the other dimension makes the product per element long enough to pay for it.
        const float *Au = A, *Bu = B;
        int64_t ldau = lda, ldbu = ldb;
        int tau = transA, tbu = transB;
        const bool pre = settings().sgemm_pretranspose != 0 && k >= 256;
        if (pre && transA && n >= 1024 && m >= 256) {
            const int64_t ldt = (m + 3) & ~3ll;
            float *At = static_cast<float *>(device_scratch(15, sizeof(float) * (size_t)ldt * k));
            if (At && transpose_f32(st, A, lda, k, m, At, ldt) == ULMB200_OK) { Au = At; ldau = ldt; tau = 0; }
        }
        if (pre && !transB && m >= 1024 && n >= 256) {
            const int64_t ldt = (n + 3) & ~3ll;
            float *Bt = static_cast<float *>(device_scratch(14, sizeof(float) * (size_t)ldt * k));
            if (Bt && transpose_f32(st, B, ldb, k, n, Bt, ldt) == ULMB200_OK) { Bu = Bt; ldbu = ldt; tbu = 1; }
        }
        int r = sgemm_ws_device(st, tau, tbu, m, n, k, alpha, Au, ldau, Bu, ldbu, beta, C, ldc);
        if (r < 0 && (Au != A || Bu != B)) r = sgemm_ws_device(st, transA, transB, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc);
        if (r >= 0) return set_status(r);
    }
    SgemmParams p;
    p.m = m; p.n = n; p.k = k; p.alpha = alpha; p.beta = beta;
    p.A = A; p.B = B; p.lda = lda; p.ldb = ldb; p.C = C; p.ldc = ldc;
    p.tiles_m = (int)((m + sg::BM - 1) / sg::BM);
    p.tiles_n = (int)((n + sg::BN - 1) / sg::BN);
    const bool vec = ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) == 0 &&
                     lda % 4 == 0 && ldb % 4 == 0;
    p.err = device_error_word();
    if (!p.err) return set_status(ULMB200_CUDA_ERROR);
    const int tiles = p.tiles_m * p.tiles_n;
    int r;
#define ULMB_SG(TA_, TB_) r = vec ? launch_fp32<TA_, TB_, true>(st, p, tiles) : launch_fp32<TA_, TB_, false>(st, p, tiles)
    if (!transA && !transB)      { ULMB_SG(false, false); }
    else if (!transA && transB)  { ULMB_SG(false, true); }
    else if (transA && !transB)  { ULMB_SG(true, false); }
    else                         { ULMB_SG(true, true); }
#undef ULMB_SG
    return set_status(r);
}

}  // namespace ulmb200

extern "C" int ulmb200_sgemm(void *stream, int mode, int transA, int transB, int64_t m, int64_t n,
                             int64_t k, float alpha, const float *dA, int64_t ldA, const float *dB,
                             int64_t ldB, float beta, float *dC, int64_t ldC)
{
    return ulmb200::sgemm_device(static_cast<cudaStream_t>(stream), mode, transA, transB, m, n, k, alpha,
                                 dA, ldA, dB, ldB, beta, dC, ldC);
}
