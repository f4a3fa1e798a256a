// The Level-3 routines the reference builds on its gemm macro-kernel, rebuilt on
// the device GEMM:
//
//   dsyrk  ulmblas/level3/syurk.tcc, sylrk.tcc (+ mkernel/msy?rk, ukernel/usy?rk):
//          the reference restricts its block loops to one triangle and masks
//          the diagonal tiles; here the GEMM kernel gets a triangle predicate
//          (whole tiles outside the triangle are never scheduled, tiles on the
//          diagonal mask their stores), so the other triangle is never touched.
//
//   dtrsm  ulmblas/level3/trlsm.tcc, trusm.tcc (+ mkernel/mtr?sm, ukernel/utr?sm,
//          pack/tr?spack): the reference solves 4x4 diagonal tiles by
//          multiplying with reciprocal diagonals and pushes everything else
//          through its gemm macro-kernel.  Here the diagonal blocks are 128x128,
//          inverted once by a small kernel, and every other flop -- applying a
//          block inverse, updating the remaining rows -- is a device GEMM,
//          arranged recursively so the updates have large inner dimensions.
#include "common.h"

namespace ulmb200 {

// ---------------------------------------------------------------------------
// syrk
// ---------------------------------------------------------------------------
int dsyrk_device(cudaStream_t st, int lower, int trans, int64_t n, int64_t k, double alpha,
                 const double *A, int64_t lda, double beta, double *C, int64_t ldc)
{
    if (n < 0 || k < 0) return set_status(ULMB200_BAD_ARGUMENT);
    const int64_t rowsA = trans ? k : n;
    if (lda < (rowsA > 1 ? rowsA : 1) || ldc < (n > 1 ? n : 1)) return set_status(ULMB200_BAD_ARGUMENT);
    // quick returns of syurk.tcc:44-51
    if (n == 0 || ((alpha == 0.0 || k == 0) && beta == 1.0)) return set_status(ULMB200_OK);
    const int tri = lower ? 2 : 1;
    // op(A) * op(A)^T: the second operand is the same array read with the opposite transposition
    return dgemm_device(st, tri, trans ? 1 : 0, trans ? 0 : 1, n, n, k, alpha, A, lda, A, lda, beta, C, ldc);
}

// ---------------------------------------------------------------------------
// trsm
// ---------------------------------------------------------------------------
constexpr int kNB = 128;          // diagonal block size

// Inverse of one triangular diagonal block per CTA, in place in shared memory.
// The block is viewed as a LOWER triangular matrix L (an upper-stored block is read
// transposed and its inverse written transposed back), padded to kNB x kNB with an identity.
//   1. eight 16 x 16 diagonal blocks are inverted by one warp each, row by row:
//          x(i,:) = (e_i - sum_{p<i} L(i,p) x(p,:)) / L(i,i),   lane j owning column j;
//   2. three doubling levels (s = 16, 32, 64) complete [[A,0],[C,B]]^-1 = [[A',0],[-B' C A', B']]
//      with two small products per pair, all 256 threads sharing the outputs:
//          W = C A'   then   C <- -B' W.
// The zeros above the diagonal are kept in shared memory, so the products need no triangle logic.
constexpr int kTrtriThreads = 256;
constexpr int kTrtriLeaf = 16;

__global__ void __launch_bounds__(kTrtriThreads)
trtri_blocks_kernel(const double *A, int64_t lda, int64_t dim, int lower, int unit, double *inv, int ldo)
{
    extern __shared__ double trtri_smem[];
    double *M = trtri_smem;                   // M[p*kNB + i] = L(i, p)
    double *W = trtri_smem + kNB * kNB;       // 64 * 64 doubles
    const int blk = blockIdx.x;
    const int64_t r0 = (int64_t)blk * kNB;
    const int len = (int)((dim - r0) < kNB ? (dim - r0) : kNB);
    const double *Ab = A + r0 + r0 * lda;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;

    // the lower view: strictly upper part zero, identity beyond len; the stored block is walked
    // column by column, and its unreferenced triangle is never read
    // eight loads in flight per thread: the walk is a chain of global-memory latencies otherwise
    for (int e0 = t; e0 < kNB * kNB; e0 += 8 * kTrtriThreads) {
        double v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int e = e0 + u * kTrtriThreads;
            const int a = e % kNB, b = e / kNB;               // stored element (a, b) of the block
            const int i = lower ? a : b, p = lower ? b : a;   // its place in the lower view
            v[u] = 0.0;
            if (i >= p) {
                if (i < len) v[u] = (unit && i == p) ? 1.0 : __ldg(Ab + a + (int64_t)b * lda);
                else if (i == p) v[u] = 1.0;
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int e = e0 + u * kTrtriThreads;
            const int a = e % kNB, b = e / kNB;
            const int i = lower ? a : b, p = lower ? b : a;
            M[p * kNB + i] = v[u];
        }
    }
    __syncthreads();

    // 1. leaves
    {
        const int b0 = warp * kTrtriLeaf;
        const int j = lane & (kTrtriLeaf - 1);
        for (int i = 0; i < kTrtriLeaf; ++i) {
            const double trow = M[(b0 + j) * kNB + b0 + i];      // L(i, j) of the leaf (zero for j > i)
            __syncwarp();
            double s = (i == j) ? 1.0 : 0.0;
            for (int p = 0; p < i; ++p) {
                const double tp = __shfl_sync(0xffffffffu, trow, p);
                s -= tp * M[(b0 + j) * kNB + b0 + p];            // x(p, j); zero for j > p
            }
            const double d = __shfl_sync(0xffffffffu, trow, i);
            if (!unit) s /= d;
            if (j > i) s = 0.0;
            __syncwarp();
            if (lane < kTrtriLeaf) M[(b0 + j) * kNB + b0 + i] = s;
            __syncwarp();
        }
    }
    __syncthreads();

    // 2. doubling: per pair 4 s threads, thread = (row i, column group g of 4); a thread walks its
    // columns g, g+4, ... four at a time so that four independent sums are in flight
    for (int s = kTrtriLeaf; s < kNB; s *= 2) {
        const int pairs = kNB / (2 * s);
        const int tpp = kTrtriThreads / pairs;                 // = 4 s
        const int q = t / tpp, tt = t % tpp;
        const int i = tt % s, g = tt / s;                      // g in 0..3
        const int o = q * 2 * s;
        const double *Ainv = M + o * kNB + o;                  // (r, c) at [c*kNB + r]
        const double *Binv = M + (o + s) * kNB + (o + s);
        double *Cb = M + o * kNB + (o + s);
        double *Wq = W + q * s * s;                            // (r, c) at [c*s + r]
        // W = C A'      (A'(p, j) = 0 for p < j)
        for (int j0 = g; j0 < s; j0 += 16) {
            double acc[4] = {0.0, 0.0, 0.0, 0.0};
            for (int p = j0; p < s; ++p) {
                const double c = Cb[p * kNB + i];
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[u] += c * Ainv[(j0 + 4 * u) * kNB + p];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) Wq[(j0 + 4 * u) * s + i] = acc[u];
        }
        __syncthreads();
        // C <- -B' W    (B'(i, p) = 0 for p > i)
        for (int j0 = g; j0 < s; j0 += 16) {
            double acc[4] = {0.0, 0.0, 0.0, 0.0};
            for (int p = 0; p <= i; ++p) {
                const double bv = Binv[p * kNB + i];
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[u] += bv * Wq[(j0 + 4 * u) * s + p];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) Cb[(j0 + 4 * u) * kNB + i] = -acc[u];
        }
        __syncthreads();
    }

    // the full kNB x kNB block goes out (zeros outside len x len and outside the triangle).  The inverses
    // of ldo x ldo diagonal blocks lie one after the other, each with leading dimension ldo: block blk
    // is the diagonal block at row and column (blk * kNB) % ldo of number blk * kNB / ldo.
    const int old_ = ldo;
    const int64_t at = (int64_t)blk * kNB;
    double *out = inv + (at / ldo) * ldo * ldo + (at % ldo) * (ldo + 1);
    for (int e = t; e < kNB * kNB; e += kTrtriThreads) {
        const int i = e % kNB, j = e / kNB;           // lower view (i, j)
        const double v = (i < len && j < len && j <= i) ? M[j * kNB + i] : 0.0;
        if (lower) out[i + j * old_] = v;
        else       out[j + i * old_] = v;
    }
}

// Completes the 256 x 256 inverses: for the pair of diagonal blocks (A, B) with off-diagonal block C,
//   lower-stored [[A,0],[C,B]]^-1 = [[A',0],[X,B']],  X = -B' C A'
//   upper-stored [[A,C],[0,B]]^-1 = [[A',X],[0,B']],  X = -A' C B'
// and the other off-diagonal block is zero.  One CTA computes a 128 x 16 strip of X: first the strip of
// the inner product (C A' or C B'), kept in shared memory, then the outer one.  A', B' are read from the
// 256 x 256 block itself, C from the matrix (rows and columns beyond its order count as zero).
constexpr int kPairStrip = 16;

__global__ void __launch_bounds__(256) trtri_pair_kernel(const double *A, int64_t lda, int64_t dim, int lower,
                                                         double *inv, int ldo)
{
    __shared__ double Ws[kPairStrip][kNB + 1];
    const int pair = blockIdx.x / (kNB / kPairStrip), strip = blockIdx.x % (kNB / kPairStrip);
    const int t = threadIdx.x, i = t & (kNB - 1), half = t >> 7;         // row i, 8 of the 16 columns
    const int LD = ldo;                                                  // the pair is a diagonal block of an ldo x ldo one
    const int64_t at = (int64_t)pair * 2 * kNB;
    double *blk = inv + (at / ldo) * ldo * ldo + (at % ldo) * (ldo + 1);
    const double *Ai = blk, *Bi = blk + kNB * LD + kNB;                  // A' and B'
    const int64_t r0 = at;                                               // first row/column of the pair in the matrix
    // C as stored: lower -> rows r0+128.., columns r0..; upper -> rows r0.., columns r0+128..
    const int64_t cr = lower ? r0 + kNB : r0, cc = lower ? r0 : r0 + kNB;
    const double *inner = lower ? Ai : Bi;                               // right factor of the inner product
    const double *outer = lower ? Bi : Ai;                               // left factor of the outer product
    const int j0 = strip * kPairStrip + half * 8;
    double acc[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) acc[u] = 0.0;
    const bool row_ok = cr + i < dim;
    for (int p0 = 0; p0 < kNB; p0 += 16) {
        // sixteen elements of the row of C at a time, so that their latencies overlap
        double c[16];
#pragma unroll
        for (int q = 0; q < 16; ++q) c[q] = (row_ok && cc + p0 + q < dim) ? __ldg(A + cr + i + (cc + p0 + q) * lda) : 0.0;
#pragma unroll
        for (int q = 0; q < 16; ++q)
#pragma unroll
            for (int u = 0; u < 8; ++u) acc[u] += c[q] * inner[(j0 + u) * LD + p0 + q];
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) Ws[half * 8 + u][i] = acc[u];
    __syncthreads();
#pragma unroll
    for (int u = 0; u < 8; ++u) acc[u] = 0.0;
    for (int p = 0; p < kNB; ++p) {
        const double o = outer[p * LD + i];
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[u] += o * Ws[half * 8 + u][p];
    }
    double *X = lower ? blk + kNB : blk + kNB * LD;                      // where X sits in the 256-block
    double *Z = lower ? blk + kNB * LD : blk + kNB;                      // the zero block
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        X[i + (j0 + u) * LD] = -acc[u];
        Z[i + (j0 + u) * LD] = 0.0;
    }
}

__global__ void copy_matrix_kernel(double *dst, int64_t ldd, const double *src, int64_t lds,
                                   int64_t rows, int64_t cols)
{
    const int64_t total = rows * cols;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = e % rows, j = e / rows;
        dst[i + j * ldd] = src[i + j * lds];
    }
}

struct TrsmCtx {
    cudaStream_t st;
    int left, lower, trans;
    int eff_lower;            // op(A) is lower triangular
    int64_t m, n;             // B is m x n
    const double *A; int64_t lda;
    double *B; int64_t ldb;
    const double *inv;        // inverses of the diagonal blocks, leaf x leaf each
    int leaf;                 // 128, or 256 when the inverses have been completed pairwise
    double *W; int64_t ldw;   // leaf result before it is copied back
    int *err;                 // error word handed to the GEMM kernels (nullptr = library default)
    int status;
};

static void launch_copy(TrsmCtx &c, double *dst, int64_t ldd, const double *src, int64_t lds,
                        int64_t rows, int64_t cols)
{
    int64_t blocks = (rows * cols + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    copy_matrix_kernel<<<(int)blocks, 256, 0, c.st>>>(dst, ldd, src, lds, rows, cols);
    count_launch();
}

// element block (i0.., j0..) of op(A): pointer + flag for the GEMM
static const double *opA_block(const TrsmCtx &c, int64_t i0, int64_t j0)
{
    return c.trans ? c.A + j0 + i0 * c.lda : c.A + i0 + j0 * c.lda;
}

static void gemm_chk(TrsmCtx &c, int ta, int tb, int64_t m, int64_t n, int64_t k, double alpha,
                     const double *A, int64_t lda, const double *B, int64_t ldb, double beta,
                     double *C, int64_t ldc)
{
    if (c.status != ULMB200_OK) return;
    c.status = dgemm_device(c.st, 0, ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, c.err);
}

// Left:  rows [r0, r0+len) of B <- op(A)[r0.., r0..]^-1 * B[r0.., :]
static void solve_left(TrsmCtx &c, int64_t r0, int64_t len)
{
    if (c.status != ULMB200_OK) return;
    if (len <= c.leaf) {
        const double *iv = c.inv + (r0 / c.leaf) * c.leaf * c.leaf;
        // in place where the operands allow it, else through the work tile and a copy back
        const int r = dgemm_leaf_inplace(c.st, 1, c.eff_lower, c.trans, len, c.n, 1.0, iv, c.leaf, c.B + r0, c.ldb, c.err);
        if (r >= 0) { c.status = r; return; }
        if (c.leaf > 2 * kNB) { c.status = ULMB200_CUDA_ERROR; return; }     // only the leaf kernel skips the unwritten blocks
        gemm_chk(c, c.trans, 0, len, c.n, len, 1.0, iv, c.leaf, c.B + r0, c.ldb, 0.0, c.W, c.ldw);
        launch_copy(c, c.B + r0, c.ldb, c.W, c.ldw, len, c.n);
        return;
    }
    const int64_t half = ((len / 2 + c.leaf - 1) / c.leaf) * c.leaf;
    const int64_t l1 = half, l2 = len - half;
    if (c.eff_lower) {
        solve_left(c, r0, l1);
        // B2 -= op(A)[r0+l1.., r0..r0+l1) * X1
        gemm_chk(c, c.trans, 0, l2, c.n, l1, -1.0, opA_block(c, r0 + l1, r0), c.lda, c.B + r0, c.ldb,
                 1.0, c.B + r0 + l1, c.ldb);
        solve_left(c, r0 + l1, l2);
    } else {
        solve_left(c, r0 + l1, l2);
        // B1 -= op(A)[r0..r0+l1, r0+l1..) * X2
        gemm_chk(c, c.trans, 0, l1, c.n, l2, -1.0, opA_block(c, r0, r0 + l1), c.lda, c.B + r0 + l1,
                 c.ldb, 1.0, c.B + r0, c.ldb);
        solve_left(c, r0, l1);
    }
}

// Right: columns [c0, c0+len) of B <- B[:, c0..] * op(A)[c0.., c0..]^-1
static void solve_right(TrsmCtx &c, int64_t c0, int64_t len)
{
    if (c.status != ULMB200_OK) return;
    if (len <= c.leaf) {
        const double *iv = c.inv + (c0 / c.leaf) * c.leaf * c.leaf;
        const int r = dgemm_leaf_inplace(c.st, 0, c.eff_lower, c.trans, len, c.m, 1.0, iv, c.leaf, c.B + c0 * c.ldb, c.ldb, c.err);
        if (r >= 0) { c.status = r; return; }
        if (c.leaf > 2 * kNB) { c.status = ULMB200_CUDA_ERROR; return; }
        gemm_chk(c, 0, c.trans, c.m, len, len, 1.0, c.B + c0 * c.ldb, c.ldb, iv, c.leaf, 0.0, c.W, c.ldw);
        launch_copy(c, c.B + c0 * c.ldb, c.ldb, c.W, c.ldw, c.m, len);
        return;
    }
    const int64_t half = ((len / 2 + c.leaf - 1) / c.leaf) * c.leaf;
    const int64_t l1 = half, l2 = len - half;
    if (c.eff_lower) {
        // X * L = B: last columns first, then B1 -= X2 * L21
        solve_right(c, c0 + l1, l2);
        gemm_chk(c, 0, c.trans, c.m, l1, l2, -1.0, c.B + (c0 + l1) * c.ldb, c.ldb,
                 opA_block(c, c0 + l1, c0), c.lda, 1.0, c.B + c0 * c.ldb, c.ldb);
        solve_right(c, c0, l1);
    } else {
        // X * U = B: first columns first, then B2 -= X1 * U12
        solve_right(c, c0, l1);
        gemm_chk(c, 0, c.trans, c.m, l2, l1, -1.0, c.B + c0 * c.ldb, c.ldb,
                 opA_block(c, c0, c0 + l1), c.lda, 1.0, c.B + (c0 + l1) * c.ldb, c.ldb);
        solve_right(c, c0 + l1, l2);
    }
}

// Doubles the order of the inverted diagonal blocks from h to 2h, for every pair whose second half
// exists: lower-stored [[A,0],[C,B]]^-1 = [[A',0],[-B' C A',B']], upper-stored [[A,C],[0,B]]^-1 =
// [[A',-A' C B'],[0,B']].  All pairs go through two batched products (inner factor into the work
// matrix pairs_w, h x h per pair side by side, then the outer one into its place).  The inverses of
// the L x L blocks lie one after the other with leading dimension L.
static int trtri_double(cudaStream_t st, const double *A, int64_t lda, int64_t dim, int lower, double *inv, int L,
                        int h, double *pairs_w)
{
    if (dim <= h) return ULMB200_OK;
    const int64_t nQ = (dim + L - 1) / L;
    BatchShape bs;
    bs.count = (int)((dim - h + 2 * h - 1) / (2 * h));
    bs.nlo = L / (2 * h);
    const int64_t wide = (int64_t)L * nQ;               // the inverses as one L x wide matrix
    const int two_h = 2 * h;
    auto set = [](int (&x)[2], int lo, int hi) { x[0] = lo; x[1] = hi; };
    // 1. pairs_w_q = C_q * A'_q (lower) or C_q * B'_q (upper)
    set(bs.a_row, two_h, L); set(bs.a_col, two_h, L);     // C_q walks down the diagonal of the matrix
    set(bs.b_row, two_h, 0); set(bs.b_col, two_h, L);     // a diagonal block of inverse number hi
    bs.c_row[0] = bs.c_row[1] = 0; bs.c_col[0] = h; bs.c_col[1] = (int64_t)h * bs.nlo;
    const double *C0 = lower ? A + h : A + (int64_t)h * lda;
    const int64_t c_rows = lower ? dim - h : dim, c_cols = lower ? dim : dim - h;
    const double *in0 = lower ? inv : inv + h + (int64_t)h * L;
    const int64_t in_rows = lower ? L : L - h, in_cols = lower ? wide : wide - h;
    int r = dgemm_batched(st, h, h, h, 1.0, C0, lda, c_rows, c_cols, in0, L, in_rows, in_cols, pairs_w, h, h, (int64_t)h * bs.count, bs);
    if (r != ULMB200_OK) return r;
    // 2. X_q = -B'_q * pairs_w_q (lower) or -A'_q * pairs_w_q (upper)
    set(bs.a_row, two_h, 0); set(bs.a_col, two_h, L);
    set(bs.b_row, 0, 0); set(bs.b_col, h, h * bs.nlo);
    bs.c_row[0] = two_h; bs.c_row[1] = 0; bs.c_col[0] = two_h; bs.c_col[1] = L;
    const double *out0 = lower ? inv + h + (int64_t)h * L : inv;
    const int64_t out_rows = lower ? L - h : L, out_cols = lower ? wide - h : wide;
    double *X0 = lower ? inv + h : inv + (int64_t)h * L;
    const int64_t x_rows = lower ? L - h : L, x_cols = lower ? wide : wide - h;
    return dgemm_batched(st, h, h, h, -1.0, out0, L, out_rows, out_cols, pairs_w, h, h, (int64_t)h * bs.count, X0, L, x_rows, x_cols, bs);
}

// Shared by the allocating entry point and any caller that brings its own
// scratch, with leaf = 128: inv holds ceil(dim/128) * 128 * 128 doubles, W 128*n (left) or m*128 (right);
// with leaf = 256 (inverses completed pairwise, half as many and larger leaf products):
// inv holds ceil(dim/256) * 256 * 256 doubles, W 256*n or m*256.  Larger leaves (512, 1024, ...: the
// inverses doubled again by batched products) need pairs as well, ceil(dim/leaf) * leaf * leaf / 4 doubles.
int dtrsm_with_scratch(cudaStream_t st, int side, int lower, int transA, int unit, int64_t m,
                       int64_t n, double alpha, const double *A, int64_t lda, double *B,
                       int64_t ldb, double *inv, double *W, int *err_word, int leaf, double *pairs)
{
    const int left = (side == 0);
    const int64_t dim = left ? m : n;
    if (alpha == 0.0)              // trlsm.tcc:46-49
        return scale_matrix_device(st, B, ldb, m, n, 0.0, 0);
    if (alpha != 1.0) {
        int s = scale_matrix_device(st, B, ldb, m, n, alpha, 0);
        if (s != ULMB200_OK) return s;
    }
    const int nblk = (int)((dim + kNB - 1) / kNB);
    static bool attr_done[kMaxDevices] = {};
    const int dev = current_device();
    const int smem = (kNB * kNB + 64 * 64) * (int)sizeof(double);
    if (!attr_done[dev]) {
        ULMB_CUDA(cudaFuncSetAttribute(trtri_blocks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_done[dev] = true;
    }
    const int64_t nleaf = (dim + leaf - 1) / leaf;
    if (leaf > 2 * kNB) {
        // the blocks above (below) the diagonal that no kernel writes are read as zeros by the batched products
        // of the next doubling step, and so is what a last block holds beyond the triangle
        ULMB_CUDA(cudaMemsetAsync(inv, 0, sizeof(double) * (size_t)nleaf * leaf * leaf, st));
    }
    trtri_blocks_kernel<<<nblk, kTrtriThreads, smem, st>>>(A, lda, dim, lower, unit, inv, leaf);
    count_launch();
    if (leaf >= 2 * kNB) {
        // an odd last block has no partner: its pair is completed against an all-zero second block,
        // which the first kernel never wrote, so clear that corner first
        const int npair = (nblk + 1) / 2;
        if ((nblk & 1) && leaf == 2 * kNB) {
            double *last = inv + (int64_t)(npair - 1) * leaf * leaf;
            ULMB_CUDA(cudaMemset2DAsync(last + kNB * leaf + kNB, sizeof(double) * leaf, 0, sizeof(double) * kNB, kNB, st));
        }
        trtri_pair_kernel<<<npair * (kNB / kPairStrip), 256, 0, st>>>(A, lda, dim, lower, inv, leaf);
        count_launch();
    }
    ULMB_CUDA(cudaGetLastError());
    for (int h = 2 * kNB; h < leaf; h *= 2) {
        const int r = trtri_double(st, A, lda, dim, lower, inv, leaf, h, pairs);
        if (r != ULMB200_OK) return r < 0 ? ULMB200_BAD_ARGUMENT : r;
    }

    TrsmCtx c;
    c.st = st; c.left = left; c.lower = lower; c.trans = transA;
    c.eff_lower = (lower != 0) != (transA != 0);
    c.m = m; c.n = n; c.A = A; c.lda = lda; c.B = B; c.ldb = ldb;
    c.inv = inv; c.W = W; c.ldw = left ? leaf : m;
    c.leaf = leaf;
    c.err = err_word;
    c.status = ULMB200_OK;
    if (left) solve_left(c, 0, m);
    else      solve_right(c, 0, n);
    return c.status;
}

// Order of the inverted diagonal blocks.  Small triangles keep 128 or 256; large ones with many right-hand
// sides take 1024, so that the products below the top of the recursion are few and large: a leaf of order
// 1024 is one launch that multiplies only the blocks of its triangle, where 256-leaves solve the same rows in
// seven launches too short to fill the machine.  The larger blocks need TMA-addressable operands for the
// batched products that build them.
// What a leaf of order L > 256 needs: TMA-addressable operands and a reader counter per leaf tile.
static bool large_leaf_ok(cudaStream_t st, int L, int64_t dim, int64_t other, const double *A, int64_t lda, const double *B,
                          int64_t ldb)
{
    const int64_t tiles = ((L < dim ? L : dim) + 127) / 128 * ((other + 127) / 128);
    return ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) == 0 && lda % 2 == 0 &&
           ldb % 2 == 0 && dim < (1ll << 31) - 4096 && other < (1ll << 31) - 4096 && lda < (1ll << 36) &&
           ldb < (1ll << 36) && tiles <= kSchedFlags && sched_words(st) != nullptr;
}

static int trsm_leaf_order(cudaStream_t st, int64_t dim, int64_t other, const double *A, int64_t lda, const double *B,
                           int64_t ldb)
{
    int leaf = dim > 2 * kNB ? 2 * kNB : kNB;
    // beyond 256 only the triangular leaf can apply the inverses, whose blocks above (below) the diagonal
    // are never written
    if (dim >= 2048 && other >= 1024 && large_leaf_ok(st, 1024, dim, other, A, lda, B, ldb)) leaf = 1024;
    const int forced = settings().trsm_leaf;
    if (forced == 128 || forced == 256 ||
        ((forced == 512 || forced == 1024 || forced == 2048) && large_leaf_ok(st, forced, dim, other, A, lda, B, ldb))) {
        leaf = forced;
        while (leaf > kNB && leaf / 2 >= dim) leaf /= 2;     // no larger than the triangle needs
    }
    return leaf;
}

int dtrsm_device(cudaStream_t st, int side, int lower, int transA, int unit, int64_t m, int64_t n,
                 double alpha, const double *A, int64_t lda, double *B, int64_t ldb)
{
    if (m < 0 || n < 0 || (side != 0 && side != 1)) return set_status(ULMB200_BAD_ARGUMENT);
    const int64_t dim = (side == 0) ? m : n;
    if (lda < (dim > 1 ? dim : 1) || ldb < (m > 1 ? m : 1)) return set_status(ULMB200_BAD_ARGUMENT);
    if (m == 0 || n == 0) return set_status(ULMB200_OK);
    if (int s = ensure_device()) return set_status(s);
    const int leaf = trsm_leaf_order(st, dim, side == 0 ? n : m, A, lda, B, ldb);
    const int64_t nblk = (dim + leaf - 1) / leaf;
    double *inv = static_cast<double *>(device_scratch(3, (size_t)nblk * leaf * leaf * sizeof(double)));
    double *W = nullptr, *pairs = nullptr;
    if (leaf > 2 * kNB) {
        // the large leaves are applied in place only: no work tile, but room for the batched products
        pairs = static_cast<double *>(device_scratch(7, (size_t)nblk * leaf * leaf / 4 * sizeof(double)));
        if (!pairs) return set_status(ULMB200_CUDA_ERROR);
    } else {
        const int64_t wel = (side == 0) ? (int64_t)leaf * n : m * (int64_t)leaf;
        W = static_cast<double *>(device_scratch(4, (size_t)wel * sizeof(double)));
        if (!W) return set_status(ULMB200_CUDA_ERROR);
    }
    if (!inv) return set_status(ULMB200_CUDA_ERROR);
    return set_status(dtrsm_with_scratch(st, side, lower, transA, unit, m, n, alpha, A, lda, B, ldb, inv, W, nullptr, leaf, pairs));
}

// ---------------------------------------------------------------------------
// syr2k:  triangle of  C <- alpha*(op(A)*op(B)^T + op(B)*op(A)^T) + beta*C
// (ulmblas/level3/syur2k.tcc:18-127, sylr2k.tcc: two passes of the gemm macro-kernel
// per block; here two passes of the device GEMM with the triangle predicate).
// ---------------------------------------------------------------------------
int dsyr2k_device(cudaStream_t st, int lower, int trans, int64_t n, int64_t k, double alpha,
                  const double *A, int64_t lda, const double *B, int64_t ldb, double beta, double *C,
                  int64_t ldc)
{
    if (n < 0 || k < 0) return set_status(ULMB200_BAD_ARGUMENT);
    const int64_t rows = trans ? k : n;
    if (lda < (rows > 1 ? rows : 1) || ldb < (rows > 1 ? rows : 1) || ldc < (n > 1 ? n : 1))
        return set_status(ULMB200_BAD_ARGUMENT);
    if (n == 0 || ((alpha == 0.0 || k == 0) && beta == 1.0)) return set_status(ULMB200_OK);   // syur2k.tcc:47-49
    const int tri = lower ? 2 : 1;
    const int ta = trans ? 1 : 0, tb = trans ? 0 : 1;
    int s = dgemm_device(st, tri, ta, tb, n, n, k, alpha, A, lda, B, ldb, beta, C, ldc);
    if (s != ULMB200_OK || alpha == 0.0 || k == 0) return s;
    return dgemm_device(st, tri, ta, tb, n, n, k, alpha, B, ldb, A, lda, 1.0, C, ldc);
}

// ---------------------------------------------------------------------------
// symm:  C <- alpha*A*B + beta*C (left) or alpha*B*A + beta*C (right), A symmetric with one
// triangle stored (ulmblas/level3/sylmm.tcc:18-100, syumm.tcc; pack/sy?pack.tcc mirrors the
// stored triangle while packing).  Here the mirror image is written once into scratch and the
// product is one device GEMM.
// ---------------------------------------------------------------------------
__global__ void symmetrize_kernel(const double *A, int64_t lda, int64_t n, int lower, double *S, int64_t lds)
{
    const int64_t total = n * n;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = e % n, j = e / n;
        const bool stored = lower ? (i >= j) : (i <= j);
        S[i + j * lds] = stored ? A[i + j * lda] : A[j + i * lda];
    }
}

int dsymm_device(cudaStream_t st, int side, int lower, int64_t m, int64_t n, double alpha, const double *A,
                 int64_t lda, const double *B, int64_t ldb, double beta, double *C, int64_t ldc)
{
    if (m < 0 || n < 0 || (side != 0 && side != 1)) return set_status(ULMB200_BAD_ARGUMENT);
    const int64_t na = side == 0 ? m : n;
    if (lda < (na > 1 ? na : 1) || ldb < (m > 1 ? m : 1) || ldc < (m > 1 ? m : 1))
        return set_status(ULMB200_BAD_ARGUMENT);
    if (m == 0 || n == 0 || (alpha == 0.0 && beta == 1.0)) return set_status(ULMB200_OK);     // sylmm.tcc:47-49
    if (int s0 = ensure_device()) return set_status(s0);
    if (alpha == 0.0) return set_status(scale_matrix_device(st, C, ldc, m, n, beta, 0));
    const int64_t lds = (na + 1) / 2 * 2;
    double *S = static_cast<double *>(device_scratch(6, sizeof(double) * (size_t)(lds * na)));
    if (!S) return set_status(ULMB200_CUDA_ERROR);
    int64_t blocks = (na * na + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    symmetrize_kernel<<<(int)blocks, 256, 0, st>>>(A, lda, na, lower, S, lds);
    count_launch();
    if (int e = check_cuda(cudaGetLastError(), "symmetrize_kernel", __FILE__, __LINE__)) return e;
    if (side == 0) return dgemm_device(st, 0, 0, 0, m, n, m, alpha, S, lds, B, ldb, beta, C, ldc);
    return dgemm_device(st, 0, 0, 0, m, n, n, alpha, B, ldb, S, lds, beta, C, ldc);
}

// ---------------------------------------------------------------------------
// trmm:  B <- alpha*op(A)*B (left) or alpha*B*op(A) (right), A triangular
// (ulmblas/level3/trlmm.tcc:18-88, trumm.tcc; pack/tr?pack.tcc zero-fills the other
// triangle while packing).  Same recursion as the solver above: the off-diagonal blocks
// are plain GEMM updates on rows/columns of B not yet overwritten, the diagonal blocks (256 x
// 256) are multiplied from zero-filled copies and go through the leaf tile.
// ---------------------------------------------------------------------------
// nbt = order of the diagonal blocks.  A CTA of min(nbt, 256) threads copies that many rows of kCleanCols
// columns of one block (grid: blocks x row parts, column chunks), all loads of a thread in flight together.
constexpr int kCleanCols = 16;
__global__ void __launch_bounds__(256)
trclean_blocks_kernel(const double *A, int64_t lda, int64_t dim, int lower, int unit, double *out, int nbt)
{
    const int parts = (nbt + (int)blockDim.x - 1) / (int)blockDim.x;
    const int blk = blockIdx.x / parts, j = (blockIdx.x % parts) * (int)blockDim.x + threadIdx.x;
    if (j >= nbt) return;
    const int64_t r0 = (int64_t)blk * nbt;
    const int len = (int)((dim - r0) < nbt ? (dim - r0) : nbt);
    const double *Ab = A + r0 + r0 * lda;
    double *o = out + (int64_t)blk * nbt * nbt;
    const int i0 = blockIdx.y * kCleanCols;
    double v[kCleanCols];
#pragma unroll
    for (int q = 0; q < kCleanCols; ++q) {
        // element (j, i): threads run down a column, coalesced
        const int i = i0 + q;
        v[q] = 0.0;
        if (i < len && j < len) {
            if (i == j) v[q] = unit ? 1.0 : Ab[j + (int64_t)i * lda];
            else if (lower ? (j > i) : (j < i)) v[q] = Ab[j + (int64_t)i * lda];
        }
    }
#pragma unroll
    for (int q = 0; q < kCleanCols; ++q)
        if (i0 + q < nbt) o[j + (int64_t)(i0 + q) * nbt] = v[q];
}

// the work tile of a leaf that cannot be multiplied in place, allocated when the first such leaf turns up
static bool trmm_work_tile(TrsmCtx &c)
{
    if (c.W) return true;
    const int64_t wel = c.left ? (int64_t)c.leaf * c.n : c.m * (int64_t)c.leaf;
    c.W = static_cast<double *>(device_scratch(4, (size_t)wel * sizeof(double)));
    if (!c.W) c.status = ULMB200_CUDA_ERROR;
    return c.W != nullptr;
}

static void mul_left(TrsmCtx &c, double alpha, int64_t r0, int64_t len)
{
    if (c.status != ULMB200_OK) return;
    if (len <= c.leaf) {
        const double *tb = c.inv + (r0 / c.leaf) * c.leaf * c.leaf;
        const int r = dgemm_leaf_inplace(c.st, 1, c.eff_lower, c.trans, len, c.n, alpha, tb, c.leaf, c.B + r0, c.ldb, c.err);
        if (r >= 0) { c.status = r; return; }
        if (!trmm_work_tile(c)) return;
        gemm_chk(c, c.trans, 0, len, c.n, len, alpha, tb, c.leaf, c.B + r0, c.ldb, 0.0, c.W, c.ldw);
        launch_copy(c, c.B + r0, c.ldb, c.W, c.ldw, len, c.n);
        return;
    }
    const int64_t l1 = ((len / 2 + c.leaf - 1) / c.leaf) * c.leaf, l2 = len - l1;
    if (c.eff_lower) {
        mul_left(c, alpha, r0 + l1, l2);               // B2 <- a*T22*B2
        gemm_chk(c, c.trans, 0, l2, c.n, l1, alpha, opA_block(c, r0 + l1, r0), c.lda, c.B + r0, c.ldb, 1.0,
                 c.B + r0 + l1, c.ldb);                // B2 += a*T21*B1 (B1 still the input)
        mul_left(c, alpha, r0, l1);
    } else {
        mul_left(c, alpha, r0, l1);                    // B1 <- a*T11*B1
        gemm_chk(c, c.trans, 0, l1, c.n, l2, alpha, opA_block(c, r0, r0 + l1), c.lda, c.B + r0 + l1, c.ldb,
                 1.0, c.B + r0, c.ldb);                // B1 += a*T12*B2 (B2 still the input)
        mul_left(c, alpha, r0 + l1, l2);
    }
}

static void mul_right(TrsmCtx &c, double alpha, int64_t c0, int64_t len)
{
    if (c.status != ULMB200_OK) return;
    if (len <= c.leaf) {
        const double *tb = c.inv + (c0 / c.leaf) * c.leaf * c.leaf;
        const int r = dgemm_leaf_inplace(c.st, 0, c.eff_lower, c.trans, len, c.m, alpha, tb, c.leaf, c.B + c0 * c.ldb, c.ldb, c.err);
        if (r >= 0) { c.status = r; return; }
        if (!trmm_work_tile(c)) return;
        gemm_chk(c, 0, c.trans, c.m, len, len, alpha, c.B + c0 * c.ldb, c.ldb, tb, c.leaf, 0.0, c.W, c.ldw);
        launch_copy(c, c.B + c0 * c.ldb, c.ldb, c.W, c.ldw, c.m, len);
        return;
    }
    const int64_t l1 = ((len / 2 + c.leaf - 1) / c.leaf) * c.leaf, l2 = len - l1;
    if (c.eff_lower) {
        mul_right(c, alpha, c0, l1);                   // B1 <- a*B1*T11
        gemm_chk(c, 0, c.trans, c.m, l1, l2, alpha, c.B + (c0 + l1) * c.ldb, c.ldb, opA_block(c, c0 + l1, c0),
                 c.lda, 1.0, c.B + c0 * c.ldb, c.ldb); // B1 += a*B2*T21 (B2 still the input)
        mul_right(c, alpha, c0 + l1, l2);
    } else {
        mul_right(c, alpha, c0 + l1, l2);              // B2 <- a*B2*T22
        gemm_chk(c, 0, c.trans, c.m, l2, l1, alpha, c.B + c0 * c.ldb, c.ldb, opA_block(c, c0, c0 + l1), c.lda,
                 1.0, c.B + (c0 + l1) * c.ldb, c.ldb); // B2 += a*B1*T12 (B1 still the input)
        mul_right(c, alpha, c0, l1);
    }
}

int dtrmm_device(cudaStream_t st, int side, int lower, int transA, int unit, int64_t m, int64_t n,
                 double alpha, const double *A, int64_t lda, double *B, int64_t ldb)
{
    if (m < 0 || n < 0 || (side != 0 && side != 1)) return set_status(ULMB200_BAD_ARGUMENT);
    const int64_t dim = (side == 0) ? m : n;
    if (lda < (dim > 1 ? dim : 1) || ldb < (m > 1 ? m : 1)) return set_status(ULMB200_BAD_ARGUMENT);
    if (m == 0 || n == 0) return set_status(ULMB200_OK);
    if (int s = ensure_device()) return set_status(s);
    if (alpha == 0.0) return set_status(scale_matrix_device(st, B, ldb, m, n, 0.0, 0));      // trlmm.tcc:46-49
    // Diagonal blocks copied with their other triangle zero-filled, multiplied in place by the triangular leaf
    // of the GEMM kernel.  256 once the triangle spans several (a leaf is then one product instead of three
    // small ones); 1024 and 2048 for large triangles with many columns, where the leaf multiplies only the
    // blocks of the triangle and the recursion above it keeps just its large updates.
    const int64_t other = (side == 0) ? n : m;
    int leaf = dim > 256 ? 256 : kNB;
    if (dim >= 2048 && other >= 1024 && large_leaf_ok(st, 1024, dim, other, A, lda, B, ldb)) leaf = 1024;
    if (dim >= 4096 && other >= 1024 && large_leaf_ok(st, 2048, dim, other, A, lda, B, ldb)) leaf = 2048;
    const int forced = settings().trsm_leaf;
    if (forced == 128 || forced == 256 ||
        ((forced == 512 || forced == 1024 || forced == 2048) && large_leaf_ok(st, forced, dim, other, A, lda, B, ldb))) {
        leaf = forced;
        while (leaf > kNB && leaf / 2 >= dim) leaf /= 2;
    }
    const int64_t nblk = (dim + leaf - 1) / leaf;
    double *blk = static_cast<double *>(device_scratch(3, (size_t)nblk * leaf * leaf * sizeof(double)));
    if (!blk) return set_status(ULMB200_CUDA_ERROR);
    const int cta = leaf < 256 ? leaf : 256;
    trclean_blocks_kernel<<<dim3((unsigned)(nblk * ((leaf + cta - 1) / cta)), (unsigned)((leaf + kCleanCols - 1) / kCleanCols)), cta, 0, st>>>(
        A, lda, dim, lower, unit, blk, leaf);
    count_launch();
    if (int e = check_cuda(cudaGetLastError(), "trclean_blocks_kernel", __FILE__, __LINE__)) return e;
    TrsmCtx c;
    c.st = st; c.left = (side == 0); c.lower = lower; c.trans = transA;
    c.eff_lower = (lower != 0) != (transA != 0);
    c.m = m; c.n = n; c.A = A; c.lda = lda; c.B = B; c.ldb = ldb;
    c.inv = blk; c.W = nullptr; c.ldw = c.left ? leaf : m;
    c.leaf = leaf;
    c.err = nullptr;
    c.status = ULMB200_OK;
    if (c.left) mul_left(c, alpha, 0, m);
    else        mul_right(c, alpha, 0, n);
    return set_status(c.status);
}

// ---------------------------------------------------------------------------
// Single-precision syrk / trsm.  The reference widens alpha (and beta) to double in these
// shims, so its ssyrk_ / strsm_ compute in double and round to float at the end of each
// block (interfaces/blas/F77/syrk.cc:30-32, trsm.cc:32).  Same here: the float operands are
// widened into scratch, the FP64 kernels above do the work, and the result is rounded once
// on the way back (only the requested triangle of C is written).
// ---------------------------------------------------------------------------
__global__ void widen_kernel(const float *X, int64_t ldx, int64_t rows, int64_t cols, double *D, int64_t ldd)
{
    const int64_t total = rows * cols;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = e % rows, j = e / rows;
        D[i + j * ldd] = (double)X[i + j * ldx];
    }
}

// tri: 0 all, 1 upper (i <= j), 2 lower (i >= j)
__global__ void narrow_kernel(const double *D, int64_t ldd, int64_t rows, int64_t cols, float *X, int64_t ldx, int tri)
{
    const int64_t total = rows * cols;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = e % rows, j = e / rows;
        if (tri == 1 && i > j) continue;
        if (tri == 2 && i < j) continue;
        X[i + j * ldx] = (float)D[i + j * ldd];
    }
}

static int grid_for(int64_t total)
{
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    return (int)(blocks > cap ? cap : (blocks < 1 ? 1 : blocks));
}

int ssyrk_device(cudaStream_t st, int lower, int trans, int64_t n, int64_t k, float alpha, const float *A,
                 int64_t lda, float beta, float *C, int64_t ldc)
{
    if (n < 0 || k < 0) return set_status(ULMB200_BAD_ARGUMENT);
    const int64_t rowsA = trans ? k : n, colsA = trans ? n : k;
    if (lda < (rowsA > 1 ? rowsA : 1) || ldc < (n > 1 ? n : 1)) return set_status(ULMB200_BAD_ARGUMENT);
    if (n == 0 || ((alpha == 0.0f || k == 0) && beta == 1.0f)) return set_status(ULMB200_OK);
    if (int s0 = ensure_device()) return set_status(s0);
    const int64_t lda_d = (rowsA + 1) / 2 * 2, ldc_d = (n + 1) / 2 * 2;
    double *buf = static_cast<double *>(device_scratch(11, sizeof(double) * (size_t)(lda_d * (colsA > 0 ? colsA : 1) + ldc_d * n)));
    if (!buf) return set_status(ULMB200_CUDA_ERROR);
    double *Ad = buf, *Cd = buf + lda_d * (colsA > 0 ? colsA : 1);
    if (rowsA > 0 && colsA > 0) { widen_kernel<<<grid_for(rowsA * colsA), 256, 0, st>>>(A, lda, rowsA, colsA, Ad, lda_d); count_launch(); }
    // the unreferenced triangle of C is widened too but never converted back
    widen_kernel<<<grid_for(n * n), 256, 0, st>>>(C, ldc, n, n, Cd, ldc_d);
    count_launch();
    int s = dsyrk_device(st, lower, trans, n, k, (double)alpha, Ad, lda_d, (double)beta, Cd, ldc_d);
    if (s != ULMB200_OK) return s;
    narrow_kernel<<<grid_for(n * n), 256, 0, st>>>(Cd, ldc_d, n, n, C, ldc, lower ? 2 : 1);
    count_launch();
    return set_status(check_cuda(cudaGetLastError(), "ssyrk", __FILE__, __LINE__));
}

int strsm_device(cudaStream_t st, int side, int lower, int transA, int unit, int64_t m, int64_t n, float alpha,
                 const float *A, int64_t lda, float *B, int64_t ldb)
{
    if (m < 0 || n < 0 || (side != 0 && side != 1)) return set_status(ULMB200_BAD_ARGUMENT);
    const int64_t dim = (side == 0) ? m : n;
    if (lda < (dim > 1 ? dim : 1) || ldb < (m > 1 ? m : 1)) return set_status(ULMB200_BAD_ARGUMENT);
    if (m == 0 || n == 0) return set_status(ULMB200_OK);
    if (int s0 = ensure_device()) return set_status(s0);
    const int64_t lda_d = (dim + 1) / 2 * 2, ldb_d = (m + 1) / 2 * 2;
    double *buf = static_cast<double *>(device_scratch(11, sizeof(double) * (size_t)(lda_d * dim + ldb_d * n)));
    if (!buf) return set_status(ULMB200_CUDA_ERROR);
    double *Ad = buf, *Bd = buf + lda_d * dim;
    // the whole square is widened; the solver reads only the referenced triangle (rogue values in
    // the other one convert to finite doubles or Inf/NaN that are never touched)
    widen_kernel<<<grid_for(dim * dim), 256, 0, st>>>(A, lda, dim, dim, Ad, lda_d);
    widen_kernel<<<grid_for(m * n), 256, 0, st>>>(B, ldb, m, n, Bd, ldb_d);
    count_launch(2);
    int s = dtrsm_device(st, side, lower, transA, unit, m, n, (double)alpha, Ad, lda_d, Bd, ldb_d);
    if (s != ULMB200_OK) return s;
    narrow_kernel<<<grid_for(m * n), 256, 0, st>>>(Bd, ldb_d, m, n, B, ldb, 0);
    count_launch();
    return set_status(check_cuda(cudaGetLastError(), "strsm", __FILE__, __LINE__));
}

}  // namespace ulmb200

extern "C" int ulmb200_dsyrk(void *stream, int lower, int trans, int64_t n, int64_t k, double alpha,
                             const double *dA, int64_t ldA, double beta, double *dC, int64_t ldC)
{
    return ulmb200::dsyrk_device(static_cast<cudaStream_t>(stream), lower, trans, n, k, alpha, dA, ldA,
                                 beta, dC, ldC);
}

extern "C" int ulmb200_dsyr2k(void *stream, int lower, int trans, int64_t n, int64_t k, double alpha,
                              const double *dA, int64_t ldA, const double *dB, int64_t ldB, double beta,
                              double *dC, int64_t ldC)
{
    return ulmb200::dsyr2k_device(static_cast<cudaStream_t>(stream), lower, trans, n, k, alpha, dA, ldA, dB,
                                  ldB, beta, dC, ldC);
}

extern "C" int ulmb200_dsymm(void *stream, int side, int lower, int64_t m, int64_t n, double alpha,
                             const double *dA, int64_t ldA, const double *dB, int64_t ldB, double beta,
                             double *dC, int64_t ldC)
{
    return ulmb200::dsymm_device(static_cast<cudaStream_t>(stream), side, lower, m, n, alpha, dA, ldA, dB, ldB,
                                 beta, dC, ldC);
}

extern "C" int ulmb200_dtrmm(void *stream, int side, int lower, int transA, int unit, int64_t m, int64_t n,
                             double alpha, const double *dA, int64_t ldA, double *dB, int64_t ldB)
{
    return ulmb200::dtrmm_device(static_cast<cudaStream_t>(stream), side, lower, transA, unit, m, n, alpha, dA,
                                 ldA, dB, ldB);
}

extern "C" int ulmb200_ssyrk(void *stream, int lower, int trans, int64_t n, int64_t k, float alpha,
                             const float *dA, int64_t ldA, float beta, float *dC, int64_t ldC)
{
    return ulmb200::ssyrk_device(static_cast<cudaStream_t>(stream), lower, trans, n, k, alpha, dA, ldA, beta, dC, ldC);
}

extern "C" int ulmb200_strsm(void *stream, int side, int lower, int transA, int unit, int64_t m, int64_t n,
                             float alpha, const float *dA, int64_t ldA, float *dB, int64_t ldB)
{
    return ulmb200::strsm_device(static_cast<cudaStream_t>(stream), side, lower, transA, unit, m, n, alpha, dA, ldA,
                                 dB, ldB);
}

extern "C" int ulmb200_dtrsm(void *stream, int side, int lower, int transA, int unit, int64_t m,
                             int64_t n, double alpha, const double *dA, int64_t ldA, double *dB,
                             int64_t ldB)
{
    return ulmb200::dtrsm_device(static_cast<cudaStream_t>(stream), side, lower, transA, unit, m, n, alpha,
                                 dA, ldA, dB, ldB);
}
