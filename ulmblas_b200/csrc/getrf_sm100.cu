// Blocked LU with partial pivoting on the device: the one in-tree caller of the
// reference's trlsm + gemm (ulmblas/lapack/getrf.tcc:30-73, getf2.tcc:15-62,
// laswp.tcc), kept right-looking with the reference's loop structure:
//
//   for each 128-column panel:   getf2 on the panel          -> getf2_panel_kernel
//                                 row swaps left and right    -> laswp_kernel
//                                 A12 <- L11^-1 A12           -> device TRSM (unit lower)
//                                 A22 <- A22 - A21 A12        -> device DGEMM
//
// The panel kernel is one cooperative launch: the CTAs split the panel's rows,
// and per column they (1) propose their largest entry, (2) after a grid-wide
// barrier agree on the pivot (first largest, as iamax does) while CTA 0 swaps the
// two rows inside the panel, (3) after a second barrier scale their part of the
// column by the reciprocal pivot (the reference's scal(1/pivot), getf2.tcc:42-44)
// and apply the rank-1 update to their rows.  Pivots are 0-based row indices as in
// the reference (piv[i] = row exchanged with row i); info is the 1-based index of
// the first exactly-zero pivot, 0 if none.
#include "common.h"

#include <cooperative_groups.h>
#include <float.h>

namespace cg = cooperative_groups;

namespace ulmb200 {

int dtrsm_device(cudaStream_t st, int side, int lower, int transA, int unit, int64_t m, int64_t n,
                 double alpha, const double *A, int64_t lda, double *B, int64_t ldb);

constexpr int kLuNB = 128;
constexpr int kLuThreads = 256;

struct PanelArgs {
    double *A;            // top-left element of the panel (row j, column j of the matrix)
    int64_t lda;
    int64_t m;            // rows of the panel
    int jb;               // columns of the panel
    int64_t row_off;      // j: added to the pivot indices and to info
    int *piv;             // device, piv[row_off + c]
    int *info;            // device, single int
    double *cand_val;     // one per CTA
    int *cand_idx;
};

// (v1, i1) beats (v2, i2) if larger, or equal and earlier: iamax returns the first maximum
__device__ __forceinline__ bool lu_better(double v1, int64_t i1, double v2, int64_t i2)
{
    return v1 > v2 || (v1 == v2 && i1 < i2);
}

// block-wide argmax: shuffles inside each warp, then one warp combines the 8 warp results
__device__ __forceinline__ void lu_block_argmax(double &v, int64_t &i, double *sv, int64_t *si)
{
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const double ov = __shfl_down_sync(0xffffffffu, v, off);
        const int64_t oi = __shfl_down_sync(0xffffffffu, i, off);
        if (lu_better(ov, oi, v, i)) { v = ov; i = oi; }
    }
    if (lane == 0) { sv[warp] = v; si[warp] = i; }
    __syncthreads();
    if (warp == 0) {
        v = lane < kLuThreads / 32 ? sv[lane] : -2.0;
        i = lane < kLuThreads / 32 ? si[lane] : INT64_MAX;
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) {
            const double ov = __shfl_down_sync(0xffffffffu, v, off);
            const int64_t oi = __shfl_down_sync(0xffffffffu, i, off);
            if (lu_better(ov, oi, v, i)) { v = ov; i = oi; }
        }
        if (lane == 0) { sv[32] = v; si[32] = i; }
    }
    __syncthreads();
    v = sv[32]; i = si[32];
    __syncthreads();
}

__global__ void __launch_bounds__(kLuThreads) getf2_panel_kernel(PanelArgs a)
{
    cg::grid_group grid = cg::this_grid();
    __shared__ double sv[kLuThreads];
    __shared__ int64_t si[kLuThreads];
    __shared__ double s_row[kLuNB];

    const int G = gridDim.x, b = blockIdx.x, t = threadIdx.x;
    const int64_t slab = ((a.m + G - 1) / G + 31) / 32 * 32;
    const int64_t lo = (int64_t)b * slab, hi = min(a.m, lo + slab);

    for (int c = 0; c < a.jb && c < a.m; ++c) {
        // (1) my candidate: largest |A(r, c)| over my rows r >= c
        double bv = -1.0;
        int64_t bi = a.m;
        for (int64_t r = max(lo, (int64_t)c) + t; r < hi; r += kLuThreads) {
            const double v = fabs(a.A[r + (int64_t)c * a.lda]);
            if (lu_better(v, r, bv, bi)) { bv = v; bi = r; }
        }
        lu_block_argmax(bv, bi, sv, si);
        if (t == 0) { a.cand_val[b] = bv; a.cand_idx[b] = (int)bi; }
        grid.sync();

        // (2) the pivot: best candidate of all CTAs (every CTA computes it); CTA 0 records and swaps
        double pv = -1.0;
        int64_t p = a.m;
        for (int g = t; g < G; g += kLuThreads) {
            const double v = a.cand_val[g];
            const int64_t i = a.cand_idx[g];
            if (lu_better(v, i, pv, p)) { pv = v; p = i; }
        }
        lu_block_argmax(pv, p, sv, si);
        const bool singular = !(pv > 0.0);          // all zero (or nothing comparable) in this column
        if (singular) p = c;
        if (b == 0) {
            if (t == 0) {
                a.piv[a.row_off + c] = (int)(p + a.row_off);
                if (singular) atomicCAS(a.info, 0, (int)(a.row_off + c + 1));
            }
            if (!singular && p != c) {
                for (int cc = t; cc < a.jb; cc += kLuThreads) {
                    double *x = a.A + c + (int64_t)cc * a.lda, *y = a.A + p + (int64_t)cc * a.lda;
                    const double tmp = *x; *x = *y; *y = tmp;
                }
            }
        }
        grid.sync();

        // (3) scale the column below the pivot and update my rows with the pivot row
        if (!singular) {
            for (int cc = c + t; cc < a.jb; cc += kLuThreads) s_row[cc] = a.A[c + (int64_t)cc * a.lda];
            __syncthreads();
            const double piv = s_row[c];
            const bool recip = fabs(piv) >= DBL_MIN;         // safeMin: getf2.tcc:42
            const double rp = 1.0 / piv;
            for (int64_t r = max(lo, (int64_t)c + 1) + t; r < hi; r += kLuThreads) {
                double *row = a.A + r;
                const double l = recip ? row[(int64_t)c * a.lda] * rp : row[(int64_t)c * a.lda] / piv;
                row[(int64_t)c * a.lda] = l;
                for (int cc = c + 1; cc < a.jb; ++cc) row[(int64_t)cc * a.lda] -= l * s_row[cc];
            }
            __syncthreads();
        }
    }
}

// The same panel factorisation with each CTA's rows held in shared memory (up to kLuSlabRows
// rows x 128 columns), used whenever the panel is short enough for that.  One grid-wide barrier
// per column: before it every CTA publishes its best candidate together with that row's
// contents, and the owner of row c publishes row c; after it every CTA knows the pivot row's
// contents without another exchange, the owners of the two rows overwrite their copies (the row
// swap), and all update their rows at shared-memory speed.  Publication buffers alternate with
// the column parity, so a CTA one column ahead never overwrites what a slower CTA still reads.
constexpr int kLuSlabRows = 192;

struct PanelSmemArgs {
    PanelArgs p;
    double *cand_rows;     // [2][G][kLuNB]
    double *rowc;          // [2][kLuNB]
    double *cval;          // [2][G]
    int *cidx;             // [2][G]
};

__global__ void __launch_bounds__(kLuThreads) getf2_panel_smem_kernel(PanelSmemArgs q)
{
    cg::grid_group grid = cg::this_grid();
    const PanelArgs &a = q.p;
    extern __shared__ double lu_smem[];
    __shared__ double sv[kLuThreads];
    __shared__ int64_t si[kLuThreads];
    __shared__ double s_row[kLuNB];
    __shared__ double s_l[kLuSlabRows];

    const int G = gridDim.x, b = blockIdx.x, t = threadIdx.x;
    const int64_t slab = (a.m + G - 1) / G;
    const int64_t lo = (int64_t)b * slab, hi = min(a.m, lo + slab);
    const int nr = (int)max((int64_t)0, hi - lo);          // my rows (<= kLuSlabRows)
    const int ldS = kLuSlabRows;
    double *S = lu_smem;                                   // S[cc*ldS + r]

    for (int e = t; e < nr * a.jb; e += kLuThreads) {
        const int r = e % nr, cc = e / nr;
        S[cc * ldS + r] = a.A[lo + r + (int64_t)cc * a.lda];
    }
    __syncthreads();

    const int ncol = (int)min((int64_t)a.jb, a.m);
    for (int c = 0; c < ncol; ++c) {
        const int par = c & 1;
        double *crow = q.cand_rows + ((size_t)par * G + b) * kLuNB;
        // (1) my candidate among rows >= c, published with its row
        double bv = -1.0;
        int64_t bi = a.m;
        for (int r = t; r < nr; r += kLuThreads) {
            const int64_t gr = lo + r;
            if (gr >= c) {
                const double v = fabs(S[c * ldS + r]);
                if (lu_better(v, gr, bv, bi)) { bv = v; bi = gr; }
            }
        }
        lu_block_argmax(bv, bi, sv, si);
        if (t == 0) { q.cval[par * G + b] = bv; q.cidx[par * G + b] = (int)bi; }
        if (bi < a.m)
            for (int cc = t; cc < a.jb; cc += kLuThreads) crow[cc] = S[cc * ldS + (int)(bi - lo)];
        if (c >= lo && c < hi)
            for (int cc = t; cc < a.jb; cc += kLuThreads) q.rowc[par * kLuNB + cc] = S[cc * ldS + (int)(c - lo)];
        __threadfence();
        grid.sync();

        // (2) the pivot and its row
        double pv = -1.0;
        int64_t p = a.m;
        for (int g = t; g < G; g += kLuThreads) {
            const double v = q.cval[par * G + g];
            const int64_t i = q.cidx[par * G + g];
            if (lu_better(v, i, pv, p)) { pv = v; p = i; }
        }
        lu_block_argmax(pv, p, sv, si);
        const bool singular = !(pv > 0.0);
        if (singular) p = c;
        if (b == 0 && t == 0) {
            a.piv[a.row_off + c] = (int)(p + a.row_off);
            if (singular) atomicCAS(a.info, 0, (int)(a.row_off + c + 1));
        }
        if (singular) continue;
        const int w = (int)min((int64_t)G - 1, p / slab);                // CTA that owns row p
        const double *prow = q.cand_rows + ((size_t)par * G + w) * kLuNB;
        for (int cc = t; cc < a.jb; cc += kLuThreads) s_row[cc] = prow[cc];
        if (p != c) {
            // the exchange: row p takes the old row c, row c takes the pivot row
            if (p >= lo && p < hi)
                for (int cc = t; cc < a.jb; cc += kLuThreads) S[cc * ldS + (int)(p - lo)] = q.rowc[par * kLuNB + cc];
            if (c >= lo && c < hi)
                for (int cc = t; cc < a.jb; cc += kLuThreads) S[cc * ldS + (int)(c - lo)] = prow[cc];
        }
        __syncthreads();

        // (3) multipliers, then the rank-1 update of my rows below c
        const double piv = s_row[c];
        const bool recip = fabs(piv) >= DBL_MIN;
        const double rp = 1.0 / piv;
        const int r_first = (int)max((int64_t)0, (int64_t)c + 1 - lo);   // first local row with global index > c
        for (int r = r_first + t; r < nr; r += kLuThreads) {
            const double x = S[c * ldS + r];
            const double l = recip ? x * rp : x / piv;
            S[c * ldS + r] = l;
            s_l[r] = l;
        }
        __syncthreads();
        const int na = nr - r_first, nc = a.jb - c - 1;
        if (na > 0)
            for (int e = t; e < na * nc; e += kLuThreads) {
                const int r = r_first + e % na, cc = c + 1 + e / na;
                S[cc * ldS + r] -= s_l[r] * s_row[cc];
            }
        __syncthreads();
    }

    for (int e = t; e < nr * a.jb; e += kLuThreads) {
        const int r = e % nr, cc = e / nr;
        a.A[lo + r + (int64_t)cc * a.lda] = S[cc * ldS + r];
    }
}

// Rows k1..k2-1 of `ncols` columns are exchanged with rows piv[k1..k2-1], in order (laswp.tcc).
__global__ void laswp_kernel(double *A, int64_t lda, int64_t ncols, int64_t k1, int64_t k2, const int *piv)
{
    for (int64_t col = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; col < ncols;
         col += (int64_t)gridDim.x * blockDim.x) {
        double *c = A + col * lda;
        for (int64_t i = k1; i < k2; ++i) {
            const int64_t p = piv[i];
            if (p != i) { const double tmp = c[i]; c[i] = c[p]; c[p] = tmp; }
        }
    }
}

// Row exchanges given as (row, other row) pairs in the order they are to be applied.
__global__ void laswp_pairs_kernel(double *A, int64_t lda, int64_t ncols, const int *pairs, int npairs)
{
    for (int64_t col = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; col < ncols;
         col += (int64_t)gridDim.x * blockDim.x) {
        double *c = A + col * lda;
        for (int q = 0; q < npairs; ++q) {
            const int i = pairs[2 * q], p = pairs[2 * q + 1];
            if (p != i) { const double tmp = c[i]; c[i] = c[p]; c[p] = tmp; }
        }
    }
}

int dlaswp_pairs_device(cudaStream_t st, double *A, int64_t lda, int64_t ncols, const int *d_pairs, int npairs)
{
    if (ncols <= 0 || npairs <= 0) return ULMB200_OK;
    int64_t blocks = (ncols + 127) / 128;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    laswp_pairs_kernel<<<(int)blocks, 128, 0, st>>>(A, lda, ncols, d_pairs, npairs);
    count_launch();
    return check_cuda(cudaGetLastError(), "laswp_pairs_kernel", __FILE__, __LINE__);
}

static void launch_laswp(cudaStream_t st, double *A, int64_t lda, int64_t ncols, int64_t k1, int64_t k2,
                         const int *piv)
{
    if (ncols <= 0) return;
    int64_t blocks = (ncols + 127) / 128;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    laswp_kernel<<<(int)blocks, 128, 0, st>>>(A, lda, ncols, k1, k2, piv);
    count_launch();
}

int dgetrf_device(cudaStream_t st, int64_t m, int64_t n, double *A, int64_t lda, int *d_piv, int *d_info)
{
    if (m < 0 || n < 0 || lda < (m > 1 ? m : 1)) return set_status(ULMB200_BAD_ARGUMENT);
    if (int s = ensure_device()) return set_status(s);
    ULMB_CUDA(cudaMemsetAsync(d_info, 0, sizeof(int), st));
    if (m == 0 || n == 0) return set_status(ULMB200_OK);

    static int max_ctas[kMaxDevices] = {};
    const int dev = current_device();
    if (max_ctas[dev] == 0) {
        int per_sm = 0;
        ULMB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, getf2_panel_kernel, kLuThreads, 0));
        max_ctas[dev] = (per_sm > 0 ? 1 : 0) * sm_count();      // one CTA per SM is plenty
        if (max_ctas[dev] <= 0) return set_status(ULMB200_CUDA_ERROR);
        ULMB_CUDA(cudaFuncSetAttribute(getf2_panel_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(sizeof(double) * kLuSlabRows * kLuNB)));
    }
    // scratch: candidates (value, index) x 2 parities, candidate rows x 2 parities, row c x 2 parities
    const size_t nG = (size_t)max_ctas[dev];
    const size_t doubles = 2 * nG + 2 * nG * kLuNB + 2 * kLuNB + nG /* ints, 2 per double */;
    double *cand_val = static_cast<double *>(device_scratch(8, sizeof(double) * doubles));
    if (!cand_val) return set_status(ULMB200_CUDA_ERROR);
    double *cand_rows = cand_val + 2 * nG;
    double *rowc = cand_rows + 2 * nG * kLuNB;
    int *cand_idx = reinterpret_cast<int *>(rowc + 2 * kLuNB);
    constexpr size_t kSlabSmem = sizeof(double) * (size_t)kLuSlabRows * kLuNB;

    const int64_t mn = m < n ? m : n;
    for (int64_t j = 0; j < mn; j += kLuNB) {
        const int jb = (int)((mn - j) < kLuNB ? (mn - j) : kLuNB);
        PanelArgs a;
        a.A = A + j + j * lda; a.lda = lda; a.m = m - j; a.jb = jb; a.row_off = j;
        a.piv = d_piv; a.info = d_info; a.cand_val = cand_val; a.cand_idx = cand_idx;
        // short panels live in shared memory (64..192 rows per CTA); taller ones work in global memory
        static const int rows_per_cta = [] { const char *e = getenv("ULMB200_LU_ROWS"); int v = e ? atoi(e) : 0;
                                             return (v >= 32 && v <= kLuSlabRows) ? v : 64; }();
        int64_t Gs = (a.m + rows_per_cta - 1) / rows_per_cta;
        if (Gs > max_ctas[dev]) Gs = max_ctas[dev];
        if (Gs < 1) Gs = 1;
        if ((a.m + Gs - 1) / Gs <= kLuSlabRows) {
            PanelSmemArgs q;
            q.p = a;
            q.cand_rows = cand_rows; q.rowc = rowc; q.cval = cand_val; q.cidx = cand_idx;
            void *args[] = {&q};
            ULMB_CUDA(cudaLaunchCooperativeKernel((const void *)getf2_panel_smem_kernel, dim3((unsigned)Gs),
                                                  dim3(kLuThreads), args, kSlabSmem, st));
        } else {
            int64_t G = (a.m + 4 * kLuThreads - 1) / (4 * kLuThreads);        // >= 1024 rows per CTA
            if (G > max_ctas[dev]) G = max_ctas[dev];
            if (G < 1) G = 1;
            void *args[] = {&a};
            ULMB_CUDA(cudaLaunchCooperativeKernel((const void *)getf2_panel_kernel, dim3((unsigned)G),
                                                  dim3(kLuThreads), args, 0, st));
        }
        count_launch();
        // the same exchanges on the columns left and right of the panel (getrf.tcc:50-57)
        launch_laswp(st, A, lda, j, j, j + jb, d_piv);
        if (j + jb < n) {
            launch_laswp(st, A + (j + jb) * lda, lda, n - j - jb, j, j + jb, d_piv);
            int s = dtrsm_device(st, 0, 1, 0, 1, jb, n - j - jb, 1.0, A + j + j * lda, lda, A + j + (j + jb) * lda, lda);
            if (s != ULMB200_OK) return set_status(s);
            if (j + jb < m) {
                s = dgemm_device(st, 0, 0, 0, m - j - jb, n - j - jb, jb, -1.0, A + (j + jb) + j * lda, lda,
                                 A + j + (j + jb) * lda, lda, 1.0, A + (j + jb) + (j + jb) * lda, lda);
                if (s != ULMB200_OK) return set_status(s);
            }
        }
    }
    return set_status(check_cuda(cudaGetLastError(), "dgetrf", __FILE__, __LINE__));
}

}  // namespace ulmb200

extern "C" int ulmb200_dgetrf(void *stream, int64_t m, int64_t n, double *dA, int64_t ldA, int *d_piv, int *d_info)
{
    return ulmb200::dgetrf_device(static_cast<cudaStream_t>(stream), m, n, dA, ldA, d_piv, d_info);
}
