// Blocked LU with partial pivoting on the device: the one in-tree caller of the
// reference's trlsm + gemm (ulmblas/lapack/getrf.tcc:30-73, getf2.tcc:15-62,
// laswp.tcc), kept right-looking with the reference's loop structure:
//
//   for each 128-column panel:   getf2 on the panel          -> getf2_cluster_reg_kernel / getf2_cluster_kernel
//                                                                (+ lu_rank_update_kernel between sub-panels)
//                                 row swaps left and right    -> lu_perm_list_kernel + laswp_gather_kernel
//                                 A12 <- L11^-1 A12           -> lu_trsm_unit_lower_kernel
//                                 A22 <- A22 - A21 A12        -> device DGEMM
//
// with look-ahead: the next panel is factored on a second stream while the rest of the trailing
// update runs (see dgetrf_device).  Panels too tall for a cluster's shared memory fall back to one
// cooperative launch: the CTAs split the panel's rows, and per column they (1) propose their
// largest entry, (2) after a grid-wide barrier agree on the pivot (first largest, as iamax does)
// while CTA 0 swaps the two rows inside the panel, (3) after a second barrier scale their part of
// the column by the reciprocal pivot (the reference's scal(1/pivot), getf2.tcc:42-44) and apply
// the rank-1 update to their rows.  Pivots are 0-based row indices as in the reference
// (piv[i] = row exchanged with row i); info is the 1-based index of the first exactly-zero pivot,
// 0 if none.
#include "common.h"

#include <cooperative_groups.h>
#include <float.h>
#include <limits.h>

namespace cg = cooperative_groups;

namespace ulmb200 {

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

// Warp-wide "first largest": every lane leaves with the largest v and, among the lanes that hold
// it, the smallest index.  Five exchange steps on the value and one hardware reduction on the index.
__device__ __forceinline__ void lu_warp_argmax(double &v, int &i)
{
    double m = v;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmax(m, __shfl_xor_sync(0xffffffffu, m, off));
    const int cand = (v == m) ? i : INT_MAX;
    i = __reduce_min_sync(0xffffffffu, cand);
    v = m;
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

// ---------------------------------------------------------------------------
// Panel factorisation inside one thread-block cluster.
//
// A grid-wide barrier costs 1.2 us on this part, a cluster barrier 0.2 us, and a CTA can write
// straight into the shared memory of the other CTAs of its cluster.  So the 128-column panel is cut
// into sub-panels of up to 32 columns, and one cluster of 16 CTAs factors a sub-panel entirely out
// of shared memory: CTA b keeps rows [b R, (b+1) R) of the sub-panel, and per column
//   1. finds its best pivot candidate,
//   2. writes the candidate (value, row index) into EVERY CTA's shared memory and parks the
//      candidate's row (and row c, if it owns it) in its own,
//   3. after one cluster barrier each CTA picks the pivot from its own copy of the 16 candidates and
//      reads the pivot row out of the winner's shared memory; the owners exchange the two rows, all
//      scale and update their rows.
// When the sub-panel is done the cluster writes it back, applies its row exchanges to the other
// columns of the 128-column panel (as one gather, no chain of dependent swaps) and solves
// U12 = L11^-1 A12 for the columns to the right, so that the only other launch per sub-panel is the
// rank-w update of those columns (lu_rank_update_kernel).
// Publication buffers alternate with the column parity: a CTA can be at most one column ahead.
// ---------------------------------------------------------------------------
constexpr int kClu = 16;           // CTAs per cluster (non-portable size, allowed explicitly)
constexpr int kCluW = 32;          // widest sub-panel

struct CluArgs {
    double *A;            // top-left element of the 128-column panel (row j, column j of the matrix)
    int64_t lda;
    int64_t m;            // rows of the panel
    int nb;               // columns of the panel
    int c0;               // first column (= first row) of the sub-panel inside the panel
    int w;                // columns of the sub-panel
    int64_t row_off;      // j: added to pivot indices and info
    int *piv;
    int *info;
    int ldS;              // pitch of the shared-memory slab (odd, >= rows per CTA)
    int R;                // rows per CTA
};

// What a cluster does once its sub-panel is factored and written back: the sub-panel's row
// exchanges, as (destination row <- source row) pairs, applied to the other columns of the
// 128-column panel, then U12 = L11^-1 A12 for the columns to its right.  `idx` is scratch shared
// memory for (rows of the sub-panel) ints.
struct CluShared {
    int s_piv[kCluW];                 // pivot of column c as a sub-panel row index
    int s_dst[2 * kCluW], s_src[2 * kCluW], s_cnt, s_info;
    double s_L11[kCluW * kCluW];
    double s_buf[2 * kCluW][8];
};

__device__ __forceinline__ void cluster_post_phase(const CluArgs &a, CluShared &sh, int *idx, int b, int ncol)
{
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int w = a.w;
    double *Asub = a.A + a.c0 + (int64_t)a.c0 * a.lda;
    // its row exchanges as (destination row <- source row) pairs: replay them on a sparse index map
    if (t < ncol) { idx[t] = t; }
    __syncthreads();
    if (t < ncol) idx[sh.s_piv[t]] = sh.s_piv[t];
    __syncthreads();
    if (t == 0) {
        for (int c = 0; c < ncol; ++c) {
            const int p = sh.s_piv[c];
            const int tmp = idx[c]; idx[c] = idx[p]; idx[p] = tmp;
        }
        sh.s_cnt = 0;
    }
    __syncthreads();
    if (t < 2 * ncol) {
        const int r = t < ncol ? t : sh.s_piv[t - ncol];
        bool first = idx[r] != r;
        for (int q = 0; q < t && first; ++q) first = (q < ncol ? q : sh.s_piv[q - ncol]) != r;
        if (first) { const int slot = atomicAdd(&sh.s_cnt, 1); sh.s_dst[slot] = r; sh.s_src[slot] = idx[r]; }
    }
    __syncthreads();
    const int cnt = sh.s_cnt;

    // my columns of the panel outside the sub-panel: exchange rows, then (right of it) U12
    for (int e = t; e < ncol * ncol; e += kLuThreads) {
        const int i = e % ncol, q = e / ncol;
        sh.s_L11[q * kCluW + i] = Asub[i + (int64_t)q * a.lda];
    }
    __syncthreads();
    const int nother = a.nb - w;
    for (int base = b * 8; base < nother; base += kClu * 8) {
        // up to 8 columns per pass; oc counts the columns outside the sub-panel
        const int ncs = min(8, nother - base);
        for (int e = t; e < cnt * ncs; e += kLuThreads) {
            const int q = e % cnt, k = e / cnt;
            const int oc = base + k, col = oc < a.c0 ? oc : oc + w;
            sh.s_buf[q][k] = a.A[a.c0 + sh.s_src[q] + (int64_t)col * a.lda];
        }
        __syncthreads();
        for (int e = t; e < cnt * ncs; e += kLuThreads) {
            const int q = e % cnt, k = e / cnt;
            const int oc = base + k, col = oc < a.c0 ? oc : oc + w;
            a.A[a.c0 + sh.s_dst[q] + (int64_t)col * a.lda] = sh.s_buf[q][k];
        }
        __threadfence_block();
        __syncthreads();
        // U12: one warp per column right of the sub-panel, lane i holds element i
        if (warp < ncs) {
            const int oc = base + warp, col = oc < a.c0 ? oc : oc + w;
            if (col >= a.c0 + w) {
                double *x = a.A + a.c0 + (int64_t)col * a.lda;
                double u = lane < ncol ? x[lane] : 0.0;
                for (int q = 0; q + 1 < ncol; ++q) {
                    const double uq = __shfl_sync(0xffffffffu, u, q);
                    if (lane > q && lane < ncol) u -= sh.s_L11[q * kCluW + lane] * uq;
                }
                if (lane < ncol) x[lane] = u;
            }
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kLuThreads, 1) getf2_cluster_kernel(CluArgs a)
{
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ double lu_smem[];
    __shared__ double sv[kLuThreads / 32];
    __shared__ double pub_val[2][kClu];
    __shared__ int pub_idx[2][kClu];
    __shared__ double pub_row[2][kCluW];         // my candidate's row, read by the others when it wins
    __shared__ double pub_rowc[2][kCluW];        // row c, parked by its owner
    __shared__ double s_row[kCluW];
    __shared__ double s_pivv[kCluW];             // pivot values (0 = column skipped as singular)
    __shared__ int s_wi[kLuThreads / 32];
    __shared__ CluShared sh;

    const int b = (int)cluster.block_rank(), t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int64_t ms = a.m - a.c0;                               // rows of the sub-panel
    const int R = a.R, ldS = a.ldS, w = a.w;
    const int64_t lo = (int64_t)b * R, hi = min(ms, lo + R);
    const int nr = (int)max((int64_t)0, hi - lo);
    double *S = lu_smem;                                        // S[cc*ldS + r]
    double *Asub = a.A + a.c0 + (int64_t)a.c0 * a.lda;          // sub-panel element (0, 0)

    for (int cc = 0; cc < w; ++cc)
        for (int r = t; r < nr; r += kLuThreads) S[cc * ldS + r] = Asub[lo + r + (int64_t)cc * a.lda];
    if (t == 0) sh.s_info = 0;
    __syncthreads();

    const int ncol = (int)min((int64_t)w, ms);
    const int msi = (int)ms;                    // the slab bound keeps the sub-panel below 2^31 rows
    for (int c = 0; c < ncol; ++c) {
        const int par = c & 1;
        // (1) candidate among my rows >= c: per lane, per warp, then every warp combines the 8 warp
        // results itself (one block barrier, no broadcast step)
        double bv = -1.0;
        int bi = msi;
        for (int r = t; r < nr; r += kLuThreads) {
            const int gr = (int)lo + r;
            if (gr >= c) {
                const double v = fabs(S[c * ldS + r]);
                if (v > bv) { bv = v; bi = gr; }          // rows ascend: the first maximum stays
            }
        }
        lu_warp_argmax(bv, bi);
        if (lane == 0) { sv[warp] = bv; s_wi[warp] = bi; }
        __syncthreads();
        bv = lane < kLuThreads / 32 ? sv[lane] : -2.0;
        bi = lane < kLuThreads / 32 ? s_wi[lane] : INT_MAX;
        lu_warp_argmax(bv, bi);
        // (2) publish the candidate into every CTA of the cluster
        if (t < kClu) {
            *cluster.map_shared_rank(&pub_val[par][b], t) = bv;
            *cluster.map_shared_rank(&pub_idx[par][b], t) = bi;
        }
        // the candidate's row and (its owner) row c are parked in this CTA's own shared memory; whoever
        // needs them after the barrier reads them from here
        if (bi < msi && t < w) pub_row[par][t] = S[t * ldS + (bi - (int)lo)];
        if (c >= lo && c < hi && t < w) pub_rowc[par][t] = S[t * ldS + (int)(c - lo)];
        cluster.sync();

        // (3) the pivot: first largest of the 16 candidates, found by every warp on its own
        double pv = lane < kClu ? pub_val[par][lane] : -2.0;
        int p = lane < kClu ? pub_idx[par][lane] : INT_MAX;
        lu_warp_argmax(pv, p);
        const bool singular = !(pv > 0.0);
        if (singular) p = c;
        // pivots and a zero-pivot report stay in shared memory until the sub-panel is done: a global
        // store here would have to drain before every cluster barrier's release
        if (t == 0) {
            sh.s_piv[c] = p;
            if (singular && sh.s_info == 0) sh.s_info = c + 1;
        }
        if (!singular) {
            const int wr = min(kClu - 1, p / R);            // CTA that owns row p
            const int oc = min(kClu - 1, c / R);            // CTA that owns row c
            if (t < w) {
                const double prow = *cluster.map_shared_rank(&pub_row[par][t], wr);
                s_row[t] = prow;
                if (t == c) {
                    s_pivv[c] = prow;                       // the pivot value, for the final scaling
                }
                if (p != c) {
                    if (p >= lo && p < hi) S[t * ldS + (p - (int)lo)] = *cluster.map_shared_rank(&pub_rowc[par][t], oc);
                    if (c >= lo && c < hi) S[t * ldS + (int)(c - lo)] = prow;
                }
            }
        } else if (t == 0) {
            s_pivv[c] = 0.0;                                // marks "column not scaled"
        }
        __syncthreads();
        if (!singular && c + 1 < w) {
            const double piv = s_row[c];
            const bool recip = fabs(piv) >= DBL_MIN;
            const double rp = 1.0 / piv;
            // rank-1 update of my rows below c, a thread per row.  Column c itself keeps the unscaled
            // entries until the write-back (later exchanges move them with their rows; the scaling
            // commutes with that), so nothing here writes what another thread reads.
            const int r_first = (int)max((int64_t)0, (int64_t)c + 1 - lo);
            for (int r = r_first + t; r < nr; r += kLuThreads) {
                const double x = S[c * ldS + r];
                const double l = recip ? x * rp : x / piv;
                for (int cc = c + 1; cc < w; ++cc) S[cc * ldS + r] -= l * s_row[cc];
            }
        }
        __syncthreads();
    }

    // the multipliers: column c of every row below the diagonal, scaled now
    for (int cc = 0; cc < ncol; ++cc) {
        const double piv = s_pivv[cc];
        if (piv == 0.0) continue;
        const bool recip = fabs(piv) >= DBL_MIN;
        const double rp = 1.0 / piv;
        const int r_first = (int)max((int64_t)0, (int64_t)cc + 1 - lo);
        for (int r = r_first + t; r < nr; r += kLuThreads) {
            const double x = S[cc * ldS + r];
            S[cc * ldS + r] = recip ? x * rp : x / piv;
        }
    }
    __syncthreads();

    // the factored sub-panel goes back, with its pivots (matrix row indices) and the first zero pivot
    if (b == 0) {
        if (t < ncol) a.piv[a.row_off + a.c0 + t] = (int)(sh.s_piv[t] + a.row_off + a.c0);
        if (t == 0 && sh.s_info != 0) atomicCAS(a.info, 0, (int)(a.row_off + a.c0 + sh.s_info));
    }
    for (int cc = 0; cc < w; ++cc)
        for (int r = t; r < nr; r += kLuThreads) Asub[lo + r + (int64_t)cc * a.lda] = S[cc * ldS + r];
    __threadfence();
    cluster.sync();

    cluster_post_phase(a, sh, reinterpret_cast<int *>(lu_smem), b, ncol);
}

// The same sub-panel factorisation with the rows held in REGISTERS: thread t of CTA b owns rows
// lo + t + 256 i (i < RPT) of the sub-panel, all 32 columns of each.  The rank-1 update then costs no
// shared-memory traffic at all, and a column needs one block barrier (inside the pivot search) and
// one cluster barrier.  Rows are not exchanged physically: each carries the position the reference's
// exchanges would have given it (which also keeps the "first largest" rule exact), and goes to that
// position when the sub-panel is written back.  Requires a full 32-column sub-panel of at least 32 rows and at most
// 16 * 256 * RPT rows; everything is unrolled so that the register arrays are indexed statically.
__device__ __forceinline__ void lu_warp_argmax_key(double &v, int &i)
{
    // v is -1 (no candidate) or a non-negative number: its bit pattern orders like the number
    const unsigned long long key = v < 0.0 ? 0ull : (unsigned long long)__double_as_longlong(v) + 1ull;
    const unsigned hi = (unsigned)(key >> 32), lo = (unsigned)key;
    const unsigned mh = __reduce_max_sync(0xffffffffu, hi);
    const unsigned ml = __reduce_max_sync(0xffffffffu, hi == mh ? lo : 0u);
    const bool mine = hi == mh && lo == ml;
    i = __reduce_min_sync(0xffffffffu, mine ? i : INT_MAX);
    const unsigned long long mk = ((unsigned long long)mh << 32) | ml;
    v = mk == 0ull ? -1.0 : __longlong_as_double((long long)(mk - 1ull));
}

template <int RPT>
__global__ void __launch_bounds__(kLuThreads, 1) getf2_cluster_reg_kernel(CluArgs a)
{
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ double lu_smem[];                           // only the post phase's index map
    __shared__ double sv[kLuThreads / 32];
    __shared__ int s_wi[kLuThreads / 32];
    __shared__ double pub_val[2][kClu];
    __shared__ int pub_idx[2][kClu];
    __shared__ double pub_row[2][kCluW];                          // my candidate's row
    __shared__ double s_roww[kLuThreads / 32][kCluW];            // the pivot row, one copy per warp
    __shared__ CluShared sh;

    constexpr int W = kCluW;
    const int b = (int)cluster.block_rank(), t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int ms = (int)(a.m - a.c0);
    const int R = a.R;
    const int lo = b * R, hi = min(ms, lo + R);
    const int nr = max(0, hi - lo);
    double *Asub = a.A + a.c0 + (int64_t)a.c0 * a.lda;

    // Rows never move between threads.  pos[i] is the position the row currently has in the
    // sub-panel (what the reference's explicit exchanges would have made it), done[i] says it has
    // served as a pivot row and is final; the rows go back to their positions at the end.
    double row[RPT][W];
    int pos[RPT];
    bool done[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int r = t + kLuThreads * i;
        pos[i] = lo + r;
        done[i] = r >= nr;                         // rows that do not exist never take part
#pragma unroll
        for (int cc = 0; cc < W; ++cc) row[i][cc] = r < nr ? Asub[lo + r + (int64_t)cc * a.lda] : 0.0;
    }
    if (t == 0) sh.s_info = 0;
    __syncthreads();

    // The column loop is a real loop (one copy of the body in the instruction cache: fully unrolled,
    // the kernel spent most of its time waiting for instruction fetches).  To keep every register
    // index static, the row registers rotate by one column per step: slot 0 is always the current
    // column, slot s holds column c + s, finished columns collect at the tail, and after 32 steps
    // everything is back in its natural place.
#pragma unroll 1
    for (int c = 0; c < W; ++c) {
        const int par = c & 1;
        // (1) candidate among my live rows: largest |value|, smallest position among equals
        double bv = -1.0;
        int bi = INT_MAX;
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            if (!done[i]) {
                const double v = fabs(row[i][0]);
                if (v > bv || (v == bv && pos[i] < bi)) { bv = v; bi = pos[i]; }
            }
        }
        lu_warp_argmax_key(bv, bi);
        if (lane == 0) { sv[warp] = bv; s_wi[warp] = bi; }
        __syncthreads();
        bv = lane < kLuThreads / 32 ? sv[lane] : -1.0;
        bi = lane < kLuThreads / 32 ? s_wi[lane] : INT_MAX;
        lu_warp_argmax_key(bv, bi);
        // (2) publish: the candidate to everyone, its row parked here by the thread that holds it
        if (t < kClu) {
            *cluster.map_shared_rank(&pub_val[par][b], t) = bv;
            *cluster.map_shared_rank(&pub_idx[par][b], t) = bi;
        }
        {
            int sel = -1;
#pragma unroll
            for (int i = 0; i < RPT; ++i) sel = (!done[i] && pos[i] == bi) ? i : sel;
            if (sel >= 0 && bv >= 0.0) {
#pragma unroll
                for (int sl = 0; sl < W; ++sl) {
                    double v = row[0][sl];
#pragma unroll
                    for (int i = 1; i < RPT; ++i) v = sel == i ? row[i][sl] : v;     // selects: static register indices
                    pub_row[par][(c + sl) & (W - 1)] = v;                             // slot sl holds column c + sl
                }
            }
        }
        cluster.sync();

        // (3) the pivot, found by every warp on its own; wr = the CTA whose candidate won
        double pv = lane < kClu ? pub_val[par][lane] : -1.0;
        int p = lane < kClu ? pub_idx[par][lane] : INT_MAX;
        const double myv = pv;
        const int myp = p;
        lu_warp_argmax_key(pv, p);
        const unsigned won = __ballot_sync(0xffffffffu, lane < kClu && myv == pv && myp == p);
        const int wr = won ? __ffs(won) - 1 : 0;
        const bool singular = !(pv > 0.0);
        if (singular) p = c;
        if (t == 0) {
            sh.s_piv[c] = p;
            if (singular && sh.s_info == 0) sh.s_info = c + 1;
        }
        if (!singular) s_roww[warp][lane] = *cluster.map_shared_rank(&pub_row[par][lane], wr);
        // the exchange of positions c and p: the pivot row becomes final at c, the row that sat at c
        // (if it is another one) now sits at p
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            if (!done[i]) {
                if (pos[i] == p) { done[i] = true; pos[i] = c; }
                else if (pos[i] == c) pos[i] = p;
            }
        }
        __syncwarp();
        if (!singular) {
            // (4) multipliers and rank-1 update of the live rows, all in registers
            const double piv = s_roww[warp][c];
            const bool recip = fabs(piv) >= DBL_MIN;
            const double rp = 1.0 / piv;
            double l[RPT];
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                l[i] = 0.0;
                if (!done[i]) {
                    l[i] = recip ? row[i][0] * rp : row[i][0] / piv;
                    row[i][0] = l[i];
                }
            }
#pragma unroll
            for (int sl = 1; sl < W; ++sl) {
                if (sl < W - c) {                                            // slots beyond hold finished columns
                    const double pr = s_roww[warp][c + sl];
#pragma unroll
                    for (int i = 0; i < RPT; ++i) row[i][sl] -= l[i] * pr;  // l = 0 leaves the row as it is
                }
            }
        }
        __syncwarp();
        // rotate: the finished column goes to the tail
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
            const double first = row[i][0];
#pragma unroll
            for (int sl = 0; sl + 1 < W; ++sl) row[i][sl] = row[i][sl + 1];
            row[i][W - 1] = first;
        }
    }

    if (b == 0) {
        if (t < W) a.piv[a.row_off + a.c0 + t] = (int)(sh.s_piv[t] + a.row_off + a.c0);
        if (t == 0 && sh.s_info != 0) atomicCAS(a.info, 0, (int)(a.row_off + a.c0 + sh.s_info));
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int r = t + kLuThreads * i;
        if (r < nr) {
#pragma unroll
            for (int cc = 0; cc < W; ++cc) Asub[pos[i] + (int64_t)cc * a.lda] = row[i][cc];
        }
    }
    __threadfence();
    cluster.sync();
    cluster_post_phase(a, sh, reinterpret_cast<int *>(lu_smem), b, W);
}

// A22 <- A22 - L21 U12 inside the 128-column panel after a sub-panel: rows below the sub-panel's
// diagonal block, columns right of it.  32 rows per CTA; U12 (w x ncr) sits in shared memory.
constexpr int kRankRows = 32;

struct RankArgs {
    double *A;            // top-left of the panel
    int64_t lda;
    int64_t m;            // rows of the panel
    int c0, w, ncr;       // sub-panel offset and width, columns right of it
};

__global__ void __launch_bounds__(kLuThreads) lu_rank_update_kernel(RankArgs a)
{
    __shared__ double U[kCluW][128 + 1];
    const int t = threadIdx.x;
    const double *U12 = a.A + a.c0 + (int64_t)(a.c0 + a.w) * a.lda;
    for (int e = t; e < kCluW * a.ncr; e += kLuThreads) {
        const int k = e % kCluW, cc = e / kCluW;
        U[k][cc] = k < a.w ? U12[k + (int64_t)cc * a.lda] : 0.0;       // rows beyond w take part as zeros
    }
    __syncthreads();
    // 32 rows per CTA (lane = row), the eight warps share the columns: twice as many CTAs as with 64
    // rows each, and four loads in flight per thread instead of one
    const int64_t r = (int64_t)a.c0 + a.w + (int64_t)blockIdx.x * kRankRows + (t & 31);
    if (r >= a.m) return;
    double l[kCluW];
#pragma unroll
    for (int k = 0; k < kCluW; ++k) l[k] = k < a.w ? a.A[r + (int64_t)(a.c0 + k) * a.lda] : 0.0;
    const int g = t >> 5;
    for (int cc = g; cc < a.ncr; cc += 32) {
        double acc[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            acc[u] = cc + 8 * u < a.ncr ? a.A[r + (int64_t)(a.c0 + a.w + cc + 8 * u) * a.lda] : 0.0;
#pragma unroll
        for (int k = 0; k < kCluW; ++k) {
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[u] -= l[k] * U[k][(cc + 8 * u) & 127];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (cc + 8 * u < a.ncr) a.A[r + (int64_t)(a.c0 + a.w + cc + 8 * u) * a.lda] = acc[u];
    }
}

// The nb row exchanges of a panel (row k1+i <-> row piv[k1+i], in order) as one simultaneous
// assignment: list = { count, dst[256], src[256] } with "row dst takes the old contents of row
// src".  Slots 0..nb-1 stand for rows k1..k1+nb-1, slot nb+q for pivot row q when it lies below
// the panel's diagonal block and q is its first occurrence; one thread replays the exchanges on
// the slot contents, which is the only sequential part.
constexpr int kPermMax = 2 * kLuNB;

__global__ void __launch_bounds__(kLuThreads) lu_perm_list_kernel(const int *piv, int64_t k1, int nb, int *list)
{
    __shared__ int s_p[kLuNB], s_slot[kLuNB], s_cont[kPermMax], s_valid[kPermMax], s_cnt;
    const int t = threadIdx.x;
    if (t < nb) s_p[t] = piv[k1 + t] - (int)k1;             // relative to the panel's first row
    if (t < kPermMax) { s_cont[t] = t; s_valid[t] = t < nb; }
    if (t == 0) s_cnt = 0;
    __syncthreads();
    if (t < nb) {
        const int p = s_p[t];
        int slot = p;
        if (p >= nb) {
            int fo = t;
            for (int q = 0; q < t; ++q) if (s_p[q] == p) { fo = q; break; }
            slot = nb + fo;
            if (fo == t) s_valid[slot] = 1;
        }
        s_slot[t] = slot;
    }
    __syncthreads();
    if (t == 0)
        for (int i = 0; i < nb; ++i) {
            const int sb = s_slot[i];
            const int tmp = s_cont[i]; s_cont[i] = s_cont[sb]; s_cont[sb] = tmp;
        }
    __syncthreads();
    if (t < kPermMax && s_valid[t] && s_cont[t] != t) {
        const int k = atomicAdd(&s_cnt, 1);
        const int src_slot = s_cont[t];
        list[1 + k] = t < nb ? t : s_p[t - nb];
        list[1 + kPermMax + k] = src_slot < nb ? src_slot : s_p[src_slot - nb];
    }
    __syncthreads();
    if (t == 0) list[0] = s_cnt;
}

// Applies such a list to columns [0, skip_from) and [skip_from + skip_count, ...) of A (ncols
// columns in all, rows relative to row0).  One warp per column: every lane first reads its
// sources, then writes its destinations, so no chain of dependent exchanges remains.
__global__ void __launch_bounds__(kLuThreads) laswp_gather_kernel(double *A, int64_t lda, int64_t ncols,
                                                                  int64_t skip_from, int64_t skip_count,
                                                                  int64_t row0, const int *list)
{
    __shared__ int s_dst[kPermMax], s_src[kPermMax];
    const int t = threadIdx.x, lane = t & 31;
    const int cnt = list[0];
    if (t < cnt) { s_dst[t] = list[1 + t]; s_src[t] = list[1 + kPermMax + t]; }
    __syncthreads();
    if (cnt == 0) return;
    const int64_t warps = (int64_t)gridDim.x * (kLuThreads / 32);
    for (int64_t oc = (int64_t)blockIdx.x * (kLuThreads / 32) + (t >> 5); oc < ncols; oc += warps) {
        const int64_t col = oc < skip_from ? oc : oc + skip_count;
        double *x = A + row0 + col * lda;
        double v[kPermMax / 32];
#pragma unroll
        for (int u = 0; u < kPermMax / 32; ++u) {
            const int q = lane + 32 * u;
            v[u] = q < cnt ? x[s_src[q]] : 0.0;
        }
        __syncwarp();
#pragma unroll
        for (int u = 0; u < kPermMax / 32; ++u) {
            const int q = lane + 32 * u;
            if (q < cnt) x[s_dst[q]] = v[u];
        }
    }
}

// U12 <- L11^-1 A12 for the columns right of a panel: L11 is the panel's unit lower triangle
// (nb <= 128), A12 its nb x ncols row block.  The generic TRSM inverts diagonal blocks and runs
// GEMMs -- four launches and ~150 us for what is 0.1 GFLOP here -- so LU has its own: L11 sits in
// shared memory, a warp solves four columns at a time by forward substitution across its lanes
// (lane = row mod 32, four rows per lane), 32 columns per CTA.
constexpr int kTrsmCols = 32;          // columns per CTA: 8 warps x 4

__global__ void __launch_bounds__(kLuThreads) lu_trsm_unit_lower_kernel(const double *L, int64_t ldl, int nb,
                                                                        double *B, int64_t ldb, int64_t ncols)
{
    extern __shared__ double Ls[];                 // Ls[p * kLuNB + i] = L(i, p)
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    for (int e = t; e < nb * kLuNB; e += kLuThreads) {
        const int i = e % kLuNB, p = e / kLuNB;
        Ls[p * kLuNB + i] = (i < nb && i > p) ? L[i + (int64_t)p * ldl] : 0.0;
    }
    __syncthreads();
    const int64_t col0 = (int64_t)blockIdx.x * kTrsmCols + warp * 4;
    double x[4][4];                                // [column][row chunk]
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int row = lane + 32 * k;
            x[j][k] = (col0 + j < ncols && row < nb) ? B[row + (col0 + j) * ldb] : 0.0;
        }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
        if (32 * kk >= nb) break;
        for (int pl = 0; pl < 32; ++pl) {
            const int p = 32 * kk + pl;
            if (p >= nb) break;
            double xp[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) xp[j] = __shfl_sync(0xffffffffu, x[j][kk], pl);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (k < kk) continue;
                const double l = Ls[p * kLuNB + lane + 32 * k];      // zero on and above the diagonal
#pragma unroll
                for (int j = 0; j < 4; ++j) x[j][k] -= l * xp[j];
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int row = lane + 32 * k;
            if (col0 + j < ncols && row < nb) B[row + (col0 + j) * ldb] = x[j][k];
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

// Occupies its stream for about ns nanoseconds (nothing is waited for: a fixed number of short sleeps).
constexpr unsigned kHeadStartNs = 12000;
__global__ void lu_head_start_kernel(unsigned ns)
{
    for (unsigned waited = 0; waited < ns; waited += 500) __nanosleep(500);
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
    static int64_t cluster_smem_max[kMaxDevices] = {};
    static bool reg_ok[kMaxDevices] = {};
    if (cluster_smem_max[dev] == 0) {
        reg_ok[dev] =
            cudaFuncSetAttribute(getf2_cluster_reg_kernel<1>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess &&
            cudaFuncSetAttribute(getf2_cluster_reg_kernel<2>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess &&
            // the index map of the post phase: 4 bytes per row of the sub-panel, up to 8192 rows
            cudaFuncSetAttribute(getf2_cluster_reg_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 40 * 1024) == cudaSuccess &&
            cudaFuncSetAttribute(getf2_cluster_reg_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 40 * 1024) == cudaSuccess;
        // what one CTA of a 16-CTA cluster may take next to the kernel's static shared memory
        cudaFuncAttributes fa;
        int optin = 0;
        ULMB_CUDA(cudaFuncGetAttributes(&fa, getf2_cluster_kernel));
        ULMB_CUDA(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        int64_t room = (int64_t)optin - (int64_t)fa.sharedSizeBytes - 1024;
        cluster_smem_max[dev] = -1;
        if (room > 16384 &&
            cudaFuncSetAttribute(getf2_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess &&
            cudaFuncSetAttribute(getf2_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)room) == cudaSuccess) {
            // the launch is only used if the device can actually co-schedule such a cluster
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(kClu); cfg.blockDim = dim3(kLuThreads); cfg.dynamicSmemBytes = (size_t)room;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = kClu; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
            cfg.attrs = at; cfg.numAttrs = 1;
            int ncl = 0;
            if (cudaOccupancyMaxActiveClusters(&ncl, getf2_cluster_kernel, &cfg) == cudaSuccess && ncl >= 1)
                cluster_smem_max[dev] = room;
        }
        cudaGetLastError();
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
    constexpr size_t kTrsmSmem = sizeof(double) * (size_t)kLuNB * kLuNB;
    static bool trsm_attr[kMaxDevices] = {};
    if (!trsm_attr[dev]) {
        ULMB_CUDA(cudaFuncSetAttribute(lu_trsm_unit_lower_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTrsmSmem));
        trsm_attr[dev] = true;
    }
    int *perm_list = static_cast<int *>(device_scratch(13, sizeof(int) * (1 + 2 * kPermMax)));
    if (!perm_list) return set_status(ULMB200_CUDA_ERROR);

    const int64_t mn = m < n ? m : n;
    // getf2 on the panel that starts at (j, j), queued on stream ps
    auto factor_panel = [&](cudaStream_t ps, int64_t j, int jb) -> int {
        PanelArgs a;
        a.A = A + j + j * lda; a.lda = lda; a.m = m - j; a.jb = jb; a.row_off = j;
        a.piv = d_piv; a.info = d_info; a.cand_val = cand_val; a.cand_idx = cand_idx;
        // Preferred: sub-panels of up to 32 columns, each factored by one 16-CTA cluster out of shared
        // memory.  The slab (rows/16 x width doubles per CTA) has to fit; narrower sub-panels for taller
        // panels, the cooperative kernels below beyond that.
        static const int use_cluster = [] { const char *e = getenv("ULMB200_LU_CLUSTER"); return e ? atoi(e) : 1; }();
        int wsub = kCluW;
        auto slab_bytes = [&](int64_t rows, int wcols) {
            const int64_t R = (rows + kClu - 1) / kClu;
            const int64_t ld = R | 1;
            const int64_t slab = (int64_t)wcols * ld * 8, map = rows * 4 + 64;
            return slab > map ? slab : map;
        };
        while (wsub > 8 && slab_bytes(a.m, wsub) > cluster_smem_max[dev]) wsub /= 2;
        if (use_cluster && cluster_smem_max[dev] > 0 && slab_bytes(a.m, wsub) <= cluster_smem_max[dev]) {
            for (int c0 = 0; c0 < jb && c0 < a.m; c0 += wsub) {
                CluArgs q;
                q.A = a.A; q.lda = lda; q.m = a.m; q.nb = jb; q.c0 = c0; q.w = (jb - c0) < wsub ? (jb - c0) : wsub;
                q.row_off = j; q.piv = d_piv; q.info = d_info;
                const int64_t rows = a.m - c0;
                q.R = (int)((rows + kClu - 1) / kClu);
                q.ldS = q.R | 1;
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = dim3(kClu); cfg.blockDim = dim3(kLuThreads);
                cfg.dynamicSmemBytes = (size_t)slab_bytes(rows, q.w);
                cfg.stream = ps;
                cudaLaunchAttribute at[1];
                at[0].id = cudaLaunchAttributeClusterDimension;
                at[0].val.clusterDim.x = kClu; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
                cfg.attrs = at; cfg.numAttrs = 1;
                // full-width sub-panels of up to 8192 rows keep their rows in registers
                static const int use_reg = [] { const char *e = getenv("ULMB200_LU_REG"); return e ? atoi(e) : 1; }();
                if (use_reg && reg_ok[dev] && q.w == kCluW && rows >= kCluW && q.R <= 2 * kLuThreads) {
                    cfg.dynamicSmemBytes = (size_t)(rows * 4 + 64);
                    if (q.R <= kLuThreads) ULMB_CUDA(cudaLaunchKernelEx(&cfg, getf2_cluster_reg_kernel<1>, q));
                    else                   ULMB_CUDA(cudaLaunchKernelEx(&cfg, getf2_cluster_reg_kernel<2>, q));
                } else {
                    ULMB_CUDA(cudaLaunchKernelEx(&cfg, getf2_cluster_kernel, q));
                }
                count_launch();
                const int ncr = jb - c0 - q.w;
                if (ncr > 0 && c0 + q.w < a.m) {
                    RankArgs r;
                    r.A = a.A; r.lda = lda; r.m = a.m; r.c0 = c0; r.w = q.w; r.ncr = ncr;
                    const int64_t below = a.m - c0 - q.w;
                    lu_rank_update_kernel<<<(unsigned)((below + kRankRows - 1) / kRankRows), kLuThreads, 0, ps>>>(r);
                    count_launch();
                }
            }
            ULMB_CUDA(cudaGetLastError());
        } else {
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
                                                  dim3(kLuThreads), args, kSlabSmem, ps));
        } else {
            int64_t G = (a.m + 4 * kLuThreads - 1) / (4 * kLuThreads);        // >= 1024 rows per CTA
            if (G > max_ctas[dev]) G = max_ctas[dev];
            if (G < 1) G = 1;
            void *args[] = {&a};
            ULMB_CUDA(cudaLaunchCooperativeKernel((const void *)getf2_panel_kernel, dim3((unsigned)G),
                                                  dim3(kLuThreads), args, 0, ps));
        }
        count_launch();
        }
        return ULMB200_OK;
    };

    // Look-ahead: once the columns of the next panel are updated, that panel is factored on a second
    // stream while the rest of the trailing update runs on the caller's.  The panel cluster needs 16
    // SMs of one GPC; it is queued first and the trailing GEMM leaves 16 SMs free, so the two run side
    // by side (if the GEMM wins the race for the SMs instead, the panel simply runs after it).
    static const int use_la = [] { const char *e = getenv("ULMB200_LU_LOOKAHEAD"); return e ? atoi(e) : 1; }();
    static cudaStream_t la_stream[kMaxDevices] = {};
    static cudaEvent_t la_ev[kMaxDevices][2] = {};
    bool la = use_la != 0 && mn > kLuNB;
    if (la && !la_stream[dev]) {
        // the panel is the critical path: its blocks go ahead of the trailing update's whenever both wait for SMs
        int prio_lo = 0, prio_hi = 0;
        cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi);
        if (cudaStreamCreateWithPriority(&la_stream[dev], cudaStreamNonBlocking, prio_hi) != cudaSuccess ||
            cudaEventCreateWithFlags(&la_ev[dev][0], cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&la_ev[dev][1], cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            la_stream[dev] = nullptr;
        }
    }
    if (!la_stream[dev]) la = false;
    const cudaStream_t sb = la_stream[dev];

    {
        const int jb0 = (int)(mn < kLuNB ? mn : kLuNB);
        if (int s0 = factor_panel(st, 0, jb0)) return set_status(s0);
    }
    for (int64_t j = 0; j < mn; j += kLuNB) {
        const int jb = (int)((mn - j) < kLuNB ? (mn - j) : kLuNB);
        // the same exchanges on the columns left and right of the panel (getrf.tcc:50-57), as one
        // gather over both column ranges
        {
            const int64_t others = n - jb;
            if (others > 0) {
                lu_perm_list_kernel<<<1, kLuThreads, 0, st>>>(d_piv, j, jb, perm_list);
                count_launch();
                int64_t blocks = (others + 7) / 8;
                const int64_t cap = (int64_t)sm_count() * 8;
                if (blocks > cap) blocks = cap;
                laswp_gather_kernel<<<(unsigned)blocks, kLuThreads, 0, st>>>(A, lda, others, j, jb, j, perm_list);
                count_launch();
            }
        }
        if (j + jb < n) {
            int s = ULMB200_OK;
            {
                const int64_t nright = n - j - jb;
                lu_trsm_unit_lower_kernel<<<(unsigned)((nright + kTrsmCols - 1) / kTrsmCols), kLuThreads, kTrsmSmem, st>>>(
                    A + j + j * lda, lda, jb, A + j + (j + jb) * lda, lda, nright);
                count_launch();
                ULMB_CUDA(cudaGetLastError());
            }
            if (j + jb < m) {
                const int64_t jn = j + jb;                              // where the next panel starts
                const int jb2 = jn < mn ? (int)((mn - jn) < kLuNB ? (mn - jn) : kLuNB) : 0;
                const int64_t mrows = m - jn, ncols = n - jn;
                const double *L21 = A + jn + j * lda, *U12 = A + j + jn * lda;
                double *A22 = A + jn + jn * lda;
                if (jb2 > 0) {
                    // the next panel's columns first, then its factorisation, then the other columns
                    s = dgemm_device(st, 0, 0, 0, mrows, jb2, jb, -1.0, L21, lda, U12, lda, 1.0, A22, lda);
                    if (s != ULMB200_OK) return set_status(s);
                    if (la) {
                        ULMB_CUDA(cudaEventRecord(la_ev[dev][0], st));
                        ULMB_CUDA(cudaStreamWaitEvent(sb, la_ev[dev][0], 0));
                        if (int sp = factor_panel(sb, jn, jb2)) return set_status(sp);
                        ULMB_CUDA(cudaEventRecord(la_ev[dev][1], sb));
                    } else {
                        if (int sp = factor_panel(st, jn, jb2)) return set_status(sp);
                    }
                    if (ncols > jb2) {
                        // Both the panel and the update become ready when the event above fires.  The update must
                        // not take its SMs first: its 132 persistent CTAs would leave the 16 free SMs scattered
                        // over all GPCs and the panel's cluster, which needs 16 SMs of one GPC, would wait for the
                        // whole update.  A few microseconds' head start lets the cluster settle on its GPC; the
                        // update then fills the other SMs and both hold their places until they are done.
                        if (la) {
                            lu_head_start_kernel<<<1, 32, 0, st>>>(kHeadStartNs);
                            count_launch();
                        }
                        const int old = la ? sm_reserve_swap(kClu) : 0;
                        s = dgemm_device(st, 0, 0, 0, mrows, ncols - jb2, jb, -1.0, L21, lda, U12 + (int64_t)jb2 * lda, lda,
                                         1.0, A22 + (int64_t)jb2 * lda, lda);
                        if (la) sm_reserve_swap(old);
                        if (s != ULMB200_OK) return set_status(s);
                    }
                    if (la) ULMB_CUDA(cudaStreamWaitEvent(st, la_ev[dev][1], 0));
                } else if (ncols > 0) {
                    s = dgemm_device(st, 0, 0, 0, mrows, ncols, jb, -1.0, L21, lda, U12, lda, 1.0, A22, lda);
                    if (s != ULMB200_OK) return set_status(s);
                }
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
