/*
 * TEST INFRASTRUCTURE -- NOT PART OF THE PRODUCT.  See ulm_oracle.h.
 *
 * The reference packs operands into MR x KC / KC x NR panels and walks 4x4
 * register tiles (ulmblas/level3/pack/gepack.tcc, mkernel/mgemm.tcc,
 * ukernel/sse/ugemm.tcc).  Packing and tiling move data but do not change
 * which IEEE operations an output element sees, so the restatement keeps only
 * what determines the bits of each C(i,j):
 *
 *   - K is cut into blocks of KC (gemm.tcc:63-65; MC for syrk, syurk.tcc:60);
 *     beta is applied on the first block, 1 afterwards;
 *   - inside a block the dot product is accumulated from zero, one k at a
 *     time, product and sum rounded separately (mulpd + addpd,
 *     ukernel/sse/ugemm.tcc:60-222; AB[] += A*B in ukernel/ref/ugemm.tcc:30-37
 *     compiled without FMA);
 *   - the block result is folded in as  C = beta*C + alpha*ab  with the two
 *     products rounded before the sum (sse/ugemm.tcc:285-374; edge tiles do
 *     gescal(beta) then geaxpy of alpha*ab, ukernel/ugemm.tcc:33-37).
 *
 * Build with -ffp-contract=off (oracle/Makefile does).
 *
 * One deliberate difference: with beta == 0 the reference's SSE kernel still
 * multiplies the old C by 0 on full tiles (so NaN/Inf in C survive), while its
 * edge tiles assign.  The oracle assigns everywhere, as the BLAS standard
 * says; on finite C the two agree bit for bit.
 */
#include "ulm_oracle.h"

#include <ctype.h>
#include <stdlib.h>
#include <string.h>

static int g_MC = 384, g_KC = 384, g_NC = 4096;
static int g_KC_z = 192;   /* BlockSize<std::complex<double>>::KC, config/blocksize.h:41 */
enum { MR = 4, NR = 4 };   /* BlockSizeUGemm<double>, ukernel/sse/ugemm.h:12-15 */

void ulm_oracle_set_blocks(int mc, int kc, int nc)
{
    if (mc > 0) g_MC = mc;
    if (kc > 0) g_KC = kc;
    if (nc > 0) g_NC = nc;
}

/* KC of the complex double type: 192 by default; the reference's test builds give every
 * type the same blocks (config/blocksize.h:11-21), so checks against them set it too.   */
void ulm_oracle_set_blocks_z(int kc)
{
    if (kc > 0) g_KC_z = kc;
}

void ulm_oracle_get_blocks(int *mc, int *kc, int *nc)
{
    if (mc) *mc = g_MC;
    if (kc) *kc = g_KC;
    if (nc) *nc = g_NC;
}

static int is_trans(char c)
{
    c = (char)toupper((unsigned char)c);
    return c == 'T' || c == 'C';
}

static int valid_trans(char c)
{
    c = (char)toupper((unsigned char)c);
    return c == 'N' || c == 'T' || c == 'C' || c == 'R';
}

static int imax(int a, int b) { return a > b ? a : b; }
static int64_t min64(int64_t a, int64_t b) { return a < b ? a : b; }

/* ---- argument checks ---------------------------------------------------- */

int ulm_oracle_gemm_info(char transA, char transB, int m, int n, int k,
                         int ldA, int ldB, int ldC)
{
    int numRowsA = !is_trans(transA) ? m : k;
    int numRowsB = !is_trans(transB) ? k : n;
    if (!valid_trans(transA)) return 1;
    if (!valid_trans(transB)) return 2;
    if (m < 0) return 3;
    if (n < 0) return 4;
    if (k < 0) return 5;
    if (ldA < imax(1, numRowsA)) return 8;
    if (ldB < imax(1, numRowsB)) return 10;
    if (ldC < imax(1, m)) return 13;
    return 0;
}

int ulm_oracle_trsm_info(char side, char uplo, char transA, char diag,
                         int m, int n, int ldA, int ldB)
{
    int s = toupper((unsigned char)side), u = toupper((unsigned char)uplo);
    int d = toupper((unsigned char)diag);
    int numRowsA = (s == 'L') ? m : n;
    if (s != 'L' && s != 'R') return 1;
    if (u != 'L' && u != 'U') return 2;
    if (!valid_trans(transA)) return 3;
    if (d != 'U' && d != 'N') return 4;
    if (m < 0) return 5;
    if (n < 0) return 6;
    if (ldA < imax(1, numRowsA)) return 9;
    if (ldB < imax(1, m)) return 11;
    return 0;
}

int ulm_oracle_syrk_info(char uplo, char trans, int n, int k, int ldA, int ldC)
{
    int u = toupper((unsigned char)uplo);
    int numRowsA = is_trans(trans) ? k : n;
    if (u != 'L' && u != 'U') return 1;
    if (!valid_trans(trans)) return 2;
    if (n < 0) return 3;
    if (k < 0) return 4;
    if (ldA < imax(1, numRowsA)) return 7;
    if (ldC < imax(1, n)) return 10;
    return 0;
}

/* ---- helpers ------------------------------------------------------------ */

/* gescal, ulmblas/level1extensions/gescal.tcc:11-39 + level1/scal.tcc:15-23 */
static void gescal_d(int64_t m, int64_t n, double beta,
                     double *C, int64_t irC, int64_t icC)
{
    if (beta == 1.0 || m <= 0 || n <= 0) return;
    for (int64_t j = 0; j < n; ++j)
        for (int64_t i = 0; i < m; ++i) {
            double *c = &C[i * irC + j * icC];
            *c = (beta == 0.0) ? 0.0 : *c * beta;
        }
}

/* dense column-major copy of op(X): rows x cols, leading dimension = rows,
 * element (i,j) taken from X[i*ir + j*ic], widened to double               */
static double *densify_d(int64_t rows, int64_t cols,
                         const double *X, int64_t ir, int64_t ic)
{
    double *D = (double *)malloc(sizeof(double) * (size_t)(rows * cols + 1));
    for (int64_t j = 0; j < cols; ++j)
        for (int64_t i = 0; i < rows; ++i)
            D[i + j * rows] = X[i * ir + j * ic];
    return D;
}

static double *densify_s(int64_t rows, int64_t cols,
                         const float *X, int64_t ir, int64_t ic)
{
    double *D = (double *)malloc(sizeof(double) * (size_t)(rows * cols + 1));
    for (int64_t j = 0; j < cols; ++j)
        for (int64_t i = 0; i < rows; ++i)
            D[i + j * rows] = (double)X[i * ir + j * ic];   /* gepack.tcc:24 */
    return D;
}

enum { STRIP = 256 };

/* ab[0..len) = sum over l in [l0,l0+kc) of Ad(i0+i, l) * Bd(l, j), sequential,
 * product and sum rounded separately.                                       */
static void block_dot(int64_t len, int64_t kc,
                      const double *Acol0, int64_t ldAd,
                      const double *Bcol, double *ab)
{
    for (int64_t i = 0; i < len; ++i) ab[i] = 0.0;
    for (int64_t l = 0; l < kc; ++l) {
        const double b = Bcol[l];
        const double *a = Acol0 + l * ldAd;
#pragma omp simd
        for (int64_t i = 0; i < len; ++i) {
            double p = a[i] * b;
            ab[i] = ab[i] + p;
        }
    }
}

/* ---- gemm --------------------------------------------------------------- */

/* ulmBLAS::gemm, ulmblas/level3/gemm.tcc:16-87, on strided operands         */
static void gemm_d(int64_t m, int64_t n, int64_t k, double alpha,
                   const double *A, int64_t irA, int64_t icA,
                   const double *B, int64_t irB, int64_t icB,
                   double beta, double *C, int64_t irC, int64_t icC)
{
    if (m <= 0 || n <= 0) return;
    if (alpha == 0.0 || k == 0) {                       /* gemm.tcc:52-55 */
        gescal_d(m, n, beta, C, irC, icC);
        return;
    }
    double *Ad = densify_d(m, k, A, irA, icA);
    double *Bd = densify_d(k, n, B, irB, icB);
    double ab[STRIP];
    const int64_t KC = g_KC;
    for (int64_t l0 = 0; l0 < k; l0 += KC) {            /* gemm.tcc:63-65 */
        const int64_t kc = min64(KC, k - l0);
        const double beta_ = (l0 == 0) ? beta : 1.0;
        for (int64_t j = 0; j < n; ++j) {
            for (int64_t i0 = 0; i0 < m; i0 += STRIP) {
                const int64_t len = min64(STRIP, m - i0);
                block_dot(len, kc, Ad + i0 + l0 * m, m, Bd + l0 + j * k, ab);
                for (int64_t i = 0; i < len; ++i) {
                    double *c = &C[(i0 + i) * irC + j * icC];
                    double t = alpha * ab[i];
                    *c = (beta_ == 0.0) ? t : (beta_ * *c) + t;
                }
            }
        }
    }
    free(Ad);
    free(Bd);
}

void ulm_oracle_dgemm(char transA, char transB, int64_t m, int64_t n, int64_t k,
                      double alpha, const double *A, int64_t ldA,
                      const double *B, int64_t ldB,
                      double beta, double *C, int64_t ldC)
{
    /* stride dispatch of interfaces/blas/F77/gemm.cc:204-248 */
    const int tA = is_trans(transA), tB = is_trans(transB);
    gemm_d(m, n, k, alpha,
           A, tA ? ldA : 1, tA ? 1 : ldA,
           B, tB ? ldB : 1, tB ? 1 : ldB,
           beta, C, 1, ldC);
}

void ulm_oracle_sgemm(char transA, char transB, int64_t m, int64_t n, int64_t k,
                      float alpha_f, const float *A, int64_t ldA,
                      const float *B, int64_t ldB,
                      float beta_f, float *C, int64_t ldC)
{
    const int tA = is_trans(transA), tB = is_trans(transB);
    const double alpha = alpha_f, beta = beta_f;         /* gemm.cc:33,36 */
    if (m <= 0 || n <= 0) return;
    if (alpha == 0.0 || k == 0) {
        if (beta == 1.0) return;
        for (int64_t j = 0; j < n; ++j)
            for (int64_t i = 0; i < m; ++i) {
                float *c = &C[i + j * ldC];
                *c = (beta == 0.0) ? 0.0f : (float)((double)*c * beta);
            }
        return;
    }
    double *Ad = densify_s(m, k, A, tA ? ldA : 1, tA ? 1 : ldA);
    double *Bd = densify_s(k, n, B, tB ? ldB : 1, tB ? 1 : ldB);
    double ab[STRIP];
    const int64_t KC = g_KC;
    for (int64_t l0 = 0; l0 < k; l0 += KC) {
        const int64_t kc = min64(KC, k - l0);
        const double beta_ = (l0 == 0) ? beta : 1.0;
        for (int64_t j = 0; j < n; ++j) {
            for (int64_t i0 = 0; i0 < m; i0 += STRIP) {
                const int64_t len = min64(STRIP, m - i0);
                block_dot(len, kc, Ad + i0 + l0 * m, m, Bd + l0 + j * k, ab);
                for (int64_t i = 0; i < len; ++i) {
                    /* every tile takes the buffered micro-kernel because the
                     * type of C differs from the compute type
                     * (ukernel/ugemm.tcc:46-61 -> :17-38): C_ = alpha*ab in
                     * double; C *= beta and C += C_ each round to float.    */
                    float *c = &C[(i0 + i) + j * ldC];
                    double t = alpha * ab[i];
                    float s = *c;
                    if (beta_ == 0.0) s = 0.0f;
                    else if (beta_ != 1.0) s = (float)((double)s * beta_);
                    *c = (float)((double)s + t);
                }
            }
        }
    }
    free(Ad);
    free(Bd);
}

/* ---- trsm --------------------------------------------------------------- */

#define A_(i, j) A[(i) * irA + (j) * icA]
#define B_(i, j) B[(i) * irB + (j) * icB]

/* rows [r, r+len) of B, column j:  B = alpha_*B - sum_{c in [c0,c0+kc)} A(row,c)*B(c,j)
 * (mgemm / ugemm with alpha = -1, beta = alpha_; trlsm.tcc:84, mtrlsm.tcc:55-59) */
static void tr_update(int64_t r, int64_t len, int64_t c0, int64_t kc, double alpha_,
                      const double *A, int64_t irA, int64_t icA,
                      double *B, int64_t irB, int64_t icB, int64_t j)
{
    for (int64_t i = 0; i < len; ++i) {
        double ab = 0.0;
        for (int64_t l = 0; l < kc; ++l) {
            double p = A_(r + i, c0 + l) * B_(c0 + l, j);
            ab = ab + p;
        }
        double t = -1.0 * ab;
        B_(r + i, j) = (alpha_ * B_(r + i, j)) + t;
    }
}

/* ulmBLAS::trlsm, ulmblas/level3/trlsm.tcc:18-92: B <- alpha * L^{-1} B     */
static void trlsm_d(int64_t m, int64_t n, double alpha, int unit,
                    const double *A, int64_t irA, int64_t icA,
                    double *B, int64_t irB, int64_t icB)
{
    if (m <= 0 || n <= 0) return;
    if (alpha == 0.0) { gescal_d(m, n, 0.0, B, irB, icB); return; }
    const int64_t MC = g_MC;
    for (int64_t r0 = 0; r0 < m; r0 += MC) {
        const int64_t mc = min64(MC, m - r0);
        const double alpha_ = (r0 == 0) ? alpha : 1.0;
        /* diagonal block: mtrlsm, mkernel/mtrlsm.tcc:36-87 */
        for (int64_t p0 = 0; p0 < mc; p0 += MR) {
            const int64_t mr = min64(MR, mc - p0);
            double inv[MR];
            for (int64_t i = 0; i < mr; ++i)    /* pack/trlspack.tcc:43-44 */
                inv[i] = unit ? 1.0 : 1.0 / A_(r0 + p0 + i, r0 + p0 + i);
            for (int64_t j = 0; j < n; ++j) {
                tr_update(r0 + p0, mr, r0, p0, alpha_, A, irA, icA, B, irB, icB, j);
                /* utrlsm, ukernel/ref/utrlsm.tcc:30-38 */
                for (int64_t i = 0; i < mr; ++i) {
                    double x = B_(r0 + p0 + i, j) * inv[i];
                    B_(r0 + p0 + i, j) = x;
                    for (int64_t l = i + 1; l < mr; ++l) {
                        double p = A_(r0 + p0 + l, r0 + p0 + i) * x;
                        B_(r0 + p0 + l, j) = B_(r0 + p0 + l, j) - p;
                    }
                }
            }
        }
        /* trailing blocks: trlsm.tcc:77-86 */
        for (int64_t r1 = r0 + MC; r1 < m; r1 += MC) {
            const int64_t mc1 = min64(MC, m - r1);
            for (int64_t j = 0; j < n; ++j)
                tr_update(r1, mc1, r0, MC, alpha_, A, irA, icA, B, irB, icB, j);
        }
    }
}

/* ulmBLAS::trusm, ulmblas/level3/trusm.tcc:21-100: B <- alpha * U^{-1} B    */
static void trusm_d(int64_t m, int64_t n, double alpha, int unit,
                    const double *A, int64_t irA, int64_t icA,
                    double *B, int64_t irB, int64_t icB)
{
    if (m <= 0 || n <= 0) return;
    if (alpha == 0.0) { gescal_d(m, n, 0.0, B, irB, icB); return; }
    const int64_t MC = g_MC;
    const int64_t mb = (m + MC - 1) / MC;
    for (int64_t ib = mb - 1; ib >= 0; --ib) {
        const int64_t r0 = ib * MC;
        const int64_t mc = min64(MC, m - r0);
        const double alpha_ = (ib == mb - 1) ? alpha : 1.0;
        /* diagonal block, bottom panel first: mkernel/mtrusm.tcc:40-84 */
        const int64_t mp = (mc + MR - 1) / MR;
        for (int64_t p = mp - 1; p >= 0; --p) {
            const int64_t p0 = p * MR;
            const int64_t mr = min64(MR, mc - p0);
            const int64_t kc = mc - p0 - mr;
            double inv[MR];
            for (int64_t i = 0; i < mr; ++i)    /* pack/truspack.tcc:24-25 */
                inv[i] = unit ? 1.0 : 1.0 / A_(r0 + p0 + i, r0 + p0 + i);
            for (int64_t j = 0; j < n; ++j) {
                tr_update(r0 + p0, mr, r0 + p0 + mr, kc, alpha_,
                          A, irA, icA, B, irB, icB, j);
                /* utrusm, ukernel/ref/utrusm.tcc:30-39 */
                for (int64_t i = mr - 1; i >= 0; --i) {
                    double x = B_(r0 + p0 + i, j) * inv[i];
                    B_(r0 + p0 + i, j) = x;
                    for (int64_t l = 0; l < i; ++l) {
                        double pr = A_(r0 + p0 + l, r0 + p0 + i) * x;
                        B_(r0 + p0 + l, j) = B_(r0 + p0 + l, j) - pr;
                    }
                }
            }
        }
        /* blocks above: trusm.tcc:88-95 */
        for (int64_t l = 0; l < ib; ++l)
            for (int64_t j = 0; j < n; ++j)
                tr_update(l * MC, MC, r0, mc, alpha_, A, irA, icA, B, irB, icB, j);
    }
}

void ulm_oracle_dtrsm(char side, char uplo, char transA, char diag,
                      int64_t m, int64_t n, double alpha,
                      const double *A, int64_t ldA, double *B, int64_t ldB)
{
    const int left = toupper((unsigned char)side) == 'L';
    const int lower = toupper((unsigned char)uplo) == 'L';
    const int tA = is_trans(transA);
    const int unit = toupper((unsigned char)diag) == 'U';
    /* dispatch of interfaces/blas/F77/trsm.cc:183-227: a transposed triangle
     * swaps lower<->upper and the two strides; the right side solves the
     * transposed system on B^T.                                             */
    if (left) {
        if (lower == !tA)
            trlsm_d(m, n, alpha, unit, A, tA ? ldA : 1, tA ? 1 : ldA, B, 1, ldB);
        else
            trusm_d(m, n, alpha, unit, A, tA ? ldA : 1, tA ? 1 : ldA, B, 1, ldB);
    } else {
        if (lower == !tA)
            trusm_d(n, m, alpha, unit, A, tA ? 1 : ldA, tA ? ldA : 1, B, ldB, 1);
        else
            trlsm_d(n, m, alpha, unit, A, tA ? 1 : ldA, tA ? ldA : 1, B, ldB, 1);
    }
}

#undef A_
#undef B_

/* ---- syrk --------------------------------------------------------------- */

/* ulmBLAS::syurk / sylrk, ulmblas/level3/syurk.tcc:18-90, sylrk.tcc:18-89:
 * the `upper` (i<=j) or lower (i>=j) triangle of  C <- beta*C + alpha*A*A^T,
 * K blocked by MC (syurk.tcc:37,60).                                        */
static void syrk_d(int upper, int64_t n, int64_t k, double alpha,
                   const double *A, int64_t irA, int64_t icA,
                   double beta, double *C, int64_t irC, int64_t icC)
{
    if (n == 0 || ((alpha == 0.0 || k == 0) && beta == 1.0)) return;
    if (alpha == 0.0 || k == 0) {            /* truscal / trlscal: syurk.tcc:48-51 */
        for (int64_t j = 0; j < n; ++j) {
            int64_t ia = upper ? 0 : j, ie = upper ? j + 1 : n;
            for (int64_t i = ia; i < ie; ++i) {
                double *c = &C[i * irC + j * icC];
                *c = (beta == 0.0) ? 0.0 : *c * beta;
            }
        }
        return;
    }
    double *Ad = densify_d(n, k, A, irA, icA);     /* n x k */
    double *At = densify_d(k, n, A, icA, irA);     /* k x n = A^T */
    double ab[STRIP];
    const int64_t KC = g_MC;
    for (int64_t l0 = 0; l0 < k; l0 += KC) {
        const int64_t kc = min64(KC, k - l0);
        const double beta_ = (l0 == 0) ? beta : 1.0;
        for (int64_t j = 0; j < n; ++j) {
            int64_t ia = upper ? 0 : j, ie = upper ? j + 1 : n;
            for (int64_t i0 = ia; i0 < ie; i0 += STRIP) {
                const int64_t len = min64(STRIP, ie - i0);
                block_dot(len, kc, Ad + i0 + l0 * n, n, At + l0 + j * k, ab);
                for (int64_t i = 0; i < len; ++i) {
                    double *c = &C[(i0 + i) * irC + j * icC];
                    double t = alpha * ab[i];
                    *c = (beta_ == 0.0) ? t : (beta_ * *c) + t;
                }
            }
        }
    }
    free(Ad);
    free(At);
}

void ulm_oracle_dsyrk(char uplo, char trans, int64_t n, int64_t k,
                      double alpha, const double *A, int64_t ldA,
                      double beta, double *C, int64_t ldC)
{
    const int lower = toupper((unsigned char)uplo) == 'L';
    const int t = is_trans(trans);
    /* interfaces/blas/F77/syrk.cc:145-157: the transposed case runs the
     * opposite-triangle routine on the transposed views of A and C.         */
    if (!t)
        syrk_d(!lower, n, k, alpha, A, 1, ldA, beta, C, 1, ldC);
    else
        syrk_d(lower, n, k, alpha, A, ldA, 1, beta, C, ldC, 1);
}


/* ---- zgemm --------------------------------------------------------------- */

/* zgemm_ : interfaces/blas/F77/gemm.cc:381-510 -> ulmblas/level3/gemm.tcc:16-87 with
 * T = std::complex<double>.  The complex type has no SSE kernel (ukernel/sse/ugemm.h:12-15
 * covers double only), so every tile runs ukernel/ref/ugemm.tcc:10-67:
 *   - K is cut into blocks of KC = 192 (config/blocksize.h:41), beta on the first block;
 *   - AB += A*B per k with std::complex's product, i.e. four real products rounded
 *     separately, one subtraction and one addition, then two additions into AB;
 *   - C = 0 (beta == 0) or C *= beta, then C += AB (alpha == 1) or C += alpha*AB.
 * Conjugation happens while packing (pack/gepack.tcc:21-33,84-96): op(A), op(B) are
 * conjugated copies, which the dense split below reproduces by negating the imaginary
 * plane.  Matrices are interleaved (re, im) pairs; leading dimensions count complex
 * elements.                                                                          */
static int is_conj(char c)
{
    c = (char)toupper((unsigned char)c);
    return c == 'C' || c == 'R';
}

static void densify_z(int64_t rows, int64_t cols, const double *X, int64_t ir, int64_t ic,
                      int conj, double **re_out, double **im_out)
{
    double *re = (double *)malloc(sizeof(double) * (size_t)(rows * cols + 1));
    double *im = (double *)malloc(sizeof(double) * (size_t)(rows * cols + 1));
    for (int64_t j = 0; j < cols; ++j)
        for (int64_t i = 0; i < rows; ++i) {
            const double *x = &X[2 * (i * ir + j * ic)];
            re[i + j * rows] = x[0];
            im[i + j * rows] = conj ? -x[1] : x[1];
        }
    *re_out = re;
    *im_out = im;
}

void ulm_oracle_zgemm(char transA, char transB, int64_t m, int64_t n, int64_t k,
                      const double *alpha, const double *A, int64_t ldA,
                      const double *B, int64_t ldB,
                      const double *beta, double *C, int64_t ldC)
{
    const int tA = is_trans(transA), tB = is_trans(transB);
    const double ar = alpha[0], ai = alpha[1];
    if (m <= 0 || n <= 0) return;
    if ((ar == 0.0 && ai == 0.0) || k == 0) {            /* gemm.tcc:52-55 -> gescal */
        const double br = beta[0], bi = beta[1];
        if (br == 1.0 && bi == 0.0) return;
        for (int64_t j = 0; j < n; ++j)
            for (int64_t i = 0; i < m; ++i) {
                double *c = &C[2 * (i + j * ldC)];
                if (br == 0.0 && bi == 0.0) { c[0] = 0.0; c[1] = 0.0; }
                else {
                    const double cr = c[0], ci = c[1];
                    c[0] = cr * br - ci * bi;
                    c[1] = cr * bi + ci * br;
                }
            }
        return;
    }
    double *Ar, *Ai, *Br, *Bi;
    densify_z(m, k, A, tA ? ldA : 1, tA ? 1 : ldA, is_conj(transA), &Ar, &Ai);
    densify_z(k, n, B, tB ? ldB : 1, tB ? 1 : ldB, is_conj(transB), &Br, &Bi);
    double abr[STRIP], abi[STRIP];
    const int64_t KC = g_KC_z;
    const int alpha_one = (ar == 1.0 && ai == 0.0);
    for (int64_t l0 = 0; l0 < k; l0 += KC) {
        const int64_t kc = min64(KC, k - l0);
        const int first = (l0 == 0);
        const double br = first ? beta[0] : 1.0, bi = first ? beta[1] : 0.0;
        for (int64_t j = 0; j < n; ++j) {
            for (int64_t i0 = 0; i0 < m; i0 += STRIP) {
                const int64_t len = min64(STRIP, m - i0);
                for (int64_t i = 0; i < len; ++i) { abr[i] = 0.0; abi[i] = 0.0; }
                for (int64_t l = 0; l < kc; ++l) {
                    const double xr = Br[l0 + l + j * k], xi = Bi[l0 + l + j * k];
                    const double *pr = Ar + i0 + (l0 + l) * m, *pi = Ai + i0 + (l0 + l) * m;
#pragma omp simd
                    for (int64_t i = 0; i < len; ++i) {
                        const double t1 = pr[i] * xr, t2 = pi[i] * xi;
                        const double t3 = pr[i] * xi, t4 = pi[i] * xr;
                        abr[i] = abr[i] + (t1 - t2);
                        abi[i] = abi[i] + (t3 + t4);
                    }
                }
                for (int64_t i = 0; i < len; ++i) {
                    double *c = &C[2 * ((i0 + i) + j * ldC)];
                    double cr, ci;
                    if (br == 0.0 && bi == 0.0) { cr = 0.0; ci = 0.0; }
                    else {
                        const double c0 = c[0], c1 = c[1];
                        cr = c0 * br - c1 * bi;
                        ci = c0 * bi + c1 * br;
                    }
                    double tr = abr[i], ti = abi[i];
                    if (!alpha_one) {
                        tr = ar * abr[i] - ai * abi[i];
                        ti = ar * abi[i] + ai * abr[i];
                    }
                    c[0] = cr + tr;
                    c[1] = ci + ti;
                }
            }
        }
    }
    free(Ar); free(Ai); free(Br); free(Bi);
}
