/*
 * TEST INFRASTRUCTURE -- NOT PART OF THE PRODUCT.
 *
 * CPU restatement (plain C, single thread) of the arithmetic that ulmBLAS's
 * Level-3 GEMM path performs, written so that every output element sees the
 * same sequence of IEEE operations as the reference's SSE3 build does.  It is
 * only ever used as a checker by the tests, by the smoke test and by the
 * bench's CPU-baseline leg.  The product library never links or calls it.
 *
 * Parity pin: the restatement is compared bit-for-bit (GEMM, SYRK) and
 * element-for-element (TRSM) against the reference compiled from its own
 * sources (oracle/_ref/libulmref.so, built by oracle/Makefile) and against
 * fixtures produced by that build (tests/golden/).
 *
 * Citations are paths inside the ulmBLAS source tree.
 */
#ifndef ULM_ORACLE_H
#define ULM_ORACLE_H 1

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Cache-block sizes MC, KC, NC of ulmblas/config/blocksize.h:27-64
 * (double: 384, 384, 4096).  The reference's test builds shrink them to
 * 8/12/12 (test/F77/config/make.testcase01.inc); so can the oracle.       */
void ulm_oracle_set_blocks(int mc, int kc, int nc);
void ulm_oracle_get_blocks(int *mc, int *kc, int *nc);
/* KC of std::complex<double> (192, blocksize.h:41; test builds: the common KC) */
void ulm_oracle_set_blocks_z(int kc);

/* dgemm_ : interfaces/blas/F77/gemm.cc:132-249 -> ulmblas/level3/gemm.tcc:16-87 */
void ulm_oracle_dgemm(char transA, char transB, int64_t m, int64_t n, int64_t k,
                      double alpha, const double *A, int64_t ldA,
                      const double *B, int64_t ldB,
                      double beta, double *C, int64_t ldC);

/* sgemm_ : interfaces/blas/F77/gemm.cc:11-128.  alpha and beta are widened to
 * double (gemm.cc:33,36), so the product is accumulated in double and rounded
 * to float once per KC block (ulmblas/level3/ukernel/ugemm.tcc:15-61).     */
void ulm_oracle_sgemm(char transA, char transB, int64_t m, int64_t n, int64_t k,
                      float alpha, const float *A, int64_t ldA,
                      const float *B, int64_t ldB,
                      float beta, float *C, int64_t ldC);

/* zgemm_ : interfaces/blas/F77/gemm.cc:381-510.  Interleaved (re, im) doubles, leading
 * dimensions in complex elements, alpha and beta as {re, im}; trans characters N, T,
 * C (conjugate transpose) and R (conjugate, no transpose).                          */
void ulm_oracle_zgemm(char transA, char transB, int64_t m, int64_t n, int64_t k,
                      const double *alpha, const double *A, int64_t ldA,
                      const double *B, int64_t ldB,
                      const double *beta, double *C, int64_t ldC);

/* dtrsm_ : interfaces/blas/F77/trsm.cc:121-228 -> ulmblas/level3/trlsm.tcc,
 * trusm.tcc.  All side/uplo/trans/diag combinations.                        */
void ulm_oracle_dtrsm(char side, char uplo, char transA, char diag,
                      int64_t m, int64_t n, double alpha,
                      const double *A, int64_t ldA, double *B, int64_t ldB);

/* dsyrk_ : interfaces/blas/F77/syrk.cc:87-158 -> ulmblas/level3/syurk.tcc,
 * sylrk.tcc.                                                               */
void ulm_oracle_dsyrk(char uplo, char trans, int64_t n, int64_t k,
                      double alpha, const double *A, int64_t ldA,
                      double beta, double *C, int64_t ldC);

/* Argument checks of the three shims: returns the 1-based index of the first
 * bad argument (what the reference hands to xerbla_), 0 if none.
 * gemm.cc:169-199, trsm.cc:154-178, syrk.cc:118-140.                        */
int ulm_oracle_gemm_info(char transA, char transB, int m, int n, int k,
                         int ldA, int ldB, int ldC);
int ulm_oracle_trsm_info(char side, char uplo, char transA, char diag,
                         int m, int n, int ldA, int ldB);
int ulm_oracle_syrk_info(char uplo, char trans, int n, int k, int ldA, int ldC);

#ifdef __cplusplus
}
#endif
#endif
