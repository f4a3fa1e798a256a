/*
 * ulmblas_b200 -- C ABI of libulmblas_b200.so
 *
 * Two layers, both plain C (pointers and sizes only):
 *
 *  1. The BLAS entry points of ulmBLAS's Level-3 GEMM path, same symbols, same
 *     argument meaning, same xerbla convention as the reference shims.  A
 *     program linked against the reference's libf77blas / libcblas for these
 *     routines links against this library unchanged.  Operand pointers may be
 *     host pointers (staged through the device) or device pointers (used in
 *     place); the call returns when the result is visible to the caller.
 *
 *  2. The device ABI behind them (ulmb200_*): operands already resident in
 *     device memory, 64-bit sizes, an explicit stream, an int status.
 *
 * Matrices are column-major with a leading dimension, as in the reference.
 * "Reference" citations are paths inside the ulmBLAS source tree.
 */
#ifndef ULMBLAS_B200_H
#define ULMBLAS_B200_H 1

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------ */
/* status codes returned by every ulmb200_* function                          */
/* ------------------------------------------------------------------------ */
enum {
    ULMB200_OK            = 0,
    ULMB200_BAD_ARGUMENT  = 1,   /* negative size, ld too small, bad flag      */
    ULMB200_CUDA_ERROR    = 2,   /* a CUDA runtime / driver call failed        */
    ULMB200_NO_DEVICE     = 3,   /* no usable sm_100 device                    */
    ULMB200_KERNEL_FAULT  = 4,   /* a kernel's bounded wait ran out            */
    ULMB200_TOO_LARGE     = 5    /* request exceeds a stated fixed limit       */
};

/* Status of the most recent ulmb200_* / BLAS call made by this thread.       */
int         ulmb200_last_status(void);
const char *ulmb200_status_string(int status);

/* ------------------------------------------------------------------------ */
/* 1. BLAS entry points (Fortran ABI: every argument by reference, 32-bit int) */
/* ------------------------------------------------------------------------ */

/* replaces F77BLAS(dgemm), interfaces/blas/F77/gemm.cc:132-249
 * xerbla_ codes {1,2,3,4,5,8,10,13}, gemm.cc:169-199                         */
void dgemm_(const char *transA, const char *transB,
            const int *m, const int *n, const int *k,
            const double *alpha, const double *A, const int *ldA,
            const double *B, const int *ldB,
            const double *beta, double *C, const int *ldC);

/* replaces F77BLAS(sgemm), interfaces/blas/F77/gemm.cc:11-128               */
void sgemm_(const char *transA, const char *transB,
            const int *m, const int *n, const int *k,
            const float *alpha, const float *A, const int *ldA,
            const float *B, const int *ldB,
            const float *beta, float *C, const int *ldC);

/* replaces F77BLAS(dtrsm), interfaces/blas/F77/trsm.cc:121-228
 * xerbla_ codes {1,2,3,4,5,6,9,11}, trsm.cc:154-178                          */
void dtrsm_(const char *side, const char *upLo, const char *transA, const char *diag,
            const int *m, const int *n, const double *alpha,
            const double *A, const int *ldA, double *B, const int *ldB);

/* replaces F77BLAS(dsyrk), interfaces/blas/F77/syrk.cc:87-158
 * xerbla_ codes {1,2,3,4,7,10}, syrk.cc:118-140                              */
void dsyrk_(const char *upLo, const char *trans, const int *n, const int *k,
            const double *alpha, const double *A, const int *ldA,
            const double *beta, double *C, const int *ldC);

/* replaces F77BLAS(dsymm), interfaces/blas/F77/symm.cc:87-150; xerbla_ codes {1,2,3,4,7,9,12} */
void dsymm_(const char *side, const char *upLo, const int *m, const int *n,
            const double *alpha, const double *A, const int *ldA,
            const double *B, const int *ldB, const double *beta, double *C, const int *ldC);

/* replaces F77BLAS(dtrmm), interfaces/blas/F77/trmm.cc:123-230; codes {1,2,3,4,5,6,9,11}    */
void dtrmm_(const char *side, const char *upLo, const char *transA, const char *diag,
            const int *m, const int *n, const double *alpha,
            const double *A, const int *ldA, double *B, const int *ldB);

/* replaces F77BLAS(dsyr2k), interfaces/blas/F77/syr2k.cc:92-170; codes {1,2,3,4,7,9,12}     */
void dsyr2k_(const char *upLo, const char *trans, const int *n, const int *k,
             const double *alpha, const double *A, const int *ldA,
             const double *B, const int *ldB, const double *beta, double *C, const int *ldC);

/* replace F77BLAS(strsm) / F77BLAS(ssyrk), interfaces/blas/F77/trsm.cc, syrk.cc: float operands,
 * arithmetic in double as in the reference (it widens alpha/beta to double there)               */
void strsm_(const char *side, const char *upLo, const char *transA, const char *diag,
            const int *m, const int *n, const float *alpha,
            const float *A, const int *ldA, float *B, const int *ldB);
void ssyrk_(const char *upLo, const char *trans, const int *n, const int *k,
            const float *alpha, const float *A, const int *ldA,
            const float *beta, float *C, const int *ldC);

/* replaces F77BLAS(zgemm), interfaces/blas/F77/gemm.cc:381-510: complex double, matrices as
 * interleaved (re, im) pairs, leading dimensions in complex elements, alpha and beta as
 * pointers to {re, im}.  trans: 'N', 'T', 'C' (conjugate transpose), 'R' (conjugate only,
 * gemm.cc:401-402).  xerbla_ codes as dgemm_, name "ZGEMM ".                                    */
void zgemm_(const char *transA, const char *transB,
            const int *m, const int *n, const int *k,
            const double *alpha, const double *A, const int *ldA,
            const double *B, const int *ldB,
            const double *beta, double *C, const int *ldC);

/* replaces F77BLAS(xerbla), interfaces/blas/F77/xerbla.cc:6-10.  Weak symbol:
 * a test harness may supply its own, exactly as the Netlib testers do.       */
void xerbla_(const char rout[6], const int *info);

/* ------------------------------------------------------------------------ */
/*    CBLAS entry points (interfaces/blas/C/cblas.h.in of the reference)      */
/* ------------------------------------------------------------------------ */
#ifndef ULMBLAS_B200_NO_CBLAS_ENUMS
enum CBLAS_ORDER     { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113,
                       AtlasConj = 114 };
enum CBLAS_UPLO      { CblasUpper = 121, CblasLower = 122 };
enum CBLAS_DIAG      { CblasNonUnit = 131, CblasUnit = 132 };
enum CBLAS_SIDE      { CblasLeft = 141, CblasRight = 142 };
#endif

/* replaces CBLAS(dgemm), interfaces/blas/C/gemm.cc:392-485 (row-major by
 * operand swap, :478-484; cblas_xerbla codes :426-466)                       */
void cblas_dgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE transA,
                 enum CBLAS_TRANSPOSE transB, int m, int n, int k,
                 double alpha, const double *A, int ldA, const double *B, int ldB,
                 double beta, double *C, int ldC);
/* replaces CBLAS(sgemm), interfaces/blas/C/gemm.cc:296-389                   */
void cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE transA,
                 enum CBLAS_TRANSPOSE transB, int m, int n, int k,
                 float alpha, const float *A, int ldA, const float *B, int ldB,
                 float beta, float *C, int ldC);
/* replaces CBLAS(dtrsm), interfaces/blas/C/trsm.cc                           */
void cblas_dtrsm(enum CBLAS_ORDER order, enum CBLAS_SIDE side, enum CBLAS_UPLO upLo,
                 enum CBLAS_TRANSPOSE transA, enum CBLAS_DIAG diag, int m, int n,
                 double alpha, const double *A, int ldA, double *B, int ldB);
/* replaces CBLAS(dsyrk), interfaces/blas/C/syrk.cc                           */
void cblas_dsyrk(enum CBLAS_ORDER order, enum CBLAS_UPLO upLo,
                 enum CBLAS_TRANSPOSE trans, int n, int k,
                 double alpha, const double *A, int ldA, double beta, double *C, int ldC);

/* replaces CBLAS(strsm), interfaces/blas/C/trsm.cc:311-384, and CBLAS(ssyrk), syrk.cc:146-203     */
void cblas_strsm(enum CBLAS_ORDER order, enum CBLAS_SIDE side, enum CBLAS_UPLO upLo,
                 enum CBLAS_TRANSPOSE transA, enum CBLAS_DIAG diag, int m, int n,
                 float alpha, const float *A, int ldA, float *B, int ldB);
void cblas_ssyrk(enum CBLAS_ORDER order, enum CBLAS_UPLO upLo,
                 enum CBLAS_TRANSPOSE trans, int n, int k,
                 float alpha, const float *A, int ldA, float beta, float *C, int ldC);

/* column-major-only twins, ULMBLAS(dgemm) interfaces/blas/C/gemm.cc:76-138 ...*/
void ulmblas_dgemm(enum CBLAS_TRANSPOSE transA, enum CBLAS_TRANSPOSE transB,
                   int m, int n, int k, double alpha, const double *A, int ldA,
                   const double *B, int ldB, double beta, double *C, int ldC);
void ulmblas_sgemm(enum CBLAS_TRANSPOSE transA, enum CBLAS_TRANSPOSE transB,
                   int m, int n, int k, float alpha, const float *A, int ldA,
                   const float *B, int ldB, float beta, float *C, int ldC);
void ulmblas_dtrsm(enum CBLAS_SIDE side, enum CBLAS_UPLO upLo,
                   enum CBLAS_TRANSPOSE transA, enum CBLAS_DIAG diag, int m, int n,
                   double alpha, const double *A, int ldA, double *B, int ldB);
void ulmblas_dsyrk(enum CBLAS_UPLO upLo, enum CBLAS_TRANSPOSE trans, int n, int k,
                   double alpha, const double *A, int ldA, double beta, double *C, int ldC);
/* ULMBLAS(strsm) interfaces/blas/C/trsm.cc:12-80, ULMBLAS(ssyrk) syrk.cc:11-39 */
void ulmblas_strsm(enum CBLAS_SIDE side, enum CBLAS_UPLO upLo,
                   enum CBLAS_TRANSPOSE transA, enum CBLAS_DIAG diag, int m, int n,
                   float alpha, const float *A, int ldA, float *B, int ldB);
void ulmblas_ssyrk(enum CBLAS_UPLO upLo, enum CBLAS_TRANSPOSE trans, int n, int k,
                   float alpha, const float *A, int ldA, float beta, float *C, int ldC);

/* replace CBLAS(zgemm) and ULMBLAS(zgemm), interfaces/blas/C/gemm.cc:584-677, :219-292;
 * AtlasConj = conjugate without transposing                                            */
void cblas_zgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE transA, enum CBLAS_TRANSPOSE transB,
                 int m, int n, int k, const double *alpha, const double *A, int ldA,
                 const double *B, int ldB, const double *beta, double *C, int ldC);
void ulmblas_zgemm(enum CBLAS_TRANSPOSE transA, enum CBLAS_TRANSPOSE transB,
                   int m, int n, int k, const double *alpha, const double *A, int ldA,
                   const double *B, int ldB, const double *beta, double *C, int ldC);

/* replace CBLAS(dsymm) / CBLAS(dtrmm) / CBLAS(dsyr2k) and their ULMBLAS() twins,
 * interfaces/blas/C/symm.cc, trmm.cc, syr2k.cc                                */
void cblas_dsymm(enum CBLAS_ORDER order, enum CBLAS_SIDE side, enum CBLAS_UPLO upLo, int m, int n,
                 double alpha, const double *A, int ldA, const double *B, int ldB,
                 double beta, double *C, int ldC);
void cblas_dtrmm(enum CBLAS_ORDER order, enum CBLAS_SIDE side, enum CBLAS_UPLO upLo,
                 enum CBLAS_TRANSPOSE transA, enum CBLAS_DIAG diag, int m, int n,
                 double alpha, const double *A, int ldA, double *B, int ldB);
void cblas_dsyr2k(enum CBLAS_ORDER order, enum CBLAS_UPLO upLo, enum CBLAS_TRANSPOSE trans,
                  int n, int k, double alpha, const double *A, int ldA,
                  const double *B, int ldB, double beta, double *C, int ldC);
void ulmblas_dsymm(enum CBLAS_SIDE side, enum CBLAS_UPLO upLo, int m, int n, double alpha,
                   const double *A, int ldA, const double *B, int ldB, double beta, double *C, int ldC);
void ulmblas_dtrmm(enum CBLAS_SIDE side, enum CBLAS_UPLO upLo, enum CBLAS_TRANSPOSE transA,
                   enum CBLAS_DIAG diag, int m, int n, double alpha,
                   const double *A, int ldA, double *B, int ldB);
void ulmblas_dsyr2k(enum CBLAS_UPLO upLo, enum CBLAS_TRANSPOSE trans, int n, int k, double alpha,
                    const double *A, int ldA, const double *B, int ldB, double beta, double *C, int ldC);

/* replaces ULMLAPACK(dgetrf), interfaces/lapack/C/getrf.cc:6-19 (blocked LU with partial
 * pivoting, ulmblas/lapack/getrf.tcc:30-73): the L and U factors overwrite A, piv[i] = 0-based row exchanged
 * with row i, returns the 1-based index of the first zero pivot or 0.  CblasColMajor only
 * (CblasRowMajor returns -1; the reference's row-major mode is consistent only for m == n).   */
int ulmblas_dgetrf(enum CBLAS_ORDER order, int m, int n, double *A, int ldA, int *piv);
/* replaces ULMLAPACK(dlaswp), interfaces/lapack/C/laswp.cc (ulmblas/lapack/laswp.tcc): exchange rows
 * i = k1..k2-1 of the n columns of A with rows piv[i*incPiv] (0-based; piv is host memory).   */
void ulmblas_dlaswp(int n, double *A, int ldA, int k1, int k2, int *piv, int incPiv);

/* replace CBLAS(xerbla) and ULMBLAS(xerbla), interfaces/blas/C/xerbla.cc:7-17 (both weak) */
void cblas_xerbla(int info, const char *rout, const char *form, ...);
void ulmblas_xerbla(int info, const char *rout, const char *form, ...);
/* interfaces/blas/C/cblas_globals.cc:3-4 (the Netlib C testers read these)   */
extern int CBLAS_CallFromC;
extern int RowMajorStrg;

/* ------------------------------------------------------------------------ */
/* 2. Device ABI: operands in device memory, work queued on `stream`          */
/*    (a cudaStream_t passed as void*, NULL = default stream), asynchronous.  */
/*    transX: 0 = as stored, 1 = transposed.                                  */
/* ------------------------------------------------------------------------ */

/* C <- alpha*op(A)*op(B) + beta*C on the FP64 tensor-core (DMMA) path.
 * Replaces ulmBLAS::gemm + gepack_A/B + mgemm + ugemm<double>
 * (ulmblas/level3/gemm.tcc:16-87, pack/gepack.tcc, mkernel/mgemm.tcc,
 * ukernel/sse/ugemm.tcc).                                                    */
int ulmb200_dgemm(void *stream, int transA, int transB,
                  int64_t m, int64_t n, int64_t k, double alpha,
                  const double *dA, int64_t ldA, const double *dB, int64_t ldB,
                  double beta, double *dC, int64_t ldC);

/* Complex double GEMM on the same tensor-core path: the operands are split into real and
 * imaginary planes (work memory: 2(mk + kn + mn) doubles, cached per device), four real
 * products follow, one pass folds alpha, beta and the result into C.  transX as above,
 * conjX: 1 = conjugate op(X).  Replaces ulmBLAS::gemm<std::complex<double>>
 * (ulmblas/level3/gemm.tcc:16-87 with conjugating pack, pack/gepack.tcc:21-33).        */
int ulmb200_zgemm(void *stream, int transA, int conjA, int transB, int conjB,
                  int64_t m, int64_t n, int64_t k, const double *alpha,
                  const double *dA, int64_t ldA, const double *dB, int64_t ldB,
                  const double *beta, double *dC, int64_t ldC);

/* SGEMM.  mode 0: FP32 FMA pipes; mode 1: opt-in 3xTF32 on tcgen05 tensor
 * cores with FP32 accumulation in tensor memory.  Replaces the float
 * instantiation of the same reference path.                                  */
enum { ULMB200_SGEMM_FP32 = 0, ULMB200_SGEMM_3XTF32 = 1 };
int ulmb200_sgemm(void *stream, int mode, int transA, int transB,
                  int64_t m, int64_t n, int64_t k, float alpha,
                  const float *dA, int64_t ldA, const float *dB, int64_t ldB,
                  float beta, float *dC, int64_t ldC);

/* B <- alpha * op(A)^-1 * B (left) or alpha * B * op(A)^-1 (right).
 * side 0 = left, 1 = right; lower 1 = lower triangle; unit 1 = unit diagonal.
 * Replaces ulmBLAS::trlsm / trusm (ulmblas/level3/trlsm.tcc, trusm.tcc).      */
int ulmb200_dtrsm(void *stream, int side, int lower, int transA, int unit,
                  int64_t m, int64_t n, double alpha,
                  const double *dA, int64_t ldA, double *dB, int64_t ldB);

/* Same operation and arguments as ulmb200_dtrsm, for callers that are not allowed to
 * allocate device memory (a latency-critical loop, a plug-in with a fixed memory budget,
 * a process whose device memory is fully committed elsewhere).  It has no counterpart in
 * the reference.  The solver's work areas live in a fixed array inside the library image
 * (about 6.3 MB on every GPU that loads the library, until exit) instead of the growing
 * cache ulmb200_dtrsm uses; no cudaMalloc/cudaFree or allocating routine is called.
 * Limits: triangle at most 2048 x 2048, the other dimension of B at most 4096; larger
 * requests return ULMB200_TOO_LARGE and launch nothing.  All calls on a GPU share the one
 * array, so calls that overlap in time on the same GPU race -- serialise them.  The first
 * call on each device resolves the array's device address and sets kernel attributes; make
 * that call before starting any stream capture.                                         */
int ulmb200_dtrsm_noalloc(void *stream, int side, int lower, int transA, int unit,
                          int64_t m, int64_t n, double alpha,
                          const double *dA, int64_t ldA, double *dB, int64_t ldB);

/* `lower`-or-upper triangle of C <- alpha*op(A)*op(A)^T + beta*C.
 * Replaces ulmBLAS::syurk / sylrk (ulmblas/level3/syurk.tcc, sylrk.tcc).      */
int ulmb200_dsyrk(void *stream, int lower, int trans, int64_t n, int64_t k,
                  double alpha, const double *dA, int64_t ldA,
                  double beta, double *dC, int64_t ldC);

/* The other gemm clients of the reference's Level 3 (same conventions as above).
 * ulmb200_dsymm  replaces ulmBLAS::sylmm / syumm   (ulmblas/level3/sylmm.tcc, syumm.tcc)
 * ulmb200_dtrmm  replaces ulmBLAS::trlmm / trumm   (ulmblas/level3/trlmm.tcc, trumm.tcc)
 * ulmb200_dsyr2k replaces ulmBLAS::sylr2k / syur2k (ulmblas/level3/sylr2k.tcc, syur2k.tcc)  */
int ulmb200_dsymm(void *stream, int side, int lower, int64_t m, int64_t n, double alpha,
                  const double *dA, int64_t ldA, const double *dB, int64_t ldB,
                  double beta, double *dC, int64_t ldC);
int ulmb200_dtrmm(void *stream, int side, int lower, int transA, int unit,
                  int64_t m, int64_t n, double alpha,
                  const double *dA, int64_t ldA, double *dB, int64_t ldB);
int ulmb200_dsyr2k(void *stream, int lower, int trans, int64_t n, int64_t k, double alpha,
                   const double *dA, int64_t ldA, const double *dB, int64_t ldB,
                   double beta, double *dC, int64_t ldC);

/* Blocked LU on device operands; d_piv (min(m,n) ints) and d_info (1 int) are device
 * pointers written asynchronously.  Replaces ulmBLAS::getrf / getf2 / laswp.                */
int ulmb200_dgetrf(void *stream, int64_t m, int64_t n, double *dA, int64_t ldA, int *d_piv, int *d_info);

/* Single-precision SYRK / TRSM on device operands: widened to FP64 scratch, computed by the FP64
 * kernels, rounded once (the reference's ssyrk_/strsm_ also compute in double).                  */
int ulmb200_ssyrk(void *stream, int lower, int trans, int64_t n, int64_t k, float alpha,
                  const float *dA, int64_t ldA, float beta, float *dC, int64_t ldC);
int ulmb200_strsm(void *stream, int side, int lower, int transA, int unit,
                  int64_t m, int64_t n, float alpha,
                  const float *dA, int64_t ldA, float *dB, int64_t ldB);

/* ------------------------------------------------------------------------ */
/* 3. One product over the GPUs of a box: C split by column blocks            */
/* ------------------------------------------------------------------------ */
/* One process per GPU; every rank makes the same calls in the same order.  Rank r owns columns
 * [j0, j1) of B and C (ulmb200_mg_column_block: near-equal blocks starting on multiples of 128);
 * A starts on the root and reaches the other ranks by NCCL broadcast in K panels, each panel's
 * product queued behind its arrival.  There is no reduction: columns of C are independent
 * (the reference walks C by column blocks in its outermost loop, ulmblas/level3/gemm.tcc:60; it
 * has no multi-device path of its own).  NCCL is looked up at run time (ULMB200_NCCL_LIB, else a
 * libnccl.so.2 already in the process, else the system's); one GPU needs none.
 *
 * Set-up: rank 0 calls ulmb200_mg_unique_id and hands the 128 bytes to the other ranks by any
 * means (MPI_Bcast, a file, a socket); every rank, with its device current, calls ulmb200_mg_init.  */
int ulmb200_mg_unique_id(char id[128]);
int ulmb200_mg_init(const char id[128], int rank, int world, void **handle);   /* id may be NULL when world == 1 */
int ulmb200_mg_finalize(void *handle);
int ulmb200_mg_column_block(int64_t n, int world, int rank, int64_t *j0, int64_t *j1);

/* Device-resident operands.  dA: m x k with ldA == m on every rank; holds A on `root`, receives it
 * elsewhere.  dB_block / dC_block: this rank's column blocks (k x nr, m x nr).  Asynchronous: the
 * work is ordered after what `stream` holds at the call and `stream` continues after it.          */
int ulmb200_mg_dgemm(void *handle, void *stream, int64_t m, int64_t n, int64_t k, double alpha,
                     double *dA, int64_t ldA, const double *dB_block, int64_t ldB,
                     double beta, double *dC_block, int64_t ldC, int root);

/* Host-resident operands (page-locked for the copies to overlap): hA is all of A, required on
 * `root`; hB_block / hC_block are this rank's column blocks; dA, dB_block, dC_block are device
 * buffers of the shapes above (dA with leading dimension m).  A travels host -> device panel by
 * panel ahead of its broadcast, the block of B row range by row range with it, and the block of C
 * returns in column pieces while the last panel is still being multiplied.  every_rank_has_a != 0
 * promises that every rank passed an hA it can read (a shared mapping, a copy): each rank then
 * brings its share of every panel over its own PCIe link and an all-gather completes the panels,
 * instead of the root pushing all of A through one link.                                            */
int ulmb200_mg_dgemm_host(void *handle, void *stream, int64_t m, int64_t n, int64_t k, double alpha,
                          const double *hA, int64_t ldhA, const double *hB_block, int64_t ldhB,
                          double beta, double *hC_block, int64_t ldhC,
                          double *dA, double *dB_block, int64_t lddB, double *dC_block, int64_t lddC,
                          int root, int every_rank_has_a);

/* Host-side wait for everything the communicator has queued, at most timeout_ms (negative: no
 * limit), watching NCCL's asynchronous error state; on an error or a timeout the communicator is
 * aborted and ULMB200_CUDA_ERROR returned (the handle is then only good for ulmb200_mg_finalize). */
int ulmb200_mg_wait(void *handle, int timeout_ms);

/* The K-panel plan as a function of sizes and rates (no device needed): widths[p] columns of A per
 * panel, reserve[p] = 1 where that panel's product leaves a few SMs to the transport.  A short first
 * panel, a second one just long enough for the rest of A to arrive behind it, one last panel with
 * the remaining K on the whole GPU.  Returns the number of panels (-1: bad argument).               */
int ulmb200_mg_plan_panels(int64_t m, int64_t n_block, int64_t k, int world, int64_t first_panel,
                           double transport_gbs, double gemm_tflops, int64_t *widths, int *reserve, int cap);
/* Plan of the communicator's last call, and the transport rates (GB/s of A reaching the ranks:
 * device-resident calls, host calls; 0 = nothing measured yet).  Every rank measures; on the second
 * and on the third call of a kind the ranks agree on the smallest of their measurements of the call before
 * (their plans must be identical) with one tiny all-reduce and a host-side wait for that call's transfers,
 * and keep the last value afterwards.                                                                  */
int ulmb200_mg_last_plan(void *handle, int64_t *widths, int *reserve, int cap,
                         double *device_rate_gbs, double *host_rate_gbs);
/* Overrides the rates the next plan uses (<= 0 leaves one as it is); every rank must pass the same.  */
int ulmb200_mg_set_rates(void *handle, double transport_gbs, double host_gbs, double gemm_tflops);
/* Per-product device times of the last ulmb200_mg_dgemm call (CUDA events on the compute stream),
 * recorded while profiling is switched on; read after the call has finished.                       */
int ulmb200_mg_profile(void *handle, int on);
int ulmb200_mg_last_gemm_ms(void *handle, double *ms, int cap);
/* When each of those products started, in ms after the call's first transfer was queued (device-resident
 * call on more than one rank; shows a product waiting for its panel).                                   */
int ulmb200_mg_last_gemm_start_ms(void *handle, double *ms, int cap);
/* Time between the end of the last product of the call before the last one and the moment the last call's
 * first transfer was queued on the device (both calls device-resident, profiled, more than one rank): what a
 * rank spends between two back-to-back calls, mostly waiting for the slowest rank.  0 on success, -1 when
 * there are no two such calls.                                                                            */
int ulmb200_mg_last_step_gap_ms(void *handle, double *ms);

/* The persistent DGEMM grid normally takes every SM.  A caller that runs a collective
 * (e.g. the NCCL broadcast of the next A panel) beside it can ask the following DGEMM
 * launches to leave `sms` SMs free so that the collective's kernels are never starved;
 * 0 restores the default.  Process-wide.                                               */
void ulmb200_set_sm_reserve(int sms);

/* Number of kernels this library has launched in this process so far.        */
int64_t ulmb200_launch_count(void);

/* Host-pointer staging used by the BLAS entry points.  0 (the default): pageable caller
 * buffers are copied as they are (buffers the caller has page-locked itself are always used
 * in place, with overlapped copies).  1: pageable buffers of 1 MB and more are page-locked
 * with cudaHostRegister for the duration of the call, which lets the copies overlap the
 * arithmetic at the price of the registration itself.  Process-wide.                       */
void ulmb200_set_pin_host(int on);

/* Waits for `stream`, then reports whether any kernel of this library gave up on one of its
 * bounded waits since the last check on the current device (ULMB200_KERNEL_FAULT, and the
 * record is cleared) or not (ULMB200_OK).  The blocking BLAS entry points check by
 * themselves; callers of the asynchronous ulmb200_* functions use this.  Allocates nothing,
 * so it also serves ulmb200_dtrsm_noalloc.                                                  */
int ulmb200_check_device_error(void *stream);

/* Cached device work memory of the current device (staging buffers of host-pointer calls, the
 * solvers' work areas): its size, and a call that waits for the device and gives all of it
 * back.  ULMB200_WORKSPACE_CAP_MB in the environment bounds the cache; a request beyond the
 * bound fails with ULMB200_CUDA_ERROR instead of allocating.                               */
int64_t ulmb200_workspace_bytes(void);
int     ulmb200_release_workspace(void);

/* Number of device allocations (cudaMalloc) the library has made in this process.          */
int64_t ulmb200_alloc_count(void);

/* The library reads its environment variables (ULMB200_TRACE, ULMB200_SGEMM,
 * ULMB200_WORKSPACE_CAP_MB and the ULMB200_DGEMM_* test hooks) once, at first use; this reads
 * them again.                                                                              */
void ulmb200_reload_env(void);

#ifdef __cplusplus
}
#endif
#endif /* ULMBLAS_B200_H */
