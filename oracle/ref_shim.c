/*
 * TEST INFRASTRUCTURE -- NOT PART OF THE PRODUCT.
 *
 * Calls into the compiled reference (oracle/_ref/libulmref*.so) through a
 * function pointer after zero-filling the stack region the callee is about to
 * use.  Reason: the reference's buffered micro-kernel hands an uninitialised
 * stack array C_[MR*NR] with beta = 0 to its SSE kernel, which still computes
 * 0*C_ + alpha*AB (ulmblas/level3/ukernel/ugemm.tcc:33-35,
 * ukernel/sse/ugemm.tcc:305-306).  If the stale stack bytes happen to be a
 * NaN/Inf bit pattern the affected edge-tile (or, for sgemm_, any-tile)
 * element comes out NaN.  Starting from a clean stack removes the dependence
 * on whatever the host interpreter left there.
 */
#include <string.h>

typedef void (*gemm_fn)(const char *, const char *, const int *, const int *, const int *,
                        const void *, const void *, const int *, const void *, const int *,
                        const void *, void *, const int *);
typedef void (*trsm_fn)(const char *, const char *, const char *, const char *,
                        const int *, const int *, const void *, const void *, const int *,
                        void *, const int *);
typedef void (*syrk_fn)(const char *, const char *, const int *, const int *,
                        const void *, const void *, const int *, const void *, void *,
                        const int *);

static void __attribute__((noinline)) scrub_stack(void)
{
    volatile char buf[1 << 18];
    memset((void *)buf, 0, sizeof buf);
    __asm__ volatile("" ::: "memory");
}

void ulm_shim_gemm(gemm_fn fn, const char *ta, const char *tb, const int *m, const int *n,
                   const int *k, const void *alpha, const void *A, const int *lda,
                   const void *B, const int *ldb, const void *beta, void *C, const int *ldc)
{
    scrub_stack();
    fn(ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc);
}

void ulm_shim_trsm(trsm_fn fn, const char *side, const char *uplo, const char *ta,
                   const char *diag, const int *m, const int *n, const void *alpha,
                   const void *A, const int *lda, void *B, const int *ldb)
{
    scrub_stack();
    fn(side, uplo, ta, diag, m, n, alpha, A, lda, B, ldb);
}

void ulm_shim_syrk(syrk_fn fn, const char *uplo, const char *trans, const int *n,
                   const int *k, const void *alpha, const void *A, const int *lda,
                   const void *beta, void *C, const int *ldc)
{
    scrub_stack();
    fn(uplo, trans, n, k, alpha, A, lda, beta, C, ldc);
}
