/*
 * ulmb200_benchsupport -- C ABI of libulmb200_benchsupport.so
 *
 * Helpers for benchmarks and tests of libulmblas_b200.so, kept out of the product library:
 * the deterministic matrix generator, register-only throughput probes that give the
 * roofline denominators, and a self test of the failure path.  The library is built from
 * the same source tree and depends on libulmblas_b200.so (same status codes, same launch
 * counter, same device error word).
 */
#ifndef ULMB200_BENCHSUPPORT_H
#define ULMB200_BENCHSUPPORT_H 1

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Deterministic test/bench matrices: element (i,j) of matrix `mat` under
 * `seed` is a pure function of (seed, mat, i, j), identical on host and device,
 * uniform in [-1,1).  Fills the rows x cols block whose top-left element has
 * global index (row0, col0).  dist 0 = uniform[-1,1); 1 = the same scaled by
 * `scale` off the diagonal and uniform[1,2) on the diagonal (triangular
 * solver inputs).  (Plays the role of ATL_gegen in bench/l3blastst.c.)        */
int ulmb200_fill_f64(void *stream, double *d, int64_t ld, int64_t rows, int64_t cols,
                     uint64_t seed, uint32_t mat, int64_t row0, int64_t col0,
                     int dist, double scale);
int ulmb200_fill_f32(void *stream, float *d, int64_t ld, int64_t rows, int64_t cols,
                     uint64_t seed, uint32_t mat, int64_t row0, int64_t col0);
void ulmb200_host_fill_f64(double *h, int64_t ld, int64_t rows, int64_t cols,
                           uint64_t seed, uint32_t mat, int64_t row0, int64_t col0,
                           int dist, double scale);
void ulmb200_host_fill_f32(float *h, int64_t ld, int64_t rows, int64_t cols,
                           uint64_t seed, uint32_t mat, int64_t row0, int64_t col0);

/* d <- |d| elementwise on a device matrix (operands of the gauge product |A||B| of the
 * componentwise error bound, formed without a host copy).                    */
int ulmb200_abs_f64(void *stream, double *d, int64_t ld, int64_t rows, int64_t cols);

/* Register-only throughput probes (FP64 DMMA shapes, FP64 FMA, FP32 FMA):
 * runs `iters` dependent-free instruction groups per warp on every SM and
 * returns achieved TFLOP/s in *tflops.  which: 0 dmma.m8n8k4, 1 dmma.m16n8k4,
 * 2 dmma.m16n8k8, 3 dmma.m16n8k16, 4 dfma, 5 ffma, 6 dmma+dfma mixed,
 * 7 packed fma.rn.f32x2.         */
int ulmb200_peak_probe(int which, int iters, double *tflops, double *ms);

/* Failure-path self test: launches a kernel whose (short, bounded) wait can never be
 * satisfied.  The kernel gives up, records it in the device error word and returns
 * normally; the call reports ULMB200_KERNEL_FAULT (as ulmb200_check_device_error
 * would) and the context stays usable.       */
int ulmb200_selftest_wait_timeout(void);
/* The same give-up, recorded in the error word of ulmb200_dtrsm_noalloc's built-in work area
 * (which exists once that entry point has been called on the device; ULMB200_BAD_ARGUMENT
 * before).  Only launches and returns ULMB200_OK: ulmb200_check_device_error() must then
 * report ULMB200_KERNEL_FAULT.                                                            */
int ulmb200_selftest_wait_timeout_noalloc_word(void);

#ifdef __cplusplus
}
#endif
#endif /* ULMB200_BENCHSUPPORT_H */
