// Complex double GEMM:  C <- alpha * op(A) * op(B) + beta * C,  op in {N, T, C, R}
// (R = conjugate without transposing, as the reference's shim accepts:
// interfaces/blas/F77/gemm.cc:401-402,428-440).
//
// The reference runs its generic micro-kernel on std::complex<double> panels that were
// conjugated while packing (ulmblas/level3/gemm.tcc:60-83, pack/gepack.tcc:21-33,
// ukernel/ref/ugemm.tcc:10-67).  Here the FP64 tensor-core GEMM does the work on split
// operands: one pass writes the real and imaginary planes of A and B (conjugation is a
// sign carried into the GEMM scalars, transposition a flag of the real GEMM), four real
// GEMMs form
//     Tr = Ar Br - sa sb Ai Bi        Ti = sb Ar Bi + sa Ai Br      (sa, sb = -1 when conjugated)
// and one pass folds  C <- alpha T + beta C  back into the interleaved matrix.  beta == 0
// never reads C.  8 m n k real flops at the DGEMM rate; the two passes are memory traffic of
// the size of the operands.
#include "common.h"

namespace ulmb200 {

__global__ void zsplit_kernel(const double2 *Z, int64_t ldz, int64_t rows, int64_t cols, double *re,
                              double *im, int64_t ldp)
{
    const int64_t total = rows * cols;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = e % rows, j = e / rows;
        const double2 z = Z[i + j * ldz];
        re[i + j * ldp] = z.x;
        im[i + j * ldp] = z.y;
    }
}

// C <- alpha * (Tr + i Ti) + beta * C;   use_t == 0: C <- beta * C only (alpha == 0 or k == 0)
__global__ void zfold_kernel(double2 *C, int64_t ldc, int64_t m, int64_t n, const double *Tr,
                             const double *Ti, int64_t ldt, double ar, double ai, double br, double bi,
                             int use_t)
{
    const int64_t total = m * n;
    const bool beta_zero = (br == 0.0 && bi == 0.0);
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = e % m, j = e / m;
        double cr = 0.0, ci = 0.0;
        if (!beta_zero) {
            const double2 c = C[i + j * ldc];
            cr = c.x * br - c.y * bi;
            ci = c.x * bi + c.y * br;
        }
        if (use_t) {
            const double tr = Tr[i + j * ldt], ti = Ti[i + j * ldt];
            cr += ar * tr - ai * ti;
            ci += ar * ti + ai * tr;
        }
        C[i + j * ldc] = make_double2(cr, ci);
    }
}

static int grid_for(int64_t total)
{
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    return (int)(blocks < 1 ? 1 : blocks);
}

static int64_t pad4(int64_t x) { return (x + 3) / 4 * 4; }

int zgemm_device(cudaStream_t st, int transA, int conjA, int transB, int conjB, int64_t m, int64_t n,
                 int64_t k, const double *alpha, const double *A, int64_t lda, const double *B,
                 int64_t ldb, const double *beta, double *C, int64_t ldc)
{
    if (m < 0 || n < 0 || k < 0) return set_status(ULMB200_BAD_ARGUMENT);
    const int64_t rowsA = transA ? k : m, colsA = transA ? m : k;
    const int64_t rowsB = transB ? n : k, colsB = transB ? k : n;
    if (lda < (rowsA > 1 ? rowsA : 1) || ldb < (rowsB > 1 ? rowsB : 1) || ldc < (m > 1 ? m : 1))
        return set_status(ULMB200_BAD_ARGUMENT);
    if (m == 0 || n == 0) return set_status(ULMB200_OK);
    if (int s0 = ensure_device()) return set_status(s0);
    const double ar = alpha[0], ai = alpha[1], br = beta[0], bi = beta[1];
    double2 *Cz = reinterpret_cast<double2 *>(C);

    if ((ar == 0.0 && ai == 0.0) || k == 0) {            // gemm.tcc:52-55: C <- beta C
        if (br == 1.0 && bi == 0.0) return set_status(ULMB200_OK);
        zfold_kernel<<<grid_for(m * n), 256, 0, st>>>(Cz, ldc, m, n, nullptr, nullptr, 0, 0.0, 0.0, br, bi, 0);
        count_launch();
        return set_status(check_cuda(cudaGetLastError(), "zfold_kernel", __FILE__, __LINE__));
    }

    // planes: Ar, Ai (rowsA x colsA), Br, Bi (rowsB x colsB), Tr, Ti (m x n); padded pitches
    const int64_t pa = pad4(rowsA), pb = pad4(rowsB), pt = pad4(m);
    const size_t na = (size_t)(pa * colsA + 32) / 32 * 32, nb = (size_t)(pb * colsB + 32) / 32 * 32;
    const size_t nt = (size_t)(pt * n + 32) / 32 * 32;
    double *W = static_cast<double *>(device_scratch(12, sizeof(double) * (2 * na + 2 * nb + 2 * nt)));
    if (!W) return set_status(ULMB200_CUDA_ERROR);
    double *Ar = W, *Ai = Ar + na, *Br = Ai + na, *Bi = Br + nb, *Tr = Bi + nb, *Ti = Tr + nt;

    zsplit_kernel<<<grid_for(rowsA * colsA), 256, 0, st>>>(reinterpret_cast<const double2 *>(A), lda, rowsA,
                                                           colsA, Ar, Ai, pa);
    count_launch();
    zsplit_kernel<<<grid_for(rowsB * colsB), 256, 0, st>>>(reinterpret_cast<const double2 *>(B), ldb, rowsB,
                                                           colsB, Br, Bi, pb);
    count_launch();
    ULMB_CUDA(cudaGetLastError());

    const double sa = conjA ? -1.0 : 1.0, sb = conjB ? -1.0 : 1.0;
    int s;
    s = dgemm_device(st, 0, transA, transB, m, n, k, 1.0, Ar, pa, Br, pb, 0.0, Tr, pt);
    if (s == ULMB200_OK) s = dgemm_device(st, 0, transA, transB, m, n, k, -sa * sb, Ai, pa, Bi, pb, 1.0, Tr, pt);
    if (s == ULMB200_OK) s = dgemm_device(st, 0, transA, transB, m, n, k, sb, Ar, pa, Bi, pb, 0.0, Ti, pt);
    if (s == ULMB200_OK) s = dgemm_device(st, 0, transA, transB, m, n, k, sa, Ai, pa, Br, pb, 1.0, Ti, pt);
    if (s != ULMB200_OK) return set_status(s);

    zfold_kernel<<<grid_for(m * n), 256, 0, st>>>(Cz, ldc, m, n, Tr, Ti, pt, ar, ai, br, bi, 1);
    count_launch();
    return set_status(check_cuda(cudaGetLastError(), "zfold_kernel", __FILE__, __LINE__));
}

}  // namespace ulmb200

extern "C" int ulmb200_zgemm(void *stream, int transA, int conjA, int transB, int conjB, int64_t m,
                             int64_t n, int64_t k, const double *alpha, const double *dA, int64_t ldA,
                             const double *dB, int64_t ldB, const double *beta, double *dC, int64_t ldC)
{
    return ulmb200::zgemm_device(static_cast<cudaStream_t>(stream), transA, conjA, transB, conjB, m, n, k,
                                 alpha, dA, ldA, dB, ldB, beta, dC, ldC);
}
