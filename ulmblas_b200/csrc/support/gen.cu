// Device and host fills built on the counter-based generator in gen.h, plus a
// few element-wise helpers the tests and the bench use on device buffers.
#include "../common.h"
#include "../../../include/ulmb200_benchsupport.h"
#include "gen.h"

namespace ulmb200 {

template <typename T>
__global__ void fill_kernel(T *d, int64_t ld, int64_t rows, int64_t cols, uint64_t seed,
                            uint32_t mat, int64_t row0, int64_t col0, int dist, double scale)
{
    const int64_t total = rows * cols;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = e % rows, j = e / rows;
        d[i + j * ld] = (T)gen_value(seed, mat, row0 + i, col0 + j, dist, scale);
    }
}

__global__ void abs_kernel(double *d, int64_t ld, int64_t rows, int64_t cols)
{
    const int64_t total = rows * cols;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total;
         e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i = e % rows, j = e / rows;
        d[i + j * ld] = fabs(d[i + j * ld]);
    }
}

template <typename T>
static int fill_device(cudaStream_t st, T *d, int64_t ld, int64_t rows, int64_t cols, uint64_t seed,
                       uint32_t mat, int64_t row0, int64_t col0, int dist, double scale)
{
    if (rows < 0 || cols < 0 || ld < (rows > 1 ? rows : 1)) return set_status(ULMB200_BAD_ARGUMENT);
    if (rows == 0 || cols == 0) return set_status(ULMB200_OK);
    if (int s = ensure_device()) return set_status(s);
    int64_t blocks = (rows * cols + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    fill_kernel<T><<<(int)blocks, 256, 0, st>>>(d, ld, rows, cols, seed, mat, row0, col0, dist, scale);
    count_launch();
    return set_status(check_cuda(cudaGetLastError(), "fill_kernel", __FILE__, __LINE__));
}

template <typename T>
static void fill_host(T *h, int64_t ld, int64_t rows, int64_t cols, uint64_t seed, uint32_t mat,
                      int64_t row0, int64_t col0, int dist, double scale)
{
    for (int64_t j = 0; j < cols; ++j)
        for (int64_t i = 0; i < rows; ++i)
            h[i + j * ld] = (T)gen_value(seed, mat, row0 + i, col0 + j, dist, scale);
}

}  // namespace ulmb200

using namespace ulmb200;

extern "C" int ulmb200_fill_f64(void *stream, double *d, int64_t ld, int64_t rows, int64_t cols,
                                uint64_t seed, uint32_t mat, int64_t row0, int64_t col0, int dist,
                                double scale)
{
    return fill_device<double>((cudaStream_t)stream, d, ld, rows, cols, seed, mat, row0, col0, dist, scale);
}

extern "C" int ulmb200_fill_f32(void *stream, float *d, int64_t ld, int64_t rows, int64_t cols,
                                uint64_t seed, uint32_t mat, int64_t row0, int64_t col0)
{
    return fill_device<float>((cudaStream_t)stream, d, ld, rows, cols, seed, mat, row0, col0, 0, 1.0);
}

extern "C" void ulmb200_host_fill_f64(double *h, int64_t ld, int64_t rows, int64_t cols,
                                      uint64_t seed, uint32_t mat, int64_t row0, int64_t col0,
                                      int dist, double scale)
{
    fill_host<double>(h, ld, rows, cols, seed, mat, row0, col0, dist, scale);
}

extern "C" void ulmb200_host_fill_f32(float *h, int64_t ld, int64_t rows, int64_t cols,
                                      uint64_t seed, uint32_t mat, int64_t row0, int64_t col0)
{
    fill_host<float>(h, ld, rows, cols, seed, mat, row0, col0, 0, 1.0);
}

extern "C" int ulmb200_abs_f64(void *stream, double *d, int64_t ld, int64_t rows, int64_t cols)
{
    if (rows <= 0 || cols <= 0) return set_status(ULMB200_OK);
    if (int s = ensure_device()) return set_status(s);
    int64_t blocks = (rows * cols + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    abs_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(d, ld, rows, cols);
    count_launch();
    return set_status(check_cuda(cudaGetLastError(), "abs_kernel", __FILE__, __LINE__));
}
