// Partition and K-panel plan of the multi-GPU DGEMM, as plain functions of sizes and rates
// (no CUDA, no NCCL), so that they can be exercised on a machine without a GPU.
#pragma once
#include <stdint.h>

namespace ulmb200 {

constexpr int kMgMaxPanels = 32;
constexpr int64_t kMgAlign = 128;          // column blocks start on CTA-tile boundaries

// [j0, j1) of rank `rank`: near-equal blocks whose starts are multiples of kMgAlign.
inline void mg_column_block(int64_t n, int world, int rank, int64_t *j0, int64_t *j1)
{
    const int64_t units = (n + kMgAlign - 1) / kMgAlign;
    const int64_t base = units / world, extra = units % world;
    const int64_t u0 = rank * base + (rank < extra ? rank : extra);
    const int64_t u1 = u0 + base + (rank < extra ? 1 : 0);
    *j0 = u0 * kMgAlign < n ? u0 * kMgAlign : n;
    *j1 = u1 * kMgAlign < n ? u1 * kMgAlign : n;
}

// K panels of A for a product m x n_block x k per rank when A (m x k doubles) reaches the ranks at
// `transport_gbs` GB/s and a GPU multiplies at `gemm_tflops`.  widths[p] = columns of A in panel p
// (multiples of 256 except the last), reserve[p] = 1 if the GEMM of panel p must leave SMs to the
// transport because later panels are still on their way.  Returns the number of panels.
//
//   one rank          one panel, nothing travels
//   panel 0           `first` columns: the only transfer nothing can hide, so it is short
//   panel 1           just long enough for the rest of A to arrive behind its product (with 15%
//                     to spare); left out when the rest arrives during panel 0's product
//   last panel        everything else; no transfer is in flight any more, so it takes the whole GPU
inline int mg_plan_panels(int64_t m, int64_t n_block, int64_t k, int world, int64_t first, double transport_gbs,
                          double gemm_tflops, int64_t *widths, int *reserve, int cap)
{
    if (k <= 0 || cap < 1) return 0;
    if (world <= 1 || cap < 3 || m <= 0 || n_block <= 0) { widths[0] = k; reserve[0] = 0; return 1; }
    if (first < 256) first = 256;
    first = first / 256 * 256;
    if (first >= k) { widths[0] = k; reserve[0] = 0; return 1; }
    if (transport_gbs <= 0.0) transport_gbs = 100.0;
    if (gemm_tflops <= 0.0) gemm_tflops = 30.0;
    const double col_arrive = 8.0 * (double)m / (transport_gbs * 1e9);                     // seconds per column of A
    const double col_gemm = 2.0 * (double)m * (double)n_block / (gemm_tflops * 1e12);      // seconds per column of K
    const double end0 = first * col_arrive + first * col_gemm;                             // panel 0's product is done
    const double all_here = 1.15 * k * col_arrive;                                         // all of A has arrived (with margin)
    int np = 0;
    widths[np] = first; reserve[np] = 1; ++np;
    int64_t left = k - first;
    if (all_here > end0) {
        int64_t w1 = (int64_t)((all_here - end0) / col_gemm) + 1;
        w1 = (w1 + 255) / 256 * 256;
        // what panel 1 multiplies must itself have arrived by the time panel 0 is done
        const int64_t here = (int64_t)(end0 / col_arrive) - first;
        if (w1 > here && here >= 256) w1 = here / 256 * 256;
        if (w1 < 256) w1 = 256;
        if (w1 < left - 256) {
            widths[np] = w1; reserve[np] = 1; ++np;
            left -= w1;
        }
    }
    widths[np] = left; reserve[np] = 0; ++np;
    return np;
}

// One GPU with a host-resident A: panels of about 512 MB only pipeline the copy of A against the
// products (the first product starts after one panel instead of after all of A).
inline int mg_plan_host_panels(int64_t m, int64_t k, int64_t *widths, int cap)
{
    if (k <= 0 || cap < 1) return 0;
    const int64_t bytes = 8 * m * k;
    int64_t np = bytes >> 29;
    if (np > 16) np = 16;
    if (np > cap) np = cap;
    while (np > 1 && k / np < 512) --np;
    if (np < 1) np = 1;
    const int64_t w = ((k + np - 1) / np + 127) / 128 * 128;
    int n = 0;
    for (int64_t l0 = 0; l0 < k && n < cap; l0 += w) widths[n++] = (w < k - l0) ? w : k - l0;
    return n;
}

}  // namespace ulmb200
