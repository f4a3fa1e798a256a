// Register-only throughput probes.  The roofline denominators for the FP64 and
// FP32 GEMM kernels are not published for this part in a form that can be
// trusted on a power-capped, shared machine, so they are measured: each probe
// keeps every SM busy with one kind of arithmetic instruction on register
// operands (no memory traffic) and reports flop/s.
#include "../common.h"
#include "../../../include/ulmb200_benchsupport.h"

namespace ulmb200 {

constexpr int kProbeAcc = 8;   // independent accumulator sets per warp (ILP)

template <int WHICH>
__global__ void __launch_bounds__(256) probe_kernel(int iters, double *sink)
{
    const double seed = 1.0 + 1e-9 * threadIdx.x;
    double acc[kProbeAcc][4];
    double a[8], b[4];
#pragma unroll
    for (int q = 0; q < 8; ++q) a[q] = seed + q;
#pragma unroll
    for (int q = 0; q < 4; ++q) b[q] = 1e-9 * (q + 1);
#pragma unroll
    for (int s = 0; s < kProbeAcc; ++s)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[s][q] = 0.0;

    float fa = 1.0f + 1e-6f * threadIdx.x, fb = 1e-6f;
    float facc[32];
#pragma unroll
    for (int q = 0; q < 32; ++q) facc[q] = 0.0f;

    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int s = 0; s < kProbeAcc; ++s) {
            if (WHICH == 0) {
                asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                             : "+d"(acc[s][0]), "+d"(acc[s][1]) : "d"(a[0]), "d"(b[0]));
            } else if (WHICH == 1) {
                asm volatile("mma.sync.aligned.m16n8k4.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                             : "+d"(acc[s][0]), "+d"(acc[s][1]), "+d"(acc[s][2]), "+d"(acc[s][3])
                             : "d"(a[0]), "d"(a[1]), "d"(b[0]));
            } else if (WHICH == 2 || WHICH == 6) {
                asm volatile("mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+d"(acc[s][0]), "+d"(acc[s][1]), "+d"(acc[s][2]), "+d"(acc[s][3])
                             : "d"(a[0]), "d"(a[1]), "d"(a[2]), "d"(a[3]), "d"(b[0]), "d"(b[1]));
                if (WHICH == 6) {
                    // same number of scalar FP64 FMAs as the tensor instruction retires per lane
#pragma unroll
                    for (int q = 0; q < 4; ++q) a[4 + q] = fma(a[4 + q], b[2], b[3]);
                }
            } else if (WHICH == 3) {
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, "
                             "{%4,%5,%6,%7,%8,%9,%10,%11}, {%12,%13,%14,%15}, {%0,%1,%2,%3};"
                             : "+d"(acc[s][0]), "+d"(acc[s][1]), "+d"(acc[s][2]), "+d"(acc[s][3])
                             : "d"(a[0]), "d"(a[1]), "d"(a[2]), "d"(a[3]), "d"(a[4]), "d"(a[5]),
                               "d"(a[6]), "d"(a[7]), "d"(b[0]), "d"(b[1]), "d"(b[2]), "d"(b[3]));
            } else if (WHICH == 4) {
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[s][q] = fma(acc[s][q], a[q], b[q]);
            } else if (WHICH == 5) {
#pragma unroll
                for (int q = 0; q < 4; ++q) facc[s * 4 + q] = fmaf(facc[s * 4 + q], fa, fb);
            } else if (WHICH == 7) {
                // packed FP32: two FMAs per lane per instruction
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    unsigned long long d, a2, b2;
                    asm("mov.b64 %0, {%1,%2};" : "=l"(d) : "f"(facc[s * 4 + 2 * q]), "f"(facc[s * 4 + 2 * q + 1]));
                    asm("mov.b64 %0, {%1,%1};" : "=l"(a2) : "f"(fa));
                    asm("mov.b64 %0, {%1,%1};" : "=l"(b2) : "f"(fb));
                    asm volatile("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(d) : "l"(a2), "l"(b2));
                    asm("mov.b64 {%0,%1}, %2;" : "=f"(facc[s * 4 + 2 * q]), "=f"(facc[s * 4 + 2 * q + 1]) : "l"(d));
                }
            }
        }
    }
    double r = 0.0;
#pragma unroll
    for (int s = 0; s < kProbeAcc; ++s)
#pragma unroll
        for (int q = 0; q < 4; ++q) r += acc[s][q];
#pragma unroll
    for (int q = 0; q < 32; ++q) r += facc[q];
#pragma unroll
    for (int q = 4; q < 8; ++q) r += a[q];
    if (r == 123.456) sink[0] = r;   // keeps the arithmetic live, never true in practice
}

template <int WHICH>
static int run_probe(int iters, int blocks, double *ms)
{
    double *sink = static_cast<double *>(device_scratch(7, 256));
    if (!sink) return ULMB200_CUDA_ERROR;
    cudaEvent_t e0, e1;
    ULMB_CUDA(cudaEventCreate(&e0));
    ULMB_CUDA(cudaEventCreate(&e1));
    probe_kernel<WHICH><<<blocks, 256>>>(iters / 8 + 1, sink);      // warm-up
    count_launch();
    ULMB_CUDA(cudaEventRecord(e0));
    probe_kernel<WHICH><<<blocks, 256>>>(iters, sink);
    count_launch();
    ULMB_CUDA(cudaEventRecord(e1));
    ULMB_CUDA(cudaEventSynchronize(e1));
    float t = 0.f;
    ULMB_CUDA(cudaEventElapsedTime(&t, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *ms = t;
    return ULMB200_OK;
}

// A wait that nothing will ever satisfy, with a short poll limit: exercises the path every
// bounded wait in the library takes when it gives up (error word written, normal return).
__global__ void wait_probe_kernel(int *err, uint32_t limit)
{
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_barrier_init();
        bool ok = false;
        for (uint32_t i = 0; i < limit && !ok; ++i) {
            ok = mbar_try_wait(&bar, 0);
            if (!ok) __nanosleep(64);
        }
        if (!ok) atomicExch(err, 301);
    }
}

}  // namespace ulmb200

using namespace ulmb200;

extern "C" int ulmb200_selftest_wait_timeout(void)
{
    if (int s = ensure_device()) return set_status(s);
    int *err = device_error_word();
    if (!err) return set_status(ULMB200_CUDA_ERROR);
    wait_probe_kernel<<<1, 32>>>(err, 20000);      // about a millisecond of polling
    count_launch();
    if (int e = check_cuda(cudaGetLastError(), "wait_probe_kernel", __FILE__, __LINE__)) return e;
    if (int e = check_cuda(cudaDeviceSynchronize(), "synchronize", __FILE__, __LINE__)) return e;
    return set_status(poll_device_error());        // ULMB200_KERNEL_FAULT is the expected answer
}

extern "C" int ulmb200_selftest_wait_timeout_noalloc_word(void)
{
    if (int s = ensure_device()) return set_status(s);
    int *err = registered_error_word(0);
    if (!err) return set_status(ULMB200_BAD_ARGUMENT);
    wait_probe_kernel<<<1, 32>>>(err, 20000);
    count_launch();
    return set_status(check_cuda(cudaGetLastError(), "wait_probe_kernel", __FILE__, __LINE__));
}

extern "C" int ulmb200_peak_probe(int which, int iters, double *tflops, double *ms_out)
{
    if (int s = ensure_device()) return set_status(s);
    if (iters <= 0 || !tflops) return set_status(ULMB200_BAD_ARGUMENT);
    const int blocks = sm_count() * 4;            // 32 warps per SM, 8 per scheduler
    double ms = 0.0;
    int st;
    // flops per warp-level instruction group (one accumulator set)
    double flops_per_set;
    switch (which) {
    case 0: st = run_probe<0>(iters, blocks, &ms); flops_per_set = 2.0 * 8 * 8 * 4; break;
    case 1: st = run_probe<1>(iters, blocks, &ms); flops_per_set = 2.0 * 16 * 8 * 4; break;
    case 2: st = run_probe<2>(iters, blocks, &ms); flops_per_set = 2.0 * 16 * 8 * 8; break;
    case 3: st = run_probe<3>(iters, blocks, &ms); flops_per_set = 2.0 * 16 * 8 * 16; break;
    case 4: st = run_probe<4>(iters, blocks, &ms); flops_per_set = 2.0 * 4 * 32; break;
    case 5: st = run_probe<5>(iters, blocks, &ms); flops_per_set = 2.0 * 4 * 32; break;
    case 6: st = run_probe<6>(iters, blocks, &ms); flops_per_set = 2.0 * 16 * 8 * 8 + 2.0 * 4 * 32; break;
    case 7: st = run_probe<7>(iters, blocks, &ms); flops_per_set = 2.0 * 4 * 32; break;
    default: return set_status(ULMB200_BAD_ARGUMENT);
    }
    if (st != ULMB200_OK) return set_status(st);
    const double total = flops_per_set * kProbeAcc * (double)iters * 8.0 /*warps*/ * blocks;
    *tflops = total / (ms * 1e-3) * 1e-12;
    if (ms_out) *ms_out = ms;
    return set_status(ULMB200_OK);
}
