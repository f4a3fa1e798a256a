// ulmb200_dtrsm_noalloc: the triangular solve for callers that must not allocate.
//
// Who needs this: code that runs where device-memory allocation is forbidden or
// would stall -- a real-time or latency-critical loop that may not take the
// allocator's locks or its implicit device synchronisation, a plug-in handed a
// fixed memory budget by its host application, a process whose device memory is
// already fully committed to another pool.  ulmb200_dtrsm keeps its work areas
// (the inverted 128x128 diagonal blocks and the 128-wide leaf tile) in a cache
// that grows with cudaMalloc; this entry point runs the same kernels on a work
// area that is part of the library image instead.
//
// The work area is a file-scope __device__ array.  Consequences the caller
// should know:
//   * Every GPU that loads the library holds it (about 6.3 MB) until exit,
//     whether or not this entry point is ever called.
//   * Sizes are capped: the triangular matrix may be at most 2048 x 2048 and
//     the other dimension of B at most 4096.  Larger requests are refused with
//     ULMB200_TOO_LARGE and nothing is launched.
//   * All calls on a device share the one area and it keeps the previous
//     call's contents.  Each call rewrites every element it later reads (the
//     block inverses are written in full, zeros included; the leaf tile is
//     produced before it is copied back), so stale contents never leak into a
//     result -- but two calls that overlap in time on the same GPU (different
//     streams, different host threads) race on it.  Serialise them.
//   * The first call on each device looks up the device addresses of the
//     arrays and raises the shared-memory limits of the kernels it launches.
//     Make that first call outside any stream capture.
//
// No cudaMalloc, cudaFree or allocating library routine is reached from here.
#include "common.h"

#include <atomic>
#include <mutex>

namespace ulmb200 {

constexpr int64_t kNoAllocMaxTri = 2048;      // side length of the triangular matrix
constexpr int64_t kNoAllocMaxOther = 4096;    // the other dimension of B
constexpr int64_t kNoAllocNB = 128;           // diagonal block size of the solver
constexpr int64_t kNoAllocInvDoubles = (kNoAllocMaxTri / kNoAllocNB) * kNoAllocNB * kNoAllocNB;
constexpr int64_t kNoAllocLeafDoubles = kNoAllocNB * kNoAllocMaxOther;

// In host code these names are only stand-ins for the device objects; the
// addresses kernels can use come from cudaGetSymbolAddress below.
static __device__ __align__(256) double g_noalloc_work[kNoAllocInvDoubles + kNoAllocLeafDoubles];
static __device__ __align__(256) int g_noalloc_err[64];

struct NoAllocDevice {
    double *work = nullptr;
    int *err = nullptr;
    std::atomic<bool> ready{false};
};
static NoAllocDevice g_noalloc[kMaxDevices];
static std::mutex g_noalloc_mu;

// Once per device, with that device current.
static int noalloc_setup(NoAllocDevice **out)
{
    const int dev = current_device();
    NoAllocDevice &d = g_noalloc[dev];
    if (!d.ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lk(g_noalloc_mu);
        if (!d.ready.load(std::memory_order_relaxed)) {
            void *w = nullptr, *e = nullptr;
            cudaError_t rc = cudaGetSymbolAddress(&w, g_noalloc_work);
            if (rc != cudaSuccess) return check_cuda(rc, "cudaGetSymbolAddress(work area)", __FILE__, __LINE__);
            rc = cudaGetSymbolAddress(&e, g_noalloc_err);
            if (rc != cudaSuccess) return check_cuda(rc, "cudaGetSymbolAddress(error word)", __FILE__, __LINE__);
            d.work = static_cast<double *>(w);
            d.err = static_cast<int *>(e);
            // ulmb200_check_device_error() reads this word too (a plain copy, no allocation)
            register_error_word(d.err);
            d.ready.store(true, std::memory_order_release);
        }
    }
    *out = &d;
    return ULMB200_OK;
}

}  // namespace ulmb200

using namespace ulmb200;

extern "C" int ulmb200_dtrsm_noalloc(void *stream, int side, int lower, int transA, int unit, int64_t m,
                                     int64_t n, double alpha, const double *dA, int64_t ldA, double *dB,
                                     int64_t ldB)
{
    if (m < 0 || n < 0 || (side != 0 && side != 1)) return set_status(ULMB200_BAD_ARGUMENT);
    const int64_t dim = (side == 0) ? m : n, other = (side == 0) ? n : m;
    if (ldA < (dim > 1 ? dim : 1) || ldB < (m > 1 ? m : 1)) return set_status(ULMB200_BAD_ARGUMENT);
    if (dim > kNoAllocMaxTri || other > kNoAllocMaxOther) {
        fprintf(stderr,
                "ulmblas_b200: ulmb200_dtrsm_noalloc handles a triangle of at most %lld and a second "
                "dimension of at most %lld (got %lld and %lld); use ulmb200_dtrsm for larger solves\n",
                (long long)kNoAllocMaxTri, (long long)kNoAllocMaxOther, (long long)dim, (long long)other);
        return set_status(ULMB200_TOO_LARGE);
    }
    if (m == 0 || n == 0) return set_status(ULMB200_OK);
    if (int s = ensure_device()) return set_status(s);
    NoAllocDevice *d = nullptr;
    if (int s = noalloc_setup(&d)) return set_status(s);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The block inverses and the leaf tile are fully rewritten by the kernels before anything reads
    // them.  The words behind the error word (the GEMM launches' tile counter) are put back to zero
    // by the kernels themselves; they are cleared here as well in case an earlier call gave up half
    // way.  The error word itself is left alone, so that a fault stays visible until
    // ulmb200_check_device_error() has reported it.
    if (int s = check_cuda(cudaMemsetAsync(d->err + 1, 0, 8 * sizeof(int), st), "cudaMemsetAsync", __FILE__, __LINE__))
        return set_status(s);
    return set_status(dtrsm_with_scratch(st, side, lower, transA, unit, m, n, alpha, dA, ldA, dB, ldB, d->work,
                                         d->work + kNoAllocInvDoubles, d->err));
}
