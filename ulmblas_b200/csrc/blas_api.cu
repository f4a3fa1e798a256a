// The reference-facing boundary: the Fortran-ABI and CBLAS symbols of
// ulmBLAS's Level-3 GEMM path (interfaces/blas/F77/{gemm,trsm,syrk,xerbla}.cc,
// interfaces/blas/C/{gemm,trsm,syrk,xerbla,cblas_globals}.cc), with the same
// argument decoding, the same first-bad-argument codes and the same xerbla
// protocol.  Behind them nothing of the reference remains: operands are used in
// place when they already live in device memory, and are staged through cached
// device buffers (column blocks of B/C pipelined against the compute) when
// they are host pointers.  There is no CPU path: without a usable sm_100 device
// the call reports through stderr and ulmb200_last_status() and leaves C alone.
//
// One deliberate difference from the reference: after reporting a bad argument
// through xerbla_ these entry points return; the reference falls through and
// computes anyway (interfaces/blas/F77/gemm.cc:197-204).
#include "common.h"

#include <algorithm>
#include <cctype>
#include <cstdarg>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <mutex>
#include <thread>
#include <time.h>
#include <vector>

namespace ulmb200 {

int sgemm_device(cudaStream_t st, int mode, int transA, int transB, int64_t m, int64_t n,
                 int64_t k, float alpha, const float *A, int64_t lda, const float *B, int64_t ldb,
                 float beta, float *C, int64_t ldc);
int dsyrk_device(cudaStream_t st, int lower, int trans, int64_t n, int64_t k, double alpha,
                 const double *A, int64_t lda, double beta, double *C, int64_t ldc);
int dtrsm_device(cudaStream_t st, int side, int lower, int transA, int unit, int64_t m, int64_t n,
                 double alpha, const double *A, int64_t lda, double *B, int64_t ldb);
int dtrmm_device(cudaStream_t st, int side, int lower, int transA, int unit, int64_t m, int64_t n,
                 double alpha, const double *A, int64_t lda, double *B, int64_t ldb);
int dgetrf_device(cudaStream_t st, int64_t m, int64_t n, double *A, int64_t lda, int *d_piv, int *d_info);
int ssyrk_device(cudaStream_t st, int lower, int trans, int64_t n, int64_t k, float alpha, const float *A,
                 int64_t lda, float beta, float *C, int64_t ldc);
int strsm_device(cudaStream_t st, int side, int lower, int transA, int unit, int64_t m, int64_t n, float alpha,
                 const float *A, int64_t lda, float *B, int64_t ldb);
int dlaswp_pairs_device(cudaStream_t st, double *A, int64_t lda, int64_t ncols, const int *d_pairs, int npairs);
int zgemm_device(cudaStream_t st, int transA, int conjA, int transB, int conjB, int64_t m, int64_t n,
                 int64_t k, const double *alpha, const double *A, int64_t lda, const double *B,
                 int64_t ldb, const double *beta, double *C, int64_t ldc);
int dsymm_device(cudaStream_t st, int side, int lower, int64_t m, int64_t n, double alpha, const double *A,
                 int64_t lda, const double *B, int64_t ldb, double beta, double *C, int64_t ldc);
int dsyr2k_device(cudaStream_t st, int lower, int trans, int64_t n, int64_t k, double alpha,
                  const double *A, int64_t lda, const double *B, int64_t ldb, double beta, double *C,
                  int64_t ldc);

static int g_pin_host = 0;

// The blocking BLAS entry points share one set of staging and work buffers per device, so calls
// from different host threads on the SAME device take turns (the reference guards its memory pool
// the same way, ulmblas/auxiliary/memorypool.tcc:43,57); calls on different devices run side by
// side, each thread on its own streams.  Callers of the asynchronous ulmb200_* device ABI order
// their own work: routines that use work buffers (dtrsm, dtrmm, dsymm, dgetrf, 3xTF32 sgemm) must
// not overlap on one device.
static std::recursive_mutex g_call_mu[kMaxDevices];
#define ULMB_SERIALISE std::lock_guard<std::recursive_mutex> ulmb_call_lock(g_call_mu[current_device()])

// wall-clock milliseconds for the trace lines
static double now_ms()
{
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec * 1e3 + ts.tv_nsec * 1e-6;
}

// ---- where does a pointer live? -------------------------------------------
static bool on_device(const void *p)
{
    if (!p) return false;
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// ---- per-thread streams and events for staged calls -------------------------
// One set per calling thread and device, created on first use with that device current.
struct Streams {
    cudaStream_t in = nullptr, run = nullptr, out = nullptr;
    cudaEvent_t ev[128] = {};
    int dev = -1;
    bool ok = false;
};
static thread_local std::vector<Streams *> t_streams;

static Streams *streams()
{
    const int dev = current_device();
    if ((int)t_streams.size() <= dev) t_streams.resize(dev + 1, nullptr);
    if (!t_streams[dev]) t_streams[dev] = new Streams;
    Streams &s = *t_streams[dev];
    if (s.ok) return &s;
    if (cudaStreamCreateWithFlags(&s.in, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaStreamCreateWithFlags(&s.run, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    if (cudaStreamCreateWithFlags(&s.out, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    for (auto &e : s.ev)
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    s.dev = dev;
    s.ok = true;
    return &s;
}

// Optional page-locking of the caller's buffers for the duration of a call.
struct HostPin {
    void *p = nullptr;
    HostPin(const void *ptr, size_t bytes)
    {
        if (g_pin_host && ptr && bytes >= (size_t)(1 << 20)) {
            cudaPointerAttributes a;
            if (cudaPointerGetAttributes(&a, ptr) == cudaSuccess && a.type == cudaMemoryTypeUnregistered &&
                cudaHostRegister(const_cast<void *>(ptr), bytes, cudaHostRegisterDefault) == cudaSuccess)
                p = const_cast<void *>(ptr);
            else
                cudaGetLastError();
        }
    }
    ~HostPin() { if (p) cudaHostUnregister(p); }
};

// ---- pageable host memory: staged through page-locked bounce buffers by worker threads ---------
// A caller of the reference hands over plain malloc'ed / Fortran arrays.  Copied directly, such
// memory moves at the speed of one driver thread's staging copy and does not overlap anything.
// Here a few worker threads copy column chunks into (out of) page-locked bounce buffers, from
// (to) which the copy engines run asynchronously: the host-side copies of different chunks run in
// parallel and overlap the transfers and the arithmetic.
class Stager {
public:
    struct Batch {
        std::mutex m;
        std::condition_variable cv;
        int pending = 0;
        cudaError_t err = cudaSuccess;
        void add(int n) { std::lock_guard<std::mutex> lk(m); pending += n; }
        void done(cudaError_t e)
        {
            std::lock_guard<std::mutex> lk(m);
            if (e != cudaSuccess && err == cudaSuccess) err = e;
            if (--pending == 0) cv.notify_all();
        }
        cudaError_t wait()
        {
            std::unique_lock<std::mutex> lk(m);
            cv.wait(lk, [&] { return pending == 0; });
            const cudaError_t e = err;
            err = cudaSuccess;
            return e;
        }
    };
    struct Task {
        int dev;
        bool in;                    // host -> device
        cudaStream_t st;
        char *dptr; size_t dpitch;  // device block
        char *hptr; size_t hpitch;  // caller's block
        size_t width, cols;         // bytes per column, columns
        Batch *batch;
    };
    static constexpr size_t kChunk = (size_t)16 << 20;

    static Stager &get()
    {
        static Stager *s = new Stager;     // never destroyed: the workers live until the process ends
        return *s;
    }
    bool usable()
    {
        std::call_once(once_, [this] { start(); });
        return !workers_.empty();
    }
    void submit(const Task &t)
    {
        {
            std::lock_guard<std::mutex> lk(mu_);
            queue_.push_back(t);
        }
        cv_.notify_one();
    }

private:
    struct Worker {
        std::thread th;
        char *buf[2] = {nullptr, nullptr};
        cudaEvent_t ev[2][kMaxDevices] = {};
        int last_dev[2] = {-1, -1};       // device whose stream used the buffer last
    };
    std::once_flag once_;
    std::mutex mu_;
    std::condition_variable cv_;
    std::deque<Task> queue_;
    std::vector<Worker *> workers_;

    void start()
    {
        unsigned hc = std::thread::hardware_concurrency();
        int n = hc >= 16 ? 8 : (hc >= 8 ? 4 : 2);
        if (const char *e = getenv("ULMB200_STAGING_THREADS")) n = std::max(0, std::min(32, atoi(e)));
        for (int i = 0; i < n; ++i) {
            Worker *w = new Worker;
            if (cudaHostAlloc(&w->buf[0], kChunk, cudaHostAllocPortable) != cudaSuccess ||
                cudaHostAlloc(&w->buf[1], kChunk, cudaHostAllocPortable) != cudaSuccess) {
                cudaGetLastError();
                delete w;
                break;
            }
            workers_.push_back(w);
            w->th = std::thread([this, w] { run(w); });
            w->th.detach();
        }
    }
    void run(Worker *w)
    {
        int cur_dev = -1, which = 0;
        for (;;) {
            Task t;
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return !queue_.empty(); });
                t = queue_.front();
                queue_.pop_front();
            }
            cudaError_t e = cudaSuccess;
            if (t.dev != cur_dev) { e = cudaSetDevice(t.dev); cur_dev = t.dev; }
            const int b = which;
            which ^= 1;
            // the buffer's previous transfer (possibly on another device's stream) must have finished
            if (e == cudaSuccess && w->last_dev[b] >= 0) e = cudaEventSynchronize(w->ev[b][w->last_dev[b]]);
            if (e == cudaSuccess && !w->ev[b][t.dev]) e = cudaEventCreateWithFlags(&w->ev[b][t.dev], cudaEventDisableTiming);
            if (e == cudaSuccess && t.in) {
                for (size_t c = 0; c < t.cols; ++c) memcpy(w->buf[b] + c * t.width, t.hptr + c * t.hpitch, t.width);
                e = cudaMemcpy2DAsync(t.dptr, t.dpitch, w->buf[b], t.width, t.width, t.cols, cudaMemcpyHostToDevice, t.st);
                if (e == cudaSuccess) e = cudaEventRecord(w->ev[b][t.dev], t.st);
                if (e == cudaSuccess) w->last_dev[b] = t.dev;
            } else if (e == cudaSuccess) {
                e = cudaMemcpy2DAsync(w->buf[b], t.width, t.dptr, t.dpitch, t.width, t.cols, cudaMemcpyDeviceToHost, t.st);
                if (e == cudaSuccess) e = cudaEventRecord(w->ev[b][t.dev], t.st);
                if (e == cudaSuccess) { w->last_dev[b] = t.dev; e = cudaEventSynchronize(w->ev[b][t.dev]); }
                if (e == cudaSuccess)
                    for (size_t c = 0; c < t.cols; ++c) memcpy(t.hptr + c * t.hpitch, w->buf[b] + c * t.width, t.width);
            }
            if (e != cudaSuccess) cudaGetLastError();
            t.batch->done(e);
        }
    }
};

// copies back to pageable memory that the current blocking call still has in flight
static thread_local Stager::Batch t_out_batch;

static bool pageable(const void *p)
{
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return true;
    }
    return a.type == cudaMemoryTypeUnregistered;
}

// true if the block went (or is going) through the bounce buffers
static bool staged_copy(bool in, char *d, size_t dpitch, char *h, size_t hpitch, size_t width, size_t cols,
                        cudaStream_t st, cudaError_t *err)
{
    *err = cudaSuccess;
    if (g_pin_host || width * cols < ((size_t)8 << 20) || width == 0 || width > Stager::kChunk || !pageable(h)) return false;
    Stager &sg = Stager::get();
    if (!sg.usable()) return false;
    const size_t per = std::max<size_t>(1, Stager::kChunk / width);
    const int chunks = (int)((cols + per - 1) / per);
    Stager::Batch local;
    Stager::Batch *batch = in ? &local : &t_out_batch;
    batch->add(chunks);
    for (size_t c0 = 0; c0 < cols; c0 += per) {
        Stager::Task t;
        t.dev = current_device(); t.in = in; t.st = st;
        t.dptr = d + c0 * dpitch; t.dpitch = dpitch;
        t.hptr = h + c0 * hpitch; t.hpitch = hpitch;
        t.width = width; t.cols = std::min(per, cols - c0);
        t.batch = batch;
        sg.submit(t);
    }
    // inbound: return once every chunk's transfer is queued on the stream, so that what the caller
    // queues next is ordered behind them; outbound chunks are waited for at the end of the call
    if (in) *err = local.wait();
    return true;
}

template <typename T>
static cudaError_t copy_in(T *d, int64_t ldd, const T *h, int64_t ldh, int64_t rows, int64_t cols,
                           cudaStream_t st)
{
    if (rows <= 0 || cols <= 0) return cudaSuccess;
    cudaError_t e;
    if (staged_copy(true, reinterpret_cast<char *>(d), ldd * sizeof(T), reinterpret_cast<char *>(const_cast<T *>(h)),
                    ldh * sizeof(T), rows * sizeof(T), (size_t)cols, st, &e))
        return e;
    return cudaMemcpy2DAsync(d, ldd * sizeof(T), h, ldh * sizeof(T), rows * sizeof(T), cols,
                             cudaMemcpyHostToDevice, st);
}

template <typename T>
static cudaError_t copy_out(T *h, int64_t ldh, const T *d, int64_t ldd, int64_t rows, int64_t cols,
                            cudaStream_t st)
{
    if (rows <= 0 || cols <= 0) return cudaSuccess;
    cudaError_t e;
    if (staged_copy(false, reinterpret_cast<char *>(const_cast<T *>(d)), ldd * sizeof(T), reinterpret_cast<char *>(h),
                    ldh * sizeof(T), rows * sizeof(T), (size_t)cols, st, &e))
        return e;
    return cudaMemcpy2DAsync(h, ldh * sizeof(T), d, ldd * sizeof(T), rows * sizeof(T), cols,
                             cudaMemcpyDeviceToHost, st);
}

static int64_t round_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

// bytes spanned by a rows x cols column-major matrix with leading dimension ld
template <typename T>
static size_t span_bytes(int64_t rows, int64_t cols, int64_t ld)
{
    return (rows > 0 && cols > 0) ? sizeof(T) * (size_t)((cols - 1) * ld + rows) : 0;
}

static int finish(Streams *s)
{
    // blocks on their way back through the bounce buffers first: their transfers may not even be
    // queued yet
    const cudaError_t staged = t_out_batch.wait();
    if (staged != cudaSuccess) return check_cuda(staged, "staged copy to host", __FILE__, __LINE__);
    cudaError_t e = cudaStreamSynchronize(s->in);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->run);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s->out);
    if (e != cudaSuccess) return check_cuda(e, "stream synchronize", __FILE__, __LINE__);
    return poll_device_error();
}

// C <- alpha*op(A)*op(B) + beta*C with host or device pointers.
// Host operands: A goes over whole; B (and C when beta != 0) go over in column
// blocks on the copy-in stream, each block's product runs on the compute
// stream as soon as its inputs have landed, and its C block returns on the
// copy-out stream while the next block computes.
template <typename T, typename Launch>
static int gemm_any(Launch launch, int transA, int transB, int64_t m, int64_t n, int64_t k,
                    const T *A, int64_t lda, const T *B, int64_t ldb, bool read_c, T *C, int64_t ldc,
                    bool scale_only)
{
    ULMB_SERIALISE;
    if (m == 0 || n == 0) return set_status(ULMB200_OK);
    if (int s0 = ensure_device()) return set_status(s0);
    // alpha == 0 or k == 0: only C <- beta*C happens and A and B are never touched, as in the
    // reference (ulmblas/level3/gemm.tcc:52-55) -- callers may pass dummy pointers for them
    if (scale_only) { A = nullptr; B = nullptr; k = 0; }
    const bool dC = on_device(C);
    const bool dA = scale_only ? dC : on_device(A), dB = scale_only ? dC : on_device(B);
    if (dA && dB && dC) {
        int st = launch(nullptr, A, lda, B, ldb, C, ldc, 0, n, 0, k, true);
        if (st != ULMB200_OK) return set_status(st);
        if (int e = check_cuda(cudaStreamSynchronize(nullptr), "synchronize", __FILE__, __LINE__)) return e;
        return set_status(poll_device_error());
    }
    Streams *s = streams();
    if (!s) return set_status(ULMB200_CUDA_ERROR);

    const int64_t rowsA = transA ? k : m, colsA = transA ? m : k;
    const int64_t rowsB = transB ? n : k, colsB = transB ? k : n;
    const int64_t dlda = round_up(std::max<int64_t>(rowsA, 1), 2);
    const int64_t dldb = round_up(std::max<int64_t>(rowsB, 1), 2);
    const int64_t dldc = round_up(m, 2);
    const T *Ad = A, *Bd = B;
    T *Cd = C;
    int64_t ua = lda, ub = ldb, uc = ldc;
    if (!dA) { Ad = static_cast<T *>(device_scratch(0, sizeof(T) * dlda * std::max<int64_t>(colsA, 1))); ua = dlda; }
    if (!dB) { Bd = static_cast<T *>(device_scratch(1, sizeof(T) * dldb * std::max<int64_t>(colsB, 1))); ub = dldb; }
    if (!dC) { Cd = static_cast<T *>(device_scratch(2, sizeof(T) * dldc * n)); uc = dldc; }
    if (!Ad || !Bd || !Cd) return set_status(ULMB200_CUDA_ERROR);

    HostPin pa(dA ? nullptr : A, span_bytes<T>(rowsA, colsA, lda));
    HostPin pb(dB ? nullptr : B, span_bytes<T>(rowsB, colsB, ldb));
    HostPin pc(dC ? nullptr : C, span_bytes<T>(m, n, ldc));

    cudaError_t e = cudaSuccess;
    // Column blocks of B and C: big enough to keep the GEMM efficient, small enough to overlap.  The
    // last block is cut into four, so that less of the final copy back to the host is exposed.
    int64_t nblk = std::min<int64_t>(16, std::max<int64_t>(1, (sizeof(T) * m * n) >> 27));
    int64_t nc = round_up((n + nblk - 1) / nblk, 128);
    nblk = (n + nc - 1) / nc;
    if (nblk > 31) { nc = round_up((n + 30) / 31, 128); nblk = (n + nc - 1) / nc; }
    struct Blk { int64_t j0, jn; };
    Blk blocks[40];
    int nblocks = 0;
    for (int64_t b = 0; b < nblk; ++b) {
        const int64_t j0 = b * nc, jn = std::min(nc, n - j0);
        if (b == nblk - 1 && nblk >= 4 && !dC && jn >= 4 * 128) {
            const int64_t q = round_up((jn + 3) / 4, 128);
            for (int64_t o = 0; o < jn; o += q) blocks[nblocks++] = {j0 + o, std::min(q, jn - o)};
        } else {
            blocks[nblocks++] = {j0, jn};
        }
    }
    // A host-resident A travels in K panels, and the first column block is multiplied panel by panel
    // as they arrive: the product starts after one panel (and the first block of B), not after all of A.
    const int64_t bytesA = (int64_t)sizeof(T) * rowsA * colsA;
    int64_t npan = (!dA && k > 0) ? std::min<int64_t>(16, bytesA >> 29) : 1;
    if (npan < 1) npan = 1;
    while (npan > 1 && k / npan < 512) --npan;
    const int64_t kp = round_up((k + npan - 1) / npan, 128);
    npan = k > 0 ? (k + kp - 1) / kp : 1;
    constexpr int kEvA = 96;                                  // events of the A panels

    // B^T blocks are row ranges of the stored matrix: ship B whole in that case
    if (!dB && transB && k > 0) {
        e = copy_in(const_cast<T *>(Bd), ub, B, ldb, rowsB, colsB, s->in);
        if (e != cudaSuccess) return check_cuda(e, "copy B", __FILE__, __LINE__);
    }
    for (int b = 0; b < nblocks; ++b) {
        const int64_t j0 = blocks[b].j0, jn = blocks[b].jn;
        if (!dB && !transB && k > 0) e = copy_in(const_cast<T *>(Bd) + j0 * ub, ub, B + j0 * ldb, ldb, rowsB, jn, s->in);
        if (e == cudaSuccess && !dC && read_c) e = copy_in(Cd + j0 * uc, uc, C + j0 * ldc, ldc, m, jn, s->in);
        if (e == cudaSuccess) e = cudaEventRecord(s->ev[2 * b], s->in);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(s->run, s->ev[2 * b], 0);
        if (e != cudaSuccess) return check_cuda(e, "stage block", __FILE__, __LINE__);
        int st = ULMB200_OK;
        if (b == 0 && !dA && k > 0) {
            // A follows the first block of B on the copy stream, one K panel at a time
            for (int64_t pn = 0; pn < npan && st == ULMB200_OK; ++pn) {
                const int64_t k0 = pn * kp, kn = std::min(kp, k - k0);
                // op(A)[:, k0:k0+kn] is a column range of A as stored, or a row range of A^T as stored
                if (!transA) e = copy_in(const_cast<T *>(Ad) + k0 * ua, ua, A + k0 * lda, lda, rowsA, kn, s->in);
                else         e = copy_in(const_cast<T *>(Ad) + k0, ua, A + k0, lda, kn, colsA, s->in);
                if (e == cudaSuccess) e = cudaEventRecord(s->ev[kEvA + pn], s->in);
                if (e == cudaSuccess) e = cudaStreamWaitEvent(s->run, s->ev[kEvA + pn], 0);
                if (e != cudaSuccess) return check_cuda(e, "stage A panel", __FILE__, __LINE__);
                st = launch(s->run, Ad, ua, Bd, ub, Cd, uc, j0, jn, k0, kn, pn == 0);
            }
        } else {
            st = launch(s->run, Ad, ua, Bd, ub, Cd, uc, j0, jn, 0, k, true);
        }
        if (st != ULMB200_OK) { finish(s); return set_status(st); }
        if (!dC) {
            e = cudaEventRecord(s->ev[2 * b + 1], s->run);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(s->out, s->ev[2 * b + 1], 0);
            if (e == cudaSuccess) e = copy_out(C + j0 * ldc, ldc, Cd + j0 * uc, uc, m, jn, s->out);
            if (e != cudaSuccess) return check_cuda(e, "return block", __FILE__, __LINE__);
        }
    }
    return set_status(finish(s));
}

static int dgemm_any(int transA, int transB, int64_t m, int64_t n, int64_t k, double alpha,
                     const double *A, int64_t lda, const double *B, int64_t ldb, double beta,
                     double *C, int64_t ldc)
{
    // columns [j0, j0+jn) of C from the K range [k0, k0+kn); beta applies on the first range only
    auto launch = [=](cudaStream_t st, const double *Ad, int64_t ua, const double *Bd, int64_t ub,
                      double *Cd, int64_t uc, int64_t j0, int64_t jn, int64_t k0, int64_t kn, bool first) {
        const double *Ablk = transA ? Ad + k0 : Ad + k0 * ua;
        const double *Bblk = transB ? Bd + j0 + k0 * ub : Bd + j0 * ub + k0;
        return dgemm_device(st, 0, transA, transB, m, jn, kn, alpha, Ablk, ua, Bblk, ub, first ? beta : 1.0,
                            Cd + j0 * uc, uc);
    };
    const double t0 = settings().trace ? now_ms() : 0.0;
    const int st = gemm_any<double>(launch, transA, transB, m, n, k, A, lda, B, ldb, beta != 0.0, C, ldc,
                                    alpha == 0.0 || k == 0);
    trace("dgemm %c%c m=%lld n=%lld k=%lld lda=%lld ldb=%lld ldc=%lld alpha=%g beta=%g status=%d %.3f ms",
          transA ? 'T' : 'N', transB ? 'T' : 'N', (long long)m, (long long)n, (long long)k, (long long)lda,
          (long long)ldb, (long long)ldc, alpha, beta, st, now_ms() - t0);
    return st;
}

static int sgemm_mode()
{
    return settings().sgemm_3xtf32 ? ULMB200_SGEMM_3XTF32 : ULMB200_SGEMM_FP32;
}

static int sgemm_any(int transA, int transB, int64_t m, int64_t n, int64_t k, float alpha,
                     const float *A, int64_t lda, const float *B, int64_t ldb, float beta, float *C,
                     int64_t ldc)
{
    const int mode = sgemm_mode();
    auto launch = [=](cudaStream_t st, const float *Ad, int64_t ua, const float *Bd, int64_t ub,
                      float *Cd, int64_t uc, int64_t j0, int64_t jn, int64_t k0, int64_t kn, bool first) {
        const float *Ablk = transA ? Ad + k0 : Ad + k0 * ua;
        const float *Bblk = transB ? Bd + j0 + k0 * ub : Bd + j0 * ub + k0;
        return sgemm_device(st, mode, transA, transB, m, jn, kn, alpha, Ablk, ua, Bblk, ub, first ? beta : 1.0f,
                            Cd + j0 * uc, uc);
    };
    const double t0 = settings().trace ? now_ms() : 0.0;
    const int st = gemm_any<float>(launch, transA, transB, m, n, k, A, lda, B, ldb, beta != 0.0f, C, ldc,
                                   alpha == 0.0f || k == 0);
    trace("sgemm %c%c m=%lld n=%lld k=%lld mode=%s status=%d %.3f ms", transA ? 'T' : 'N', transB ? 'T' : 'N',
          (long long)m, (long long)n, (long long)k, mode == ULMB200_SGEMM_3XTF32 ? "3xtf32" : "fp32", st,
          now_ms() - t0);
    return st;
}

// Staging for the two-operand routines (whole matrices; no pipelining).
static int dsyrk_any(int lower, int trans, int64_t n, int64_t k, double alpha, const double *A,
                     int64_t lda, double beta, double *C, int64_t ldc)
{
    ULMB_SERIALISE;
    if (n == 0) return set_status(ULMB200_OK);
    if (int s0 = ensure_device()) return set_status(s0);
    // alpha == 0 or k == 0 only scales the triangle; A is not touched (syurk.tcc:44-51)
    const bool scale_only = alpha == 0.0 || k == 0;
    if (scale_only) { k = 0; alpha = 0.0; }
    const bool dC = on_device(C), dA = scale_only ? true : on_device(A);
    Streams *s = streams();
    if (!s) return set_status(ULMB200_CUDA_ERROR);
    const int64_t rowsA = trans ? k : n, colsA = trans ? n : k;
    const double *Ad = scale_only ? C : A;
    double *Cd = C;
    int64_t ua = lda, uc = ldc;
    if (!dA) { ua = round_up(std::max<int64_t>(rowsA, 1), 2); Ad = static_cast<double *>(device_scratch(0, 8 * ua * std::max<int64_t>(colsA, 1))); }
    if (!dC) { uc = round_up(n, 2); Cd = static_cast<double *>(device_scratch(2, 8 * uc * n)); }
    if (!Ad || !Cd) return set_status(ULMB200_CUDA_ERROR);
    cudaError_t e = cudaSuccess;
    if (!dA && k > 0) e = copy_in(const_cast<double *>(Ad), ua, A, lda, rowsA, colsA, s->run);
    // the whole square goes over and comes back; the kernel only writes the triangle,
    // so the other triangle returns bit-identical
    if (e == cudaSuccess && !dC) e = copy_in(Cd, uc, C, ldc, n, n, s->run);
    if (e != cudaSuccess) return check_cuda(e, "copy in", __FILE__, __LINE__);
    int st = dsyrk_device(s->run, lower, trans, n, k, alpha, Ad, ua, beta, Cd, uc);
    if (st != ULMB200_OK) { finish(s); return set_status(st); }
    if (!dC) {
        e = copy_out(C, ldc, Cd, uc, n, n, s->run);
        if (e != cudaSuccess) return check_cuda(e, "copy out", __FILE__, __LINE__);
    }
    return set_status(finish(s));
}

static int dtrsm_any(int side, int lower, int transA, int unit, int64_t m, int64_t n, double alpha,
                     const double *A, int64_t lda, double *B, int64_t ldb)
{
    ULMB_SERIALISE;
    if (m == 0 || n == 0) return set_status(ULMB200_OK);
    if (int s0 = ensure_device()) return set_status(s0);
    // alpha == 0 assigns zeros to B and reads neither A nor B (trlsm.tcc:46-49)
    const bool zero_only = alpha == 0.0;
    const bool dB = on_device(B), dA = zero_only ? true : on_device(A);
    Streams *s = streams();
    if (!s) return set_status(ULMB200_CUDA_ERROR);
    const int64_t dim = side == 0 ? m : n;
    const double *Ad = zero_only ? B : A;
    double *Bd = B;
    int64_t ua = lda, ub = ldb;
    if (!dA) { ua = round_up(dim, 2); Ad = static_cast<double *>(device_scratch(0, 8 * ua * dim)); }
    if (!dB) { ub = round_up(m, 2); Bd = static_cast<double *>(device_scratch(2, 8 * ub * n)); }
    if (!Ad || !Bd) return set_status(ULMB200_CUDA_ERROR);
    cudaError_t e = cudaSuccess;
    // The whole square of A is shipped, but the kernels only ever read the
    // referenced triangle (and skip the diagonal when it is unit).
    if (!dA) e = copy_in(const_cast<double *>(Ad), ua, A, lda, dim, dim, s->run);
    if (e == cudaSuccess && !dB && !zero_only) e = copy_in(Bd, ub, B, ldb, m, n, s->run);
    if (e != cudaSuccess) return check_cuda(e, "copy in", __FILE__, __LINE__);
    int st = dtrsm_device(s->run, side, lower, transA, unit, m, n, alpha, Ad, ua, Bd, ub);
    if (st != ULMB200_OK) { finish(s); return set_status(st); }
    if (!dB) {
        e = copy_out(B, ldb, Bd, ub, m, n, s->run);
        if (e != cudaSuccess) return check_cuda(e, "copy out", __FILE__, __LINE__);
    }
    return set_status(finish(s));
}

// One staged operand: device pointers pass through, host matrices are copied into a cached
// device buffer (slot) before the call and, when `back`, copied out after it.
template <typename T>
struct StagedT {
    const T *host = nullptr;
    T *dev = nullptr;
    int64_t ldh = 0, ldd = 0, rows = 0, cols = 0;
    bool staged = false;
};
typedef StagedT<double> Staged;

template <typename T>
static int stage_in(StagedT<T> &o, const T *p, int64_t ld, int64_t rows, int64_t cols, int slot, bool copy,
                    cudaStream_t st)
{
    o.host = p; o.ldh = ld; o.rows = rows; o.cols = cols;
    if (on_device(p) || rows <= 0 || cols <= 0) { o.dev = const_cast<T *>(p); o.ldd = ld; return ULMB200_OK; }
    o.ldd = round_up(rows, 4);
    o.dev = static_cast<T *>(device_scratch(slot, sizeof(T) * (size_t)(o.ldd * cols)));
    if (!o.dev) return ULMB200_CUDA_ERROR;
    o.staged = true;
    if (copy) return check_cuda(copy_in(o.dev, o.ldd, p, ld, rows, cols, st), "copy in", __FILE__, __LINE__);
    return ULMB200_OK;
}

template <typename T>
static int stage_out(const StagedT<T> &o, cudaStream_t st)
{
    if (!o.staged) return ULMB200_OK;
    return check_cuda(copy_out(const_cast<T *>(o.host), o.ldh, o.dev, o.ldd, o.rows, o.cols, st), "copy out",
                      __FILE__, __LINE__);
}

static int ssyrk_any(int lower, int trans, int64_t n, int64_t k, float alpha, const float *A, int64_t lda,
                     float beta, float *C, int64_t ldc)
{
    ULMB_SERIALISE;
    if (n == 0) return set_status(ULMB200_OK);
    if (int s0 = ensure_device()) return set_status(s0);
    Streams *s = streams();
    if (!s) return set_status(ULMB200_CUDA_ERROR);
    const int64_t rows = trans ? k : n, cols = trans ? n : k;
    StagedT<float> a, c;
    int st = stage_in(a, A, lda, rows, cols, 0, true, s->run);
    if (st == ULMB200_OK) st = stage_in(c, C, ldc, n, n, 2, true, s->run);
    if (st == ULMB200_OK) st = ssyrk_device(s->run, lower, trans, n, k, alpha, a.dev, a.ldd, beta, c.dev, c.ldd);
    if (st == ULMB200_OK) st = stage_out(c, s->run);
    const int fin = finish(s);
    return set_status(st != ULMB200_OK ? st : fin);
}

static int strsm_any(int side, int lower, int transA, int unit, int64_t m, int64_t n, float alpha,
                     const float *A, int64_t lda, float *B, int64_t ldb)
{
    ULMB_SERIALISE;
    if (m == 0 || n == 0) return set_status(ULMB200_OK);
    if (int s0 = ensure_device()) return set_status(s0);
    Streams *s = streams();
    if (!s) return set_status(ULMB200_CUDA_ERROR);
    const int64_t dim = side == 0 ? m : n;
    StagedT<float> a, b;
    int st = stage_in(a, A, lda, dim, dim, 0, true, s->run);
    if (st == ULMB200_OK) st = stage_in(b, B, ldb, m, n, 2, true, s->run);
    if (st == ULMB200_OK) st = strsm_device(s->run, side, lower, transA, unit, m, n, alpha, a.dev, a.ldd, b.dev, b.ldd);
    if (st == ULMB200_OK) st = stage_out(b, s->run);
    const int fin = finish(s);
    return set_status(st != ULMB200_OK ? st : fin);
}

static int dtrmm_any(int side, int lower, int transA, int unit, int64_t m, int64_t n, double alpha,
                     const double *A, int64_t lda, double *B, int64_t ldb)
{
    ULMB_SERIALISE;
    if (m == 0 || n == 0) return set_status(ULMB200_OK);
    if (int s0 = ensure_device()) return set_status(s0);
    Streams *s = streams();
    if (!s) return set_status(ULMB200_CUDA_ERROR);
    const int64_t dim = side == 0 ? m : n;
    Staged a, b;
    int st = stage_in(a, A, lda, dim, dim, 0, true, s->run);
    if (st == ULMB200_OK) st = stage_in(b, B, ldb, m, n, 2, true, s->run);
    if (st == ULMB200_OK) st = dtrmm_device(s->run, side, lower, transA, unit, m, n, alpha, a.dev, a.ldd, b.dev, b.ldd);
    if (st == ULMB200_OK) st = stage_out(b, s->run);
    const int fin = finish(s);
    return set_status(st != ULMB200_OK ? st : fin);
}

static int dsymm_any(int side, int lower, int64_t m, int64_t n, double alpha, const double *A, int64_t lda,
                     const double *B, int64_t ldb, double beta, double *C, int64_t ldc)
{
    ULMB_SERIALISE;
    if (m == 0 || n == 0) return set_status(ULMB200_OK);
    if (int s0 = ensure_device()) return set_status(s0);
    Streams *s = streams();
    if (!s) return set_status(ULMB200_CUDA_ERROR);
    const int64_t na = side == 0 ? m : n;
    Staged a, b, c;
    int st = stage_in(a, A, lda, na, na, 0, true, s->run);
    if (st == ULMB200_OK) st = stage_in(b, B, ldb, m, n, 1, true, s->run);
    if (st == ULMB200_OK) st = stage_in(c, C, ldc, m, n, 2, beta != 0.0, s->run);
    if (st == ULMB200_OK) st = dsymm_device(s->run, side, lower, m, n, alpha, a.dev, a.ldd, b.dev, b.ldd, beta, c.dev, c.ldd);
    if (st == ULMB200_OK) st = stage_out(c, s->run);
    const int fin = finish(s);
    return set_status(st != ULMB200_OK ? st : fin);
}

static int dsyr2k_any(int lower, int trans, int64_t n, int64_t k, double alpha, const double *A, int64_t lda,
                      const double *B, int64_t ldb, double beta, double *C, int64_t ldc)
{
    ULMB_SERIALISE;
    if (n == 0) return set_status(ULMB200_OK);
    if (int s0 = ensure_device()) return set_status(s0);
    Streams *s = streams();
    if (!s) return set_status(ULMB200_CUDA_ERROR);
    const int64_t rows = trans ? k : n, cols = trans ? n : k;
    Staged a, b, c;
    int st = stage_in(a, A, lda, rows, cols, 0, true, s->run);
    if (st == ULMB200_OK) st = stage_in(b, B, ldb, rows, cols, 1, true, s->run);
    // the whole square travels both ways; the kernels only touch the requested triangle
    if (st == ULMB200_OK) st = stage_in(c, C, ldc, n, n, 2, true, s->run);
    if (st == ULMB200_OK) st = dsyr2k_device(s->run, lower, trans, n, k, alpha, a.dev, a.ldd, b.dev, b.ldd, beta, c.dev, c.ldd);
    if (st == ULMB200_OK) st = stage_out(c, s->run);
    const int fin = finish(s);
    return set_status(st != ULMB200_OK ? st : fin);
}

// Complex double GEMM with host or device operands (interleaved re/im, ld in complex elements).
static int zgemm_any(int transA, int conjA, int transB, int conjB, int64_t m, int64_t n, int64_t k,
                     const double *alpha, const double *A, int64_t lda, const double *B, int64_t ldb,
                     const double *beta, double *C, int64_t ldc)
{
    ULMB_SERIALISE;
    if (m == 0 || n == 0) return set_status(ULMB200_OK);
    if (int s0 = ensure_device()) return set_status(s0);
    Streams *s = streams();
    if (!s) return set_status(ULMB200_CUDA_ERROR);
    const bool scale_only = (alpha[0] == 0.0 && alpha[1] == 0.0) || k == 0;
    const bool beta_zero = beta[0] == 0.0 && beta[1] == 0.0;
    StagedT<double2> a, b, c;
    int st = ULMB200_OK;
    if (!scale_only) {
        st = stage_in(a, reinterpret_cast<const double2 *>(A), lda, transA ? k : m, transA ? m : k, 0, true, s->run);
        if (st == ULMB200_OK)
            st = stage_in(b, reinterpret_cast<const double2 *>(B), ldb, transB ? n : k, transB ? k : n, 1, true, s->run);
    } else {
        a.dev = nullptr; a.ldd = std::max<int64_t>(1, transA ? k : m);
        b.dev = nullptr; b.ldd = std::max<int64_t>(1, transB ? n : k);
    }
    if (st == ULMB200_OK)
        st = stage_in(c, reinterpret_cast<const double2 *>(C), ldc, m, n, 2, !beta_zero, s->run);
    if (st == ULMB200_OK)
        st = zgemm_device(s->run, transA, conjA, transB, conjB, m, n, k, alpha,
                          reinterpret_cast<const double *>(a.dev), a.ldd,
                          reinterpret_cast<const double *>(b.dev), b.ldd, beta,
                          reinterpret_cast<double *>(c.dev), c.ldd);
    if (st == ULMB200_OK) st = stage_out(c, s->run);
    const int fin = finish(s);
    return set_status(st != ULMB200_OK ? st : fin);
}

// ---- argument decoding shared by the shims ---------------------------------
static inline int up(const char *c) { return std::toupper((unsigned char)*c); }
static inline bool is_trans(const char *c) { int u = up(c); return u == 'T' || u == 'C'; }
static inline bool is_conj(const char *c) { int u = up(c); return u == 'C' || u == 'R'; }
static inline bool valid_trans(const char *c) { int u = up(c); return u == 'N' || u == 'T' || u == 'C' || u == 'R'; }

static int gemm_info(const char *ta, const char *tb, int m, int n, int k, int lda, int ldb, int ldc)
{
    const int rowsA = !is_trans(ta) ? m : k, rowsB = !is_trans(tb) ? k : n;
    if (!valid_trans(ta)) return 1;
    if (!valid_trans(tb)) return 2;
    if (m < 0) return 3;
    if (n < 0) return 4;
    if (k < 0) return 5;
    if (lda < std::max(1, rowsA)) return 8;
    if (ldb < std::max(1, rowsB)) return 10;
    if (ldc < std::max(1, m)) return 13;
    return 0;
}

}  // namespace ulmb200

using namespace ulmb200;

extern "C" {

int CBLAS_CallFromC = 0;
int RowMajorStrg = 0;

__attribute__((weak)) void xerbla_(const char rout[6], const int *info)
{
    // same text as interfaces/blas/F77/xerbla.cc:9; rout is 6 blank-padded characters
    fprintf(stderr, "Parameter %d to routine %.6s was incorrect\n", *info, rout);
}

__attribute__((weak)) void cblas_xerbla(int info, const char *rout, const char *form, ...)
{
    (void)form;
    fprintf(stderr, "Parameter %d to routine %s was incorrect\n", info, rout);
}

// ULMBLAS(xerbla), interfaces/blas/C/xerbla.cc:7-11: the reference's libcblas exports it beside
// CBLAS(xerbla) with the same text
__attribute__((weak)) void ulmblas_xerbla(int info, const char *rout, const char *form, ...)
{
    (void)form;
    fprintf(stderr, "Parameter %d to routine %s was incorrect\n", info, rout);
}

void ulmb200_set_pin_host(int on) { g_pin_host = on ? 1 : 0; }

// ---------------------------- Fortran ABI -----------------------------------

void dgemm_(const char *transA, const char *transB, const int *m, const int *n, const int *k,
            const double *alpha, const double *A, const int *ldA, const double *B, const int *ldB,
            const double *beta, double *C, const int *ldC)
{
    int info = gemm_info(transA, transB, *m, *n, *k, *ldA, *ldB, *ldC);
    if (info != 0) {
        xerbla_("DGEMM ", &info);
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    dgemm_any(is_trans(transA), is_trans(transB), *m, *n, *k, *alpha, A, *ldA, B, *ldB, *beta, C, *ldC);
}

// interfaces/blas/F77/gemm.cc:381-510.  'C' = conjugate transpose, 'R' = conjugate only.
void zgemm_(const char *transA, const char *transB, const int *m, const int *n, const int *k,
            const double *alpha, const double *A, const int *ldA, const double *B, const int *ldB,
            const double *beta, double *C, const int *ldC)
{
    int info = gemm_info(transA, transB, *m, *n, *k, *ldA, *ldB, *ldC);
    if (info != 0) {
        xerbla_("ZGEMM ", &info);
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    zgemm_any(is_trans(transA), is_conj(transA), is_trans(transB), is_conj(transB), *m, *n, *k, alpha, A,
              *ldA, B, *ldB, beta, C, *ldC);
}

void sgemm_(const char *transA, const char *transB, const int *m, const int *n, const int *k,
            const float *alpha, const float *A, const int *ldA, const float *B, const int *ldB,
            const float *beta, float *C, const int *ldC)
{
    int info = gemm_info(transA, transB, *m, *n, *k, *ldA, *ldB, *ldC);
    if (info != 0) {
        xerbla_("SGEMM ", &info);
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    sgemm_any(is_trans(transA), is_trans(transB), *m, *n, *k, *alpha, A, *ldA, B, *ldB, *beta, C, *ldC);
}

void dtrsm_(const char *side, const char *upLo, const char *transA, const char *diag, const int *m,
            const int *n, const double *alpha, const double *A, const int *ldA, double *B,
            const int *ldB)
{
    const bool left = up(side) == 'L';
    const int rowsA = left ? *m : *n;
    int info = 0;
    if (up(side) != 'L' && up(side) != 'R') info = 1;
    else if (up(upLo) != 'L' && up(upLo) != 'U') info = 2;
    else if (!valid_trans(transA)) info = 3;
    else if (up(diag) != 'U' && up(diag) != 'N') info = 4;
    else if (*m < 0) info = 5;
    else if (*n < 0) info = 6;
    else if (*ldA < std::max(1, rowsA)) info = 9;
    else if (*ldB < std::max(1, *m)) info = 11;
    if (info != 0) {
        xerbla_("DTRSM ", &info);
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    dtrsm_any(left ? 0 : 1, up(upLo) == 'L', is_trans(transA), up(diag) == 'U', *m, *n, *alpha, A, *ldA, B, *ldB);
}

void dsyrk_(const char *upLo, const char *trans, const int *n, const int *k, const double *alpha,
            const double *A, const int *ldA, const double *beta, double *C, const int *ldC)
{
    const int rowsA = is_trans(trans) ? *k : *n;
    int info = 0;
    if (up(upLo) != 'L' && up(upLo) != 'U') info = 1;
    else if (!valid_trans(trans)) info = 2;
    else if (*n < 0) info = 3;
    else if (*k < 0) info = 4;
    else if (*ldA < std::max(1, rowsA)) info = 7;
    else if (*ldC < std::max(1, *n)) info = 10;
    if (info != 0) {
        xerbla_("DSYRK ", &info);
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    dsyrk_any(up(upLo) == 'L', is_trans(trans), *n, *k, *alpha, A, *ldA, *beta, C, *ldC);
}

// replaces F77BLAS(dsymm), interfaces/blas/F77/symm.cc:87-150
void dsymm_(const char *side, const char *upLo, const int *m, const int *n, const double *alpha,
            const double *A, const int *ldA, const double *B, const int *ldB, const double *beta,
            double *C, const int *ldC)
{
    const bool left = up(side) == 'L';
    const int rowsA = left ? *m : *n;
    int info = 0;
    if (up(side) != 'L' && up(side) != 'R') info = 1;
    else if (up(upLo) != 'L' && up(upLo) != 'U') info = 2;
    else if (*m < 0) info = 3;
    else if (*n < 0) info = 4;
    else if (*ldA < std::max(1, rowsA)) info = 7;
    else if (*ldB < std::max(1, *m)) info = 9;
    else if (*ldC < std::max(1, *m)) info = 12;
    if (info != 0) {
        xerbla_("DSYMM ", &info);
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    dsymm_any(left ? 0 : 1, up(upLo) == 'L', *m, *n, *alpha, A, *ldA, B, *ldB, *beta, C, *ldC);
}

// replaces F77BLAS(dtrmm), interfaces/blas/F77/trmm.cc:123-230
void dtrmm_(const char *side, const char *upLo, const char *transA, const char *diag, const int *m,
            const int *n, const double *alpha, const double *A, const int *ldA, double *B,
            const int *ldB)
{
    const bool left = up(side) == 'L';
    const int rowsA = left ? *m : *n;
    int info = 0;
    if (up(side) != 'L' && up(side) != 'R') info = 1;
    else if (up(upLo) != 'L' && up(upLo) != 'U') info = 2;
    else if (!valid_trans(transA)) info = 3;
    else if (up(diag) != 'U' && up(diag) != 'N') info = 4;
    else if (*m < 0) info = 5;
    else if (*n < 0) info = 6;
    else if (*ldA < std::max(1, rowsA)) info = 9;
    else if (*ldB < std::max(1, *m)) info = 11;
    if (info != 0) {
        xerbla_("DTRMM ", &info);
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    dtrmm_any(left ? 0 : 1, up(upLo) == 'L', is_trans(transA), up(diag) == 'U', *m, *n, *alpha, A, *ldA, B, *ldB);
}

// replaces F77BLAS(dsyr2k), interfaces/blas/F77/syr2k.cc:92-170
void dsyr2k_(const char *upLo, const char *trans, const int *n, const int *k, const double *alpha,
             const double *A, const int *ldA, const double *B, const int *ldB, const double *beta,
             double *C, const int *ldC)
{
    const int rows = is_trans(trans) ? *k : *n;
    int info = 0;
    if (up(upLo) != 'L' && up(upLo) != 'U') info = 1;
    else if (!valid_trans(trans)) info = 2;
    else if (*n < 0) info = 3;
    else if (*k < 0) info = 4;
    else if (*ldA < std::max(1, rows)) info = 7;
    else if (*ldB < std::max(1, rows)) info = 9;
    else if (*ldC < std::max(1, *n)) info = 12;
    if (info != 0) {
        xerbla_("DSYR2K", &info);
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    dsyr2k_any(up(upLo) == 'L', is_trans(trans), *n, *k, *alpha, A, *ldA, B, *ldB, *beta, C, *ldC);
}

// replaces F77BLAS(strsm), interfaces/blas/F77/trsm.cc (float operands, double arithmetic)
void strsm_(const char *side, const char *upLo, const char *transA, const char *diag, const int *m,
            const int *n, const float *alpha, const float *A, const int *ldA, float *B, const int *ldB)
{
    const bool left = up(side) == 'L';
    const int rowsA = left ? *m : *n;
    int info = 0;
    if (up(side) != 'L' && up(side) != 'R') info = 1;
    else if (up(upLo) != 'L' && up(upLo) != 'U') info = 2;
    else if (!valid_trans(transA)) info = 3;
    else if (up(diag) != 'U' && up(diag) != 'N') info = 4;
    else if (*m < 0) info = 5;
    else if (*n < 0) info = 6;
    else if (*ldA < std::max(1, rowsA)) info = 9;
    else if (*ldB < std::max(1, *m)) info = 11;
    if (info != 0) {
        xerbla_("STRSM ", &info);
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    strsm_any(left ? 0 : 1, up(upLo) == 'L', is_trans(transA), up(diag) == 'U', *m, *n, *alpha, A, *ldA, B, *ldB);
}

// replaces F77BLAS(ssyrk), interfaces/blas/F77/syrk.cc (float operands, double arithmetic)
void ssyrk_(const char *upLo, const char *trans, const int *n, const int *k, const float *alpha,
            const float *A, const int *ldA, const float *beta, float *C, const int *ldC)
{
    const int rowsA = is_trans(trans) ? *k : *n;
    int info = 0;
    if (up(upLo) != 'L' && up(upLo) != 'U') info = 1;
    else if (!valid_trans(trans)) info = 2;
    else if (*n < 0) info = 3;
    else if (*k < 0) info = 4;
    else if (*ldA < std::max(1, rowsA)) info = 7;
    else if (*ldC < std::max(1, *n)) info = 10;
    if (info != 0) {
        xerbla_("SSYRK ", &info);
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    ssyrk_any(up(upLo) == 'L', is_trans(trans), *n, *k, *alpha, A, *ldA, *beta, C, *ldC);
}

// ------------------------------- CBLAS ---------------------------------------

static inline bool c_notrans(int t) { return t == CblasNoTrans || t == AtlasConj; }
static inline bool c_valid_trans(int t)
{
    return t == CblasNoTrans || t == CblasTrans || t == AtlasConj || t == CblasConjTrans;
}

void ulmblas_dgemm(enum CBLAS_TRANSPOSE transA, enum CBLAS_TRANSPOSE transB, int m, int n, int k,
                   double alpha, const double *A, int ldA, const double *B, int ldB, double beta,
                   double *C, int ldC)
{
    dgemm_any(!c_notrans(transA), !c_notrans(transB), m, n, k, alpha, A, ldA, B, ldB, beta, C, ldC);
}

void ulmblas_sgemm(enum CBLAS_TRANSPOSE transA, enum CBLAS_TRANSPOSE transB, int m, int n, int k,
                   float alpha, const float *A, int ldA, const float *B, int ldB, float beta,
                   float *C, int ldC)
{
    sgemm_any(!c_notrans(transA), !c_notrans(transB), m, n, k, alpha, A, ldA, B, ldB, beta, C, ldC);
}

// interfaces/blas/C/gemm.cc:219-292
void ulmblas_zgemm(enum CBLAS_TRANSPOSE transA, enum CBLAS_TRANSPOSE transB, int m, int n, int k,
                   const double *alpha, const double *A, int ldA, const double *B, int ldB,
                   const double *beta, double *C, int ldC)
{
    const bool conjA = (transA == AtlasConj || transA == CblasConjTrans);
    const bool conjB = (transB == AtlasConj || transB == CblasConjTrans);
    zgemm_any(!c_notrans(transA), conjA, !c_notrans(transB), conjB, m, n, k, alpha, A, ldA, B, ldB, beta, C, ldC);
}

// first-bad-argument code of CBLAS(dgemm)/CBLAS(sgemm), interfaces/blas/C/gemm.cc:426-466
static int cblas_gemm_info(int order, int transA, int transB, int m, int n, int k, int ldA, int ldB, int ldC)
{
    int rowsA, rowsB;
    if (order == CblasColMajor) {
        rowsA = c_notrans(transA) ? m : k;
        rowsB = c_notrans(transB) ? k : n;
    } else {
        rowsB = c_notrans(transB) ? n : k;
        rowsA = c_notrans(transA) ? k : m;
    }
    if (order != CblasColMajor && order != CblasRowMajor) return 1;
    if (!c_valid_trans(transA)) return 2;
    if (!c_valid_trans(transB)) return 3;
    if (order == CblasColMajor) {
        if (m < 0) return 4;
        if (n < 0) return 5;
        if (k < 0) return 6;
        if (ldA < std::max(1, rowsA)) return 9;
        if (ldB < std::max(1, rowsB)) return 11;
        if (ldC < std::max(1, m)) return 14;
    } else {
        if (n < 0) return 4;
        if (m < 0) return 5;
        if (k < 0) return 6;
        if (ldB < std::max(1, rowsB)) return 9;
        if (ldA < std::max(1, rowsA)) return 11;
        if (ldC < std::max(1, n)) return 14;
    }
    return 0;
}

void cblas_dgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE transA, enum CBLAS_TRANSPOSE transB,
                 int m, int n, int k, double alpha, const double *A, int ldA, const double *B,
                 int ldB, double beta, double *C, int ldC)
{
    int info = cblas_gemm_info(order, transA, transB, m, n, k, ldA, ldB, ldC);
    if (info != 0) {
        cblas_xerbla(info, "cblas_dgemm", "");
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    // row-major C = A*B is column-major C^T = B^T * A^T: swap the operands (gemm.cc:478-484)
    if (order == CblasColMajor) ulmblas_dgemm(transA, transB, m, n, k, alpha, A, ldA, B, ldB, beta, C, ldC);
    else                        ulmblas_dgemm(transB, transA, n, m, k, alpha, B, ldB, A, ldA, beta, C, ldC);
}

// interfaces/blas/C/gemm.cc:584-677 (same codes and the same operand swap as the real types)
void cblas_zgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE transA, enum CBLAS_TRANSPOSE transB,
                 int m, int n, int k, const double *alpha, const double *A, int ldA, const double *B,
                 int ldB, const double *beta, double *C, int ldC)
{
    int info = cblas_gemm_info(order, transA, transB, m, n, k, ldA, ldB, ldC);
    if (info != 0) {
        cblas_xerbla(info, "cblas_zgemm", "");
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    if (order == CblasColMajor) ulmblas_zgemm(transA, transB, m, n, k, alpha, A, ldA, B, ldB, beta, C, ldC);
    else                        ulmblas_zgemm(transB, transA, n, m, k, alpha, B, ldB, A, ldA, beta, C, ldC);
}

void cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE transA, enum CBLAS_TRANSPOSE transB,
                 int m, int n, int k, float alpha, const float *A, int ldA, const float *B, int ldB,
                 float beta, float *C, int ldC)
{
    int info = cblas_gemm_info(order, transA, transB, m, n, k, ldA, ldB, ldC);
    if (info != 0) {
        cblas_xerbla(info, "cblas_sgemm", "");
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    if (order == CblasColMajor) ulmblas_sgemm(transA, transB, m, n, k, alpha, A, ldA, B, ldB, beta, C, ldC);
    else                        ulmblas_sgemm(transB, transA, n, m, k, alpha, B, ldB, A, ldA, beta, C, ldC);
}

// First bad argument of CBLAS(?trsm), interfaces/blas/C/trsm.cc:325-371 (s) and :400-446 (d): the same
// order of tests for both types; m and n change places in the row-major numbering.
static int cblas_trsm_info(int order, int side, int upLo, int transA, int diag, int m, int n, int ldA, int ldB)
{
    const int rowsA = (side == CblasLeft) ? m : n;
    if (order != CblasColMajor && order != CblasRowMajor) return 1;
    if (side != CblasLeft && side != CblasRight) return 2;
    if (upLo != CblasLower && upLo != CblasUpper) return 3;
    if (!c_valid_trans((enum CBLAS_TRANSPOSE)transA)) return 4;
    if (diag != CblasUnit && diag != CblasNonUnit) return 5;
    if (order == CblasColMajor) {
        if (m < 0) return 6;
        if (n < 0) return 7;
        if (ldA < std::max(1, rowsA)) return 10;
        if (ldB < std::max(1, m)) return 12;
    } else {
        if (n < 0) return 6;
        if (m < 0) return 7;
        if (ldA < std::max(1, rowsA)) return 10;
        if (ldB < std::max(1, n)) return 12;
    }
    return 0;
}

// First bad argument of CBLAS(?syrk), interfaces/blas/C/syrk.cc:158-190 (s) and :218-250 (d).
static int cblas_syrk_info(int order, int upLo, int trans, int n, int k, int ldA, int ldC)
{
    if (order != CblasColMajor && order != CblasRowMajor) return 1;
    if (upLo != CblasLower && upLo != CblasUpper) return 2;
    if (!c_valid_trans((enum CBLAS_TRANSPOSE)trans)) return 3;
    const bool no = c_notrans((enum CBLAS_TRANSPOSE)trans);
    const int rowsA = order == CblasColMajor ? (no ? n : k) : (no ? k : n);
    if (n < 0) return 4;
    if (k < 0) return 5;
    if (ldA < std::max(1, rowsA)) return 8;
    if (ldC < std::max(1, n)) return 11;
    return 0;
}

void ulmblas_dtrsm(enum CBLAS_SIDE side, enum CBLAS_UPLO upLo, enum CBLAS_TRANSPOSE transA,
                   enum CBLAS_DIAG diag, int m, int n, double alpha, const double *A, int ldA,
                   double *B, int ldB)
{
    dtrsm_any(side == CblasLeft ? 0 : 1, upLo == CblasLower, !c_notrans(transA), diag == CblasUnit, m, n,
              alpha, A, ldA, B, ldB);
}

void cblas_dtrsm(enum CBLAS_ORDER order, enum CBLAS_SIDE side, enum CBLAS_UPLO upLo,
                 enum CBLAS_TRANSPOSE transA, enum CBLAS_DIAG diag, int m, int n, double alpha,
                 const double *A, int ldA, double *B, int ldB)
{
    const int info = cblas_trsm_info(order, side, upLo, transA, diag, m, n, ldA, ldB);
    if (info != 0) {
        cblas_xerbla(info, "cblas_dtrsm", "");
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    if (order == CblasColMajor) {
        ulmblas_dtrsm(side, upLo, transA, diag, m, n, alpha, A, ldA, B, ldB);
    } else {
        // interfaces/blas/C/trsm.cc:455-457
        ulmblas_dtrsm(side == CblasLeft ? CblasRight : CblasLeft,
                      upLo == CblasUpper ? CblasLower : CblasUpper, transA, diag, n, m, alpha, A, ldA, B, ldB);
    }
}

void ulmblas_dsyrk(enum CBLAS_UPLO upLo, enum CBLAS_TRANSPOSE trans, int n, int k, double alpha,
                   const double *A, int ldA, double beta, double *C, int ldC)
{
    dsyrk_any(upLo == CblasLower, !c_notrans(trans), n, k, alpha, A, ldA, beta, C, ldC);
}

void cblas_dsyrk(enum CBLAS_ORDER order, enum CBLAS_UPLO upLo, enum CBLAS_TRANSPOSE trans, int n,
                 int k, double alpha, const double *A, int ldA, double beta, double *C, int ldC)
{
    const int info = cblas_syrk_info(order, upLo, trans, n, k, ldA, ldC);
    if (info != 0) {
        cblas_xerbla(info, "cblas_dsyrk", "");
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    if (order == CblasColMajor) {
        ulmblas_dsyrk(upLo, trans, n, k, alpha, A, ldA, beta, C, ldC);
    } else {
        // interfaces/blas/C/syrk.cc:259-261
        ulmblas_dsyrk(upLo == CblasUpper ? CblasLower : CblasUpper,
                      c_notrans(trans) ? CblasTrans : CblasNoTrans, n, k, alpha, A, ldA, beta, C, ldC);
    }
}

// ---- single precision: CBLAS(strsm) interfaces/blas/C/trsm.cc:311-384, CBLAS(ssyrk) syrk.cc:146-203 ----
// (the kernels accumulate in double and round once, as the Fortran entry points strsm_ / ssyrk_ do)

void ulmblas_strsm(enum CBLAS_SIDE side, enum CBLAS_UPLO upLo, enum CBLAS_TRANSPOSE transA,
                   enum CBLAS_DIAG diag, int m, int n, float alpha, const float *A, int ldA, float *B, int ldB)
{
    strsm_any(side == CblasLeft ? 0 : 1, upLo == CblasLower, !c_notrans(transA), diag == CblasUnit, m, n,
              alpha, A, ldA, B, ldB);
}

void cblas_strsm(enum CBLAS_ORDER order, enum CBLAS_SIDE side, enum CBLAS_UPLO upLo,
                 enum CBLAS_TRANSPOSE transA, enum CBLAS_DIAG diag, int m, int n, float alpha,
                 const float *A, int ldA, float *B, int ldB)
{
    const int info = cblas_trsm_info(order, side, upLo, transA, diag, m, n, ldA, ldB);
    if (info != 0) {
        cblas_xerbla(info, "cblas_strsm", "");
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    if (order == CblasColMajor) {
        ulmblas_strsm(side, upLo, transA, diag, m, n, alpha, A, ldA, B, ldB);
    } else {
        // interfaces/blas/C/trsm.cc:380-382
        ulmblas_strsm(side == CblasLeft ? CblasRight : CblasLeft,
                      upLo == CblasUpper ? CblasLower : CblasUpper, transA, diag, n, m, alpha, A, ldA, B, ldB);
    }
}

void ulmblas_ssyrk(enum CBLAS_UPLO upLo, enum CBLAS_TRANSPOSE trans, int n, int k, float alpha,
                   const float *A, int ldA, float beta, float *C, int ldC)
{
    ssyrk_any(upLo == CblasLower, !c_notrans(trans), n, k, alpha, A, ldA, beta, C, ldC);
}

void cblas_ssyrk(enum CBLAS_ORDER order, enum CBLAS_UPLO upLo, enum CBLAS_TRANSPOSE trans, int n,
                 int k, float alpha, const float *A, int ldA, float beta, float *C, int ldC)
{
    const int info = cblas_syrk_info(order, upLo, trans, n, k, ldA, ldC);
    if (info != 0) {
        cblas_xerbla(info, "cblas_ssyrk", "");
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    if (order == CblasColMajor) {
        ulmblas_ssyrk(upLo, trans, n, k, alpha, A, ldA, beta, C, ldC);
    } else {
        // interfaces/blas/C/syrk.cc:199-201
        ulmblas_ssyrk(upLo == CblasUpper ? CblasLower : CblasUpper,
                      c_notrans(trans) ? CblasTrans : CblasNoTrans, n, k, alpha, A, ldA, beta, C, ldC);
    }
}

// ---- CBLAS twins of the three further gemm clients -----------------------------------------

void ulmblas_dsymm(enum CBLAS_SIDE side, enum CBLAS_UPLO upLo, int m, int n, double alpha, const double *A,
                   int ldA, const double *B, int ldB, double beta, double *C, int ldC)
{
    dsymm_any(side == CblasLeft ? 0 : 1, upLo == CblasLower, m, n, alpha, A, ldA, B, ldB, beta, C, ldC);
}

// replaces CBLAS(dsymm), interfaces/blas/C/symm.cc
void cblas_dsymm(enum CBLAS_ORDER order, enum CBLAS_SIDE side, enum CBLAS_UPLO upLo, int m, int n,
                 double alpha, const double *A, int ldA, const double *B, int ldB, double beta, double *C,
                 int ldC)
{
    const int rowsA = (side == CblasLeft) ? m : n;
    int info = 0;
    if (order != CblasColMajor && order != CblasRowMajor) info = 1;
    else if (side != CblasLeft && side != CblasRight) info = 2;
    else if (upLo != CblasLower && upLo != CblasUpper) info = 3;
    else if (order == CblasColMajor) {
        if (m < 0) info = 4;
        else if (n < 0) info = 5;
        else if (ldA < std::max(1, rowsA)) info = 8;
        else if (ldB < std::max(1, m)) info = 10;
        else if (ldC < std::max(1, m)) info = 13;
    } else {
        if (n < 0) info = 4;
        else if (m < 0) info = 5;
        else if (ldA < std::max(1, rowsA)) info = 8;
        else if (ldB < std::max(1, n)) info = 10;
        else if (ldC < std::max(1, n)) info = 13;
    }
    if (info != 0) {
        cblas_xerbla(info, "cblas_dsymm", "");
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    if (order == CblasColMajor) ulmblas_dsymm(side, upLo, m, n, alpha, A, ldA, B, ldB, beta, C, ldC);
    else ulmblas_dsymm(side == CblasLeft ? CblasRight : CblasLeft, upLo == CblasUpper ? CblasLower : CblasUpper,
                       n, m, alpha, A, ldA, B, ldB, beta, C, ldC);
}

void ulmblas_dtrmm(enum CBLAS_SIDE side, enum CBLAS_UPLO upLo, enum CBLAS_TRANSPOSE transA,
                   enum CBLAS_DIAG diag, int m, int n, double alpha, const double *A, int ldA, double *B,
                   int ldB)
{
    dtrmm_any(side == CblasLeft ? 0 : 1, upLo == CblasLower, !c_notrans(transA), diag == CblasUnit, m, n, alpha,
              A, ldA, B, ldB);
}

// replaces CBLAS(dtrmm), interfaces/blas/C/trmm.cc
void cblas_dtrmm(enum CBLAS_ORDER order, enum CBLAS_SIDE side, enum CBLAS_UPLO upLo,
                 enum CBLAS_TRANSPOSE transA, enum CBLAS_DIAG diag, int m, int n, double alpha,
                 const double *A, int ldA, double *B, int ldB)
{
    const int rowsA = (side == CblasLeft) ? m : n;
    int info = 0;
    if (order != CblasColMajor && order != CblasRowMajor) info = 1;
    else if (side != CblasLeft && side != CblasRight) info = 2;
    else if (upLo != CblasLower && upLo != CblasUpper) info = 3;
    else if (!c_valid_trans(transA)) info = 4;
    else if (diag != CblasUnit && diag != CblasNonUnit) info = 5;
    else if (order == CblasColMajor) {
        if (m < 0) info = 6;
        else if (n < 0) info = 7;
        else if (ldA < std::max(1, rowsA)) info = 10;
        else if (ldB < std::max(1, m)) info = 12;
    } else {
        if (n < 0) info = 6;
        else if (m < 0) info = 7;
        else if (ldA < std::max(1, rowsA)) info = 10;
        else if (ldB < std::max(1, n)) info = 12;
    }
    if (info != 0) {
        cblas_xerbla(info, "cblas_dtrmm", "");
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    if (order == CblasColMajor) ulmblas_dtrmm(side, upLo, transA, diag, m, n, alpha, A, ldA, B, ldB);
    else ulmblas_dtrmm(side == CblasLeft ? CblasRight : CblasLeft, upLo == CblasUpper ? CblasLower : CblasUpper,
                       transA, diag, n, m, alpha, A, ldA, B, ldB);
}

void ulmblas_dsyr2k(enum CBLAS_UPLO upLo, enum CBLAS_TRANSPOSE trans, int n, int k, double alpha,
                    const double *A, int ldA, const double *B, int ldB, double beta, double *C, int ldC)
{
    dsyr2k_any(upLo == CblasLower, !c_notrans(trans), n, k, alpha, A, ldA, B, ldB, beta, C, ldC);
}

// replaces CBLAS(dsyr2k), interfaces/blas/C/syr2k.cc
void cblas_dsyr2k(enum CBLAS_ORDER order, enum CBLAS_UPLO upLo, enum CBLAS_TRANSPOSE trans, int n, int k,
                  double alpha, const double *A, int ldA, const double *B, int ldB, double beta, double *C,
                  int ldC)
{
    int rows;
    if (order == CblasColMajor) rows = c_notrans(trans) ? n : k;
    else                        rows = c_notrans(trans) ? k : n;
    int info = 0;
    if (order != CblasColMajor && order != CblasRowMajor) info = 1;
    else if (upLo != CblasLower && upLo != CblasUpper) info = 2;
    else if (!c_valid_trans(trans)) info = 3;
    else if (n < 0) info = 4;
    else if (k < 0) info = 5;
    else if (ldA < std::max(1, rows)) info = 8;
    else if (ldB < std::max(1, rows)) info = 10;
    else if (ldC < std::max(1, n)) info = 13;
    if (info != 0) {
        cblas_xerbla(info, "cblas_dsyr2k", "");
        set_status(ULMB200_BAD_ARGUMENT);
        return;
    }
    if (order == CblasColMajor) ulmblas_dsyr2k(upLo, trans, n, k, alpha, A, ldA, B, ldB, beta, C, ldC);
    else ulmblas_dsyr2k(upLo == CblasUpper ? CblasLower : CblasUpper, c_notrans(trans) ? CblasTrans : CblasNoTrans,
                        n, k, alpha, B, ldB, A, ldA, beta, C, ldC);
}

// replaces ULMLAPACK(dgetrf), interfaces/lapack/C/getrf.cc:6-19 -> ulmBLAS::getrf
// (ulmblas/lapack/getrf.tcc:30-73).  Column-major only: for CblasRowMajor the reference runs
// getrf(n, m, A, ldA, 1), which addresses the array consistently only when m == n; that mode is
// refused here (return value -1) rather than imitated.  piv holds 0-based row indices, the
// return value is the 1-based index of the first zero pivot or 0.
int ulmblas_dgetrf(enum CBLAS_ORDER order, int m, int n, double *A, int ldA, int *piv)
{
    ULMB_SERIALISE;
    if (order != CblasColMajor || m < 0 || n < 0 || ldA < std::max(1, m)) {
        int info = order != CblasColMajor ? 1 : (m < 0 ? 2 : (n < 0 ? 3 : 5));
        cblas_xerbla(info, "ulmblas_dgetrf", "");
        set_status(ULMB200_BAD_ARGUMENT);
        return -info;
    }
    if (m == 0 || n == 0) { set_status(ULMB200_OK); return 0; }
    if (ensure_device() != ULMB200_OK) { set_status(ULMB200_NO_DEVICE); return -100; }
    Streams *s = streams();
    if (!s) { set_status(ULMB200_CUDA_ERROR); return -100; }
    const int mn = std::min(m, n);
    int *dints = static_cast<int *>(device_scratch(9, sizeof(int) * (size_t)(mn + 1)));
    if (!dints) { set_status(ULMB200_CUDA_ERROR); return -100; }
    Staged a;
    int st = stage_in(a, A, ldA, m, n, 2, true, s->run);
    if (st == ULMB200_OK) st = dgetrf_device(s->run, m, n, a.dev, a.ldd, dints, dints + mn);
    if (st == ULMB200_OK) st = stage_out(a, s->run);
    int info = 0;
    if (st == ULMB200_OK)
        st = check_cuda(cudaMemcpyAsync(piv, dints, sizeof(int) * mn, cudaMemcpyDeviceToHost, s->run), "piv", __FILE__, __LINE__);
    if (st == ULMB200_OK)
        st = check_cuda(cudaMemcpyAsync(&info, dints + mn, sizeof(int), cudaMemcpyDeviceToHost, s->run), "info", __FILE__, __LINE__);
    const int fin = finish(s);
    set_status(st != ULMB200_OK ? st : fin);
    return (st == ULMB200_OK && fin == ULMB200_OK) ? info : -100;
}

// replaces ULMLAPACK(dlaswp), interfaces/lapack/C/laswp.cc -> ulmBLAS::laswp (ulmblas/lapack/laswp.tcc):
// rows i = k1 .. k2-1 of the n columns of A are exchanged with rows piv[i*incPiv], in increasing
// order of i for incPiv > 0 and decreasing for incPiv < 0.  piv is read on the host.
void ulmblas_dlaswp(int n, double *A, int ldA, int k1, int k2, int *piv, int incPiv)
{
    ULMB_SERIALISE;
    if (incPiv == 0 || n <= 0 || k2 <= k1) { set_status(ULMB200_OK); return; }
    if (ensure_device() != ULMB200_OK) { set_status(ULMB200_NO_DEVICE); return; }
    Streams *s = streams();
    if (!s) { set_status(ULMB200_CUDA_ERROR); return; }
    std::vector<int> pairs;
    int rows = k2;
    const int inc = incPiv > 0 ? 1 : -1;
    for (int i = incPiv > 0 ? k1 : k2 - 1; incPiv > 0 ? i < k2 : i >= k1; i += inc) {
        const int ip = piv[(long)i * incPiv];
        pairs.push_back(i); pairs.push_back(ip);
        rows = std::max(rows, ip + 1);
    }
    int *dp = static_cast<int *>(device_scratch(10, sizeof(int) * pairs.size()));
    if (!dp) { set_status(ULMB200_CUDA_ERROR); return; }
    Staged a;
    int st = stage_in(a, A, ldA, rows, n, 2, true, s->run);
    if (st == ULMB200_OK)
        st = check_cuda(cudaMemcpyAsync(dp, pairs.data(), sizeof(int) * pairs.size(), cudaMemcpyHostToDevice, s->run),
                        "pairs", __FILE__, __LINE__);
    if (st == ULMB200_OK) st = dlaswp_pairs_device(s->run, a.dev, a.ldd, n, dp, (int)(pairs.size() / 2));
    if (st == ULMB200_OK) st = stage_out(a, s->run);
    const int fin = finish(s);      // also keeps `pairs` alive until the copy has been consumed
    set_status(st != ULMB200_OK ? st : fin);
}

}  // extern "C"
