// Large DGEMM split over the GPUs of one box by column blocks of C:
//
//     C[:, J_r] <- alpha * A * B[:, J_r] + beta * C[:, J_r]        on rank r
//
// One process per GPU.  Rank r owns the column block J_r of B and C for good; A lives on the
// root rank and reaches the others by NCCL broadcast over NVLink, cut into K panels
// A[:, l0:l1] (contiguous in column-major storage).  The broadcasts are queued ahead on a
// communication stream; the product of panel l is queued on a compute stream behind "panel l
// has arrived", so later panels travel while earlier ones multiply.  No reduction and no
// other exchange: columns of C are independent.
//
// The reference has no multi-device path (it is single-threaded CPU code); the partition
// follows its own outermost loop, which already walks C by column blocks
// (ulmblas/level3/gemm.tcc:60).  Every product is the library's device DGEMM.
//
// NCCL is not a link-time dependency: its few entry points are looked up at run time
// (ULMB200_NCCL_LIB, else a libnccl.so.2 the process has already loaded, else the system's).
//
// The persistent GEMM grid would starve NCCL's kernels -- and a starved NCCL kernel on one
// rank keeps its peers' spinning -- so while panels still travel the grid leaves a few SMs
// free.  That costs those GEMMs about 5%, so the K panels are planned such that it touches
// little of the work: a short first panel (its transfer is the only one nothing hides), a
// second panel just long enough for the rest of A to arrive behind it, and one last panel
// with all the remaining K, which runs on the whole GPU because nothing travels any more.
// The transport rate the plan needs is measured by every rank; the ranks agree on one value (their
// collectives must match, so must their plans) early on and keep it.
#include "common.h"
#include "mg_plan.h"

#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include <algorithm>
#include <mutex>
#include <vector>

namespace ulmb200 {

// ---- NCCL, bound at run time ----------------------------------------------------------------
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;                       // 0 = ncclSuccess
constexpr int kNcclFloat64 = 8, kNcclMin = 3;

struct NcclApi {
    void *dl = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    ncclResult_t (*Broadcast)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

static NcclApi *nccl_api()
{
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char *env = getenv("ULMB200_NCCL_LIB");
        if (env && *env) api.dl = dlopen(env, RTLD_NOW | RTLD_LOCAL);
        if (!api.dl) api.dl = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);    // one the process already has
        if (!api.dl) api.dl = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (!api.dl) {
            fprintf(stderr, "ulmblas_b200: libnccl.so.2 not found (set ULMB200_NCCL_LIB): %s\n", dlerror());
            return;
        }
        bool all = true;
        auto sym = [&](const char *name) {
            void *p = dlsym(api.dl, name);
            if (!p) { fprintf(stderr, "ulmblas_b200: %s missing from NCCL\n", name); all = false; }
            return p;
        };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
        api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
        api.Broadcast = reinterpret_cast<decltype(api.Broadcast)>(sym("ncclBroadcast"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        api.ok = all;
    });
    return api.ok ? &api : nullptr;
}

static int check_nccl(NcclApi *n, ncclResult_t r, const char *what)
{
    if (r == 0) return ULMB200_OK;
    fprintf(stderr, "ulmblas_b200: %s failed: %s\n", what, n->GetErrorString ? n->GetErrorString(r) : "NCCL error");
    return set_status(ULMB200_CUDA_ERROR);
}

// ---- one rank's state ---------------------------------------------------------------------
constexpr int kMgEvents = 3 * kMgMaxPanels + 64;

struct MgComm {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1, dev = 0;
    cudaStream_t comm_stream = nullptr, compute = nullptr, h2d = nullptr, d2h = nullptr;
    cudaEvent_t ev[kMgEvents] = {};
    cudaEvent_t t0 = nullptr, t1 = nullptr;      // transport timing: first panel queued .. last panel landed
    bool timed = false;
    int timed_which = 0;                         // which kind of call (device / host operands) the events belong to
    double timed_bytes = 0.0;
    double rate_gbs[2] = {0.0, 0.0};             // transport rate the plans use: [0] device-resident, [1] host staging
    double seen_gbs[2] = {0.0, 0.0};             // what this rank has measured itself since the ranks last agreed
    int calls[2] = {0, 0};
    double *agree = nullptr;                     // one double in device memory for the ranks' agreement
    double gemm_tflops = 35.0;
    int reserve_sms = 8;
    int64_t first = 1024;
    // per-GEMM device times of the last device-resident call, when asked for (ulmb200_mg_profile)
    bool profile = false;
    cudaEvent_t g0[kMgMaxPanels] = {}, g1[kMgMaxPanels] = {};
    int profiled = 0;
    cudaEvent_t gend[2] = {};                    // end of the last product of the two latest profiled calls
    int ended = 0;
    // what the last call did (ulmb200_mg_last_plan)
    int last_npanels = 0;
    int64_t last_widths[kMgMaxPanels] = {};
    int last_reserve[kMgMaxPanels] = {};
};

// The K-panel plan must be the same on every rank -- the ranks' collectives have to match -- so the
// rate it is computed from is never a rank's own measurement.  Each rank measures the transport of its
// calls; on the second and on the third call of a kind the ranks agree on the smallest of their latest
// measurements (one tiny all-reduce and a host-side wait), and the last value stands from then on.
// The ranks agree on the transport rate at the start of their second and third call of a kind.
constexpr int kAgreeCalls = 2;

static int fold_rate(MgComm *c, int which, NcclApi *N)
{
    const int call = c->calls[which]++;
    // The plan of a call rests on the transport rate seen in the call before it, under that call's own plan
    // and beside its products.  Every call first waits (host side) for the previous call's transfers -- they
    // end early in a call, and the host still has the whole of that call's last product to queue this one --
    // and takes their rate.  On the second and third call the ranks then agree on the smallest rate (one tiny
    // all-reduce, which has to wait for an SM until the previous call's last product is done): ranks'
    // collectives must match, so must their plans.  Later calls keep the agreed rate.
    const bool agree_now = c->world > 1 && N && c->agree && call >= 1 && call <= kAgreeCalls;
    if (c->timed && c->timed_which == which) {
        if (c->world > 1) ULMB_CUDA(cudaStreamSynchronize(c->comm_stream));
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, c->t0, c->t1) == cudaSuccess && ms > 0.f) {
            c->seen_gbs[which] = c->timed_bytes / (ms * 1e-3) * 1e-9;
            c->timed = false;
        } else {
            cudaGetLastError();          // still under way: the rate stays what it was
        }
    }
    if (!agree_now) return ULMB200_OK;
    double mine = c->seen_gbs[which] > 0.0 ? c->seen_gbs[which] : 1e9;       // "no opinion"
    ULMB_CUDA(cudaMemcpyAsync(c->agree, &mine, sizeof mine, cudaMemcpyHostToDevice, c->comm_stream));
    if (int s = check_nccl(N, N->AllReduce(c->agree, c->agree, 1, kNcclFloat64, kNcclMin, c->comm, c->comm_stream), "ncclAllReduce"))
        return s;
    double all = 0.0;
    ULMB_CUDA(cudaMemcpyAsync(&all, c->agree, sizeof all, cudaMemcpyDeviceToHost, c->comm_stream));
    ULMB_CUDA(cudaStreamSynchronize(c->comm_stream));
    if (all > 0.0 && all < 1e8) c->rate_gbs[which] = all;
    return ULMB200_OK;
}

static int next_event(MgComm *c, int &cursor, cudaEvent_t *out)
{
    if (cursor >= kMgEvents) return ULMB200_TOO_LARGE;
    *out = c->ev[cursor++];
    return ULMB200_OK;
}

#define MG_CUDA(call) ULMB_CUDA(call)
#define MG_TRY(expr)                                   \
    do {                                               \
        int st__ = (expr);                             \
        if (st__ != ULMB200_OK) return set_status(st__); \
    } while (0)

// b waits for everything queued on a so far
static int stream_after(MgComm *c, int &cursor, cudaStream_t b, cudaStream_t a)
{
    cudaEvent_t e;
    if (int s = next_event(c, cursor, &e)) return s;
    MG_CUDA(cudaEventRecord(e, a));
    MG_CUDA(cudaStreamWaitEvent(b, e, 0));
    return ULMB200_OK;
}

static int plan_for(MgComm *c, int64_t m, int64_t nr, int64_t k, int which, int64_t *widths, int *reserve)
{
    // before anything has been measured: NVLink broadcast next to a busy GPU / one PCIe link
    const double guess = which == 0 ? 150.0 : 40.0;
    const double rate = c->rate_gbs[which] > 0.0 ? c->rate_gbs[which] : guess;
    const int np = mg_plan_panels(m, nr, k, c->world, c->first, rate, c->gemm_tflops, widths, reserve, kMgMaxPanels);
    c->last_npanels = np;
    for (int i = 0; i < np; ++i) { c->last_widths[i] = widths[i]; c->last_reserve[i] = reserve[i]; }
    return np;
}

// Device-resident: A (m x k, ld = ldA) holds data on the root and is a buffer elsewhere.
static int mg_dgemm_device(MgComm *c, cudaStream_t user, int64_t m, int64_t n, int64_t k, double alpha, double *dA,
                           int64_t ldA, const double *dB, int64_t ldB, double beta, double *dC, int64_t ldC, int root)
{
    NcclApi *N = c->world > 1 ? nccl_api() : nullptr;
    if (c->world > 1 && !N) return set_status(ULMB200_CUDA_ERROR);
    int64_t j0, j1;
    mg_column_block(n, c->world, c->rank, &j0, &j1);
    const int64_t nr = j1 - j0;
    int64_t nr_max = 0;
    for (int r = 0; r < c->world; ++r) {
        int64_t a, b;
        mg_column_block(n, c->world, r, &a, &b);
        nr_max = std::max(nr_max, b - a);
    }
    MG_TRY(fold_rate(c, 0, N));
    int64_t widths[kMgMaxPanels];
    int reserve[kMgMaxPanels];
    const int np = plan_for(c, m, nr_max, k, 0, widths, reserve);
    int cursor = 0;
    MG_TRY(stream_after(c, cursor, c->compute, user));
    if (c->world > 1) {
        MG_TRY(stream_after(c, cursor, c->comm_stream, user));
        // contiguous panels only: a broadcast moves one block of memory
        if (ldA != m) return set_status(ULMB200_BAD_ARGUMENT);
        MG_CUDA(cudaEventRecord(c->t0, c->comm_stream));
        cudaEvent_t arrived[kMgMaxPanels];
        int64_t l0 = 0;
        for (int p = 0; p < np; ++p) {
            double *panel = dA + l0 * ldA;
            MG_TRY(check_nccl(N, N->Broadcast(panel, panel, (size_t)(m * widths[p]), kNcclFloat64, root, c->comm, c->comm_stream),
                              "ncclBroadcast"));
            MG_TRY(next_event(c, cursor, &arrived[p]));
            MG_CUDA(cudaEventRecord(arrived[p], c->comm_stream));
            l0 += widths[p];
        }
        MG_CUDA(cudaEventRecord(c->t1, c->comm_stream));
        c->timed = true;
        c->timed_which = 0;
        c->timed_bytes = 8.0 * (double)m * (double)k;
        l0 = 0;
        for (int p = 0; p < np; ++p) {
            MG_CUDA(cudaStreamWaitEvent(c->compute, arrived[p], 0));
            if (nr > 0) {
                if (c->profile) MG_CUDA(cudaEventRecord(c->g0[p], c->compute));
                const int prev = sm_reserve_swap(reserve[p] ? c->reserve_sms : 0);
                const int st = dgemm_device(c->compute, 0, 0, 0, m, nr, widths[p], alpha, dA + l0 * ldA, ldA, dB + l0, ldB,
                                            p == 0 ? beta : 1.0, dC, ldC);
                sm_reserve_swap(prev);
                MG_TRY(st);
                if (c->profile) MG_CUDA(cudaEventRecord(c->g1[p], c->compute));
            }
            l0 += widths[p];
        }
        c->profiled = (c->profile && nr > 0) ? np : 0;
        if (c->profile) {
            MG_CUDA(cudaEventRecord(c->gend[c->ended & 1], c->compute));
            ++c->ended;
        } else {
            c->ended = 0;
        }
        MG_TRY(stream_after(c, cursor, user, c->comm_stream));
    } else if (nr > 0) {
        if (c->profile) MG_CUDA(cudaEventRecord(c->g0[0], c->compute));
        MG_TRY(dgemm_device(c->compute, 0, 0, 0, m, nr, k, alpha, dA, ldA, dB, ldB, beta, dC, ldC));
        if (c->profile) MG_CUDA(cudaEventRecord(c->g1[0], c->compute));
        c->profiled = c->profile ? 1 : 0;
    }
    MG_TRY(stream_after(c, cursor, user, c->compute));
    return set_status(ULMB200_OK);
}

// Host-resident operands.  hA: the whole of A (m x k, ld = ldhA).  On the root it must be given.
// A rank that can read A itself (a mapping of the same host memory, a copy) passes it too; when
// every rank does, each one brings a share of the rows of every panel over its own PCIe link and
// the shares are exchanged by all-gather, instead of the root pushing all of A through one link.
// hB / hC: this rank's column blocks.  dA, dB, dC: device buffers of the same shapes as in the
// device-resident call (dA m x k with ld = m).
static int mg_dgemm_host(MgComm *c, cudaStream_t user, int64_t m, int64_t n, int64_t k, double alpha, const double *hA,
                         int64_t ldhA, const double *hB, int64_t ldhB, double beta, double *hC, int64_t ldhC,
                         double *dA, double *dB, int64_t lddB, double *dC, int64_t lddC, int root, int all_have_a)
{
    NcclApi *N = c->world > 1 ? nccl_api() : nullptr;
    if (c->world > 1 && !N) return set_status(ULMB200_CUDA_ERROR);
    int64_t j0, j1;
    mg_column_block(n, c->world, c->rank, &j0, &j1);
    const int64_t nr = j1 - j0;
    int64_t nr_max = 0;
    for (int r = 0; r < c->world; ++r) {
        int64_t a, b;
        mg_column_block(n, c->world, r, &a, &b);
        nr_max = std::max(nr_max, b - a);
    }
    if (c->rank == root && !hA) return set_status(ULMB200_BAD_ARGUMENT);
    const bool slabs = c->world > 1 && all_have_a && hA != nullptr;
    MG_TRY(fold_rate(c, 1, N));
    int64_t widths[kMgMaxPanels];
    int reserve[kMgMaxPanels];
    int np;
    if (c->world == 1) {
        // one GPU: the panels only pipeline the copy of A against the products
        np = mg_plan_host_panels(m, k, widths, kMgMaxPanels);
        for (int i = 0; i < np; ++i) reserve[i] = 0;
        c->last_npanels = np;
        for (int i = 0; i < np; ++i) { c->last_widths[i] = widths[i]; c->last_reserve[i] = 0; }
    } else {
        np = plan_for(c, m, nr_max, k, 1, widths, reserve);
    }
    int cursor = 0;
    MG_TRY(stream_after(c, cursor, c->compute, user));
    MG_TRY(stream_after(c, cursor, c->comm_stream, user));
    MG_TRY(stream_after(c, cursor, c->h2d, user));
    MG_TRY(stream_after(c, cursor, c->d2h, user));
    MG_CUDA(cudaEventRecord(c->t0, c->h2d));
    cudaEvent_t arrived[kMgMaxPanels];
    int64_t l0 = 0;
    for (int p = 0; p < np; ++p) {
        double *panel = dA + l0 * m;
        const int64_t w = widths[p];
        // the rows of this rank's block of B that panel p multiplies (and, before the first product, its block of C)
        if (nr > 0) {
            MG_CUDA(cudaMemcpy2DAsync(dB + l0, lddB * 8, hB + l0, ldhB * 8, (size_t)w * 8, (size_t)nr, cudaMemcpyHostToDevice, c->h2d));
            if (p == 0 && beta != 0.0)
                MG_CUDA(cudaMemcpy2DAsync(dC, lddC * 8, hC, ldhC * 8, (size_t)m * 8, (size_t)nr, cudaMemcpyHostToDevice, c->h2d));
        }
        if (slabs && w % c->world == 0) {
            // columns of a column-major panel are contiguous: this rank brings its share of them over its own
            // PCIe link, straight into place, and the all-gather (in place) completes the panel on every rank
            const int64_t cw = w / c->world;
            double *mine = panel + (size_t)c->rank * cw * m;
            MG_CUDA(cudaMemcpy2DAsync(mine, m * 8, hA + (l0 + c->rank * cw) * ldhA, ldhA * 8, (size_t)m * 8, (size_t)cw,
                                      cudaMemcpyHostToDevice, c->h2d));
            MG_TRY(stream_after(c, cursor, c->comm_stream, c->h2d));
            MG_TRY(check_nccl(N, N->AllGather(mine, panel, (size_t)(cw * m), kNcclFloat64, c->comm, c->comm_stream),
                              "ncclAllGather"));
        } else {
            if (c->rank == root) {
                MG_CUDA(cudaMemcpy2DAsync(panel, m * 8, hA + l0 * ldhA, ldhA * 8, (size_t)m * 8, (size_t)w,
                                          cudaMemcpyHostToDevice, c->h2d));
            }
            MG_TRY(stream_after(c, cursor, c->comm_stream, c->h2d));
            if (c->world > 1)
                MG_TRY(check_nccl(N, N->Broadcast(panel, panel, (size_t)(m * w), kNcclFloat64, root, c->comm, c->comm_stream),
                                  "ncclBroadcast"));
        }
        MG_TRY(next_event(c, cursor, &arrived[p]));
        MG_CUDA(cudaEventRecord(arrived[p], c->comm_stream));
        l0 += w;
    }
    MG_CUDA(cudaEventRecord(c->t1, c->comm_stream));
    c->timed = c->world > 1;
    c->timed_which = 1;
    c->timed_bytes = 8.0 * (double)m * (double)k;

    // All panels but the last are applied to the whole column block; the last one -- by plan the
    // bulk of K -- goes column piece by column piece, so that finished pieces of C leave for the host
    // while the next ones are still being multiplied.
    l0 = 0;
    for (int p = 0; p < np; ++p) {
        MG_CUDA(cudaStreamWaitEvent(c->compute, arrived[p], 0));
        const bool last = p == np - 1;
        int pieces = 1;
        if (last && nr >= 8 * 128) pieces = 8;
        const int64_t q = ((nr + pieces - 1) / pieces + 127) / 128 * 128;
        for (int64_t c0 = 0; c0 < nr; c0 += (last ? q : nr)) {
            const int64_t cn = last ? std::min(q, nr - c0) : nr;
            const int prev = sm_reserve_swap(reserve[p] ? c->reserve_sms : 0);
            const int st = dgemm_device(c->compute, 0, 0, 0, m, cn, widths[p], alpha, dA + l0 * m, m, dB + l0 + c0 * lddB, lddB,
                                        p == 0 ? beta : 1.0, dC + c0 * lddC, lddC);
            sm_reserve_swap(prev);
            MG_TRY(st);
            if (last) {
                MG_TRY(stream_after(c, cursor, c->d2h, c->compute));
                MG_CUDA(cudaMemcpy2DAsync(hC + c0 * ldhC, ldhC * 8, dC + c0 * lddC, lddC * 8, (size_t)m * 8, (size_t)cn,
                                          cudaMemcpyDeviceToHost, c->d2h));
            }
        }
        l0 += widths[p];
    }
    MG_TRY(stream_after(c, cursor, user, c->compute));
    MG_TRY(stream_after(c, cursor, user, c->comm_stream));
    MG_TRY(stream_after(c, cursor, user, c->h2d));
    MG_TRY(stream_after(c, cursor, user, c->d2h));
    return set_status(ULMB200_OK);
}

}  // namespace ulmb200

using namespace ulmb200;

extern "C" int ulmb200_mg_column_block(int64_t n, int world, int rank, int64_t *j0, int64_t *j1)
{
    if (world <= 0 || rank < 0 || rank >= world || n < 0 || !j0 || !j1) return set_status(ULMB200_BAD_ARGUMENT);
    mg_column_block(n, world, rank, j0, j1);
    return set_status(ULMB200_OK);
}

extern "C" int ulmb200_mg_plan_panels(int64_t m, int64_t n_block, int64_t k, int world, int64_t first, double transport_gbs,
                                      double gemm_tflops, int64_t *widths, int *reserve, int cap)
{
    if (m < 0 || n_block < 0 || k < 0 || world <= 0 || !widths || !reserve || cap <= 0) return -1;
    return mg_plan_panels(m, n_block, k, world, first, transport_gbs, gemm_tflops, widths, reserve, cap);
}

extern "C" int ulmb200_mg_unique_id(char id[128])
{
    NcclApi *N = nccl_api();
    if (!N || !id) return set_status(ULMB200_CUDA_ERROR);
    ncclUniqueId u;
    if (int s = check_nccl(N, N->GetUniqueId(&u), "ncclGetUniqueId")) return s;
    memcpy(id, u.internal, 128);
    return set_status(ULMB200_OK);
}

extern "C" int ulmb200_mg_init(const char id[128], int rank, int world, void **handle)
{
    if (!handle || world <= 0 || rank < 0 || rank >= world) return set_status(ULMB200_BAD_ARGUMENT);
    *handle = nullptr;
    if (int s = ensure_device()) return set_status(s);
    MgComm *c = new MgComm;
    c->rank = rank; c->world = world; c->dev = current_device();
    if (const char *e = getenv("ULMB200_MG_RESERVE_SMS")) c->reserve_sms = std::max(0, atoi(e));
    if (const char *e = getenv("ULMB200_MG_FIRST_PANEL")) c->first = std::max(128, atoi(e));
    auto fail = [&](int st) { delete c; return set_status(st); };
    if (world > 1) {
        NcclApi *N = nccl_api();
        if (!N || !id) return fail(ULMB200_CUDA_ERROR);
        ncclUniqueId u;
        memcpy(u.internal, id, 128);
        if (check_nccl(N, N->CommInitRank(&c->comm, world, u, rank), "ncclCommInitRank")) return fail(ULMB200_CUDA_ERROR);
    }
    cudaError_t e = cudaStreamCreateWithFlags(&c->comm_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->compute, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->h2d, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->d2h, cudaStreamNonBlocking);
    for (int i = 0; i < kMgEvents && e == cudaSuccess; ++i) e = cudaEventCreateWithFlags(&c->ev[i], cudaEventDisableTiming);
    for (int i = 0; i < kMgMaxPanels && e == cudaSuccess; ++i) {
        e = cudaEventCreate(&c->g0[i]);
        if (e == cudaSuccess) e = cudaEventCreate(&c->g1[i]);
    }
    if (e == cudaSuccess && world > 1) e = cudaMalloc(&c->agree, 64);
    if (e == cudaSuccess) e = cudaEventCreate(&c->t0);
    if (e == cudaSuccess) e = cudaEventCreate(&c->t1);
    if (e == cudaSuccess) e = cudaEventCreate(&c->gend[0]);
    if (e == cudaSuccess) e = cudaEventCreate(&c->gend[1]);
    if (e != cudaSuccess) { check_cuda(e, "stream/event creation", __FILE__, __LINE__); return fail(ULMB200_CUDA_ERROR); }
    *handle = c;
    return set_status(ULMB200_OK);
}

extern "C" int ulmb200_mg_finalize(void *handle)
{
    MgComm *c = static_cast<MgComm *>(handle);
    if (!c) return set_status(ULMB200_OK);
    cudaDeviceSynchronize();
    if (c->comm) {
        NcclApi *N = nccl_api();
        if (N) N->CommDestroy(c->comm);
    }
    for (cudaStream_t s : {c->comm_stream, c->compute, c->h2d, c->d2h})
        if (s) cudaStreamDestroy(s);
    for (cudaEvent_t e : c->ev)
        if (e) cudaEventDestroy(e);
    for (int i = 0; i < kMgMaxPanels; ++i) {
        if (c->g0[i]) cudaEventDestroy(c->g0[i]);
        if (c->g1[i]) cudaEventDestroy(c->g1[i]);
    }
    if (c->agree) cudaFree(c->agree);
    if (c->t0) cudaEventDestroy(c->t0);
    if (c->t1) cudaEventDestroy(c->t1);
    for (cudaEvent_t e : c->gend)
        if (e) cudaEventDestroy(e);
    delete c;
    return set_status(ULMB200_OK);
}

extern "C" int ulmb200_mg_dgemm(void *handle, void *stream, int64_t m, int64_t n, int64_t k, double alpha, double *dA,
                                int64_t ldA, const double *dB_block, int64_t ldB, double beta, double *dC_block,
                                int64_t ldC, int root)
{
    MgComm *c = static_cast<MgComm *>(handle);
    if (!c || m < 0 || n < 0 || k < 0 || root < 0 || root >= c->world) return set_status(ULMB200_BAD_ARGUMENT);
    if (ldA < std::max<int64_t>(1, m) || ldB < std::max<int64_t>(1, k) || ldC < std::max<int64_t>(1, m))
        return set_status(ULMB200_BAD_ARGUMENT);
    if (m == 0 || n == 0) return set_status(ULMB200_OK);
    return mg_dgemm_device(c, static_cast<cudaStream_t>(stream), m, n, k, alpha, dA, ldA, dB_block, ldB, beta, dC_block,
                           ldC, root);
}

extern "C" int ulmb200_mg_dgemm_host(void *handle, void *stream, int64_t m, int64_t n, int64_t k, double alpha,
                                     const double *hA, int64_t ldhA, const double *hB_block, int64_t ldhB, double beta,
                                     double *hC_block, int64_t ldhC, double *dA, double *dB_block, int64_t lddB,
                                     double *dC_block, int64_t lddC, int root, int every_rank_has_a)
{
    MgComm *c = static_cast<MgComm *>(handle);
    if (!c || m < 0 || n < 0 || k < 0 || root < 0 || root >= c->world) return set_status(ULMB200_BAD_ARGUMENT);
    if (ldhA < std::max<int64_t>(1, m) || ldhB < std::max<int64_t>(1, k) || ldhC < std::max<int64_t>(1, m) ||
        lddB < std::max<int64_t>(1, k) || lddC < std::max<int64_t>(1, m))
        return set_status(ULMB200_BAD_ARGUMENT);
    if (m == 0 || n == 0) return set_status(ULMB200_OK);
    return mg_dgemm_host(c, static_cast<cudaStream_t>(stream), m, n, k, alpha, hA, ldhA, hB_block, ldhB, beta, hC_block, ldhC,
                         dA, dB_block, lddB, dC_block, lddC, root, every_rank_has_a);
}

extern "C" int ulmb200_mg_last_plan(void *handle, int64_t *widths, int *reserve, int cap, double *device_rate_gbs,
                                    double *host_rate_gbs)
{
    MgComm *c = static_cast<MgComm *>(handle);
    if (!c) return -1;
    for (int i = 0; i < c->last_npanels && i < cap; ++i) {
        if (widths) widths[i] = c->last_widths[i];
        if (reserve) reserve[i] = c->last_reserve[i];
    }
    if (device_rate_gbs) *device_rate_gbs = c->rate_gbs[0] > 0.0 ? c->rate_gbs[0] : c->seen_gbs[0];
    if (host_rate_gbs) *host_rate_gbs = c->rate_gbs[1] > 0.0 ? c->rate_gbs[1] : c->seen_gbs[1];
    return c->last_npanels;
}

extern "C" int ulmb200_mg_profile(void *handle, int on)
{
    MgComm *c = static_cast<MgComm *>(handle);
    if (!c) return set_status(ULMB200_BAD_ARGUMENT);
    if (on && !c->profile) c->profiled = 0;
    c->profile = on != 0;
    return set_status(ULMB200_OK);
}

extern "C" int ulmb200_mg_last_gemm_start_ms(void *handle, double *ms, int cap)
{
    MgComm *c = static_cast<MgComm *>(handle);
    if (!c || !ms) return -1;
    int n = 0;
    for (; n < c->profiled && n < cap; ++n) {
        float t = 0.f;
        if (cudaEventElapsedTime(&t, c->t0, c->g0[n]) != cudaSuccess) { cudaGetLastError(); return -1; }
        ms[n] = t;
    }
    return n;
}

extern "C" int ulmb200_mg_last_step_gap_ms(void *handle, double *ms)
{
    MgComm *c = static_cast<MgComm *>(handle);
    if (!c || !ms || c->world < 2 || c->ended < 2) return -1;
    float t = 0.f;
    if (cudaEventElapsedTime(&t, c->gend[c->ended & 1], c->t0) != cudaSuccess) { cudaGetLastError(); return -1; }
    *ms = t;
    return 0;
}

extern "C" int ulmb200_mg_last_gemm_ms(void *handle, double *ms, int cap)
{
    MgComm *c = static_cast<MgComm *>(handle);
    if (!c || !ms) return -1;
    int n = 0;
    for (; n < c->profiled && n < cap; ++n) {
        float t = 0.f;
        if (cudaEventElapsedTime(&t, c->g0[n], c->g1[n]) != cudaSuccess) { cudaGetLastError(); return -1; }
        ms[n] = t;
    }
    return n;
}

// Waits (host side, at most timeout_ms) for everything this communicator has queued, watching NCCL's
// asynchronous error state meanwhile.  A transport error or the timeout aborts the communicator -- the
// handle is then only good for ulmb200_mg_finalize -- and returns ULMB200_CUDA_ERROR.
extern "C" int ulmb200_mg_wait(void *handle, int timeout_ms)
{
    MgComm *c = static_cast<MgComm *>(handle);
    if (!c) return set_status(ULMB200_BAD_ARGUMENT);
    NcclApi *N = c->comm ? nccl_api() : nullptr;
    timespec t0;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (;;) {
        bool busy = false;
        for (cudaStream_t s : {c->comm_stream, c->compute, c->h2d, c->d2h}) {
            cudaError_t e = cudaStreamQuery(s);
            if (e == cudaErrorNotReady) busy = true;
            else if (e != cudaSuccess) return check_cuda(e, "cudaStreamQuery", __FILE__, __LINE__);
        }
        if (N) {
            ncclResult_t async = 0;
            if (N->CommGetAsyncError(c->comm, &async) != 0 || async != 0) {
                fprintf(stderr, "ulmblas_b200: NCCL reports an asynchronous error; aborting the communicator\n");
                N->CommAbort(c->comm);
                c->comm = nullptr;
                return set_status(ULMB200_CUDA_ERROR);
            }
        }
        if (!busy) return set_status(poll_device_error());
        timespec t1;
        clock_gettime(CLOCK_MONOTONIC, &t1);
        const double ms = (t1.tv_sec - t0.tv_sec) * 1e3 + (t1.tv_nsec - t0.tv_nsec) * 1e-6;
        if (timeout_ms >= 0 && ms > timeout_ms) {
            fprintf(stderr, "ulmblas_b200: sharded call still running after %d ms; aborting the communicator\n", timeout_ms);
            if (N) { N->CommAbort(c->comm); c->comm = nullptr; }
            return set_status(ULMB200_CUDA_ERROR);
        }
        timespec nap = {0, 200000};
        nanosleep(&nap, nullptr);
    }
}

extern "C" int ulmb200_mg_set_rates(void *handle, double transport_gbs, double host_gbs, double gemm_tflops)
{
    MgComm *c = static_cast<MgComm *>(handle);
    if (!c) return set_status(ULMB200_BAD_ARGUMENT);
    if (transport_gbs > 0.0) c->rate_gbs[0] = transport_gbs;
    if (host_gbs > 0.0) c->rate_gbs[1] = host_gbs;
    if (gemm_tflops > 0.0) c->gemm_tflops = gemm_tflops;
    return set_status(ULMB200_OK);
}
