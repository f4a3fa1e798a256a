// Host-side plumbing shared by every entry point: per-thread status, launch
// accounting, the per-device error word and scratch cache, tensor-map encoding.
#include "common.h"

#include <atomic>
#include <mutex>
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>
#include <unordered_map>

namespace ulmb200 {

static thread_local int t_last_status = ULMB200_OK;
static std::atomic<int64_t> g_launches{0};

int set_status(int st)
{
    t_last_status = st;
    return st;
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int check_cuda(cudaError_t e, const char *what, const char *file, int line)
{
    if (e == cudaSuccess) return ULMB200_OK;
    fprintf(stderr, "ulmblas_b200: %s failed: %s (%s:%d)\n", what, cudaGetErrorString(e), file, line);
    cudaGetLastError();      // a launch error is reported once, not again by the next call
    return set_status(ULMB200_CUDA_ERROR);
}

int current_device()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) dev = 0;
    return dev < kMaxDevices ? dev : kMaxDevices - 1;
}

struct DeviceState {
    int checked = 0;          // 0 unknown, 1 usable, -1 not usable
    int sms = 0;
    int *err_word = nullptr;
    int *extra_err[4] = {};   // error words that live elsewhere (a __device__ array of the library)
    void *scratch[16] = {};
    size_t scratch_bytes[16] = {};
    int *sched = nullptr;     // kSchedSlots blocks of kSchedWords ints
    int sched_used = 0;
    std::unordered_map<unsigned long long, int> sched_of_stream;
};
static DeviceState g_dev[kMaxDevices];
static std::mutex g_mu;
static std::atomic<int64_t> g_allocs{0};

int64_t alloc_count() { return g_allocs.load(std::memory_order_relaxed); }

// ---- settings from the environment ---------------------------------------------------
static Settings g_settings;
static std::atomic<int> g_settings_read{0};

static void read_settings()
{
    Settings s;
    if (const char *e = getenv("ULMB200_TRACE")) s.trace = atoi(e);
    if (const char *e = getenv("ULMB200_SGEMM")) s.sgemm_3xtf32 = (e[0] == '3' || e[0] == 't');
    if (const char *e = getenv("ULMB200_WORKSPACE_CAP_MB")) s.workspace_cap = (int64_t)atoll(e) << 20;
    if (const char *e = getenv("ULMB200_DGEMM_TILE")) s.dgemm_tile = atoi(e);
    if (const char *e = getenv("ULMB200_DGEMM_PATH")) s.dgemm_ldg = (e[0] == 'l');
    if (const char *e = getenv("ULMB200_DGEMM_SPLITK")) s.dgemm_split = atoi(e);
    if (const char *e = getenv("ULMB200_DGEMM_EPI")) s.dgemm_epi = atoi(e);
    if (const char *e = getenv("ULMB200_TRSM_LEAF")) s.trsm_leaf = atoi(e);
    if (const char *e = getenv("ULMB200_SGEMM_PRETRANSPOSE")) s.sgemm_pretranspose = atoi(e);
    if (const char *e = getenv("ULMB200_SGEMM_PATH")) s.sgemm_path = (e[0] == 'l');
    g_settings = s;
}

const Settings &settings()
{
    if (!g_settings_read.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_settings_read.load(std::memory_order_relaxed)) {
            read_settings();
            g_settings_read.store(1, std::memory_order_release);
        }
    }
    return g_settings;
}

void trace(const char *fmt, ...)
{
    if (!settings().trace) return;
    char line[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(line, sizeof line, fmt, ap);
    va_end(ap);
    fprintf(stderr, "ulmb200: %s\n", line);
}

int ensure_device()
{
    const int dev = current_device();
    DeviceState &d = g_dev[dev];
    if (d.checked == 1) return ULMB200_OK;
    std::lock_guard<std::mutex> lk(g_mu);
    if (d.checked == 0) {
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            fprintf(stderr, "ulmblas_b200: no CUDA device visible; this library has no CPU path\n");
            d.checked = -1;
        } else {
            int major = 0, sms = 0;
            cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (major != 10) {
                fprintf(stderr, "ulmblas_b200: device %d has compute capability %d.x; "
                                "the kernels are built for sm_100a only\n", dev, major);
                d.checked = -1;
            } else {
                d.sms = sms;
                d.checked = 1;
            }
        }
    }
    return d.checked == 1 ? ULMB200_OK : ULMB200_NO_DEVICE;
}

int sm_count()
{
    const int s = g_dev[current_device()].sms;
    return s > 0 ? s : 148;
}

int *device_error_word()
{
    DeviceState &d = g_dev[current_device()];
    if (d.err_word) return d.err_word;
    std::lock_guard<std::mutex> lk(g_mu);
    if (!d.err_word) {
        int *p = nullptr;
        if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
        g_allocs.fetch_add(1, std::memory_order_relaxed);
        cudaMemset(p, 0, 256);
        cudaDeviceSynchronize();
        d.err_word = p;
    }
    return d.err_word;
}

void register_error_word(int *dev_word)
{
    DeviceState &d = g_dev[current_device()];
    std::lock_guard<std::mutex> lk(g_mu);
    for (int *&w : d.extra_err) {
        if (w == dev_word) return;
        if (!w) { w = dev_word; return; }
    }
}

int *registered_error_word(int i)
{
    DeviceState &d = g_dev[current_device()];
    std::lock_guard<std::mutex> lk(g_mu);
    return (i >= 0 && i < 4) ? d.extra_err[i] : nullptr;
}

// Reads every error word this device has (the library's own, if it was ever created, and the
// registered ones) with blocking copies; allocates nothing.
int poll_device_error()
{
    DeviceState &d = g_dev[current_device()];
    int *words[5];
    int nw = 0;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (d.err_word) words[nw++] = d.err_word;
        for (int *w : d.extra_err)
            if (w) words[nw++] = w;
    }
    int found = 0;
    for (int i = 0; i < nw; ++i) {
        int v = 0;
        if (cudaMemcpy(&v, words[i], sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return ULMB200_CUDA_ERROR;
        if (v != 0) {
            fprintf(stderr, "ulmblas_b200: a kernel gave up on a bounded wait (code %d)\n", v);
            cudaMemset(words[i], 0, sizeof v);
            found = v;
        }
    }
    if (found) {
        // a kernel that gave up may have left scheduler words behind
        std::lock_guard<std::mutex> lk(g_mu);
        if (d.sched) cudaMemset(d.sched, 0, sizeof(int) * (size_t)kSchedSlots * kSchedWords);
        return ULMB200_KERNEL_FAULT;
    }
    return ULMB200_OK;
}

int *sched_words(cudaStream_t st)
{
    DeviceState &d = g_dev[current_device()];
    unsigned long long id = 0;
    if (cudaStreamGetId(st, &id) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    std::lock_guard<std::mutex> lk(g_mu);
    if (!d.sched) {
        int *p = nullptr;
        const size_t bytes = sizeof(int) * (size_t)kSchedSlots * kSchedWords;
        if (cudaMalloc(&p, bytes) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        g_allocs.fetch_add(1, std::memory_order_relaxed);
        // the memset runs on the legacy default stream, which non-blocking streams do not wait for: make sure
        // the words are zero before any launch on any stream can see them
        cudaMemset(p, 0, bytes);
        cudaDeviceSynchronize();
        d.sched = p;
    }
    auto it = d.sched_of_stream.find(id);
    if (it != d.sched_of_stream.end()) return d.sched + (size_t)it->second * kSchedWords;
    if (d.sched_used >= kSchedSlots) return nullptr;
    const int slot = d.sched_used++;
    d.sched_of_stream.emplace(id, slot);
    return d.sched + (size_t)slot * kSchedWords;
}

static size_t cached_bytes(const DeviceState &d)
{
    size_t t = 0;
    for (size_t b : d.scratch_bytes) t += b;
    return t;
}

void *device_scratch(int slot, size_t bytes)
{
    const int64_t cap = settings().workspace_cap;
    DeviceState &d = g_dev[current_device()];
    std::lock_guard<std::mutex> lk(g_mu);
    if (d.scratch_bytes[slot] >= bytes && d.scratch[slot]) return d.scratch[slot];
    if (cap >= 0 && (int64_t)(cached_bytes(d) - d.scratch_bytes[slot] + bytes) > cap) {
        fprintf(stderr, "ulmblas_b200: work memory request of %zu bytes exceeds ULMB200_WORKSPACE_CAP_MB\n", bytes);
        return nullptr;
    }
    if (d.scratch[slot]) {
        cudaDeviceSynchronize();       // earlier work may still read the old buffer
        cudaFree(d.scratch[slot]);
        d.scratch[slot] = nullptr;
        d.scratch_bytes[slot] = 0;
    }
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    g_allocs.fetch_add(1, std::memory_order_relaxed);
    d.scratch[slot] = p;
    d.scratch_bytes[slot] = bytes;
    return p;
}

int release_workspace(int64_t *freed)
{
    DeviceState &d = g_dev[current_device()];
    if (d.checked != 1) { if (freed) *freed = 0; return ULMB200_OK; }
    cudaError_t e = cudaDeviceSynchronize();   // nothing queued may still use the buffers
    if (e != cudaSuccess) return check_cuda(e, "synchronize", __FILE__, __LINE__);
    std::lock_guard<std::mutex> lk(g_mu);
    int64_t total = 0;
    for (int s = 0; s < 16; ++s) {
        if (d.scratch[s]) {
            cudaFree(d.scratch[s]);
            total += (int64_t)d.scratch_bytes[s];
            d.scratch[s] = nullptr;
            d.scratch_bytes[s] = 0;
        }
    }
    if (freed) *freed = total;
    return ULMB200_OK;
}

int64_t workspace_bytes()
{
    DeviceState &d = g_dev[current_device()];
    std::lock_guard<std::mutex> lk(g_mu);
    return (int64_t)cached_bytes(d);
}

EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    });
    return fn;
}

bool make_tmap_2d(CUtensorMap *map, CUtensorMapDataType dt, int elem_bytes, const void *base,
                  uint64_t d0, uint64_t d1, uint64_t ld, uint32_t b0, uint32_t b1, CUtensorMapSwizzle swizzle)
{
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return false;
    cuuint64_t dims[2] = {d0, d1};
    cuuint64_t strides[1] = {ld * (uint64_t)elem_bytes};
    cuuint32_t box[2] = {b0, b1};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace ulmb200

extern "C" int ulmb200_last_status(void) { return ulmb200::t_last_status; }

extern "C" const char *ulmb200_status_string(int st)
{
    switch (st) {
    case ULMB200_OK: return "ok";
    case ULMB200_BAD_ARGUMENT: return "bad argument";
    case ULMB200_CUDA_ERROR: return "CUDA error";
    case ULMB200_NO_DEVICE: return "no sm_100 device (this library has no CPU path)";
    case ULMB200_KERNEL_FAULT: return "kernel gave up on a bounded wait";
    case ULMB200_TOO_LARGE: return "request exceeds a fixed limit";
    default: return "unknown status";
    }
}

extern "C" int64_t ulmb200_launch_count(void) { return ulmb200::g_launches.load(); }

extern "C" int64_t ulmb200_alloc_count(void) { return ulmb200::alloc_count(); }

extern "C" int64_t ulmb200_workspace_bytes(void) { return ulmb200::workspace_bytes(); }

extern "C" int ulmb200_release_workspace(void)
{
    return ulmb200::set_status(ulmb200::release_workspace(nullptr));
}

extern "C" void ulmb200_reload_env(void)
{
    std::lock_guard<std::mutex> lk(ulmb200::g_mu);
    ulmb200::read_settings();
    ulmb200::g_settings_read.store(1, std::memory_order_release);
}

extern "C" int ulmb200_check_device_error(void *stream)
{
    if (int s = ulmb200::ensure_device()) return ulmb200::set_status(s);
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return ulmb200::check_cuda(e, "stream synchronize", __FILE__, __LINE__);
    return ulmb200::set_status(ulmb200::poll_device_error());
}
