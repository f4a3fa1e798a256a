// Host-side plumbing shared by every entry point: per-thread status, launch
// accounting, the per-device error word and scratch cache, tensor-map encoding.
#include "common.h"

#include <atomic>
#include <mutex>
#include <string.h>

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
    void *scratch[16] = {};
    size_t scratch_bytes[16] = {};
};
static DeviceState g_dev[kMaxDevices];
static std::mutex g_mu;

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
        cudaMemset(p, 0, 256);
        d.err_word = p;
    }
    return d.err_word;
}

int poll_device_error()
{
    int *w = device_error_word();
    if (!w) return ULMB200_CUDA_ERROR;
    int v = 0;
    if (cudaMemcpy(&v, w, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return ULMB200_CUDA_ERROR;
    if (v != 0) {
        fprintf(stderr, "ulmblas_b200: a kernel gave up on a bounded wait (code %d)\n", v);
        cudaMemset(w, 0, sizeof v);
        return ULMB200_KERNEL_FAULT;
    }
    return ULMB200_OK;
}

void *device_scratch(int slot, size_t bytes)
{
    DeviceState &d = g_dev[current_device()];
    std::lock_guard<std::mutex> lk(g_mu);
    if (d.scratch_bytes[slot] >= bytes && d.scratch[slot]) return d.scratch[slot];
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
    d.scratch[slot] = p;
    d.scratch_bytes[slot] = bytes;
    return p;
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
                  uint64_t d0, uint64_t d1, uint64_t ld, uint32_t b0, uint32_t b1)
{
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return false;
    cuuint64_t dims[2] = {d0, d1};
    cuuint64_t strides[1] = {ld * (uint64_t)elem_bytes};
    cuuint32_t box[2] = {b0, b1};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
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
