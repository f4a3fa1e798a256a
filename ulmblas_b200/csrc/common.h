// Shared host/device helpers of libulmblas_b200: status plumbing, launch
// accounting, and the sm_100a PTX wrappers (mbarrier, TMA) the kernels use.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/ulmblas_b200.h"

namespace ulmb200 {

// ---- host-side status ------------------------------------------------------

int  set_status(int st);                 // records the thread's last status, returns it
void count_launch(int n = 1);            // feeds ulmb200_launch_count()
int  check_cuda(cudaError_t e, const char *what, const char *file, int line);
int  ensure_device();                    // 0 if the current device is sm_100
constexpr int kMaxDevices = 64;
int  current_device();                   // cudaGetDevice, clamped to [0, kMaxDevices)
int  sm_count();                         // SMs of the current device

#define ULMB_CUDA(call)                                                            \
    do {                                                                           \
        int st__ = ::ulmb200::check_cuda((call), #call, __FILE__, __LINE__);        \
        if (st__ != ULMB200_OK) return st__;                                       \
    } while (0)

// Device-side error word (one per device, zero-initialised).  A kernel whose
// bounded wait runs out stores a non-zero code here and returns normally.
int *device_error_word();                // device pointer, for the current device
void register_error_word(int *dev_word); // a further word poll_device_error() should read (current device)
int *registered_error_word(int i);       // i-th registered word of the current device or nullptr
int  poll_device_error();                // syncs nothing; reads the words with blocking copies, allocates nothing
int  release_workspace(int64_t *freed_bytes);
int64_t workspace_bytes();

// Cached scratch buffers in device memory (one set per device, grown on demand, given back
// by ulmb200_release_workspace), the counterpart of the reference's MemoryPool
// (ulmblas/auxiliary/memorypool.tcc).  Returns nullptr when the allocation fails or would
// take the cache beyond ULMB200_WORKSPACE_CAP_MB.
void *device_scratch(int slot, size_t bytes);
int64_t alloc_count();                   // device allocations made by the library so far

// Scheduler words of the persistent GEMM kernels: per CUDA stream one zero-initialised block of
// kSchedWords ints in device memory -- [0] tile counter, [1] CTAs that have finished,
// [2 ...] fold flags of tiles shared by several CTAs.  Kernels leave every word at zero when
// they end, so launches that follow each other on one stream reuse the block without a
// memset, and launches on different streams never share one.  nullptr when no block is left
// (more than kSchedSlots streams in use on the device): the caller then schedules statically.
constexpr int kSchedFlags = 4096;
constexpr int kSchedWords = 4160;
constexpr int kSchedSlots = 256;
int *sched_words(cudaStream_t st);

// Settings taken from the environment, read at first use and again by ulmb200_reload_env():
//   ULMB200_TRACE=1              one line per call on stderr
//   ULMB200_SGEMM=fp32|3xtf32    arithmetic of sgemm_ / cblas_sgemm
//   ULMB200_WORKSPACE_CAP_MB=n   upper limit of the cached device work memory
//   ULMB200_DGEMM_TILE=64|128|12864, ULMB200_DGEMM_PATH=ldg, ULMB200_DGEMM_SPLITK=0|2,
//   ULMB200_DGEMM_EPI=n (epilogue cost, in pipeline stages, assumed by the share planner)   (test hooks)
//   ULMB200_SGEMM_PRETRANSPOSE=0   never copy K-contiguous operands of sgemm (test hook)
//   ULMB200_TRSM_LEAF=128|256|512|1024|2048   order of the diagonal blocks (leaves) of dtrsm and dtrmm (test hook)
struct Settings {
    int trace = 0;
    int sgemm_3xtf32 = 0;
    int64_t workspace_cap = -1;          // bytes, -1 = none
    int dgemm_tile = 0, dgemm_ldg = 0, dgemm_split = 1;
    int dgemm_epi = 0;            // test hook: epilogue cost (in pipeline stages) the share planner assumes, 0 = built in
    int sgemm_path = 0;                  // 0 auto, 1 force the plain-load kernel
    int sgemm_pretranspose = 1;          // 0: K-contiguous operands are always transposed inside the kernel
    int trsm_leaf = 0;                   // 0 auto
};
const Settings &settings();
void trace(const char *fmt, ...) __attribute__((format(printf, 1, 2)));

// cuTensorMapEncodeTiled fetched through the runtime (no link against libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();

// 2-D tensor map over a column-major matrix: dim0 = contiguous dimension
// (extent d0), dim1 = the strided one (extent d1, stride ld elements), box
// b0 x b1 elements, 128-byte swizzle unless told otherwise.  Returns false if the driver refuses.
bool make_tmap_2d(CUtensorMap *map, CUtensorMapDataType dt, int elem_bytes, const void *base,
                  uint64_t d0, uint64_t d1, uint64_t ld, uint32_t b0, uint32_t b1,
                  CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B);

// C <- alpha*op(A)*op(B) + beta*C on device operands (dgemm_sm100.cu).  tri: 0 full, 1 upper
// triangle only, 2 lower.  err_word: device word a kernel writes when a bounded wait runs out;
// nullptr selects the library's own per-device word.
int dgemm_device(cudaStream_t st, int tri, int transA, int transB, int64_t m, int64_t n, int64_t k,
                 double alpha, const double *A, int64_t lda, const double *B, int64_t ldb, double beta,
                 double *C, int64_t ldc, int *err_word = nullptr);
// X <- alpha * op(T) * X (left) or alpha * X * op(T) (right) in place, T triangular of any order with zeros in the
// other triangle of its 128 x 128 diagonal blocks (dgemm_sm100.cu); -1 when the operands do not qualify
int dgemm_leaf_inplace(cudaStream_t st, int left, int lower_op, int transT, int64_t dim, int64_t other, double alpha,
                       const double *T, int64_t ldt, double *X, int64_t ldx, int *err_word);
// Where product b = hi * nlo + lo of a batch finds its blocks: lo * x[0] + hi * x[1] rows or columns past the
// blocks of product 0, for the rows and columns of the stored A, B and C.
struct BatchShape {
    int count, nlo;
    int a_row[2], a_col[2], b_row[2], b_col[2];
    int64_t c_row[2], c_col[2];
};
// count products C_b <- alpha * A_b * B_b of one shape in one launch (dgemm_sm100.cu); a_rows .. b_cols are the
// extents of the stored matrices the blocks are cut from (likewise c_rows, c_cols); -1 when the operands do not qualify
int dgemm_batched(cudaStream_t st, int64_t m, int64_t n, int64_t k, double alpha, const double *A, int64_t lda,
                  int64_t a_rows, int64_t a_cols, const double *B, int64_t ldb, int64_t b_rows, int64_t b_cols,
                  double *C, int64_t ldc, int64_t c_rows, int64_t c_cols, const BatchShape &bs);
// sets the number of SMs the persistent DGEMM grid leaves free; returns the previous value
int sm_reserve_swap(int sms);
int scale_matrix_device(cudaStream_t st, double *C, int64_t ldc, int64_t m, int64_t n, double beta, int tri);
// B <- alpha*op(A)^-1*B (side 0) or alpha*B*op(A)^-1 (side 1) with caller-provided scratch
// (level3_sm100.cu): inv holds ceil(dim/leaf)*leaf*leaf doubles, W leaf*n (left) or m*leaf (right);
// leaf = 128 or 256, or a larger power of two with pairs = ceil(dim/leaf)*leaf*leaf/4 more doubles.
int dtrsm_with_scratch(cudaStream_t st, int side, int lower, int transA, int unit, int64_t m, int64_t n,
                       double alpha, const double *A, int64_t lda, double *B, int64_t ldb, double *inv,
                       double *W, int *err_word = nullptr, int leaf = 128, double *pairs = nullptr);

#ifdef __CUDACC__
// ---- device-side PTX wrappers ---------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Release of a buffer the caller has read with shared loads.  `seen` is computed from the registers those
// loads wrote; it is stored to `sink` (a word of shared memory nobody reads) before the arrive, so the
// store cannot issue before the loads have returned, and the arrive -- a release -- follows the store.
__device__ __forceinline__ void mbar_arrive_after(uint64_t *bar, uint32_t seen, volatile uint32_t *sink)
{
    asm volatile("st.shared.u32 [%1], %2;\n\t"
                 "mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)), "r"(smem_u32(const_cast<uint32_t *>(sink))), "r"(seen)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: every mbarrier wait in this library gives up after a fixed
// number of polls (seconds of wall time, far beyond any legitimate wait) and
// reports failure instead of spinning forever.
constexpr uint32_t kWaitPollLimit = 1u << 24;

__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity)
{
    for (uint32_t i = 0; i < kWaitPollLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(64);
    }
    return false;
}

// One 2-D TMA tile load for this CTA alone; completion is signalled on `bar`.
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int32_t x,
                                            int32_t y, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y),
        "r"(smem_u32(bar))
        : "memory");
}

// One 2-D TMA tile store from shared memory (rows and columns outside the tensor are clipped); part of
// the thread's current bulk group.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int32_t x, int32_t y, const void *smem_src)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(smem_src))
                 : "memory");
}

// The same tile added to what global memory holds (one IEEE addition per element, done in the memory
// system); part of the thread's current bulk group.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap *map, int32_t x, int32_t y, const void *smem_src)
{
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(smem_src))
                 : "memory");
}

__device__ __forceinline__ void bulk_commit_group()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// every bulk group of this thread has read its shared-memory source
__device__ __forceinline__ void bulk_wait_read_all()
{
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// every bulk group of this thread is complete
__device__ __forceinline__ void bulk_wait_all()
{
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

__device__ __forceinline__ void prefetch_tmap(const CUtensorMap *map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

// Warp-uniform election of one lane.
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
#endif  // __CUDACC__

}  // namespace ulmb200
