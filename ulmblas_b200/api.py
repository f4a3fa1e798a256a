"""Bindings of libulmblas_b200.so (imported lazily by the package).

The product is ``libulmblas_b200.so`` (built in-tree by ``python -m ulmblas_b200.build``):
hand-written sm_100a kernels behind a plain C ABI (``include/ulmblas_b200.h``).  This
module is the thin host-side mirror of the reference's interface for that path:

* ``dgemm / sgemm / dtrsm / dsyrk`` take numpy column-major arrays and go through the
  very symbols a Fortran or C caller of the reference binds (``dgemm_`` ...,
  interfaces/blas/F77/gemm.cc:132, trsm.cc:121, syrk.cc:87 of the reference), host
  pointers and all.
* ``dev_dgemm / dev_sgemm / dev_dtrsm / dev_dsyrk`` take device pointers (ints, e.g.
  ``tensor.data_ptr()``) and a CUDA stream handle and call the device ABI.

There is no CPU implementation here and no fallback: if the shared library is missing
the import fails, and without an sm_100 device every call reports status 3.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libulmblas_b200.so")
SUPPORT_LIB_PATH = os.path.join(_HERE, "libulmb200_benchsupport.so")

OK, BAD_ARGUMENT, CUDA_ERROR, NO_DEVICE, KERNEL_FAULT, TOO_LARGE = range(6)
SGEMM_FP32, SGEMM_3XTF32 = 0, 1


class LibraryMissing(ImportError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise LibraryMissing(
            f"{LIB_PATH} is missing: build it with `python -m ulmblas_b200.build` "
            "(needs nvcc); there is no CPU fallback")
    return C.CDLL(LIB_PATH)


lib = _load()


def _load_support():
    """libulmb200_benchsupport.so: generator, probes and self tests (not part of the product)."""
    if not os.path.exists(SUPPORT_LIB_PATH):
        raise LibraryMissing(f"{SUPPORT_LIB_PATH} is missing: build it with `python -m ulmblas_b200.build`")
    return C.CDLL(SUPPORT_LIB_PATH)


sup = _load_support()

_i64, _dbl, _flt, _int, _vp, _u64, _u32 = (C.c_int64, C.c_double, C.c_float, C.c_int, C.c_void_p,
                                           C.c_uint64, C.c_uint32)
_pi, _pd, _pf, _cp = C.POINTER(C.c_int), C.POINTER(C.c_double), C.POINTER(C.c_float), C.c_char_p

lib.ulmb200_last_status.restype = _int
lib.ulmb200_status_string.restype = C.c_char_p
lib.ulmb200_status_string.argtypes = [_int]
lib.ulmb200_launch_count.restype = _i64
sup.ulmb200_selftest_wait_timeout.restype = _int
sup.ulmb200_selftest_wait_timeout_noalloc_word.restype = _int
lib.ulmb200_alloc_count.restype = _i64
lib.ulmb200_workspace_bytes.restype = _i64
lib.ulmb200_release_workspace.restype = _int
lib.ulmb200_check_device_error.argtypes = [_vp]
lib.ulmb200_check_device_error.restype = _int
lib.ulmb200_reload_env.restype = None
lib.ulmb200_dgemm.argtypes = [_vp, _int, _int, _i64, _i64, _i64, _dbl, _vp, _i64, _vp, _i64, _dbl, _vp, _i64]
lib.ulmb200_sgemm.argtypes = [_vp, _int, _int, _int, _i64, _i64, _i64, _flt, _vp, _i64, _vp, _i64, _flt, _vp, _i64]
lib.ulmb200_dtrsm.argtypes = [_vp, _int, _int, _int, _int, _i64, _i64, _dbl, _vp, _i64, _vp, _i64]
lib.ulmb200_dtrsm_noalloc.argtypes = [_vp, _int, _int, _int, _int, _i64, _i64, _dbl, _vp, _i64, _vp, _i64]
lib.ulmb200_dsyrk.argtypes = [_vp, _int, _int, _i64, _i64, _dbl, _vp, _i64, _dbl, _vp, _i64]
sup.ulmb200_fill_f64.argtypes = [_vp, _vp, _i64, _i64, _i64, _u64, _u32, _i64, _i64, _int, _dbl]
sup.ulmb200_fill_f32.argtypes = [_vp, _vp, _i64, _i64, _i64, _u64, _u32, _i64, _i64]
sup.ulmb200_host_fill_f64.argtypes = [_vp, _i64, _i64, _i64, _u64, _u32, _i64, _i64, _int, _dbl]
sup.ulmb200_host_fill_f64.restype = None
sup.ulmb200_host_fill_f32.argtypes = [_vp, _i64, _i64, _i64, _u64, _u32, _i64, _i64]
sup.ulmb200_host_fill_f32.restype = None
sup.ulmb200_abs_f64.argtypes = [_vp, _vp, _i64, _i64, _i64]
sup.ulmb200_peak_probe.argtypes = [_int, _int, _pd, _pd]
lib.ulmb200_set_sm_reserve.argtypes = [_int]
lib.ulmb200_set_sm_reserve.restype = None
lib.ulmb200_set_pin_host.argtypes = [_int]
lib.ulmb200_set_pin_host.restype = None
lib.ulmb200_dgetrf.argtypes = [_vp, _i64, _i64, _vp, _i64, _vp, _vp]
lib.ulmblas_dgetrf.argtypes = [_int, _int, _int, _vp, _int, _vp]
lib.ulmblas_dgetrf.restype = _int
lib.ulmblas_dlaswp.argtypes = [_int, _vp, _int, _int, _int, _vp, _int]
lib.ulmblas_dlaswp.restype = None
lib.ulmb200_dsymm.argtypes = [_vp, _int, _int, _i64, _i64, _dbl, _vp, _i64, _vp, _i64, _dbl, _vp, _i64]
lib.ulmb200_dtrmm.argtypes = [_vp, _int, _int, _int, _int, _i64, _i64, _dbl, _vp, _i64, _vp, _i64]
lib.ulmb200_dsyr2k.argtypes = [_vp, _int, _int, _i64, _i64, _dbl, _vp, _i64, _vp, _i64, _dbl, _vp, _i64]
lib.ulmb200_ssyrk.argtypes = [_vp, _int, _int, _i64, _i64, _flt, _vp, _i64, _flt, _vp, _i64]
lib.ulmb200_strsm.argtypes = [_vp, _int, _int, _int, _int, _i64, _i64, _flt, _vp, _i64, _vp, _i64]
for _name in ("strsm_", "ssyrk_", "dsymm_", "dtrmm_", "dsyr2k_", "dgemm_", "sgemm_", "dtrsm_", "dsyrk_", "cblas_dgemm", "cblas_sgemm", "cblas_dtrsm",
              "cblas_dsyrk", "ulmblas_dgemm", "ulmblas_sgemm", "ulmblas_dtrsm", "ulmblas_dsyrk"):
    getattr(lib, _name).restype = None
lib.cblas_dgemm.argtypes = [_int, _int, _int, _int, _int, _int, _dbl, _vp, _int, _vp, _int, _dbl, _vp, _int]
lib.cblas_sgemm.argtypes = [_int, _int, _int, _int, _int, _int, _flt, _vp, _int, _vp, _int, _flt, _vp, _int]
lib.cblas_dtrsm.argtypes = [_int, _int, _int, _int, _int, _int, _int, _dbl, _vp, _int, _vp, _int]
lib.cblas_dsymm.argtypes = [_int, _int, _int, _int, _int, _dbl, _vp, _int, _vp, _int, _dbl, _vp, _int]
lib.cblas_dtrmm.argtypes = [_int, _int, _int, _int, _int, _int, _int, _dbl, _vp, _int, _vp, _int]
lib.cblas_dsyr2k.argtypes = [_int, _int, _int, _int, _int, _dbl, _vp, _int, _vp, _int, _dbl, _vp, _int]
for _name in ("cblas_dsymm", "cblas_dtrmm", "cblas_dsyr2k"):
    getattr(lib, _name).restype = None
lib.cblas_dsyrk.argtypes = [_int, _int, _int, _int, _int, _dbl, _vp, _int, _dbl, _vp, _int]
lib.ulmb200_zgemm.argtypes = [_vp, _int, _int, _int, _int, _i64, _i64, _i64, _vp, _vp, _i64, _vp, _i64, _vp, _vp, _i64]
lib.cblas_zgemm.argtypes = [_int, _int, _int, _int, _int, _int, _vp, _vp, _int, _vp, _int, _vp, _vp, _int]
lib.ulmblas_zgemm.argtypes = [_int, _int, _int, _int, _int, _vp, _vp, _int, _vp, _int, _vp, _vp, _int]
for _name in ("zgemm_", "cblas_zgemm", "ulmblas_zgemm"):
    getattr(lib, _name).restype = None

_pi64 = C.POINTER(C.c_int64)
lib.ulmb200_mg_unique_id.argtypes = [C.c_char_p]
lib.ulmb200_mg_init.argtypes = [C.c_char_p, _int, _int, C.POINTER(_vp)]
lib.ulmb200_mg_finalize.argtypes = [_vp]
lib.ulmb200_mg_column_block.argtypes = [_i64, _int, _int, _pi64, _pi64]
lib.ulmb200_mg_dgemm.argtypes = [_vp, _vp, _i64, _i64, _i64, _dbl, _vp, _i64, _vp, _i64, _dbl, _vp, _i64, _int]
lib.ulmb200_mg_dgemm_host.argtypes = [_vp, _vp, _i64, _i64, _i64, _dbl, _vp, _i64, _vp, _i64, _dbl, _vp, _i64,
                                      _vp, _vp, _i64, _vp, _i64, _int, _int]
lib.ulmb200_mg_wait.argtypes = [_vp, _int]
lib.ulmb200_mg_plan_panels.argtypes = [_i64, _i64, _i64, _int, _i64, _dbl, _dbl, _pi64, _pi, _int]
lib.ulmb200_mg_last_plan.argtypes = [_vp, _pi64, _pi, _int, _pd, _pd]
lib.ulmb200_mg_set_rates.argtypes = [_vp, _dbl, _dbl, _dbl]
lib.ulmb200_mg_profile.argtypes = [_vp, _int]
lib.ulmb200_mg_last_gemm_ms.argtypes = [_vp, _pd, _int]
lib.ulmb200_mg_last_gemm_start_ms.argtypes = [_vp, _pd, _int]
lib.ulmb200_mg_last_step_gap_ms.argtypes = [_vp, _pd]

CblasRowMajor, CblasColMajor = 101, 102
CblasNoTrans, CblasTrans, CblasConjTrans, AtlasConj = 111, 112, 113, 114
CblasUpper, CblasLower = 121, 122
CblasNonUnit, CblasUnit = 131, 132
CblasLeft, CblasRight = 141, 142


class Ulmb200Error(RuntimeError):
    def __init__(self, status, where):
        self.status = status
        super().__init__(f"{where}: status {status} ({status_string(status)})")


def last_status():
    return lib.ulmb200_last_status()


def status_string(st):
    return lib.ulmb200_status_string(st).decode()


def launch_count():
    return lib.ulmb200_launch_count()


def _check(st, where):
    if st != OK:
        raise Ulmb200Error(st, where)


def _ld(a):
    if a.ndim != 2 or (a.shape[0] > 1 and a.strides[0] != a.itemsize):
        raise ValueError("matrices must be 2-D and column-major (unit stride down a column)")
    return max(1, a.shape[0], a.strides[1] // a.itemsize if a.shape[1] > 0 else 1)


def _p(a):
    return a.ctypes.data_as(_vp)


def _c(ch):
    return ch.encode() if isinstance(ch, str) else ch


def _ri(v):
    return C.byref(C.c_int(v))


# --------------------------------------------------------------------------- host-pointer calls
# (the reference's Fortran ABI: every argument by reference, 32-bit int)

def dgemm(transA, transB, m, n, k, alpha, A, B, beta, Cm, lda=None, ldb=None, ldc=None):
    """C <- alpha*op(A)*op(B) + beta*C through ``dgemm_`` (numpy arrays, in place on ``Cm``)."""
    lib.dgemm_(_cp(_c(transA)), _cp(_c(transB)), _ri(m), _ri(n), _ri(k), C.byref(_dbl(alpha)),
               _p(A), _ri(lda or _ld(A)), _p(B), _ri(ldb or _ld(B)), C.byref(_dbl(beta)), _p(Cm),
               _ri(ldc or _ld(Cm)))
    return last_status()


def _z2(z):
    z = complex(z)
    return (_dbl * 2)(z.real, z.imag)


def zgemm(transA, transB, m, n, k, alpha, A, B, beta, Cm, lda=None, ldb=None, ldc=None):
    """C <- alpha*op(A)*op(B) + beta*C through ``zgemm_`` (complex128 arrays; trans N, T, C or R)."""
    lib.zgemm_(_cp(_c(transA)), _cp(_c(transB)), _ri(m), _ri(n), _ri(k), _z2(alpha),
               _p(A), _ri(lda or _ld(A)), _p(B), _ri(ldb or _ld(B)), _z2(beta), _p(Cm),
               _ri(ldc or _ld(Cm)))
    return last_status()


def cblas_zgemm(order, transA, transB, m, n, k, alpha, A, lda, B, ldb, beta, Cm, ldc):
    lib.cblas_zgemm(order, transA, transB, m, n, k, _z2(alpha), _p(A), lda, _p(B), ldb, _z2(beta), _p(Cm), ldc)
    return last_status()


def dev_zgemm(transA, conjA, transB, conjB, m, n, k, alpha, dA, lda, dB, ldb, beta, dC, ldc, stream=0):
    _check(lib.ulmb200_zgemm(stream, int(transA), int(conjA), int(transB), int(conjB), m, n, k, _z2(alpha),
                             dA, lda, dB, ldb, _z2(beta), dC, ldc), "ulmb200_zgemm")


def sgemm(transA, transB, m, n, k, alpha, A, B, beta, Cm, lda=None, ldb=None, ldc=None):
    """C <- alpha*op(A)*op(B) + beta*C through ``sgemm_`` (float32)."""
    lib.sgemm_(_cp(_c(transA)), _cp(_c(transB)), _ri(m), _ri(n), _ri(k), C.byref(_flt(alpha)),
               _p(A), _ri(lda or _ld(A)), _p(B), _ri(ldb or _ld(B)), C.byref(_flt(beta)), _p(Cm),
               _ri(ldc or _ld(Cm)))
    return last_status()


def dtrsm(side, uplo, transA, diag, m, n, alpha, A, B, lda=None, ldb=None):
    """B <- alpha*op(A)^-1*B or alpha*B*op(A)^-1 through ``dtrsm_``."""
    lib.dtrsm_(_cp(_c(side)), _cp(_c(uplo)), _cp(_c(transA)), _cp(_c(diag)), _ri(m), _ri(n),
               C.byref(_dbl(alpha)), _p(A), _ri(lda or _ld(A)), _p(B), _ri(ldb or _ld(B)))
    return last_status()


def dsyrk(uplo, trans, n, k, alpha, A, beta, Cm, lda=None, ldc=None):
    """One triangle of C <- alpha*op(A)*op(A)^T + beta*C through ``dsyrk_``."""
    lib.dsyrk_(_cp(_c(uplo)), _cp(_c(trans)), _ri(n), _ri(k), C.byref(_dbl(alpha)), _p(A),
               _ri(lda or _ld(A)), C.byref(_dbl(beta)), _p(Cm), _ri(ldc or _ld(Cm)))
    return last_status()


def ssyrk(uplo, trans, n, k, alpha, A, beta, Cm, lda=None, ldc=None):
    """Single-precision SYRK through ``ssyrk_`` (float32 arrays)."""
    lib.ssyrk_(_cp(_c(uplo)), _cp(_c(trans)), _ri(n), _ri(k), C.byref(_flt(alpha)), _p(A),
               _ri(lda or _ld(A)), C.byref(_flt(beta)), _p(Cm), _ri(ldc or _ld(Cm)))
    return last_status()


def strsm(side, uplo, transA, diag, m, n, alpha, A, B, lda=None, ldb=None):
    """Single-precision TRSM through ``strsm_`` (float32 arrays)."""
    lib.strsm_(_cp(_c(side)), _cp(_c(uplo)), _cp(_c(transA)), _cp(_c(diag)), _ri(m), _ri(n),
               C.byref(_flt(alpha)), _p(A), _ri(lda or _ld(A)), _p(B), _ri(ldb or _ld(B)))
    return last_status()


def dsymm(side, uplo, m, n, alpha, A, B, beta, Cm, lda=None, ldb=None, ldc=None):
    """C <- alpha*A*B + beta*C (side 'L') or alpha*B*A + beta*C ('R'), A symmetric, through ``dsymm_``."""
    lib.dsymm_(_cp(_c(side)), _cp(_c(uplo)), _ri(m), _ri(n), C.byref(_dbl(alpha)), _p(A), _ri(lda or _ld(A)),
               _p(B), _ri(ldb or _ld(B)), C.byref(_dbl(beta)), _p(Cm), _ri(ldc or _ld(Cm)))
    return last_status()


def dtrmm(side, uplo, transA, diag, m, n, alpha, A, B, lda=None, ldb=None):
    """B <- alpha*op(A)*B or alpha*B*op(A), A triangular, through ``dtrmm_``."""
    lib.dtrmm_(_cp(_c(side)), _cp(_c(uplo)), _cp(_c(transA)), _cp(_c(diag)), _ri(m), _ri(n),
               C.byref(_dbl(alpha)), _p(A), _ri(lda or _ld(A)), _p(B), _ri(ldb or _ld(B)))
    return last_status()


def dsyr2k(uplo, trans, n, k, alpha, A, B, beta, Cm, lda=None, ldb=None, ldc=None):
    """One triangle of C <- alpha*(op(A)*op(B)^T + op(B)*op(A)^T) + beta*C through ``dsyr2k_``."""
    lib.dsyr2k_(_cp(_c(uplo)), _cp(_c(trans)), _ri(n), _ri(k), C.byref(_dbl(alpha)), _p(A), _ri(lda or _ld(A)),
                _p(B), _ri(ldb or _ld(B)), C.byref(_dbl(beta)), _p(Cm), _ri(ldc or _ld(Cm)))
    return last_status()


def dgetrf(A, lda=None):
    """LU with partial pivoting in place on a numpy column-major matrix through ``ulmblas_dgetrf``;
    returns (piv, info) with the reference's 0-based pivots."""
    m, n = A.shape
    piv = np.zeros(max(1, min(m, n)), dtype=np.int32)
    info = lib.ulmblas_dgetrf(CblasColMajor, m, n, _p(A), lda or _ld(A), piv.ctypes.data_as(_vp))
    return piv[:min(m, n)].astype(np.int64), info


# --------------------------------------------------------------------------- device-pointer calls

def dev_dgemm(transA, transB, m, n, k, alpha, dA, lda, dB, ldb, beta, dC, ldc, stream=0):
    _check(lib.ulmb200_dgemm(stream, int(transA), int(transB), m, n, k, alpha, dA, lda, dB, ldb, beta,
                             dC, ldc), "ulmb200_dgemm")


def dev_sgemm(mode, transA, transB, m, n, k, alpha, dA, lda, dB, ldb, beta, dC, ldc, stream=0):
    _check(lib.ulmb200_sgemm(stream, mode, int(transA), int(transB), m, n, k, alpha, dA, lda, dB, ldb,
                             beta, dC, ldc), "ulmb200_sgemm")


def dev_dtrsm(side, lower, transA, unit, m, n, alpha, dA, lda, dB, ldb, stream=0):
    _check(lib.ulmb200_dtrsm(stream, int(side), int(lower), int(transA), int(unit), m, n, alpha, dA, lda,
                             dB, ldb), "ulmb200_dtrsm")


def dev_dtrsm_noalloc(side, lower, transA, unit, m, n, alpha, dA, lda, dB, ldb, stream=0):
    """ulmb200_dtrsm on the library's built-in work area: never allocates device memory.
    Triangle <= 2048, other dimension <= 4096 (status TOO_LARGE beyond); calls on one GPU
    must not overlap in time.  Returns the status instead of raising."""
    return lib.ulmb200_dtrsm_noalloc(stream, int(side), int(lower), int(transA), int(unit), m, n, alpha,
                                     dA, lda, dB, ldb)


def dev_dsyrk(lower, trans, n, k, alpha, dA, lda, beta, dC, ldc, stream=0):
    _check(lib.ulmb200_dsyrk(stream, int(lower), int(trans), n, k, alpha, dA, lda, beta, dC, ldc),
           "ulmb200_dsyrk")


def dev_fill_f64(d, ld, rows, cols, seed, mat, row0=0, col0=0, dist=0, scale=1.0, stream=0):
    _check(sup.ulmb200_fill_f64(stream, d, ld, rows, cols, seed, mat, row0, col0, dist, scale),
           "ulmb200_fill_f64")


def dev_fill_f32(d, ld, rows, cols, seed, mat, row0=0, col0=0, stream=0):
    _check(sup.ulmb200_fill_f32(stream, d, ld, rows, cols, seed, mat, row0, col0), "ulmb200_fill_f32")


def host_fill(a, seed, mat, row0=0, col0=0, dist=0, scale=1.0):
    """Fill a numpy column-major matrix with the library's deterministic generator."""
    rows, cols = a.shape
    if a.dtype == np.float64:
        sup.ulmb200_host_fill_f64(_p(a), _ld(a), rows, cols, seed, mat, row0, col0, dist, scale)
    elif a.dtype == np.float32:
        sup.ulmb200_host_fill_f32(_p(a), _ld(a), rows, cols, seed, mat, row0, col0)
    else:
        raise TypeError("float64 or float32 only")
    return a


def reload_env():
    """The library reads its ULMB200_* environment variables once; read them again."""
    lib.ulmb200_reload_env()


def check_device_error(stream=0):
    """Waits for `stream`; KERNEL_FAULT if a kernel gave up on a bounded wait since the last check."""
    return lib.ulmb200_check_device_error(stream)


def alloc_count():
    return lib.ulmb200_alloc_count()


def workspace_bytes():
    return lib.ulmb200_workspace_bytes()


def release_workspace():
    return lib.ulmb200_release_workspace()


def mg_column_block(n, world, rank):
    """[j0, j1): the columns of B and C that rank `rank` of `world` owns (ulmb200_mg_column_block)."""
    j0, j1 = C.c_int64(0), C.c_int64(0)
    _check(lib.ulmb200_mg_column_block(n, world, rank, C.byref(j0), C.byref(j1)), "ulmb200_mg_column_block")
    return j0.value, j1.value


def mg_plan_panels(m, n_block, k, world, first=1024, transport_gbs=150.0, gemm_tflops=35.0):
    """([width of each K panel], [1 where that panel's product leaves SMs to the transport])."""
    w, r = (C.c_int64 * 32)(), (C.c_int * 32)()
    n = lib.ulmb200_mg_plan_panels(m, n_block, k, world, first, transport_gbs, gemm_tflops, w, r, 32)
    if n < 0:
        raise ValueError("bad argument to ulmb200_mg_plan_panels")
    return [int(w[i]) for i in range(n)], [int(r[i]) for i in range(n)]


def set_sm_reserve(sms):
    """Leave `sms` SMs free in the following persistent DGEMM launches (0 = use them all)."""
    lib.ulmb200_set_sm_reserve(int(sms))


def peak_probe(which, iters=2000):
    """Register-only throughput probe: returns (TFLOP/s, ms)."""
    tf, ms = _dbl(0.0), _dbl(0.0)
    _check(sup.ulmb200_peak_probe(which, iters, C.byref(tf), C.byref(ms)), "ulmb200_peak_probe")
    return tf.value, ms.value


def fmat(rows, cols, ld=None, dtype=np.float64, fill=None):
    """rows x cols column-major view over an ld x cols allocation; returns (view, base)."""
    ld = max(ld or rows, rows, 1)
    base = np.empty((ld, max(cols, 1)), dtype=dtype, order="F")
    if fill is not None:
        base[...] = fill
    return base[:rows, :cols], base
