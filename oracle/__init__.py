"""TEST INFRASTRUCTURE -- NOT PART OF THE PRODUCT.

ctypes front-ends for the two CPU checkers:

* ``Port``  -- ``oracle/libulm_oracle.so``, the plain-C restatement of the
  arithmetic of ulmBLAS's Level-3 GEMM path (``oracle/ulm_oracle.c``).
* ``Ref``   -- ``oracle/_ref/libulmref*.so``, ulmBLAS itself, compiled from its
  own sources by ``oracle/Makefile`` (Fortran-ABI symbols ``dgemm_`` ...,
  interfaces/blas/F77/gemm.cc:132, trsm.cc:121, syrk.cc:87 of the reference).

Only the tests, the smoke test and the bench's CPU-baseline leg may import
this package.  All matrices are numpy arrays in Fortran (column-major) order;
the leading dimension is ``a.strides[1] // a.itemsize`` so a view of the first
``m`` rows of a taller array exercises ``ld > m``.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

_i64, _dbl, _flt, _chr, _int = C.c_int64, C.c_double, C.c_float, C.c_char, C.c_int
_vp = C.c_void_p


def reference_tree():
    """Root of the ulmBLAS source tree: $ULMBLAS_REF, else a `reference` directory beside the
    repository; None when neither holds the sources."""
    cands = [os.environ.get("ULMBLAS_REF"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "interfaces", "blas", "F77", "gemm.cc")):
            return c
    return None


def build(ref=True):
    """Compile the restatement and, if the reference tree is present, the reference."""
    tree = reference_tree() if ref else None
    cmd = ["make", "-j8", "-C", _HERE, "all" if ref else "port"]
    if tree:
        cmd.append("REF=" + tree)
    subprocess.run(cmd, check=True, stdout=subprocess.DEVNULL)


def _ld(a):
    assert a.ndim == 2 and (a.shape[0] <= 1 or a.strides[0] == a.itemsize), "need a column-major matrix"
    return max(1, a.shape[0], a.strides[1] // a.itemsize if a.shape[1] > 0 else 1)


def _p(a):
    return a.ctypes.data_as(_vp)


def _c(ch):
    return ch.encode() if isinstance(ch, str) else ch


class Port:
    """The C restatement (``oracle/ulm_oracle.c``)."""

    def __init__(self, path=None):
        path = path or os.path.join(_HERE, "libulm_oracle.so")
        if not os.path.exists(path):
            build(ref=False)
        L = self.lib = C.CDLL(path)
        L.ulm_oracle_set_blocks.argtypes = [_int] * 3
        L.ulm_oracle_dgemm.argtypes = [_chr, _chr, _i64, _i64, _i64, _dbl, _vp, _i64,
                                       _vp, _i64, _dbl, _vp, _i64]
        L.ulm_oracle_sgemm.argtypes = [_chr, _chr, _i64, _i64, _i64, _flt, _vp, _i64,
                                       _vp, _i64, _flt, _vp, _i64]
        L.ulm_oracle_zgemm.argtypes = [_chr, _chr, _i64, _i64, _i64, _vp, _vp, _i64, _vp, _i64, _vp, _vp, _i64]
        L.ulm_oracle_zgemm.restype = None
        L.ulm_oracle_dtrsm.argtypes = [_chr] * 4 + [_i64, _i64, _dbl, _vp, _i64, _vp, _i64]
        L.ulm_oracle_dsyrk.argtypes = [_chr, _chr, _i64, _i64, _dbl, _vp, _i64, _dbl, _vp, _i64]
        L.ulm_oracle_gemm_info.argtypes = [_chr, _chr] + [_int] * 6
        L.ulm_oracle_trsm_info.argtypes = [_chr] * 4 + [_int] * 4
        L.ulm_oracle_syrk_info.argtypes = [_chr, _chr] + [_int] * 4
        for f in (L.ulm_oracle_dgemm, L.ulm_oracle_sgemm, L.ulm_oracle_dtrsm,
                  L.ulm_oracle_dsyrk, L.ulm_oracle_set_blocks):
            f.restype = None

    def set_blocks(self, mc=384, kc=384, nc=4096, kc_z=192):
        """Cache blocks of the real types and KC of complex double (defaults = the reference's)."""
        self.lib.ulm_oracle_set_blocks(mc, kc, nc)
        self.lib.ulm_oracle_set_blocks_z(kc_z)

    def dgemm(self, ta, tb, m, n, k, alpha, A, B, beta, Cm, lda=None, ldb=None, ldc=None):
        self.lib.ulm_oracle_dgemm(_c(ta), _c(tb), m, n, k, alpha, _p(A), lda or _ld(A),
                                  _p(B), ldb or _ld(B), beta, _p(Cm), ldc or _ld(Cm))

    def sgemm(self, ta, tb, m, n, k, alpha, A, B, beta, Cm, lda=None, ldb=None, ldc=None):
        self.lib.ulm_oracle_sgemm(_c(ta), _c(tb), m, n, k, alpha, _p(A), lda or _ld(A),
                                  _p(B), ldb or _ld(B), beta, _p(Cm), ldc or _ld(Cm))

    def zgemm(self, ta, tb, m, n, k, alpha, A, B, beta, Cm, lda=None, ldb=None, ldc=None):
        """complex128 column-major arrays; alpha, beta Python complex."""
        al, be = (_dbl * 2)(alpha.real, alpha.imag), (_dbl * 2)(beta.real, beta.imag)
        self.lib.ulm_oracle_zgemm(_c(ta), _c(tb), m, n, k, al, _p(A), lda or _ld(A),
                                  _p(B), ldb or _ld(B), be, _p(Cm), ldc or _ld(Cm))

    def dtrsm(self, side, uplo, ta, diag, m, n, alpha, A, B, lda=None, ldb=None):
        self.lib.ulm_oracle_dtrsm(_c(side), _c(uplo), _c(ta), _c(diag), m, n, alpha,
                                  _p(A), lda or _ld(A), _p(B), ldb or _ld(B))

    def dsyrk(self, uplo, trans, n, k, alpha, A, beta, Cm, lda=None, ldc=None):
        self.lib.ulm_oracle_dsyrk(_c(uplo), _c(trans), n, k, alpha, _p(A), lda or _ld(A),
                                  beta, _p(Cm), ldc or _ld(Cm))

    def gemm_info(self, ta, tb, m, n, k, lda, ldb, ldc):
        return self.lib.ulm_oracle_gemm_info(_c(ta), _c(tb), m, n, k, lda, ldb, ldc)

    def trsm_info(self, side, uplo, ta, diag, m, n, lda, ldb):
        return self.lib.ulm_oracle_trsm_info(_c(side), _c(uplo), _c(ta), _c(diag), m, n, lda, ldb)

    def syrk_info(self, uplo, trans, n, k, lda, ldc):
        return self.lib.ulm_oracle_syrk_info(_c(uplo), _c(trans), n, k, lda, ldc)


def ref_path(variant=""):
    name = {"": "libulmref.so", "tiny": "libulmref_tiny.so", "plain": "libulmref_plain.so", "lapack": "libulmref_lapack.so",
            "cblas": "libulmref_cblas.so", "nox": "libulmref_nox.so", "cblas_nox": "libulmref_cblas_nox.so"}[variant]
    return os.path.join(_HERE, "_ref", name)


def have_ref(variant=""):
    return os.path.exists(ref_path(variant))


class Ref:
    """ulmBLAS itself through its Fortran-ABI symbols (every argument by reference).

    Calls go through ``oracle/ref_shim.c``, which hands the reference a zeroed
    stack: its buffered micro-kernel reads an uninitialised stack tile and can
    otherwise emit NaN on finite inputs.
    """

    def __init__(self, variant=""):
        path = ref_path(variant)
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path}: run `make -C oracle ref` where the reference tree exists")
        self.lib = C.CDLL(path)     # RTLD_LOCAL: its dgemm_ never shadows the product's
        self.shim = Port().lib
        for f in (self.shim.ulm_shim_gemm, self.shim.ulm_shim_trsm, self.shim.ulm_shim_syrk):
            f.restype = None

    @staticmethod
    def _r(v, t):
        return C.byref(t(v))

    def _fn(self, name):
        return C.cast(getattr(self.lib, name), _vp)

    def _gemm(self, name, ft, ta, tb, m, n, k, alpha, A, B, beta, Cm, lda, ldb, ldc):
        r = self._r
        self.shim.ulm_shim_gemm(
            self._fn(name), C.c_char_p(_c(ta)), C.c_char_p(_c(tb)), r(m, _int), r(n, _int),
            r(k, _int), r(alpha, ft), _p(A), r(lda or _ld(A), _int), _p(B),
            r(ldb or _ld(B), _int), r(beta, ft), _p(Cm), r(ldc or _ld(Cm), _int))

    def dgemm(self, ta, tb, m, n, k, alpha, A, B, beta, Cm, lda=None, ldb=None, ldc=None):
        self._gemm("dgemm_", _dbl, ta, tb, m, n, k, alpha, A, B, beta, Cm, lda, ldb, ldc)

    def sgemm(self, ta, tb, m, n, k, alpha, A, B, beta, Cm, lda=None, ldb=None, ldc=None):
        self._gemm("sgemm_", _flt, ta, tb, m, n, k, alpha, A, B, beta, Cm, lda, ldb, ldc)

    def zgemm(self, ta, tb, m, n, k, alpha, A, B, beta, Cm, lda=None, ldb=None, ldc=None):
        """zgemm_ (interfaces/blas/F77/gemm.cc:381): complex128 arrays, alpha/beta by reference as {re, im}."""
        r = self._r
        al, be = (_dbl * 2)(alpha.real, alpha.imag), (_dbl * 2)(beta.real, beta.imag)
        self.shim.ulm_shim_gemm(
            self._fn("zgemm_"), C.c_char_p(_c(ta)), C.c_char_p(_c(tb)), r(m, _int), r(n, _int),
            r(k, _int), al, _p(A), r(lda or _ld(A), _int), _p(B),
            r(ldb or _ld(B), _int), be, _p(Cm), r(ldc or _ld(Cm), _int))

    def dtrsm(self, side, uplo, ta, diag, m, n, alpha, A, B, lda=None, ldb=None):
        r = self._r
        self.shim.ulm_shim_trsm(
            self._fn("dtrsm_"), C.c_char_p(_c(side)), C.c_char_p(_c(uplo)), C.c_char_p(_c(ta)),
            C.c_char_p(_c(diag)), r(m, _int), r(n, _int), r(alpha, _dbl),
            _p(A), r(lda or _ld(A), _int), _p(B), r(ldb or _ld(B), _int))

    def dsyrk(self, uplo, trans, n, k, alpha, A, beta, Cm, lda=None, ldc=None):
        r = self._r
        self.shim.ulm_shim_syrk(
            self._fn("dsyrk_"), C.c_char_p(_c(uplo)), C.c_char_p(_c(trans)), r(n, _int),
            r(k, _int), r(alpha, _dbl), _p(A), r(lda or _ld(A), _int), r(beta, _dbl),
            _p(Cm), r(ldc or _ld(Cm), _int))


def _ref_extra(self):
    r = self._r

    def dsymm(side, uplo, m, n, alpha, A, B, beta, Cm, lda=None, ldb=None, ldc=None):
        self.lib.dsymm_(C.c_char_p(_c(side)), C.c_char_p(_c(uplo)), r(m, _int), r(n, _int), r(alpha, _dbl),
                        _p(A), r(lda or _ld(A), _int), _p(B), r(ldb or _ld(B), _int), r(beta, _dbl), _p(Cm),
                        r(ldc or _ld(Cm), _int))

    def dtrmm(side, uplo, ta, diag, m, n, alpha, A, B, lda=None, ldb=None):
        self.lib.dtrmm_(C.c_char_p(_c(side)), C.c_char_p(_c(uplo)), C.c_char_p(_c(ta)), C.c_char_p(_c(diag)),
                        r(m, _int), r(n, _int), r(alpha, _dbl), _p(A), r(lda or _ld(A), _int), _p(B),
                        r(ldb or _ld(B), _int))

    def dsyr2k(uplo, trans, n, k, alpha, A, B, beta, Cm, lda=None, ldb=None, ldc=None):
        self.lib.dsyr2k_(C.c_char_p(_c(uplo)), C.c_char_p(_c(trans)), r(n, _int), r(k, _int), r(alpha, _dbl),
                         _p(A), r(lda or _ld(A), _int), _p(B), r(ldb or _ld(B), _int), r(beta, _dbl), _p(Cm),
                         r(ldc or _ld(Cm), _int))

    def ssyrk(uplo, trans, n, k, alpha, A, beta, Cm, lda=None, ldc=None):
        self.lib.ssyrk_(C.c_char_p(_c(uplo)), C.c_char_p(_c(trans)), r(n, _int), r(k, _int), r(alpha, _flt),
                        _p(A), r(lda or _ld(A), _int), r(beta, _flt), _p(Cm), r(ldc or _ld(Cm), _int))

    def strsm(side, uplo, ta, diag, m, n, alpha, A, B, lda=None, ldb=None):
        self.lib.strsm_(C.c_char_p(_c(side)), C.c_char_p(_c(uplo)), C.c_char_p(_c(ta)), C.c_char_p(_c(diag)),
                        r(m, _int), r(n, _int), r(alpha, _flt), _p(A), r(lda or _ld(A), _int), _p(B),
                        r(ldb or _ld(B), _int))

    return dsymm, dtrmm, dsyr2k, ssyrk, strsm


def _ref_getattr(self, name):
    """dsymm / dtrmm / dsyr2k / ssyrk / strsm of the compiled reference (interfaces/blas/F77/symm.cc:87,
    trmm.cc:123, syr2k.cc:92), bound on first use."""
    if name in ("dsymm", "dtrmm", "dsyr2k", "ssyrk", "strsm"):
        fns = dict(zip(("dsymm", "dtrmm", "dsyr2k", "ssyrk", "strsm"), _ref_extra(self)))
        self.__dict__.update(fns)
        return fns[name]
    raise AttributeError(name)


Ref.__getattr__ = _ref_getattr


def ref_dgetrf(A, lda=None):
    """ulmblas_dgetrf of the compiled reference (interfaces/lapack/C/getrf.cc:6-19), column-major,
    in place on the numpy matrix A; returns (piv, info) with the reference's 0-based pivots."""
    L = C.CDLL(ref_path("lapack"))
    m, n = A.shape
    piv = (C.c_int * max(1, min(m, n)))()
    L.ulmblas_dgetrf.restype = _int
    info = L.ulmblas_dgetrf(C.c_int(102), C.c_int(m), C.c_int(n), _p(A), C.c_int(lda or _ld(A)), piv)
    return np.array(piv[:min(m, n)], dtype=np.int64), int(info)


def fmat(rows, cols, ld=None, dtype=np.float64, fill=None):
    """Column-major rows x cols view on top of an ld x cols allocation (padding = ``fill``)."""
    ld = max(ld or rows, rows, 1)
    base = np.empty((ld, max(cols, 1)), dtype=dtype, order="F")
    if fill is not None:
        base[...] = fill
    return base[:rows, :cols], base
