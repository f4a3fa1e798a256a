"""The CBLAS entry points in both storage orders, and their column-major twins, on the GPU.

Procedure of the reference's C tester (test/C/c_dblas3.c:14-75 dgemm, :130-176 dsyrk, :284-333
dtrsm): for CblasRowMajor the operands are copied into transposed (row-major) buffers whose
leading dimension is one more than the row length; the padding is filled with the tester's rogue
value and must come back untouched, inputs must come back bit-identical, and for triangular and
symmetric operands the unreferenced triangle holds the rogue value too.  Results are compared
with the compiled reference's own cblas_* (oracle/_ref/libulmref_cblas.so, interfaces/blas/C/
gemm.cc:296-485, trsm.cc:311-459, syrk.cc:146-263) wherever that is finite, and against a float64
numpy expectation under the componentwise bound everywhere."""
import ctypes as C
import itertools

import numpy as np
import pytest

import oracle
from helpers import EPS32, EPS64, ROGUE, bound_ratio, det_uniform

pytestmark = pytest.mark.gpu

ROW, COL = 101, 102
NT, TR, CT = 111, 112, 113
UP, LO = 121, 122
NU, UN = 131, 132
LE, RI = 141, 142


def _reflib():
    if not oracle.have_ref("cblas"):
        return None
    L = C.CDLL(oracle.ref_path("cblas"))
    for name in ("cblas_dgemm", "cblas_sgemm", "cblas_dtrsm", "cblas_dsyrk", "cblas_strsm", "cblas_ssyrk"):
        getattr(L, name).restype = None
    return L


REF = _reflib()


class Mat:
    """rows x cols values in the given storage order inside an allocation with ld = row length + 1
    (what the C tester does), padding = rogue."""

    def __init__(self, order, values, extra=1):
        self.order = order
        r, c = values.shape
        if order == COL:
            self.ld = r + extra
            self.base = np.full((self.ld, max(c, 1)), ROGUE, dtype=values.dtype, order="F")
            self.view = self.base[:r, :c]
        else:
            self.ld = c + extra
            self.base = np.full((max(r, 1), self.ld), ROGUE, dtype=values.dtype, order="C")
            self.view = self.base[:r, :c]
        self.view[...] = values
        self.before = self.base.copy(order="K")

    @property
    def ptr(self):
        return self.base.ctypes.data_as(C.c_void_p)

    def copy(self):
        m = Mat.__new__(Mat)
        m.order, m.ld = self.order, self.ld
        m.base = self.base.copy(order="K")
        r, c = self.view.shape
        m.view = m.base[:r, :c]
        m.before = self.before
        return m

    def padding_untouched(self):
        mask = np.ones(self.base.shape, bool)
        r, c = self.view.shape
        mask[:r, :c] = False
        return np.array_equal(self.base[mask], self.before[mask])

    def unchanged(self):
        return np.array_equal(self.base, self.before)


def opm(M, t):
    return M.T if t in (TR, CT) else M


def _real(ft):
    return C.c_float if ft == np.float32 else C.c_double


# ------------------------------------------------------------------------------------ gemm

def _gemm_case(ulm, routine, order, ta, tb, m, n, k, alpha, beta, seed, dtype, twin=False):
    A = det_uniform(seed, *((m, k) if ta == NT else (k, m)), dtype)
    B = det_uniform(seed + 1, *((k, n) if tb == NT else (n, k)), dtype)
    C0 = det_uniform(seed + 2, m, n, dtype)
    mA, mB, mC = Mat(order, A), Mat(order, B), Mat(order, C0)
    ft = _real(dtype)
    got = mC.copy()
    if twin:
        f = getattr(ulm.lib, routine)
        f.restype = None
        f(C.c_int(ta), C.c_int(tb), C.c_int(m), C.c_int(n), C.c_int(k), ft(alpha), mA.ptr, C.c_int(mA.ld), mB.ptr,
          C.c_int(mB.ld), ft(beta), got.ptr, C.c_int(got.ld))
    else:
        f = getattr(ulm.lib, routine)
        f.restype = None
        f(C.c_int(order), C.c_int(ta), C.c_int(tb), C.c_int(m), C.c_int(n), C.c_int(k), ft(alpha), mA.ptr,
          C.c_int(mA.ld), mB.ptr, C.c_int(mB.ld), ft(beta), got.ptr, C.c_int(got.ld))
    assert ulm.last_status() == ulm.OK, (routine, order, ta, tb, m, n, k)
    assert mA.unchanged() and mB.unchanged(), "an input operand was modified"
    assert got.padding_untouched(), "padding of C was written"
    eps = EPS32 if dtype == np.float32 else EPS64
    oa, ob = opm(A, ta).astype(np.float64), opm(B, tb).astype(np.float64)
    want = alpha * (oa @ ob) + beta * C0.astype(np.float64)
    gauge = abs(alpha) * (np.abs(oa) @ np.abs(ob)) + abs(beta) * np.abs(C0).astype(np.float64)
    ratio = bound_ratio(got.view, want, gauge, k, eps)
    # the float64 expectation is exact to 2^-52, the float result is rounded once more
    assert ratio <= 1.0 + (0.5 if dtype == np.float32 else 0.0), (routine, order, ta, tb, m, n, k, ratio)
    if REF is not None and not twin:
        ref = mC.copy()
        getattr(REF, routine)(C.c_int(order), C.c_int(ta), C.c_int(tb), C.c_int(m), C.c_int(n), C.c_int(k),
                              ft(alpha), mA.ptr, C.c_int(mA.ld), mB.ptr, C.c_int(mB.ld), ft(beta), ref.ptr,
                              C.c_int(ref.ld))
        fin = np.isfinite(ref.view)          # the reference's SSE build can emit NaN on edge tiles
        r2 = bound_ratio(np.where(fin, got.view, 0), np.where(fin, ref.view, 0), gauge, k, eps)
        assert r2 <= 1.0, (routine, "vs reference", order, ta, tb, m, n, k, r2)


SHAPES = [(7, 12, 31), (31, 7, 12), (1, 31, 2), (65, 130, 33), (129, 65, 17), (300, 260, 100)]


@pytest.mark.parametrize("routine,dtype", [("cblas_dgemm", np.float64), ("cblas_sgemm", np.float32)])
@pytest.mark.parametrize("order", [COL, ROW])
def test_cblas_gemm_both_orders(ulm, routine, dtype, order):
    seed = 41000 + (7 if order == ROW else 0)
    for (m, n, k) in SHAPES:
        for ta, tb in itertools.product((NT, TR), (NT, TR)):
            for alpha, beta in [(0.7, 1.3), (1.0, 0.0)]:
                seed += 3
                _gemm_case(ulm, routine, order, ta, tb, m, n, k, alpha, beta, seed, dtype)
    # conjugate-transpose is a transpose for the real types (gemm.cc:93-94)
    _gemm_case(ulm, routine, order, CT, NT, 31, 12, 7, 0.7, 1.3, seed + 3, dtype)


@pytest.mark.parametrize("routine,dtype", [("ulmblas_dgemm", np.float64), ("ulmblas_sgemm", np.float32)])
def test_column_major_gemm_twins(ulm, routine, dtype):
    """ULMBLAS(dgemm) / ULMBLAS(sgemm), interfaces/blas/C/gemm.cc:76-138, :10-72: no order argument."""
    seed = 42000
    for (m, n, k) in SHAPES[:4]:
        for ta, tb in itertools.product((NT, TR), (NT, TR)):
            seed += 3
            _gemm_case(ulm, routine, COL, ta, tb, m, n, k, 0.7, 1.3, seed, dtype, twin=True)


# ------------------------------------------------------------------------------------ trsm

def _tri(seed, na, upper_view, unit):
    """Well conditioned triangular matrix (values in the `upper_view` triangle of the logical
    matrix), rogue in the other triangle, rogue on the diagonal when it is declared unit."""
    A = det_uniform(seed, na, na) / max(na, 1)
    A[np.arange(na), np.arange(na)] = 1.5 + 0.25 * det_uniform(seed + 7, na, 1)[:, 0]
    T = np.triu(A) if upper_view else np.tril(A)
    stored = T.copy()
    other = np.tril(np.ones((na, na), bool), -1) if upper_view else np.triu(np.ones((na, na), bool), 1)
    stored[other] = ROGUE
    if unit:
        T[np.arange(na), np.arange(na)] = 1.0
        stored[np.arange(na), np.arange(na)] = ROGUE
    return T, stored


def _trsm_case(ulm, order, side, uplo, ta, diag, m, n, alpha, seed, twin=False, dtype=np.float64):
    na = m if side == LE else n
    T, stored = _tri(seed, na, uplo == UP, diag == UN)
    B0 = det_uniform(seed + 1, m, n)
    single = dtype == np.float32
    if single:
        # the values the routine sees are the rounded ones; the expectation is formed from those in float64
        T, stored, B0 = (x.astype(np.float32) for x in (T, stored, B0))
    name = "strsm" if single else "dtrsm"
    eps = EPS32 if single else EPS64
    mA, mB = Mat(order, stored), Mat(order, B0)
    got = mB.copy()
    args = [C.c_int(side), C.c_int(uplo), C.c_int(ta), C.c_int(diag), C.c_int(m), C.c_int(n), _real(dtype)(alpha),
            mA.ptr, C.c_int(mA.ld), got.ptr, C.c_int(got.ld)]
    T, B0 = T.astype(np.float64), B0.astype(np.float64)
    f = getattr(ulm.lib, ("ulmblas_" if twin else "cblas_") + name)
    f.restype = None
    f(*(args if twin else [C.c_int(order)] + args))
    assert ulm.last_status() == ulm.OK
    assert mA.unchanged(), "the triangular operand was modified"
    assert got.padding_untouched(), "padding of B was written"
    X = got.view.astype(np.float64)
    assert np.isfinite(X).all(), "the unreferenced triangle (rogue) leaked into the result"
    oT = opm(T, ta)
    # multiply back, the reference tester's check (test/F77/dblat3.f:1130-1155)
    back = oT @ X if side == LE else X @ oT
    gauge = (np.abs(oT) @ np.abs(X) if side == LE else np.abs(X) @ np.abs(oT)) + abs(alpha) * np.abs(B0)
    assert bound_ratio(back, alpha * B0, gauge, na, eps) <= 1.0, (name, order, side, uplo, ta, diag, m, n)
    if REF is not None and not twin:
        ref = mB.copy()
        getattr(REF, "cblas_" + name)(C.c_int(order), *args[:7], mA.ptr, C.c_int(mA.ld), ref.ptr, C.c_int(ref.ld))
        fin = np.isfinite(ref.view)          # the reference's SSE build can emit NaN on edge tiles
        assert fin.mean() > 0.5
        scale = max(1.0, np.abs(ref.view[fin]).max())
        # the C interface's single-precision solve works in float throughout (trsm.cc:12-80): na roundings
        tol = 16 * na * EPS32 if single else 1e-10
        assert np.abs(X[fin] - ref.view[fin]).max() <= tol * scale, (name, order, side, uplo, ta, diag)


@pytest.mark.parametrize("order", [COL, ROW])
def test_cblas_dtrsm_both_orders(ulm, order):
    """All sixteen side/uplo/trans/diag variants in each order; the row-major call becomes the
    column-major one with side and uplo exchanged and m, n swapped (trsm.cc:455-457)."""
    seed = 43000 + (5 if order == ROW else 0)
    for (m, n) in [(31, 12), (12, 31), (130, 70), (257, 40)]:
        for side, uplo, ta, diag in itertools.product((LE, RI), (UP, LO), (NT, TR), (NU, UN)):
            seed += 11
            _trsm_case(ulm, order, side, uplo, ta, diag, m, n, 0.7 if (seed % 2) else 1.0, seed)


def test_column_major_dtrsm_twin(ulm):
    seed = 43900
    for side, uplo, ta, diag in itertools.product((LE, RI), (UP, LO), (NT, TR), (NU, UN)):
        seed += 11
        _trsm_case(ulm, COL, side, uplo, ta, diag, 70, 45, 0.7, seed, twin=True)


@pytest.mark.parametrize("order", [COL, ROW])
def test_cblas_strsm_both_orders(ulm, order):
    """Single precision through CBLAS(strsm) (trsm.cc:311-384) and its column-major twin: same sixteen
    variants, multiply-back bound with the single-precision epsilon."""
    seed = 45000 + (5 if order == ROW else 0)
    for (m, n) in [(31, 12), (130, 70), (70, 257)]:
        for side, uplo, ta, diag in itertools.product((LE, RI), (UP, LO), (NT, TR), (NU, UN)):
            seed += 11
            _trsm_case(ulm, order, side, uplo, ta, diag, m, n, 0.7 if (seed % 2) else 1.0, seed, dtype=np.float32)
    if order == COL:
        for side, uplo in itertools.product((LE, RI), (UP, LO)):
            seed += 11
            _trsm_case(ulm, COL, side, uplo, TR, NU, 70, 45, 0.7, seed, twin=True, dtype=np.float32)


# ------------------------------------------------------------------------------------ syrk

def _syrk_case(ulm, order, uplo, tr, n, k, alpha, beta, seed, twin=False, dtype=np.float64):
    A = det_uniform(seed, *((n, k) if tr == NT else (k, n)), dtype)
    C0 = det_uniform(seed + 1, n, n, dtype)
    single = dtype == np.float32
    name = "ssyrk" if single else "dsyrk"
    eps = EPS32 if single else EPS64
    ft = _real(dtype)
    tri = np.triu(np.ones((n, n), bool)) if uplo == UP else np.tril(np.ones((n, n), bool))
    stored = np.where(tri, C0, dtype(ROGUE)).astype(dtype)
    mA, mC = Mat(order, A), Mat(order, stored)
    got = mC.copy()
    args = [C.c_int(uplo), C.c_int(tr), C.c_int(n), C.c_int(k), ft(alpha), mA.ptr, C.c_int(mA.ld),
            ft(beta), got.ptr, C.c_int(got.ld)]
    A, C0 = A.astype(np.float64), C0.astype(np.float64)
    f = getattr(ulm.lib, ("ulmblas_" if twin else "cblas_") + name)
    f.restype = None
    f(*(args if twin else [C.c_int(order)] + args))
    assert ulm.last_status() == ulm.OK
    assert mA.unchanged() and got.padding_untouched()
    assert np.array_equal(got.view[~tri], stored[~tri]), "the other triangle of C was written"
    oa = opm(A, tr)
    want = alpha * (oa @ oa.T) + beta * C0
    gauge = abs(alpha) * (np.abs(oa) @ np.abs(oa.T)) + abs(beta) * np.abs(C0)
    r = bound_ratio(np.where(tri, got.view, 0), np.where(tri, want, 0), gauge, k, eps)
    # the float64 expectation is exact to 2^-52, the float result is rounded once more
    assert r <= 1.0 + (0.5 if single else 0.0), (name, order, uplo, tr, n, k, r)
    if REF is not None and not twin:
        ref = mC.copy()
        getattr(REF, "cblas_" + name)(C.c_int(order), *args[:6], C.c_int(mA.ld), ft(beta), ref.ptr, C.c_int(ref.ld))
        fin = np.isfinite(ref.view) & tri
        r2 = bound_ratio(np.where(fin, got.view, 0), np.where(fin, ref.view, 0), gauge, k, eps)
        assert r2 <= 1.0, (name, "vs reference", order, uplo, tr, n, k, r2)


@pytest.mark.parametrize("order", [COL, ROW])
def test_cblas_dsyrk_both_orders(ulm, order):
    """Row-major: uplo flipped and trans toggled before the column-major routine (syrk.cc:259-261)."""
    seed = 44000 + (5 if order == ROW else 0)
    for (n, k) in [(31, 12), (12, 31), (130, 70), (257, 33)]:
        for uplo, tr in itertools.product((UP, LO), (NT, TR)):
            for alpha, beta in [(0.7, 1.3), (1.0, 0.0)]:
                seed += 5
                _syrk_case(ulm, order, uplo, tr, n, k, alpha, beta, seed)


def test_column_major_dsyrk_twin(ulm):
    seed = 44900
    for uplo, tr in itertools.product((UP, LO), (NT, TR)):
        seed += 5
        _syrk_case(ulm, COL, uplo, tr, 70, 45, 0.7, 1.3, seed, twin=True)


@pytest.mark.parametrize("order", [COL, ROW])
def test_cblas_ssyrk_both_orders(ulm, order):
    """Single precision through CBLAS(ssyrk) (syrk.cc:146-203) and its column-major twin."""
    seed = 46000 + (5 if order == ROW else 0)
    for (n, k) in [(31, 12), (130, 70), (257, 33)]:
        for uplo, tr in itertools.product((UP, LO), (NT, TR)):
            for alpha, beta in [(0.75, 1.25), (1.0, 0.0)]:
                seed += 5
                _syrk_case(ulm, order, uplo, tr, n, k, alpha, beta, seed, dtype=np.float32)
    if order == COL:
        for uplo, tr in itertools.product((UP, LO), (NT, TR)):
            seed += 5
            _syrk_case(ulm, COL, uplo, tr, 70, 45, 0.75, 1.25, seed, twin=True, dtype=np.float32)


# ------------------------------------------------------------------- quick paths with dummy operands

def test_alpha_zero_never_touches_a_or_b(ulm):
    """alpha == 0 (or k == 0) only scales C -- the reference returns before looking at A or B
    (ulmblas/level3/gemm.tcc:52-55, trlsm.tcc:46-49, syurk.tcc:44-51), so callers may pass dummy
    pointers for them."""
    m, n = 50, 40
    C0 = det_uniform(45000, m, n)
    got = C0.copy(order="F")
    one, zero, beta = C.c_double(1.0), C.c_double(0.0), C.c_double(1.3)
    ri = lambda v: C.byref(C.c_int(v))      # noqa: E731
    ulm.lib.dgemm_(b"N", b"N", ri(m), ri(n), ri(7), C.byref(zero), None, ri(m), None, ri(7), C.byref(beta),
                   got.ctypes.data_as(C.c_void_p), ri(m))
    assert ulm.last_status() == ulm.OK and np.array_equal(got, C0 * 1.3)
    got = C0.copy(order="F")
    ulm.lib.dgemm_(b"N", b"N", ri(m), ri(n), ri(0), C.byref(one), None, ri(m), None, ri(1), C.byref(zero),
                   got.ctypes.data_as(C.c_void_p), ri(m))
    assert ulm.last_status() == ulm.OK and not got.any()
    S0 = det_uniform(45001, n, n)
    got = S0.copy(order="F")
    ulm.lib.dsyrk_(b"U", b"N", ri(n), ri(9), C.byref(zero), None, ri(n), C.byref(beta),
                   got.ctypes.data_as(C.c_void_p), ri(n))
    up = np.triu(np.ones((n, n), bool))
    assert ulm.last_status() == ulm.OK
    assert np.array_equal(got[up], (S0 * 1.3)[up]) and np.array_equal(got[~up], S0[~up])
    got = C0.copy(order="F")
    ulm.lib.dtrsm_(b"L", b"L", b"N", b"N", ri(m), ri(n), C.byref(zero), None, ri(m), got.ctypes.data_as(C.c_void_p), ri(m))
    assert ulm.last_status() == ulm.OK and not got.any()
