"""Blocked LU (ulmblas_dgetrf) on the GPU against the reference's own getrf
(ulmblas/lapack/getrf.tcc), the in-tree caller of trlsm + gemm."""
import numpy as np
import pytest

import oracle
from helpers import EPS64, det_uniform, padded

pytestmark = pytest.mark.gpu


def apply_piv(A, piv):
    P = A.copy()
    for i, p in enumerate(piv):
        if p != i:
            P[[i, p]] = P[[p, i]]
    return P


def check_lu(ulm, m, n, seed, extra=3):
    A0 = det_uniform(seed, m, n)
    Av, Ab = padded(A0, m + extra)
    got = Ab.copy(order="F")
    piv, info = ulm.dgetrf(got[:m, :n], lda=m + extra)
    assert ulm.last_status() == ulm.OK and info == 0
    assert np.array_equal(got[m:, :], Ab[m:, :]), "padding rows written"
    mn = min(m, n)
    LU = got[:m, :n]
    L = np.tril(LU, -1)[:, :mn] + np.eye(m, mn)
    U = np.triu(LU)[:mn, :]
    assert np.abs(np.tril(LU, -1)).max() <= 1.0 + 1e-12, "partial pivoting keeps |l_ij| <= 1"
    # backward error of the factorisation: |P A - L U| <= c * mn * eps * |L||U|
    resid = np.abs(apply_piv(A0, piv) - L @ U)
    bound = 4.0 * mn * EPS64 * (np.abs(L) @ np.abs(U))
    assert (resid <= bound + 1e-300).all(), (m, n, float((resid / np.maximum(bound, 1e-300)).max()))
    if oracle.have_ref("lapack"):
        want = Ab.copy(order="F")
        rpiv, rinfo = oracle.ref_dgetrf(want[:m, :n], lda=m + extra)
        assert rinfo == 0
        # same pivot sequence (first-largest rule) and factors equal up to rounding
        assert np.array_equal(piv, rpiv), (m, n)
        scale = np.abs(L) @ np.abs(U)
        assert (np.abs(LU - want[:m, :n]) <= 8.0 * mn * EPS64 * np.maximum(scale, 1.0)).all(), (m, n)


def test_dgetrf_shapes(ulm):
    for i, (m, n) in enumerate([(1, 1), (7, 5), (5, 7), (31, 31), (130, 130), (300, 200), (200, 300),
                                (513, 513), (1100, 700),
                                (5000, 300),        # more than 4096 rows: two rows per thread in the register panel
                                (9000, 160),        # more than 8192 rows: the cluster panel held in shared memory
                                (14000, 40),        # ... with 16-column sub-panels
                                (30000, 40),        # ... with 8-column sub-panels
                                (60000, 20)]):      # too tall for a cluster's shared memory: cooperative panel
        check_lu(ulm, m, n, 70000 + i)


def test_dgetrf_ties_follow_the_first_largest_rule(ulm):
    """A = [B; B]: every row has a bit-identical twin, and twins stay bit-identical under elimination
    (same operations on the same numbers), so every pivot search ends in an exact tie between two
    rows.  The first of the two in the CURRENT row order has to win, as in the reference
    (iamax returns the first maximum)."""
    for i, (k, n) in enumerate([(32, 20), (300, 200), (5000, 96)]):
        B = det_uniform(72000 + i, k, n)
        A0 = np.asfortranarray(np.vstack([B, B]))
        m = 2 * k
        got = A0.copy(order="F")
        piv, info = ulm.dgetrf(got)
        assert ulm.last_status() == ulm.OK and info == 0
        if oracle.have_ref("lapack"):
            want = A0.copy(order="F")
            rpiv, rinfo = oracle.ref_dgetrf(want)
            assert rinfo == 0
            assert np.array_equal(piv, rpiv), (k, n, int(np.argmax(piv != rpiv)))
        mn = min(m, n)
        L = np.tril(got, -1)[:, :mn] + np.eye(m, mn)
        U = np.triu(got)[:mn, :]
        resid = np.abs(apply_piv(A0, piv) - L @ U)
        assert (resid <= 4.0 * mn * EPS64 * (np.abs(L) @ np.abs(U)) + 1e-300).all()
        # each pivot row's twin has a multiplier of 1 up to the rounding of the reciprocal
        assert (np.sum(np.abs(np.tril(got, -1) - 1.0) <= 4 * EPS64, axis=0)[:mn] >= 1).all()


def test_dgetrf_2048_and_zero_pivot(ulm):
    check_lu(ulm, 2048, 2048, 71000, extra=0)
    # an exactly singular matrix: column 2 is zero -> info = 3 (1-based), as the reference reports
    A = det_uniform(71001, 6, 6)
    A[:, 2] = 0.0
    W = A.copy(order="F")
    piv, info = ulm.dgetrf(W)
    assert info == 3
    if oracle.have_ref("lapack"):
        W2 = A.copy(order="F")
        rpiv, rinfo = oracle.ref_dgetrf(W2)
        assert rinfo == info and np.array_equal(piv, rpiv)


def test_dgetrf_row_major_is_refused(ulm):
    A = np.zeros((4, 4), order="F")
    piv = np.zeros(4, dtype=np.int32)
    assert ulm.lib.ulmblas_dgetrf(ulm.CblasRowMajor, 4, 4, A.ctypes.data, 4, piv.ctypes.data) == -1
    assert ulm.last_status() == ulm.BAD_ARGUMENT


def test_dlaswp_forward_and_backward(ulm):
    """ulmblas_dlaswp against the row exchanges done in numpy; incPiv = -1 walks the rows backwards
    and reads piv[-i] (ulmblas/lapack/laswp.tcc:22-24), which undoes a forward pass."""
    rng = np.random.default_rng(9)
    m, n, k1, k2 = 40, 300, 3, 29
    A0 = det_uniform(72000, m, n)
    piv = np.arange(m, dtype=np.int32)
    piv[k1:k2] = rng.integers(k1, m, k2 - k1)
    want = A0.copy()
    for i in range(k1, k2):
        want[[i, piv[i]]] = want[[piv[i], i]]
    Av, Ab = padded(A0, m + 3)
    ulm.lib.ulmblas_dlaswp(n, Av.ctypes.data, m + 3, k1, k2, piv.ctypes.data, 1)
    assert ulm.last_status() == ulm.OK
    assert np.array_equal(Av, want) and np.all(Ab[m:, :] == -1e10)
    # backwards: the reference indexes piv[i*incPiv], i.e. piv[-i]; hand it a mirrored array
    mirrored = np.zeros(2 * m, dtype=np.int32)
    mirrored[m - np.arange(m)] = piv            # mirrored[m - i] = piv[i]
    base = mirrored[m:]                         # base[-i] == piv[i]
    ulm.lib.ulmblas_dlaswp(n, Av.ctypes.data, m + 3, k1, k2, base.ctypes.data, -1)
    assert np.array_equal(Av, A0)
