"""DSYMM, DTRMM and DSYR2K on the GPU: the other clients of the reference's gemm macro-kernel
(ulmblas/level3/sy?mm.tcc, tr?mm.tcc, sy?r2k.tcc).  Checked against the compiled reference where
oracle/_ref is present and against a float64 numpy product otherwise, under the same componentwise
bound as GEMM; unreferenced triangles are filled with a rogue value and must be neither read nor
written."""
import itertools

import numpy as np
import pytest

from helpers import EPS64, ROGUE, bound_ratio, det_uniform, padded, ref

pytestmark = pytest.mark.gpu


def op(M, t):
    return M.T if t in "TC" else M


def tri_mask(n, uplo):
    return np.triu(np.ones((n, n), bool)) if uplo == "U" else np.tril(np.ones((n, n), bool))


def sym_from_triangle(A, uplo):
    T = np.where(tri_mask(A.shape[0], uplo), A, 0.0)
    return T + T.T - np.diag(np.diag(A))


def test_dsymm_all_variants(ulm):
    seed = 40000
    R = ref("plain")
    for (m, n) in [(1, 1), (7, 5), (31, 12), (130, 70), (300, 129)]:
        for side, uplo in itertools.product("LR", "UL"):
            for alpha, beta in [(1.0, 0.0), (0.7, 1.3), (0.0, 0.5)]:
                seed += 3
                na = m if side == "L" else n
                A = det_uniform(seed, na, na)
                A[~tri_mask(na, uplo)] = ROGUE
                Av, Ab = padded(A, na + 1)
                Bv, Bb = padded(det_uniform(seed + 1, m, n), m + 2)
                Cv, Cb = padded(det_uniform(seed + 2, m, n), m + 3)
                S = sym_from_triangle(np.where(tri_mask(na, uplo), A, 0.0), uplo)
                want = alpha * (S @ Bv if side == "L" else Bv @ S) + beta * Cv
                gauge = abs(alpha) * (np.abs(S) @ np.abs(Bv) if side == "L" else np.abs(Bv) @ np.abs(S)) + abs(beta) * np.abs(Cv)
                if R is not None:
                    w2 = Cb.copy(order="F")
                    R.dsymm(side, uplo, m, n, alpha, Av, Bv, beta, w2[:m, :n], lda=na + 1, ldb=m + 2, ldc=m + 3)
                    assert bound_ratio(w2[:m, :n], want, gauge, na, EPS64) <= 1.0      # the reference agrees with numpy
                    want = w2[:m, :n]
                got = Cb.copy(order="F")
                Ab0 = Ab.copy(order="F")
                assert ulm.dsymm(side, uplo, m, n, alpha, Av, Bv, beta, got[:m, :n], lda=na + 1, ldb=m + 2, ldc=m + 3) == ulm.OK
                assert np.array_equal(Ab, Ab0) and np.array_equal(got[m:, :], Cb[m:, :])
                assert np.isfinite(got[:m, :n]).all(), "the unreferenced triangle of A was read"
                ratio = bound_ratio(got[:m, :n], want, gauge, na, EPS64)
                assert ratio <= 1.0, (side, uplo, m, n, alpha, beta, ratio)


def test_dtrmm_all_variants(ulm):
    seed = 50000
    R = ref("plain")
    for (m, n) in [(1, 1), (7, 5), (31, 12), (130, 70), (300, 129), (257, 260)]:
        for side, uplo, tr, diag in itertools.product("LR", "UL", "NT", "NU"):
            seed += 2
            alpha = 0.7 if (m + n) % 2 else 1.0
            na = m if side == "L" else n
            A = det_uniform(seed, na, na)
            A[~tri_mask(na, uplo)] = ROGUE
            Av, Ab = padded(A, na + 2)
            Bv, Bb = padded(det_uniform(seed + 1, m, n), m + 2)
            T = np.where(tri_mask(na, uplo), A, 0.0)
            if diag == "U":
                T = T - np.diag(np.diag(T)) + np.eye(na)
            T = op(T, tr)
            want = alpha * (T @ Bv if side == "L" else Bv @ T)
            gauge = abs(alpha) * (np.abs(T) @ np.abs(Bv) if side == "L" else np.abs(Bv) @ np.abs(T))
            if R is not None:
                w2 = Bb.copy(order="F")
                R.dtrmm(side, uplo, tr, diag, m, n, alpha, Av, w2[:m, :n], lda=na + 2, ldb=m + 2)
                assert bound_ratio(w2[:m, :n], want, gauge, na, EPS64) <= 1.0
                want = w2[:m, :n]
            got = Bb.copy(order="F")
            Ab0 = Ab.copy(order="F")
            assert ulm.dtrmm(side, uplo, tr, diag, m, n, alpha, Av, got[:m, :n], lda=na + 2, ldb=m + 2) == ulm.OK
            assert np.array_equal(Ab, Ab0) and np.array_equal(got[m:, :], Bb[m:, :])
            assert np.isfinite(got[:m, :n]).all(), "the unreferenced triangle of A was read"
            ratio = bound_ratio(got[:m, :n], want, gauge, na, EPS64)
            assert ratio <= 1.0, (side, uplo, tr, diag, m, n, ratio)
    # alpha == 0 zeroes B
    Bv, Bb = padded(det_uniform(1, 9, 4), 11)
    A = np.asfortranarray(np.eye(9))
    assert ulm.dtrmm("L", "L", "N", "N", 9, 4, 0.0, A, Bv) == ulm.OK
    assert np.all(Bv == 0.0)


def test_dsyr2k_all_variants(ulm):
    """The reference's sy?r2k ignores B's own strides (ulmblas/level3/syur2k.tcc:25-26 declares
    incRowB/incColB and never uses them), so its dsyr2k_ is only right when ldB == ldA.  The
    reference is therefore consulted with equal leading dimensions; the unequal case is checked
    against the float64 numpy product alone (extra = 1)."""
    seed = 60000
    for (n, k) in [(1, 1), (7, 3), (31, 12), (200, 65), (300, 401), (129, 0)]:
        for uplo, tr in itertools.product("UL", "NT"):
            for (alpha, beta), extra in itertools.product([(1.0, 0.5), (-0.7, 0.0), (0.0, 1.3)], (2, 1)):
                R = ref("plain") if extra == 2 else None
                seed += 3
                ra, ca = (n, k) if tr == "N" else (k, n)
                Av, Ab = padded(det_uniform(seed, ra, ca), ra + 2)
                Bv, Bb = padded(det_uniform(seed + 1, ra, ca), ra + extra)
                Cv, Cb = padded(det_uniform(seed + 2, n, n), n + 2)
                mask = tri_mask(n, uplo)
                Cb[:n, :n][~mask] = ROGUE
                oA, oB = op(Av, "N" if tr == "N" else "T"), op(Bv, "N" if tr == "N" else "T")
                C0 = np.where(mask, Cb[:n, :n], 0.0)
                want = alpha * (oA @ oB.T + oB @ oA.T) + beta * C0
                gauge = abs(alpha) * (np.abs(oA) @ np.abs(oB).T + np.abs(oB) @ np.abs(oA).T) + abs(beta) * np.abs(C0)
                if R is not None:
                    w2 = Cb.copy(order="F")
                    R.dsyr2k(uplo, tr, n, k, alpha, Av, Bv, beta, w2[:n, :n], lda=ra + 2, ldb=ra + extra, ldc=n + 2)
                    assert bound_ratio(np.where(mask, w2[:n, :n], 0), np.where(mask, want, 0), gauge, 2 * k, EPS64) <= 1.0
                    want = w2[:n, :n]
                got = Cb.copy(order="F")
                assert ulm.dsyr2k(uplo, tr, n, k, alpha, Av, Bv, beta, got[:n, :n], lda=ra + 2, ldb=ra + extra, ldc=n + 2) == ulm.OK
                assert np.array_equal(got[n:, :], Cb[n:, :])
                assert np.all(got[:n, :n][~mask] == ROGUE), "opposite triangle was written"
                ratio = bound_ratio(np.where(mask, got[:n, :n], 0), np.where(mask, want, 0), gauge, 2 * k, EPS64)
                assert ratio <= 1.0, (n, k, uplo, tr, alpha, beta, ratio)
