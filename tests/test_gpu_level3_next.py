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


def trmm_cases(ulm, shapes, seed, variants=None):
    R = ref("plain")
    for (m, n) in shapes:
        for side, uplo, tr, diag in (variants or itertools.product("LR", "UL", "NT", "NU")):
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


def test_dtrmm_all_variants(ulm):
    # the last two shapes have several 256-wide diagonal blocks and a ragged last one
    trmm_cases(ulm, [(1, 1), (7, 5), (31, 12), (130, 70), (300, 129), (257, 260), (1100, 33), (33, 1300)], 50000)
    # alpha == 0 zeroes B
    Bv, Bb = padded(det_uniform(1, 9, 4), 11)
    A = np.asfortranarray(np.eye(9))
    assert ulm.dtrmm("L", "L", "N", "N", 9, 4, 0.0, A, Bv) == ulm.OK
    assert np.all(Bv == 0.0)


@pytest.mark.parametrize("leaf,dim,other", [(512, 1100, 150), (1024, 2200, 136), (2048, 2100, 130)])
def test_dtrmm_large_leaves(ulm, monkeypatch, leaf, dim, other):
    """Leaves of order 512, 1024 and 2048: zero-filled copies of the diagonal blocks multiplied in place by the
    triangular leaf of the GEMM kernel, a ragged last block, every side / uplo / trans / diag."""
    monkeypatch.setenv("ULMB200_TRSM_LEAF", str(leaf))
    ulm.reload_env()
    for side in "LR":
        m, n = (dim, other) if side == "L" else (other, dim)
        trmm_cases(ulm, [(m, n)], 51000 + leaf + ord(side), [(side,) + v for v in itertools.product("UL", "NT", "NU")])


def test_dtrmm_chosen_leaf_order_many_strips(ulm):
    """The library's own choice (1024 from 2048 rows, 2048 from 4096 rows on, with at least 1024 columns)."""
    trmm_cases(ulm, [(2304, 1500)], 52000, [("L", "L", "N", "N"), ("L", "U", "T", "U")])
    trmm_cases(ulm, [(1500, 2304)], 52100, [("R", "U", "N", "N"), ("R", "L", "T", "N")])
    trmm_cases(ulm, [(4200, 1100)], 52200, [("L", "U", "N", "N")])


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


def test_cblas_row_major_symm_trmm_syr2k(ulm):
    """Row-major CBLAS calls = the column-major routine on the transposed problem
    (interfaces/blas/C/symm.cc, trmm.cc, syr2k.cc); checked against numpy on C-ordered arrays."""
    rng = np.random.default_rng(5)
    m, n, k = 40, 65, 23
    A = rng.uniform(-1, 1, (m, m)); B = rng.uniform(-1, 1, (m, n)); C0 = rng.uniform(-1, 1, (m, n))
    S = np.triu(A) + np.triu(A, 1).T
    got = C0.copy()
    ulm.lib.cblas_dsymm(ulm.CblasRowMajor, ulm.CblasLeft, ulm.CblasUpper, m, n, 0.5, A.ctypes.data, m,
                        B.ctypes.data, n, 2.0, got.ctypes.data, n)
    assert ulm.last_status() == ulm.OK
    want = 0.5 * S @ B + 2.0 * C0
    assert bound_ratio(got, want, 0.5 * np.abs(S) @ np.abs(B) + 2.0 * np.abs(C0), m, EPS64) <= 1.0
    T = np.tril(A)
    got = B.copy()
    ulm.lib.cblas_dtrmm(ulm.CblasRowMajor, ulm.CblasLeft, ulm.CblasLower, ulm.CblasTrans, ulm.CblasNonUnit, m, n,
                        1.5, A.ctypes.data, m, got.ctypes.data, n)
    assert ulm.last_status() == ulm.OK
    assert bound_ratio(got, 1.5 * T.T @ B, 1.5 * np.abs(T.T) @ np.abs(B), m, EPS64) <= 1.0
    A2 = rng.uniform(-1, 1, (n, k)); B2 = rng.uniform(-1, 1, (n, k)); C2 = rng.uniform(-1, 1, (n, n))
    got = C2.copy()
    ulm.lib.cblas_dsyr2k(ulm.CblasRowMajor, ulm.CblasLower, ulm.CblasNoTrans, n, k, 1.0, A2.ctypes.data, k,
                         B2.ctypes.data, k, 0.5, got.ctypes.data, n)
    assert ulm.last_status() == ulm.OK
    want = A2 @ B2.T + B2 @ A2.T + 0.5 * C2
    low = np.tril(np.ones((n, n), bool))
    gauge = np.abs(A2) @ np.abs(B2).T + np.abs(B2) @ np.abs(A2).T + 0.5 * np.abs(C2)
    assert bound_ratio(np.where(low, got, 0), np.where(low, want, 0), gauge, 2 * k, EPS64) <= 1.0
    assert np.array_equal(got[~low], C2[~low])


def test_single_precision_syrk_and_trsm(ulm):
    """ssyrk_ / strsm_: float operands, double arithmetic -- as in the reference, whose shims widen
    alpha and beta to double (interfaces/blas/F77/syrk.cc:30-32, trsm.cc:32).  Checked against the
    compiled reference (portable build) and the fp32 componentwise bound."""
    from helpers import EPS32
    R = ref("plain")
    seed = 80000
    for (n, k) in [(7, 3), (130, 70), (300, 401)]:
        for uplo, tr in itertools.product("UL", "NT"):
            seed += 2
            ra, ca = (n, k) if tr == "N" else (k, n)
            A = det_uniform(seed, ra, ca, np.float32)
            Cv, Cb = padded(det_uniform(seed + 1, n, n, np.float32), n + 3)
            mask = tri_mask(n, uplo)
            Cb[:n, :n][~mask] = ROGUE
            oA = op(A.astype(np.float64), tr)
            C0 = np.where(mask, Cb[:n, :n], 0.0).astype(np.float64)
            want = 0.7 * (oA @ oA.T) + 1.3 * C0
            gauge = 0.7 * (np.abs(oA) @ np.abs(oA).T) + 1.3 * np.abs(C0)
            if R is not None:
                w2 = Cb.copy(order="F")
                R.ssyrk(uplo, tr, n, k, 0.7, A, 1.3, w2[:n, :n], ldc=n + 3)
                want = w2[:n, :n]
            got = Cb.copy(order="F")
            assert ulm.ssyrk(uplo, tr, n, k, 0.7, A, 1.3, got[:n, :n], ldc=n + 3) == ulm.OK
            assert np.array_equal(got[n:, :], Cb[n:, :]) and np.all(got[:n, :n][~mask] == np.float32(ROGUE))
            assert bound_ratio(np.where(mask, got[:n, :n], 0), np.where(mask, want, 0), gauge, k, EPS32) <= 1.0
    for (m, n) in [(7, 5), (130, 70), (300, 129)]:
        for side, uplo, tr, diag in itertools.product("LR", "UL", "NT", "NU"):
            seed += 2
            na = m if side == "L" else n
            A = det_uniform(seed, na, na).astype(np.float64)
            d = np.diag(A).copy()
            A = A / na
            A[np.arange(na), np.arange(na)] = 1.5 + 0.25 * d
            Af = np.asfortranarray(A.astype(np.float32))
            Af[~tri_mask(na, uplo)] = ROGUE
            Bv, Bb = padded(det_uniform(seed + 1, m, n, np.float32), m + 1)
            T = np.where(tri_mask(na, uplo), Af, 0).astype(np.float64)
            if diag == "U":
                T = T - np.diag(np.diag(T)) + np.eye(na)
            T = op(T, tr)
            got = Bb.copy(order="F")
            assert ulm.strsm(side, uplo, tr, diag, m, n, 0.5, Af, got[:m, :n], ldb=m + 1) == ulm.OK
            X = got[:m, :n].astype(np.float64)
            assert np.isfinite(X).all() and np.array_equal(got[m:, :], Bb[m:, :])
            lhs = T @ X if side == "L" else X @ T
            gauge = (np.abs(T) @ np.abs(X) if side == "L" else np.abs(X) @ np.abs(T)) + 0.5 * np.abs(Bv)
            assert bound_ratio(lhs, 0.5 * Bv.astype(np.float64), gauge, na, EPS32) <= 1.0, (side, uplo, tr, diag, m, n)
            if R is not None:
                w2 = Bb.copy(order="F")
                R.strsm(side, uplo, tr, diag, m, n, 0.5, Af, w2[:m, :n], ldb=m + 1)
                assert np.abs(X - w2[:m, :n]).max() <= 2e-5 * max(1.0, np.abs(X).max())
