"""SGEMM, DTRSM and DSYRK parity on the GPU against the reference."""
import itertools

import numpy as np
import pytest

from helpers import (EPS32, EPS64, ROGUE, bound_ratio, det_uniform, gemm_gauge, golden_inputs, load_golden,
                     padded, port, ref, repair_nonfinite)

pytestmark = pytest.mark.gpu


def op(M, t):
    return M.T if t in "TC" else M


def reference_sgemm(ta, tb, m, n, k, alpha, A, B, beta, C0):
    want = C0.copy(order="F")
    R = ref("")
    if R is not None:
        R.sgemm(ta, tb, m, n, k, alpha, A, B, beta, want)
        if not np.isfinite(want).all():
            alt = C0.copy(order="F")
            port().sgemm(ta, tb, m, n, k, alpha, A, B, beta, alt)
            repair_nonfinite(want, alt)
    else:
        port().sgemm(ta, tb, m, n, k, alpha, A, B, beta, want)
    return want


@pytest.mark.parametrize("mode", ["fp32", "3xtf32"])
def test_config2_sgemm_4096_tn(ulm, mode, monkeypatch):
    """SGEMM m=n=k=4096, transA='T', transB='N', alpha=1, beta=0, seed 7; both arithmetic modes."""
    monkeypatch.setenv("ULMB200_SGEMM", mode)
    ulm.reload_env()
    m = n = k = 4096
    A, _ = ulm.fmat(k, m, dtype=np.float32); B, _ = ulm.fmat(k, n, dtype=np.float32)
    ulm.host_fill(A, 7, 0); ulm.host_fill(B, 7, 1)
    C0 = np.zeros((m, n), dtype=np.float32, order="F")
    got = C0.copy(order="F")
    assert ulm.sgemm("T", "N", m, n, k, 1.0, A, B, 0.0, got) == ulm.OK
    # the CPU reference needs ~10 s for the full product: check 512 sampled columns of it
    cols = np.sort(np.random.default_rng(0).choice(n, 512, replace=False))
    Bs = np.asfortranarray(B[:, cols])
    want = reference_sgemm("T", "N", m, len(cols), k, 1.0, A, Bs, 0.0, np.zeros((m, len(cols)), np.float32, order="F"))
    ratio = bound_ratio(got[:, cols], want, gemm_gauge(1.0, A.T, Bs, 0.0, want), k, EPS32)
    assert ratio <= 1.0, ratio


@pytest.mark.parametrize("mode", ["fp32", "3xtf32"])
def test_sgemm_shapes_and_transposes(ulm, mode, monkeypatch):
    monkeypatch.setenv("ULMB200_SGEMM", mode)
    ulm.reload_env()
    seed = 9000
    for (m, n, k) in [(1, 1, 1), (7, 12, 31), (129, 65, 17), (300, 260, 100), (128, 256, 64), (200, 1, 33)]:
        for ta, tb in itertools.product("NT", "NT"):
            for alpha, beta in [(1.0, 0.0), (0.7, 1.3)]:
                seed += 3
                ra, ca = (m, k) if ta == "N" else (k, m)
                rb, cb = (k, n) if tb == "N" else (n, k)
                A, Ab = padded(det_uniform(seed, ra, ca, np.float32), ra + 1)
                B, Bb = padded(det_uniform(seed + 1, rb, cb, np.float32), rb + 4)
                C0v, C0b = padded(det_uniform(seed + 2, m, n, np.float32), m + 3)
                want = reference_sgemm(ta, tb, m, n, k, alpha, A, B, beta, np.asfortranarray(C0v))
                got = C0b.copy(order="F")
                st = ulm.sgemm(ta, tb, m, n, k, alpha, A, B, beta, got[:m, :n], lda=ra + 1, ldb=rb + 4, ldc=m + 3)
                assert st == ulm.OK
                assert np.array_equal(got[m:, :], C0b[m:, :]), "padding rows of C were written"
                ratio = bound_ratio(got[:m, :n], want, gemm_gauge(alpha, op(A, ta), op(B, tb), beta, C0v), k, EPS32)
                assert ratio <= 1.0, (mode, m, n, k, ta, tb, alpha, beta, ratio)


@pytest.mark.parametrize("pre", ["1", "0"])
def test_sgemm_large_k_contiguous_operands(ulm, pre, monkeypatch):
    """From 1024 rows (columns) of the other operand on, a K-contiguous operand (A with transA = T, B with
    transB = N) is copied once into the M/N-contiguous layout TMA can feed straight to the consumers;
    ULMB200_SGEMM_PRETRANSPOSE=0 keeps the transposition inside the kernel.  Ragged sizes, padded leading
    dimensions, all four transpositions, both settings."""
    monkeypatch.setenv("ULMB200_SGEMM", "fp32")
    monkeypatch.setenv("ULMB200_SGEMM_PRETRANSPOSE", pre)
    ulm.reload_env()
    seed = 9500
    for (m, n, k) in [(1100, 1300, 300), (1027, 1025, 259)]:
        for ta, tb in itertools.product("NT", "NT"):
            seed += 3
            ra, ca = (m, k) if ta == "N" else (k, m)
            rb, cb = (k, n) if tb == "N" else (n, k)
            A, Ab = padded(det_uniform(seed, ra, ca, np.float32), ra + 3)
            B, Bb = padded(det_uniform(seed + 1, rb, cb, np.float32), rb + 4)
            C0v, C0b = padded(det_uniform(seed + 2, m, n, np.float32), m + 4)
            want = reference_sgemm(ta, tb, m, n, k, 0.7, A, B, 1.3, np.asfortranarray(C0v))
            got = C0b.copy(order="F")
            Ab0, Bb0 = Ab.copy(order="F"), Bb.copy(order="F")
            assert ulm.sgemm(ta, tb, m, n, k, 0.7, A, B, 1.3, got[:m, :n], lda=ra + 3, ldb=rb + 4, ldc=m + 4) == ulm.OK
            assert np.array_equal(Ab, Ab0) and np.array_equal(Bb, Bb0), "an input operand was modified"
            assert np.array_equal(got[m:, :], C0b[m:, :]), "padding rows of C were written"
            ratio = bound_ratio(got[:m, :n], want, gemm_gauge(0.7, op(A, ta), op(B, tb), 1.3, C0v), k, EPS32)
            assert ratio <= 1.0, (pre, m, n, k, ta, tb, ratio)


def test_sgemm_split_k_tail(ulm, monkeypatch):
    """Tile counts a little above a multiple of the SM count: the FP32 kernel gives the last few tiles
    to several CTAs each, one K range per CTA, added in a fixed order.  Checked on sampled columns
    against the reference, and for run-to-run reproducibility (bit-identical results)."""
    monkeypatch.setenv("ULMB200_SGEMM", "fp32")
    ulm.reload_env()
    for (m, n, k, ta, tb, alpha, beta) in [(3328, 1536, 1100, "N", "N", 1.0, 0.0),      # 156 tiles: 8 left over, 8 K ranges
                                           (3300, 1500, 300, "T", "N", 0.7, 1.3),       # ragged edges, 2 K ranges
                                           (2560, 2304, 515, "N", "T", -1.0, 1.0)]:     # 180 tiles: 32 left over, 4 ranges
        ra, ca = (m, k) if ta == "N" else (k, m)
        rb, cb = (k, n) if tb == "N" else (n, k)
        A = np.asfortranarray(det_uniform(31, ra, ca, np.float32))
        B = np.asfortranarray(det_uniform(32, rb, cb, np.float32))
        C0 = np.asfortranarray(det_uniform(33, m, n, np.float32))
        got = C0.copy(order="F")
        assert ulm.sgemm(ta, tb, m, n, k, alpha, A, B, beta, got) == ulm.OK
        again = C0.copy(order="F")
        assert ulm.sgemm(ta, tb, m, n, k, alpha, A, B, beta, again) == ulm.OK
        assert np.array_equal(got, again), "the split-K tail must not depend on timing"
        cols = np.unique(np.concatenate([np.arange(n - 40, n), np.random.default_rng(4).choice(n, 60, replace=False)]))
        Bs = np.asfortranarray(B[:, cols]) if tb == "N" else np.asfortranarray(B[cols, :])
        Cs = np.asfortranarray(C0[:, cols])
        want = reference_sgemm(ta, tb, m, len(cols), k, alpha, A, Bs, beta, Cs)
        ratio = bound_ratio(got[:, cols], want, gemm_gauge(alpha, op(A, ta), op(Bs, tb), beta, Cs), k, EPS32)
        assert ratio <= 1.0, (m, n, k, ta, tb, ratio)


def test_golden_sgemm_cases_on_gpu(ulm):
    for name, c in load_golden().items():
        if c["kind"] != "sgemm":
            continue
        A, B, C0 = golden_inputs(c)
        got = C0.copy(order="F")
        assert ulm.sgemm(c["ta"], c["tb"], c["m"], c["n"], c["k"], c["alpha"], A, B, c["beta"], got) == ulm.OK
        ratio = bound_ratio(got, c["C"], gemm_gauge(c["alpha"], op(A, c["ta"]), op(B, c["tb"]), c["beta"], C0),
                            c["k"], EPS32)
        assert ratio <= 1.0, (name, ratio)


# ------------------------------------------------------------------------------- dsyrk

def syrk_reference(uplo, tr, n, k, alpha, A, beta, Cb, ldc):
    want = Cb.copy(order="F")
    R = ref("")
    if R is not None:
        R.dsyrk(uplo, tr, n, k, alpha, A, beta, want[:n, :n], ldc=ldc)
        if not np.isfinite(want[:n, :n]).all():
            alt = Cb.copy(order="F")
            port().dsyrk(uplo, tr, n, k, alpha, A, beta, alt[:n, :n], ldc=ldc)
            repair_nonfinite(want, alt)
    else:
        port().dsyrk(uplo, tr, n, k, alpha, A, beta, want[:n, :n], ldc=ldc)
    return want


def tri_mask(n, uplo):
    return np.triu(np.ones((n, n), bool)) if uplo == "U" else np.tril(np.ones((n, n), bool))


def test_dsyrk_all_variants(ulm):
    seed = 12000
    for (n, k) in [(1, 1), (7, 3), (31, 12), (200, 65), (390, 401), (129, 0)]:
        for uplo, tr in itertools.product("UL", "NT"):
            for alpha, beta in [(1.0, 0.5), (-0.7, 0.0), (0.0, 1.3)]:
                seed += 2
                ra, ca = (n, k) if tr == "N" else (k, n)
                A, Ab = padded(det_uniform(seed, ra, ca), ra + 2)
                Cv, Cb = padded(det_uniform(seed + 1, n, n), n + 2)
                mask = tri_mask(n, uplo)
                Cb[:n, :n][~mask] = ROGUE          # the unreferenced triangle must be neither read nor written
                want = syrk_reference(uplo, tr, n, k, alpha, A, beta, Cb, n + 2)
                got = Cb.copy(order="F")
                assert ulm.dsyrk(uplo, tr, n, k, alpha, A, beta, got[:n, :n], lda=ra + 2, ldc=n + 2) == ulm.OK
                assert np.array_equal(got[n:, :], Cb[n:, :])
                assert np.all(got[:n, :n][~mask] == ROGUE), "opposite triangle was written"
                opA = op(A, tr)
                gauge = gemm_gauge(alpha, opA, opA.T, beta, np.where(mask, Cb[:n, :n], 0.0))
                g, w = np.where(mask, got[:n, :n], 0.0), np.where(mask, want[:n, :n], 0.0)
                ratio = bound_ratio(g, w, gauge, k, EPS64)
                assert ratio <= 1.0, (n, k, uplo, tr, alpha, beta, ratio)


def test_dsyrk_tail_split(ulm):
    """n = 2176 is 17 tile rows: 153 tiles in the triangle, 5 more than the 148 SMs, so the last five
    are shared by several CTAs (K ranges added in a fixed order).  Both triangles, full comparison."""
    n, k = 2176, 1024
    for i, (uplo, tr, alpha, beta) in enumerate([("U", "N", 1.0, 0.5), ("L", "T", -0.7, 1.3)]):
        ra, ca = (n, k) if tr == "N" else (k, n)
        A = np.asfortranarray(det_uniform(12500 + i, ra, ca))
        C0 = np.asfortranarray(det_uniform(12600 + i, n, n))
        mask = tri_mask(n, uplo)
        C0[~mask] = ROGUE
        want = syrk_reference(uplo, tr, n, k, alpha, A, beta, C0, n)
        got, again = C0.copy(order="F"), C0.copy(order="F")
        assert ulm.dsyrk(uplo, tr, n, k, alpha, A, beta, got) == ulm.OK
        assert ulm.dsyrk(uplo, tr, n, k, alpha, A, beta, again) == ulm.OK
        assert np.array_equal(got, again)
        assert np.all(got[~mask] == ROGUE), "opposite triangle was written"
        opA = op(A, tr)
        gauge = gemm_gauge(alpha, opA, opA.T, beta, np.where(mask, C0, 0.0))
        ratio = bound_ratio(np.where(mask, got, 0.0), np.where(mask, want, 0.0), gauge, k, EPS64)
        assert ratio <= 1.0, (uplo, tr, ratio)


def test_config4_dsyrk_8192_sampled_blocks(ulm, torch_cuda):
    """DSYRK uplo=U trans=N n=8192 k=4096 (alpha=1, beta=0.5), device-resident.  The CPU reference
    would need ~20 s for all of it; diagonal and off-diagonal 512-blocks are checked instead
    (each output element's arithmetic in the reference depends on its own row/column only)."""
    torch = torch_cuda
    n, k, nb = 8192, 4096, 512
    dA = torch.empty((k, n), dtype=torch.float64, device="cuda")
    dC = torch.empty((n, n), dtype=torch.float64, device="cuda")
    ulm.dev_fill_f64(dA.data_ptr(), n, n, k, 3, 0)
    ulm.dev_fill_f64(dC.data_ptr(), n, n, n, 3, 2)
    dC0 = dC.clone()
    ulm.dev_dsyrk(0, 0, n, k, 1.0, dA.data_ptr(), n, 0.5, dC.data_ptr(), n)
    torch.cuda.synchronize()
    low = torch.tril(torch.ones((n, n), dtype=torch.bool, device="cuda"), -1).T   # storage is transposed
    assert torch.equal(dC[low], dC0[low]), "strictly lower triangle was written"
    R = ref("") or port()
    for (bi, bj) in [(0, 0), (3, 3), (15, 15), (0, 15), (2, 9), (7, 8)]:
        Ai, _ = ulm.fmat(nb, k); Aj, _ = ulm.fmat(nb, k); C0, _ = ulm.fmat(nb, nb)
        ulm.host_fill(Ai, 3, 0, row0=bi * nb); ulm.host_fill(Aj, 3, 0, row0=bj * nb)
        ulm.host_fill(C0, 3, 2, row0=bi * nb, col0=bj * nb)
        want = C0.copy(order="F")
        if bi == bj:
            R.dsyrk("U", "N", nb, k, 1.0, Ai, 0.5, want)
        else:
            R.dgemm("N", "T", nb, nb, k, 1.0, Ai, Aj, 0.5, want)
        alt = C0.copy(order="F")
        if not np.isfinite(want).all():
            (port().dsyrk("U", "N", nb, k, 1.0, Ai, 0.5, alt) if bi == bj
             else port().dgemm("N", "T", nb, nb, k, 1.0, Ai, Aj, 0.5, alt))
            repair_nonfinite(want, alt)
        got = dC[bj * nb:(bj + 1) * nb, bi * nb:(bi + 1) * nb].cpu().numpy().T
        mask = tri_mask(nb, "U") if bi == bj else np.ones((nb, nb), bool)
        gauge = gemm_gauge(1.0, Ai, Aj.T, 0.5, C0)
        ratio = bound_ratio(np.where(mask, got, 0), np.where(mask, want, 0), gauge, k, EPS64)
        assert ratio <= 1.0, (bi, bj, ratio)


# ------------------------------------------------------------------------------- dtrsm

def tri_matrix(seed, na, uplo, rogue_other=True):
    """Diagonal uniform[1.25,1.75], referenced triangle uniform[-1,1]/na, the other triangle rogue."""
    A = det_uniform(seed, na, na)
    d = np.diag(A).copy()
    A = np.asfortranarray(A / max(na, 1))
    A[np.arange(na), np.arange(na)] = 1.5 + 0.25 * d
    if rogue_other:
        other = np.triu(np.ones((na, na), bool), 1) if uplo == "L" else np.tril(np.ones((na, na), bool), -1)
        A[other] = ROGUE
    return A


def trsm_check(ulm, side, uplo, tr, diag, m, n, alpha, seed):
    na = m if side == "L" else n
    A = tri_matrix(seed, na, uplo)
    Av, Ab = padded(A, na + 2)
    Bv, Bb = padded(det_uniform(seed + 1, m, n), m + 2)
    want = Bb.copy(order="F")
    R = ref("")
    if R is not None:
        R.dtrsm(side, uplo, tr, diag, m, n, alpha, Av, want[:m, :n], lda=na + 2, ldb=m + 2)
    if R is None or not np.isfinite(want[:m, :n]).all():
        alt = Bb.copy(order="F")
        port().dtrsm(side, uplo, tr, diag, m, n, alpha, Av, alt[:m, :n], lda=na + 2, ldb=m + 2)
        if R is None:
            want = alt
        else:
            repair_nonfinite(want, alt)
    got = Bb.copy(order="F")
    Ab0 = Ab.copy(order="F")
    st = ulm.dtrsm(side, uplo, tr, diag, m, n, alpha, Av, got[:m, :n], lda=na + 2, ldb=m + 2)
    assert st == ulm.OK
    assert np.array_equal(Ab, Ab0) and np.array_equal(got[m:, :], Bb[m:, :])
    X = got[:m, :n]
    assert np.isfinite(X).all(), "the unreferenced (rogue) triangle of A leaked into the result"
    # the tester's check: multiply back (test/F77/dblat3.f:1130-1155)
    T = np.tril(Av) if uplo == "L" else np.triu(Av)
    if diag == "U":
        T = T - np.diag(np.diag(T)) + np.eye(na)
    T = op(T, tr)
    lhs = T @ X if side == "L" else X @ T
    gauge = (np.abs(T) @ np.abs(X) if side == "L" else np.abs(X) @ np.abs(T)) + abs(alpha) * np.abs(Bv)
    resid = bound_ratio(lhs, alpha * Bv, gauge, na, EPS64)
    assert resid <= 1.0, (side, uplo, tr, diag, m, n, alpha, resid)
    # and directly against the reference's solution (A is well conditioned by construction)
    assert np.abs(X - want[:m, :n]).max() <= 1e-10, (side, uplo, tr, diag, m, n)


def test_dtrsm_all_variants(ulm):
    seed = 20000
    # (700, 20) / (20, 700): three 256-wide diagonal blocks, the last one ragged and without a partner
    for (m, n) in [(1, 1), (7, 5), (31, 12), (130, 70), (300, 129), (700, 20), (20, 700)]:
        for side, uplo, tr, diag in itertools.product("LR", "UL", "NT", "NU"):
            seed += 2
            trsm_check(ulm, side, uplo, tr, diag, m, n, 0.7 if (m + n) % 2 else 1.0, seed)
    trsm_check(ulm, "L", "L", "N", "N", 390, 33, 0.0, seed + 2)      # alpha == 0 zeroes B


@pytest.mark.parametrize("leaf,dim,other", [(512, 1100, 200), (1024, 2200, 136), (2048, 2100, 130)])
def test_dtrsm_large_inverted_blocks(ulm, monkeypatch, leaf, dim, other):
    """Diagonal blocks of order 512, 1024 and 2048 inverted (by batched products from the 256-inverses)
    and applied in place by the leaf kernel, which multiplies only the blocks of the triangle: every
    side / uplo / trans / diag, a ragged last block, leading dimensions with padding."""
    monkeypatch.setenv("ULMB200_TRSM_LEAF", str(leaf))
    ulm.reload_env()
    seed = 21000 + leaf
    for side, uplo, tr, diag in itertools.product("LR", "UL", "NT", "NU"):
        seed += 2
        m, n = (dim, other) if side == "L" else (other, dim)
        trsm_check(ulm, side, uplo, tr, diag, m, n, 0.7 if uplo == "U" else 1.0, seed)


def test_dtrsm_chosen_block_order_many_strips(ulm):
    """The library's own choice (order 1024 from 2048 rows and 1024 right-hand sides on) with more
    leaf tiles than CTAs, so that tiles are handed out while others still wait for their readers."""
    trsm_check(ulm, "L", "L", "N", "N", 2304, 2700, 1.0, 21900)
    trsm_check(ulm, "R", "U", "T", "U", 2700, 2304, 0.7, 21902)
    trsm_check(ulm, "R", "L", "N", "N", 2700, 2100, 1.0, 21904)
    trsm_check(ulm, "L", "U", "N", "N", 2100, 2700, 1.0, 21906)


def test_dtrsm_device_resident_odd_orders_keep_padding(ulm, torch_cuda):
    """Device-resident B with an odd number of rows and rogue padding rows below them (leading dimensions
    even, so TMA addresses everything): the in-place leaves store whole tiles by TMA, whose row clipping
    works in units of 16 bytes.  Padding stays bit for bit, the solution satisfies the tester's bound."""
    torch = torch_cuda
    seed = 22000
    for (side, uplo, tr, m, n) in [("L", "L", "N", 2201, 1301), ("R", "U", "T", 1301, 2201), ("L", "U", "T", 301, 77),
                                   ("R", "L", "N", 2049, 2048)]:
        seed += 2
        na = m if side == "L" else n
        A = tri_matrix(seed, na, uplo)
        B = det_uniform(seed + 1, m, n)
        lda, ldb = na + 2 + (na % 2), m + 4 + (m % 2)

        def dev(h, ld):
            t = torch.full((h.shape[1], ld), ROGUE, dtype=torch.float64, device="cuda")
            t[:, :h.shape[0]] = torch.from_numpy(np.ascontiguousarray(h.T)).cuda()
            return t
        dA, dB = dev(A, lda), dev(B, ldb)
        ulm.dev_dtrsm(0 if side == "L" else 1, uplo == "L", tr == "T", 0, m, n, 1.0, dA.data_ptr(), lda, dB.data_ptr(), ldb)
        torch.cuda.synchronize()
        assert ulm.check_device_error() == 0
        got = dB.cpu().numpy().T
        assert (got[m:, :] == ROGUE).all(), (side, uplo, tr, m, n, "padding rows of B were written")
        X = got[:m, :]
        assert np.isfinite(X).all()
        T = op(np.tril(A) if uplo == "L" else np.triu(A), tr)
        lhs = T @ X if side == "L" else X @ T
        gauge = (np.abs(T) @ np.abs(X) if side == "L" else np.abs(X) @ np.abs(T)) + np.abs(B)
        resid = bound_ratio(lhs, B, gauge, na, EPS64)
        assert resid <= 1.0, (side, uplo, tr, m, n, resid)


def test_config4_dtrsm_8192_sampled_columns(ulm, torch_cuda):
    """DTRSM side=L uplo=L trans=N diag=N, m=n=8192, seed 3, device-resident: diagonal uniform[1,2),
    strict lower uniform[-1,1)/n, strict upper rogue.  Columns of X are independent, so the
    reference solves 48 sampled columns (m=8192, n=48) and the multiply-back residual is
    evaluated on those columns in numpy."""
    torch = torch_cuda
    m = n = 8192
    dA = torch.empty((m, m), dtype=torch.float64, device="cuda")
    dB = torch.empty((n, m), dtype=torch.float64, device="cuda")
    ulm.dev_fill_f64(dA.data_ptr(), m, m, m, 3, 0, dist=1, scale=1.0 / m)
    upper = torch.triu(torch.ones((m, m), dtype=torch.bool, device="cuda"), 1).T
    dA[upper] = ROGUE
    ulm.dev_fill_f64(dB.data_ptr(), m, m, n, 3, 1)
    ulm.dev_dtrsm(0, 1, 0, 0, m, n, 1.0, dA.data_ptr(), m, dB.data_ptr(), m)
    torch.cuda.synchronize()
    cols = np.sort(np.random.default_rng(1).choice(n, 48, replace=False))
    A, _ = ulm.fmat(m, m)
    ulm.host_fill(A, 3, 0, dist=1, scale=1.0 / m)
    B0 = np.empty((m, len(cols)), order="F")
    for j, c in enumerate(cols):
        ulm.host_fill(B0[:, j:j + 1], 3, 1, col0=int(c))
    want = B0.copy(order="F")
    (ref("") or port()).dtrsm("L", "L", "N", "N", m, len(cols), 1.0, A, want)
    alt = None
    if not np.isfinite(want).all():
        alt = B0.copy(order="F")
        port().dtrsm("L", "L", "N", "N", m, len(cols), 1.0, A, alt)
        repair_nonfinite(want, alt)
    X = dB[torch.from_numpy(cols).cuda(), :].cpu().numpy().T
    assert np.isfinite(X).all()
    L = np.tril(A)
    resid = bound_ratio(L @ X, B0, np.abs(L) @ np.abs(X) + np.abs(B0), m, EPS64)
    assert resid <= 1.0, resid
    assert np.abs(X - want).max() <= 1e-10
