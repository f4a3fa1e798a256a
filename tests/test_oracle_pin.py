"""The CPU restatement (oracle/ulm_oracle.c) against the reference itself.

1. Against golden outputs the compiled reference produced (tests/golden, runs anywhere).
2. Bit for bit against the compiled reference where oracle/_ref is present: the
   portable-kernel build everywhere, the SSE build on every finite entry, and the
   reference's own tiny-block test configuration.
"""
import itertools

import numpy as np
import pytest

from helpers import (ROGUE, det_uniform, golden_inputs, load_golden, padded, port, ref)


def _run_port(c):
    P = port()
    P.set_blocks(384, 384, 4096)
    kind = c["kind"]
    if kind in ("dgemm", "sgemm"):
        A, B, C0 = golden_inputs(c)
        out = C0.copy(order="F")
        fn = P.dgemm if kind == "dgemm" else P.sgemm
        fn(c["ta"], c["tb"], c["m"], c["n"], c["k"], c["alpha"], A, B, c["beta"], out)
        return out
    if kind == "dsyrk":
        A, C0 = golden_inputs(c)
        out = C0.copy(order="F")
        P.dsyrk(c["uplo"], c["trans"], c["n"], c["k"], c["alpha"], A, c["beta"], out)
        return out
    A, B0 = golden_inputs(c)
    out = B0.copy(order="F")
    P.dtrsm(c["side"], c["uplo"], c["trans"], c["diag"], c["m"], c["n"], c["alpha"], A, out)
    return out


def test_port_reproduces_reference_golden_outputs():
    cases = load_golden()
    assert len(cases) > 100
    for name, c in cases.items():
        want = c["C"] if "C" in c else c["B"]
        got = _run_port(c)
        assert np.array_equal(got, want), f"{name}: restatement differs from the reference's output"


needs_ref = pytest.mark.skipif(ref("plain") is None, reason="oracle/_ref not built (no reference tree here)")


def _mk(seed, r, c, extra):
    return padded(det_uniform(seed, r, c), r + extra)


@needs_ref
@pytest.mark.parametrize("variant", ["plain", ""])
def test_port_equals_compiled_reference_dgemm(variant):
    R, P = ref(variant), port()
    P.set_blocks(384, 384, 4096)
    seed = 7
    for (m, n, k) in [(1, 1, 1), (4, 4, 0), (5, 0, 3), (33, 17, 401), (400, 390, 800), (385, 4, 769)]:
        for ta, tb in itertools.product("NT", "NT"):
            for alpha, beta in [(1.5, 0.5), (1.0, 0.0), (0.0, 0.7), (0.7, 1.0)]:
                seed += 3
                A, _ = _mk(seed, m if ta == "N" else k, k if ta == "N" else m, 3)
                B, _ = _mk(seed + 1, k if tb == "N" else n, n if tb == "N" else k, 1)
                _, Cb = _mk(seed + 2, m, n, 2)
                c1, c2 = Cb.copy(order="F"), Cb.copy(order="F")
                R.dgemm(ta, tb, m, n, k, alpha, A, B, beta, c1[:m, :n], ldc=m + 2)
                P.dgemm(ta, tb, m, n, k, alpha, A, B, beta, c2[:m, :n], ldc=m + 2)
                ok = np.isfinite(c1)
                if variant == "plain":
                    assert ok.all()
                assert np.array_equal(c1[ok], c2[ok]), (m, n, k, ta, tb, alpha, beta)
                assert np.all(c2[m:, :] == ROGUE), "padding rows written"


@needs_ref
def test_port_equals_reference_tiny_block_build():
    """The reference's own test configuration: MC=8, KC=12, NC=12 (test/F77/config/make.testcase01.inc)."""
    R, P = ref("tiny"), port()
    P.set_blocks(8, 12, 12)
    try:
        seed = 100
        for (m, n, k) in [(7, 5, 3), (33, 17, 41), (31, 31, 31), (12, 24, 36)]:
            for ta, tb in itertools.product("NT", "NT"):
                for alpha, beta in [(1.0, 0.0), (0.7, 1.3)]:
                    seed += 3
                    A = det_uniform(seed, m if ta == "N" else k, k if ta == "N" else m)
                    B = det_uniform(seed + 1, k if tb == "N" else n, n if tb == "N" else k)
                    C0 = det_uniform(seed + 2, m, n)
                    c1, c2 = C0.copy(order="F"), C0.copy(order="F")
                    R.dgemm(ta, tb, m, n, k, alpha, A, B, beta, c1)
                    P.dgemm(ta, tb, m, n, k, alpha, A, B, beta, c2)
                    assert np.array_equal(c1, c2)
        for (m, n) in [(7, 5), (33, 17), (12, 30)]:
            for side, uplo, tr, diag in itertools.product("LR", "UL", "NT", "NU"):
                seed += 2
                na = m if side == "L" else n
                A = det_uniform(seed, na, na) / na
                A[np.arange(na), np.arange(na)] = 1.5
                A = np.asfortranarray(A)
                B0 = det_uniform(seed + 1, m, n)
                b1, b2 = B0.copy(order="F"), B0.copy(order="F")
                R.dtrsm(side, uplo, tr, diag, m, n, 0.7, A, b1)
                P.dtrsm(side, uplo, tr, diag, m, n, 0.7, A, b2)
                assert np.array_equal(b1, b2), (m, n, side, uplo, tr, diag)
    finally:
        P.set_blocks(384, 384, 4096)


@needs_ref
def test_port_equals_compiled_reference_sgemm_syrk_trsm():
    R, P = ref("plain"), port()
    P.set_blocks(384, 384, 4096)
    seed = 500
    for (m, n, k) in [(7, 5, 3), (70, 33, 790)]:
        for ta, tb in itertools.product("NT", "NT"):
            seed += 3
            A = det_uniform(seed, m if ta == "N" else k, k if ta == "N" else m, np.float32)
            B = det_uniform(seed + 1, k if tb == "N" else n, n if tb == "N" else k, np.float32)
            C0 = det_uniform(seed + 2, m, n, np.float32)
            c1, c2 = C0.copy(order="F"), C0.copy(order="F")
            R.sgemm(ta, tb, m, n, k, 0.7, A, B, 1.3, c1)
            P.sgemm(ta, tb, m, n, k, 0.7, A, B, 1.3, c2)
            assert np.array_equal(c1, c2)
    for (n, k) in [(7, 3), (400, 390)]:
        for uplo, tr in itertools.product("UL", "NT"):
            seed += 2
            A = det_uniform(seed, n if tr == "N" else k, k if tr == "N" else n)
            _, Cb = _mk(seed + 1, n, n, 2)
            c1, c2 = Cb.copy(order="F"), Cb.copy(order="F")
            R.dsyrk(uplo, tr, n, k, -0.7, A, 1.3, c1[:n, :n], ldc=n + 2)
            P.dsyrk(uplo, tr, n, k, -0.7, A, 1.3, c2[:n, :n], ldc=n + 2)
            assert np.array_equal(c1, c2)
            other = np.tril(np.ones((n, n), bool), -1) if uplo == "U" else np.triu(np.ones((n, n), bool), 1)
            assert np.array_equal(c2[:n, :n][other], Cb[:n, :n][other]), "opposite triangle written"
    for (m, n) in [(400, 9), (9, 400)]:
        for side, uplo, tr, diag in itertools.product("LR", "UL", "NT", "NU"):
            seed += 2
            na = m if side == "L" else n
            A = det_uniform(seed, na, na) / na
            A[np.arange(na), np.arange(na)] = 1.25
            A = np.asfortranarray(A)
            B0 = det_uniform(seed + 1, m, n)
            b1, b2 = B0.copy(order="F"), B0.copy(order="F")
            R.dtrsm(side, uplo, tr, diag, m, n, 1.0, A, b1)
            P.dtrsm(side, uplo, tr, diag, m, n, 1.0, A, b2)
            assert np.array_equal(b1, b2), (m, n, side, uplo, tr, diag)


def test_port_argument_checks_follow_the_reference_order():
    P = port()
    # first offending argument wins, in the reference's order (interfaces/blas/F77/gemm.cc:169-199)
    assert P.gemm_info("X", "N", 1, 1, 1, 1, 1, 1) == 1
    assert P.gemm_info("N", "Q", 1, 1, 1, 1, 1, 1) == 2
    assert P.gemm_info("N", "N", -1, 1, 1, 1, 1, 1) == 3
    assert P.gemm_info("N", "N", 1, -1, 1, 1, 1, 1) == 4
    assert P.gemm_info("N", "N", 1, 1, -1, 1, 1, 1) == 5
    assert P.gemm_info("N", "N", 4, 1, 1, 3, 1, 4) == 8
    assert P.gemm_info("T", "N", 4, 1, 7, 6, 7, 4) == 8
    assert P.gemm_info("N", "N", 4, 1, 7, 4, 6, 4) == 10
    assert P.gemm_info("N", "T", 4, 9, 7, 4, 8, 4) == 10
    assert P.gemm_info("N", "N", 4, 1, 7, 4, 7, 3) == 13
    assert P.gemm_info("r", "c", 4, 1, 7, 4, 1, 4) == 0      # 'R' is accepted as "not transposed"
    assert P.trsm_info("L", "L", "N", "N", 3, 2, 3, 3) == 0
    assert [P.trsm_info(*a) for a in [("X", "L", "N", "N", 1, 1, 1, 1), ("L", "X", "N", "N", 1, 1, 1, 1),
                                      ("L", "L", "X", "N", 1, 1, 1, 1), ("L", "L", "N", "X", 1, 1, 1, 1),
                                      ("L", "L", "N", "N", -1, 1, 1, 1), ("L", "L", "N", "N", 1, -1, 1, 1),
                                      ("L", "L", "N", "N", 3, 1, 2, 3), ("R", "L", "N", "N", 3, 5, 4, 3),
                                      ("L", "L", "N", "N", 3, 1, 3, 2)]] == [1, 2, 3, 4, 5, 6, 9, 9, 11]
    assert [P.syrk_info(*a) for a in [("X", "N", 1, 1, 1, 1), ("U", "X", 1, 1, 1, 1), ("U", "N", -1, 1, 1, 1),
                                      ("U", "N", 1, -1, 1, 1), ("U", "N", 3, 1, 2, 3), ("U", "T", 3, 5, 4, 3),
                                      ("U", "N", 3, 1, 3, 2)]] == [1, 2, 3, 4, 7, 7, 10]


# ---------------------------------------------------------------------------
# complex double GEMM
# ---------------------------------------------------------------------------
def _same_z(a, b):
    return np.array_equal(a.real, b.real) and np.array_equal(a.imag, b.imag)


def test_port_reproduces_reference_golden_zgemm():
    """Outputs the compiled reference's zgemm_ produced (tests/golden/ulmblas_zgemm.npz), bit for bit."""
    P = port()
    P.set_blocks()
    cases = load_golden("ulmblas_zgemm.npz")
    assert len(cases) == 20
    for name, c in cases.items():
        A, B, C0 = golden_inputs(c)
        got = C0.copy(order="F")
        P.zgemm(c["ta"], c["tb"], c["m"], c["n"], c["k"], complex(c["alpha_re"], c["alpha_im"]), A, B,
                complex(c["beta_re"], c["beta_im"]), got)
        want = c["C_re"] + 1j * c["C_im"]
        assert _same_z(got, want), name


@needs_ref
@pytest.mark.parametrize("variant,blocks", [("", (384, 384, 4096, 192)), ("plain", (384, 384, 4096, 384)),
                                            ("tiny", (8, 12, 12, 12))])
def test_port_equals_compiled_reference_zgemm(variant, blocks):
    R, P = ref(variant), port()
    P.set_blocks(*blocks)
    try:
        seed = 7000
        for (m, n, k) in [(1, 1, 1), (5, 7, 3), (33, 21, 50), (70, 45, 401)]:
            for ta, tb in itertools.product("NTCR", "NTCR"):
                for al, be in [(1 + 0j, 0j), (0.7 - 0.3j, 1.3 + 0.2j)]:
                    seed += 6
                    ra, ca = (k, m) if ta in "TC" else (m, k)
                    rb, cb = (n, k) if tb in "TC" else (k, n)
                    A = np.asfortranarray(det_uniform(seed, ra + 2, ca) + 1j * det_uniform(seed + 1, ra + 2, ca))
                    B = np.asfortranarray(det_uniform(seed + 2, rb + 1, cb) + 1j * det_uniform(seed + 3, rb + 1, cb))
                    C0 = np.asfortranarray(det_uniform(seed + 4, m + 3, n) + 1j * det_uniform(seed + 5, m + 3, n))
                    c1, c2 = C0.copy(order="F"), C0.copy(order="F")
                    R.zgemm(ta, tb, m, n, k, al, A, B, be, c1, lda=ra + 2, ldb=rb + 1, ldc=m + 3)
                    P.zgemm(ta, tb, m, n, k, al, A, B, be, c2, lda=ra + 2, ldb=rb + 1, ldc=m + 3)
                    assert _same_z(c1, c2), (variant, m, n, k, ta, tb, al, be)
                    assert _same_z(c2[m:, :], C0[m:, :]), "padding rows written"
    finally:
        P.set_blocks()
