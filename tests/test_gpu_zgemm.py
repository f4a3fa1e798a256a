"""Complex double GEMM on the GPU against the reference's zgemm_.

Bound: the one the reference's own tester applies (test/F77/zblat3.f:3003-3160, ZMMCH), with the
constant 2 k eps used for the real routines: |C - C_ref|_1 <= 2 k eps (|alpha|_1 (|A|_1 |B|_1) + |beta|_1 |C0|_1), where
|z|_1 = |re z| + |im z| elementwise."""
import itertools

import numpy as np
import pytest

from helpers import EPS64, det_uniform, golden_inputs, load_golden, port, ref

pytestmark = pytest.mark.gpu

OPS = {"N": lambda X: X, "T": lambda X: X.T, "C": lambda X: X.conj().T, "R": lambda X: X.conj()}


def abs1(Z):
    return np.abs(Z.real) + np.abs(Z.imag)


def zmat(seed, r, c, ld=None):
    ld = ld or r
    base = np.full((ld, c), -1e10 - 1e10j, dtype=np.complex128, order="F")
    base[:r, :] = det_uniform(seed, r, c) + 1j * det_uniform(seed + 1, r, c)
    return base[:r, :], base


def ratio(got, want, ta, tb, k, alpha, A, B, beta, C0):
    gauge = abs1(np.array(alpha)) * (abs1(OPS[ta](A)) @ abs1(OPS[tb](B))) + abs1(np.array(beta)) * abs1(C0)
    bound = 2.0 * max(k, 1) * EPS64 * gauge
    err = abs1(got - want)
    ok = bound > 0
    r = float((err[ok] / bound[ok]).max()) if ok.any() else 0.0
    assert np.all(err[~ok] == 0.0)
    return r


def reference_zgemm(ta, tb, m, n, k, alpha, A, B, beta, C0, **ld):
    want = C0.copy(order="F")
    (ref("") or port()).zgemm(ta, tb, m, n, k, alpha, A, B, beta, want, **ld)
    return want


def test_golden_zgemm_cases_on_gpu(ulm):
    for name, c in load_golden("ulmblas_zgemm.npz").items():
        A, B, C0 = golden_inputs(c)
        al, be = complex(c["alpha_re"], c["alpha_im"]), complex(c["beta_re"], c["beta_im"])
        got = C0.copy(order="F")
        assert ulm.zgemm(c["ta"], c["tb"], c["m"], c["n"], c["k"], al, A, B, be, got) == ulm.OK
        want = c["C_re"] + 1j * c["C_im"]
        assert ratio(got, want, c["ta"], c["tb"], c["k"], al, A, B, be, C0) <= 1.0, name


def test_zgemm_all_modes_padded_lds(ulm):
    seed = 52000
    for (m, n, k) in [(1, 1, 1), (7, 5, 3), (130, 67, 201), (300, 129, 64)]:
        for ta, tb in itertools.product("NTCR", "NTCR"):
            seed += 6
            ra, ca = (k, m) if ta in "TC" else (m, k)
            rb, cb = (n, k) if tb in "TC" else (k, n)
            A, Ab = zmat(seed, ra, ca, ra + 3)
            B, Bb = zmat(seed + 2, rb, cb, rb + 1)
            C0, Cb = zmat(seed + 4, m, n, m + 2)
            al, be = (0.7 - 0.3j, 1.3 + 0.2j) if (m + ord(ta)) % 2 else (1.0 + 0j, -0.5j)
            want = reference_zgemm(ta, tb, m, n, k, al, A, B, be, C0, lda=ra + 3, ldb=rb + 1)
            got_b = Cb.copy(order="F")
            A0, B0 = Ab.copy(order="F"), Bb.copy(order="F")
            assert ulm.zgemm(ta, tb, m, n, k, al, A, B, be, got_b[:m, :n], lda=ra + 3, ldb=rb + 1, ldc=m + 2) == ulm.OK
            assert ratio(got_b[:m, :n], want, ta, tb, k, al, A, B, be, C0) <= 1.0, (m, n, k, ta, tb)
            # padding rows and the inputs stay bit-identical
            assert np.array_equal(got_b[m:, :].real, Cb[m:, :].real) and np.array_equal(got_b[m:, :].imag, Cb[m:, :].imag)
            assert np.array_equal(Ab.real, A0.real) and np.array_equal(Bb.imag, B0.imag)


def test_zgemm_quick_paths_and_beta_zero(ulm):
    m, n, k = 40, 30, 20
    A, _ = zmat(1, m, k); B, _ = zmat(3, k, n); C0, _ = zmat(5, m, n)
    # beta == 0 never reads C
    Cn = np.full((m, n), np.nan + 1j * np.nan, dtype=np.complex128, order="F")
    assert ulm.zgemm("N", "N", m, n, k, 1.0, A, B, 0.0, Cn) == ulm.OK
    assert np.isfinite(Cn.real).all() and np.isfinite(Cn.imag).all()
    assert ratio(Cn, A @ B, "N", "N", k, 1.0 + 0j, A, B, 0j, C0 * 0) <= 1.0
    # alpha == 0 and k == 0 only scale (gemm.tcc:52-55)
    for kk, al in ((k, 0.0), (0, 1.0)):
        got = C0.copy(order="F")
        assert ulm.zgemm("N", "N", m, n, kk, al, A, B, 0.5 - 2j, got) == ulm.OK
        want = reference_zgemm("N", "N", m, n, kk, complex(al), A, B, 0.5 - 2j, C0)
        assert np.abs(got - want).max() <= 4 * EPS64 * np.abs(want).max()
    got = C0.copy(order="F")
    assert ulm.zgemm("N", "N", m, n, 0, 1.0, A, B, 1.0, got) == ulm.OK
    assert np.array_equal(got.real, C0.real) and np.array_equal(got.imag, C0.imag)


def test_cblas_zgemm_row_major_and_conj(ulm):
    m, n, k = 37, 22, 51
    # row-major operands are C-ordered arrays; CblasConjTrans on A, AtlasConj on B
    Ar = (det_uniform(11, k, m) + 1j * det_uniform(12, k, m)).copy(order="C")     # op(A) = A^H: stored k x m
    Br = (det_uniform(13, k, n) + 1j * det_uniform(14, k, n)).copy(order="C")
    C0 = (det_uniform(15, m, n) + 1j * det_uniform(16, m, n)).copy(order="C")
    got = C0.copy(order="C")
    al, be = 0.3 + 0.9j, -1.1 + 0.4j
    st = ulm.cblas_zgemm(ulm.CblasRowMajor, 113, 114, m, n, k, al, Ar, m, Br, n, be, got, n)
    assert st == ulm.OK
    want = al * (Ar.conj().T @ Br.conj()) + be * C0
    gauge = abs1(np.array(al)) * (abs1(Ar.T) @ abs1(Br)) + abs1(np.array(be)) * abs1(C0)
    assert (abs1(got - want) <= 2 * k * EPS64 * gauge).all()


def test_zgemm_1024_device_resident(ulm, torch_cuda):
    """1024^3, op(A) = A^H, device pointers through ulmb200_zgemm; the CPU oracle checks 64 sampled columns."""
    torch = torch_cuda
    m = n = k = 1024
    A, _ = zmat(21, k, m); B, _ = zmat(23, k, n); C0, _ = zmat(25, m, n)
    dA = torch.from_numpy(np.ascontiguousarray(A.T)).cuda()
    dB = torch.from_numpy(np.ascontiguousarray(B.T)).cuda()
    dC = torch.from_numpy(np.ascontiguousarray(C0.T)).cuda()
    al, be = 0.7 - 0.3j, 1.3 + 0.2j
    ulm.dev_zgemm(1, 1, 0, 0, m, n, k, al, dA.data_ptr(), k, dB.data_ptr(), k, be, dC.data_ptr(), m)
    torch.cuda.synchronize()
    got = dC.cpu().numpy().T
    cols = np.sort(np.random.default_rng(2).choice(n, 64, replace=False))
    Bs, Cs = np.asfortranarray(B[:, cols]), np.asfortranarray(C0[:, cols])
    want = reference_zgemm("C", "N", m, len(cols), k, al, A, Bs, be, Cs)
    assert ratio(got[:, cols], want, "C", "N", k, al, A, Bs, be, Cs) <= 1.0
