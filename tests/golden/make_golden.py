"""Generates tests/golden/*.npz from the reference itself.

Run where the ulmBLAS source tree is available (``make -C oracle ref`` must have built
``oracle/_ref/libulmref*.so``):

    python tests/golden/make_golden.py

Each fixture stores the inputs and the output the compiled reference produced for one
call on the Level-3 GEMM path.  Two builds of the reference are used: the SSE build
(reference's own flags) and the portable-kernel build at the same block sizes; they
agree bit for bit except where the SSE build returns NaN on finite inputs (its
buffered micro-kernel reads an uninitialised tile) -- those entries are taken from
the portable build, and the number replaced is recorded in the fixture.
"""
import itertools
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from tests.helpers import det_uniform  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
_seed = [1000]


def mat(rng, r, c, ld, dtype=np.float64):
    """Inputs come from tests.helpers.det_uniform(seed, ...) with consecutive seeds, so the
    fixture only has to store the seeds and the reference's outputs."""
    _seed[0] += 1
    v, base = oracle.fmat(r, c, ld, dtype=dtype, fill=-1e10)
    v[...] = det_uniform(_seed[0], r, c, dtype)
    return v, base, _seed[0]


def merged(sse, plain):
    bad = ~np.isfinite(sse)
    assert np.array_equal(sse[~bad], plain[~bad]), "the two reference builds disagree on finite entries"
    out = sse.copy(order="F")
    out[bad] = plain[bad]
    return out, int(bad.sum())


def main():
    sse, plain = oracle.Ref(""), oracle.Ref("plain")
    rng = np.random.default_rng(20241125)
    fx = {}

    # dgemm: shapes that straddle the 384/384/4096 cache blocks and the 4x4 register tile
    for idx, ((m, n, k), (ta, tb), (al, be)) in enumerate(itertools.product(
            [(5, 7, 3), (33, 17, 401), (390, 9, 30)], itertools.product("NT", "NT"),
            [(1.5, 0.5), (-0.7, 1.3), (1.0, 0.0)])):
        A, _, sa = mat(rng, m if ta == "N" else k, k if ta == "N" else m, (m if ta == "N" else k) + 3)
        B, _, sb = mat(rng, k if tb == "N" else n, n if tb == "N" else k, (k if tb == "N" else n) + 1)
        C0, Cb, sc = mat(rng, m, n, m + 2)
        c1, c2 = Cb.copy(order="F"), Cb.copy(order="F")
        sse.dgemm(ta, tb, m, n, k, al, A, B, be, c1[:m, :n], ldc=m + 2)
        plain.dgemm(ta, tb, m, n, k, al, A, B, be, c2[:m, :n], ldc=m + 2)
        out, nbad = merged(c1, c2)
        fx[f"dgemm_{idx}"] = dict(kind="dgemm", ta=ta, tb=tb, m=m, n=n, k=k, alpha=al, beta=be,
                                  seedA=sa, seedB=sb, seedC=sc, C=out[:m, :n], nan_replaced=nbad)

    # sgemm (the Fortran-ABI entry point accumulates in double)
    for idx, ((m, n, k), (ta, tb), (al, be)) in enumerate(itertools.product(
            [(9, 6, 5), (70, 33, 790)], itertools.product("NT", "NT"), [(1.0, 0.0), (0.7, 1.3)])):
        A, _, sa = mat(rng, m if ta == "N" else k, k if ta == "N" else m, None, np.float32)
        B, _, sb = mat(rng, k if tb == "N" else n, n if tb == "N" else k, None, np.float32)
        C0, Cb, sc = mat(rng, m, n, m + 1, np.float32)
        c1, c2 = Cb.copy(order="F"), Cb.copy(order="F")
        sse.sgemm(ta, tb, m, n, k, al, A, B, be, c1[:m, :n], ldc=m + 1)
        plain.sgemm(ta, tb, m, n, k, al, A, B, be, c2[:m, :n], ldc=m + 1)
        out, nbad = merged(c1, c2)
        fx[f"sgemm_{idx}"] = dict(kind="sgemm", ta=ta, tb=tb, m=m, n=n, k=k, alpha=al, beta=be,
                                  seedA=sa, seedB=sb, seedC=sc, C=out[:m, :n], nan_replaced=nbad)

    # dsyrk
    for idx, ((n, k), (uplo, tr), (al, be)) in enumerate(itertools.product(
            [(7, 5), (40, 401)], itertools.product("UL", "NT"), [(1.0, 0.5), (-0.7, 0.0)])):
        A, _, sa = mat(rng, n if tr == "N" else k, k if tr == "N" else n, (n if tr == "N" else k) + 1)
        C0, Cb, sc = mat(rng, n, n, n + 2)
        c1, c2 = Cb.copy(order="F"), Cb.copy(order="F")
        sse.dsyrk(uplo, tr, n, k, al, A, be, c1[:n, :n], ldc=n + 2)
        plain.dsyrk(uplo, tr, n, k, al, A, be, c2[:n, :n], ldc=n + 2)
        out, nbad = merged(c1, c2)
        fx[f"dsyrk_{idx}"] = dict(kind="dsyrk", uplo=uplo, trans=tr, n=n, k=k, alpha=al, beta=be,
                                  seedA=sa, seedC=sc, C=out[:n, :n], nan_replaced=nbad)

    # dtrsm: every side/uplo/trans/diag combination, one size above the 384 block
    for idx, ((m, n), (side, uplo, tr, diag), al) in enumerate(itertools.product(
            [(9, 6), (390, 5), (5, 390)], itertools.product("LR", "UL", "NT", "NU"), [0.7])):
        na = m if side == "L" else n
        A, _, sa = mat(rng, na, na, na + 1)
        d = A[np.arange(na), np.arange(na)].copy()
        A[...] = A / na
        A[np.arange(na), np.arange(na)] = 1.5 + 0.5 * d
        B0, Bb, sb = mat(rng, m, n, m + 2)
        b1, b2 = Bb.copy(order="F"), Bb.copy(order="F")
        sse.dtrsm(side, uplo, tr, diag, m, n, al, A, b1[:m, :n], ldb=m + 2)
        plain.dtrsm(side, uplo, tr, diag, m, n, al, A, b2[:m, :n], ldb=m + 2)
        out, nbad = merged(b1, b2)
        fx[f"dtrsm_{idx}"] = dict(kind="dtrsm", side=side, uplo=uplo, trans=tr, diag=diag, m=m, n=n,
                                  alpha=al, seedA=sa, seedB=sb, B=out[:m, :n], nan_replaced=nbad)

    flat = {}
    for name, d in fx.items():
        for key, val in d.items():
            flat[f"{name}/{key}"] = np.asarray(val)
    path = os.path.join(OUT, "ulmblas_level3.npz")
    np.savez_compressed(path, **flat)
    print(path, os.path.getsize(path) // 1024, "KiB,", len(fx), "cases,",
          sum(int(d["nan_replaced"]) for d in fx.values()), "NaN entries replaced")


def main_z():
    """zgemm_ cases into their own file (seeds continue from a fixed base, independent of main())."""
    sse, plain = oracle.Ref(""), oracle.Ref("plain")
    _seed[0] = 9000
    fx = {}
    cases = [((5, 7, 3), "N", "N"), ((5, 7, 3), "C", "R"), ((33, 17, 401), "N", "N"), ((33, 17, 401), "T", "N"),
             ((33, 17, 401), "N", "C"), ((33, 17, 401), "C", "T"), ((33, 17, 401), "R", "N"),
             ((200, 9, 190), "C", "N"), ((200, 9, 190), "N", "T"), ((9, 200, 30), "T", "R")]
    scal = [(1.0 + 0.0j, 0.0j), (0.7 - 0.3j, 1.3 + 0.2j)]
    for idx, (((m, n, k), ta, tb), (al, be)) in enumerate(itertools.product(cases, scal)):
        ra, ca = (k, m) if ta in "TC" else (m, k)
        rb, cb = (n, k) if tb in "TC" else (k, n)
        seeds = []
        def zmat(r, c, ld):
            re, _, s1 = mat(None, r, c, r)
            im, _, s2 = mat(None, r, c, r)
            seeds.append((s1, s2))
            base = np.full((ld, c), -1e10 - 1e10j, dtype=np.complex128, order="F")
            base[:r, :] = re + 1j * im
            return base[:r, :], base
        A, _ = zmat(ra, ca, ra + 3)
        B, _ = zmat(rb, cb, rb + 1)
        C0, Cb = zmat(m, n, m + 2)
        c1, c2 = Cb.copy(order="F"), Cb.copy(order="F")
        sse.zgemm(ta, tb, m, n, k, al, A, B, be, c1[:m, :n], lda=ra + 3, ldb=rb + 1, ldc=m + 2)
        plain_kc = 192     # the portable-kernel build uses KC = 384 for every type: only k <= 384 agree in general
        plain.zgemm(ta, tb, m, n, k, al, A, B, be, c2[:m, :n], lda=ra + 3, ldb=rb + 1, ldc=m + 2)
        assert np.isfinite(c1.real).all() and np.isfinite(c1.imag).all()
        if k <= plain_kc:
            assert np.array_equal(c1.real, c2.real) and np.array_equal(c1.imag, c2.imag)
        assert np.array_equal(c1[m:, :].real, Cb[m:, :].real), "padding rows written"
        fx[f"zgemm_{idx}"] = dict(kind="zgemm", ta=ta, tb=tb, m=m, n=n, k=k, alpha_re=al.real, alpha_im=al.imag,
                                  beta_re=be.real, beta_im=be.imag, seedA=seeds[0], seedB=seeds[1], seedC=seeds[2],
                                  C_re=c1[:m, :n].real, C_im=c1[:m, :n].imag)
    flat = {}
    for name, d in fx.items():
        for key, val in d.items():
            flat[f"{name}/{key}"] = np.asarray(val)
    path = os.path.join(OUT, "ulmblas_zgemm.npz")
    np.savez_compressed(path, **flat)
    print(path, os.path.getsize(path) // 1024, "KiB,", len(fx), "cases")


if __name__ == "__main__":
    if "--zgemm-only" not in sys.argv:
        main()
    main_z()
