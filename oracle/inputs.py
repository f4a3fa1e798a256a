"""TEST INFRASTRUCTURE -- NOT PART OF THE PRODUCT.

numpy twins of two things the checkers need without loading any library of the product:

* ``gen_uniform`` -- the counter-based matrix generator of the bench and the tests
  (ulmblas_b200/csrc/support/gen.h): element (i, j) of matrix ``mat`` under ``seed`` is a pure
  function of (seed, mat, i, j), so any block of any operand can be regenerated anywhere, bit
  for bit.  (The role ATL_gegen plays in the reference's timers, bench/l3blastst.c.)
* ``bound_ratio`` / ``gemm_gauge`` -- the componentwise error bound
  |C - Cref| <= 2 k eps (|alpha| |A||B| + |beta| |C|), with the gauge of the reference's tester
  (test/F77/dblat3.f:2496-2545) and eps as it defines it (dblat3.f:183-193).
"""
import numpy as np

EPS64 = 2.0 ** -52
EPS32 = 2.0 ** -23

_U = np.uint64


def _mix64(z):
    z = (z + _U(0x9E3779B97F4A7C15)).astype(np.uint64)
    z = ((z ^ (z >> _U(30))) * _U(0xBF58476D1CE4E5B9)).astype(np.uint64)
    z = ((z ^ (z >> _U(27))) * _U(0x94D049BB133111EB)).astype(np.uint64)
    return z ^ (z >> _U(31))


def gen_u01(seed, mat, rows, cols, row0=0, col0=0):
    """rows x cols block of uniform[0,1) values with 53 random bits, top-left element (row0, col0)."""
    with np.errstate(over="ignore"):
        key = _mix64(np.array([np.uint64(seed) ^ (np.uint64(mat) * _U(0xD1B54A32D192ED03))], dtype=np.uint64))[0]
        i = (np.arange(rows, dtype=np.int64) + row0).astype(np.uint64) & _U(0xFFFFFFFF)
        j = (np.arange(cols, dtype=np.int64) + col0).astype(np.uint64) << _U(32)
        h = _mix64(key ^ (j[None, :] | i[:, None]))
    return (h >> _U(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def gen_uniform(seed, mat, rows, cols, row0=0, col0=0, dtype=np.float64, dist=0, scale=1.0):
    """Column-major block of the generator's matrix: dist 0 uniform[-1,1); dist 1 uniform[1,2) on
    the diagonal and uniform[-1,1) * scale elsewhere (triangular solver inputs)."""
    u = gen_u01(seed, mat, rows, cols, row0, col0)
    v = 2.0 * u - 1.0
    if dist == 1:
        v = v * scale
        gi = np.arange(rows)[:, None] + row0
        gj = np.arange(cols)[None, :] + col0
        v = np.where(gi == gj, 1.0 + u, v)
    return np.asfortranarray(v.astype(dtype))


def gemm_gauge(alpha, opA, opB, beta, C0):
    """|alpha| * |op(A)| |op(B)| + |beta| * |C0|."""
    g = abs(alpha) * (np.abs(opA).astype(np.float64) @ np.abs(opB).astype(np.float64))
    if beta != 0:
        g = g + abs(beta) * np.abs(C0).astype(np.float64)
    return g


def bound_ratio(C, Cref, gauge, k, eps):
    """max_ij |C - Cref| / (2*k*eps*gauge_ij); parity holds iff the result is <= 1."""
    err = np.abs(C.astype(np.float64) - Cref.astype(np.float64))
    lim = 2.0 * max(k, 1) * eps * gauge
    with np.errstate(divide="ignore", invalid="ignore"):
        ratio = np.where(lim > 0, err / lim, np.where(err == 0, 0.0, np.inf))
    return float(ratio.max()) if ratio.size else 0.0
