"""Shared test utilities: deterministic inputs, the componentwise error bound, and the
reference checkers (oracle/ is test infrastructure; the product never imports it)."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from oracle.inputs import EPS32, EPS64, bound_ratio, gemm_gauge, gen_uniform  # noqa: E402,F401
# EPS: smallest power of two with 1 + eps != 1, as the reference's tester defines it
# (test/F77/dblat3.f:183-193); bound_ratio: the componentwise parity bound
ROGUE = -1e10           # padding / unreferenced-triangle fill of the reference's tester (dblat3.f:2365)


def _mix64(z):
    z = (z + np.uint64(0x9E3779B97F4A7C15)).astype(np.uint64)
    z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)).astype(np.uint64)
    z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)).astype(np.uint64)
    return z ^ (z >> np.uint64(31))


def det_uniform(seed, rows, cols, dtype=np.float64):
    """rows x cols column-major matrix, uniform[-1,1), a pure function of (seed, i, j);
    independent of numpy's own random streams so fixtures stay reproducible."""
    with np.errstate(over="ignore"):
        idx = (np.arange(cols, dtype=np.uint64)[None, :] << np.uint64(32)) | np.arange(rows, dtype=np.uint64)[:, None]
        h = _mix64(_mix64(np.uint64(seed)) ^ idx)
    u = (h >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)
    return np.asfortranarray((2.0 * u - 1.0).astype(dtype))


def padded(values, ld, fill=ROGUE):
    """Copy `values` into the top rows of an ld-row column-major allocation filled with `fill`."""
    r, c = values.shape
    view, base = oracle.fmat(r, c, ld, dtype=values.dtype, fill=fill)
    view[...] = values
    return view, base


_port = None
_refs = {}


def port():
    global _port
    if _port is None:
        _port = oracle.Port()
    return _port


def ref(variant=""):
    """The compiled reference, or None when oracle/_ref has not been built."""
    if variant not in _refs:
        _refs[variant] = oracle.Ref(variant) if oracle.have_ref(variant) else None
    return _refs[variant]


def repair_nonfinite(out_ref, out_port):
    """The reference's SSE build can return NaN on finite inputs (its buffered micro-kernel
    reads an uninitialised stack tile, ulmblas/level3/ukernel/ugemm.tcc:33).  The C
    restatement is bit-identical to the reference elsewhere, so its value stands in for
    such entries.  Returns the number of entries replaced."""
    bad = ~np.isfinite(out_ref)
    n = int(bad.sum())
    if n:
        out_ref[bad] = out_port[bad]
    return n


# --------------------------------------------------------------------------- golden fixtures

def load_golden(name="ulmblas_level3.npz"):
    """tests/golden/<name> -> {case name: {field: value}} (made by make_golden.py)."""
    z = np.load(os.path.join(ROOT, "tests", "golden", name))
    cases = {}
    for key in z.files:
        name, field = key.split("/")
        v = z[key]
        cases.setdefault(name, {})[field] = v.item() if v.ndim == 0 else v
    return cases


def golden_inputs(c):
    """Rebuild the inputs of a fixture case from its seeds (same recipe as make_golden.py)."""
    kind = c["kind"]
    if kind in ("dgemm", "sgemm"):
        dt = np.float64 if kind == "dgemm" else np.float32
        m, n, k = c["m"], c["n"], c["k"]
        A = det_uniform(c["seedA"], m if c["ta"] == "N" else k, k if c["ta"] == "N" else m, dt)
        B = det_uniform(c["seedB"], k if c["tb"] == "N" else n, n if c["tb"] == "N" else k, dt)
        return A, B, det_uniform(c["seedC"], m, n, dt)
    if kind == "zgemm":
        m, n, k = c["m"], c["n"], c["k"]
        ra, ca = (k, m) if c["ta"] in "TC" else (m, k)
        rb, cb = (n, k) if c["tb"] in "TC" else (k, n)

        def z(seeds, r, cc):
            return np.asfortranarray(det_uniform(int(seeds[0]), r, cc) + 1j * det_uniform(int(seeds[1]), r, cc))
        return z(c["seedA"], ra, ca), z(c["seedB"], rb, cb), z(c["seedC"], m, n)
    if kind == "dsyrk":
        n, k = c["n"], c["k"]
        A = det_uniform(c["seedA"], n if c["trans"] == "N" else k, k if c["trans"] == "N" else n)
        return A, det_uniform(c["seedC"], n, n)
    if kind == "dtrsm":
        m, n = c["m"], c["n"]
        na = m if c["side"] == "L" else n
        A = det_uniform(c["seedA"], na, na)
        d = A[np.arange(na), np.arange(na)].copy()
        A = np.asfortranarray(A / na)
        A[np.arange(na), np.arange(na)] = 1.5 + 0.5 * d
        return A, det_uniform(c["seedB"], m, n)
    raise ValueError(kind)
