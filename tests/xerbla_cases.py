"""Bad-argument cases for the error exits of the Level-3 entry points, shared by the script that
records what the compiled reference reports (tests/golden/make_golden_errors.py) and by the test
that holds libulmblas_b200.so to the same answers.

The method is the reference tester's (test/F77/dblat3.f:1801 DCHKE, test/C/c_d3chke.c): start from
a valid call, make ONE argument illegal, and expect the routine's name and the 1-based index of
that argument in the caller-supplied xerbla.  A few cases break two arguments at once: the first
one must be reported.  Both storage orders for the CBLAS entry points.

A case is (routine, args): characters/enum values and integers only.  Scalars (alpha, beta) and the
matrix operands are supplied by `call`: 1.0 and 16 x 16 arrays, large enough for every size used
here, so that the reference -- which reports the bad argument and then computes anyway
(interfaces/blas/F77/gemm.cc:197-204) -- stays inside them.
"""
import ctypes as C

import numpy as np

ROW, COL = 101, 102
NT, TR, CT, AC = 111, 112, 113, 114
UP, LO = 121, 122
NU, UN = 131, 132
LE, RI = 141, 142
BAD = 7            # no CBLAS enum has this value


def _variants(base, bad_values, extra=()):
    """base with argument i replaced by its bad value, for every i that has one."""
    out = []
    for i, bad in enumerate(bad_values):
        if bad is None:
            continue
        for b in (bad if isinstance(bad, (list, tuple)) else [bad]):
            a = list(base)
            a[i] = b
            out.append(tuple(a))
    out.extend(extra)
    return out


def cases():
    cs = []
    # ---- Fortran ABI --------------------------------------------------------------------
    # ?gemm_(ta, tb, m, n, k, lda, ldb, ldc)
    for r in ("dgemm_", "sgemm_", "zgemm_"):
        for base in [("N", "N", 4, 3, 5, 4, 5, 4), ("T", "N", 4, 3, 5, 5, 5, 4), ("N", "T", 4, 3, 5, 4, 3, 4),
                     ("c", "t", 4, 3, 5, 5, 3, 4)]:
            lda_bad = (4 if base[0] in "Nn" else 5) - 1
            ldb_bad = (5 if base[1] in "Nn" else 3) - 1
            cs += [(r, a) for a in _variants(base, ["X", "Q", -1, -1, -1, lda_bad, ldb_bad, 3])]
        cs += [(r, ("X", "Y", -1, 3, 5, 4, 5, 4)), (r, ("N", "N", 4, -2, -1, 1, 1, 1)), (r, ("N", "N", 0, 0, 0, 0, 1, 1)),
               (r, ("N", "N", 0, 0, 0, 1, 0, 1)), (r, ("N", "N", 0, 0, 0, 1, 1, 0))]
    # ?trsm_/dtrmm_(side, uplo, ta, diag, m, n, lda, ldb)
    for r in ("dtrsm_", "strsm_", "dtrmm_"):
        for base in [("L", "L", "N", "N", 4, 3, 4, 4), ("R", "U", "T", "U", 4, 3, 3, 4), ("l", "u", "c", "n", 2, 5, 2, 2)]:
            dim = base[4] if base[0] in "Ll" else base[5]
            cs += [(r, a) for a in _variants(base, ["X", "X", "X", "X", -1, -1, dim - 1, base[4] - 1])]
        cs += [(r, ("X", "X", "N", "N", 4, 3, 4, 4)), (r, ("L", "L", "N", "N", -1, -1, 0, 0)),
               (r, ("L", "L", "N", "N", 0, 0, 0, 1)), (r, ("L", "L", "N", "N", 0, 0, 1, 0))]
    # ?syrk_(uplo, trans, n, k, lda, ldc)
    for r in ("dsyrk_", "ssyrk_"):
        for base in [("U", "N", 4, 3, 4, 4), ("L", "T", 4, 3, 3, 4), ("u", "c", 3, 5, 5, 3)]:
            rows = base[2] if base[1] in "Nn" else base[3]
            cs += [(r, a) for a in _variants(base, ["X", "X", -1, -1, rows - 1, base[2] - 1])]
        cs += [(r, ("X", "X", 4, 3, 4, 4)), (r, ("U", "N", 0, 0, 0, 1)), (r, ("U", "N", 0, 0, 1, 0))]
    # dsymm_(side, uplo, m, n, lda, ldb, ldc)
    for base in [("L", "U", 4, 3, 4, 4, 4), ("R", "L", 4, 3, 3, 4, 4)]:
        dim = base[2] if base[0] == "L" else base[3]
        cs += [("dsymm_", a) for a in _variants(base, ["X", "X", -1, -1, dim - 1, 3, 3])]
    cs += [("dsymm_", ("L", "U", 0, 0, 0, 1, 1)), ("dsymm_", ("L", "U", 0, 0, 1, 0, 1)), ("dsymm_", ("L", "U", 0, 0, 1, 1, 0))]
    # dsyr2k_(uplo, trans, n, k, lda, ldb, ldc)
    for base in [("U", "N", 4, 3, 4, 4, 4), ("L", "T", 4, 3, 3, 3, 4)]:
        rows = base[2] if base[1] == "N" else base[3]
        cs += [("dsyr2k_", a) for a in _variants(base, ["X", "X", -1, -1, rows - 1, rows - 1, 3])]
    # ---- CBLAS ----------------------------------------------------------------------------
    # cblas_?gemm(order, ta, tb, m, n, k, lda, ldb, ldc)
    for r in ("cblas_dgemm", "cblas_sgemm", "cblas_zgemm"):
        for order in (COL, ROW):
            for ta, tb in [(NT, NT), (TR, NT), (NT, CT), (AC, TR)]:
                m, n, k = 4, 3, 5
                na, nb = ta in (NT, AC), tb in (NT, AC)
                if order == COL:
                    lda, ldb, ldc = (m if na else k), (k if nb else n), m
                else:
                    lda, ldb, ldc = (k if na else m), (n if nb else k), n
                base = (order, ta, tb, m, n, k, lda, ldb, ldc)
                cs += [(r, a) for a in _variants(base, [BAD, BAD, BAD, -1, -1, -1, lda - 1, ldb - 1, ldc - 1])]
            cs += [(r, (order, BAD, BAD, -1, 3, 5, 4, 5, 4)), (r, (order, NT, NT, -1, -1, 5, 1, 1, 1)),
                   (r, (order, NT, NT, 4, 3, 5, 1, 1, 1))]
        cs += [(r, (BAD, BAD, NT, 4, 3, 5, 4, 5, 4))]
    # cblas_?trsm / cblas_dtrmm(order, side, uplo, ta, diag, m, n, lda, ldb)
    for r in ("cblas_dtrsm", "cblas_strsm", "cblas_dtrmm"):
        for order in (COL, ROW):
            for side, uplo, ta, diag in [(LE, LO, NT, NU), (RI, UP, TR, UN), (LE, UP, CT, NU), (RI, LO, AC, UN)]:
                m, n = 4, 3
                dim = m if side == LE else n
                ldb = m if order == COL else n
                base = (order, side, uplo, ta, diag, m, n, dim, ldb)
                cs += [(r, a) for a in _variants(base, [BAD, BAD, BAD, BAD, BAD, -1, -1, dim - 1, ldb - 1])]
            cs += [(r, (order, LE, LO, NT, NU, -1, -1, 4, 4)), (r, (order, BAD, BAD, NT, NU, 4, 3, 4, 4)),
                   (r, (order, LE, LO, NT, NU, 4, 3, 1, 1))]
    # cblas_?syrk(order, uplo, trans, n, k, lda, ldc)
    for r in ("cblas_dsyrk", "cblas_ssyrk"):
        for order in (COL, ROW):
            for uplo, tr in [(UP, NT), (LO, TR), (UP, CT), (LO, AC)]:
                n, k = 4, 3
                no = tr in (NT, AC)
                rows = (n if no else k) if order == COL else (k if no else n)
                base = (order, uplo, tr, n, k, rows, n)
                cs += [(r, a) for a in _variants(base, [BAD, BAD, BAD, -1, -1, rows - 1, n - 1])]
            cs += [(r, (order, UP, NT, -1, -1, 1, 1)), (r, (order, UP, NT, 4, 3, 1, 1))]
    # cblas_dsymm(order, side, uplo, m, n, lda, ldb, ldc)
    for order in (COL, ROW):
        for side, uplo in [(LE, UP), (RI, LO)]:
            m, n = 4, 3
            dim = m if side == LE else n
            ld = m if order == COL else n
            base = (order, side, uplo, m, n, dim, ld, ld)
            cs += [("cblas_dsymm", a) for a in _variants(base, [BAD, BAD, BAD, -1, -1, dim - 1, ld - 1, ld - 1])]
    # cblas_dsyr2k(order, uplo, trans, n, k, lda, ldb, ldc)
    for order in (COL, ROW):
        for uplo, tr in [(UP, NT), (LO, TR)]:
            n, k = 4, 3
            no = tr in (NT, AC)
            rows = (n if no else k) if order == COL else (k if no else n)
            base = (order, uplo, tr, n, k, rows, rows, n)
            cs += [("cblas_dsyr2k", a) for a in _variants(base, [BAD, BAD, BAD, -1, -1, rows - 1, rows - 1, n - 1])]
    return cs


class Operands:
    """Scalars and 16 x 16 operands (identity: triangular solves stay finite) of every type."""

    def __init__(self):
        self.d = [np.asfortranarray(np.eye(16)) for _ in range(3)]
        self.s = [np.asfortranarray(np.eye(16, dtype=np.float32)) for _ in range(3)]
        self.z = [np.asfortranarray(np.eye(16, dtype=np.complex128)) for _ in range(3)]
        self.one_z = (C.c_double * 2)(1.0, 0.0)

    def of(self, routine):
        t = routine.replace("cblas_", "")[0]
        return {"d": self.d, "s": self.s, "z": self.z}[t]


def call(lib, routine, args, ops):
    """Calls `routine` of `lib` with the case's characters/integers and the stock operands."""
    f = getattr(lib, routine)
    f.restype = None
    A, B, Cm = (x.ctypes.data_as(C.c_void_p) for x in ops.of(routine))
    t = routine.replace("cblas_", "")[0]
    ft = C.c_float if t == "s" else C.c_double
    ints = [a for a in args if isinstance(a, int)]
    chars = [a for a in args if isinstance(a, str)]
    if routine.endswith("_"):                       # Fortran ABI: everything by reference
        ch = [C.c_char_p(c.encode()) for c in chars]
        iv = [C.byref(C.c_int(v)) for v in ints]
        one = ops.one_z if t == "z" else C.byref(ft(1.0))
        kind = routine[1:-1]
        if kind == "gemm":
            f(ch[0], ch[1], iv[0], iv[1], iv[2], one, A, iv[3], B, iv[4], one, Cm, iv[5])
        elif kind in ("trsm", "trmm"):
            f(ch[0], ch[1], ch[2], ch[3], iv[0], iv[1], one, A, iv[2], B, iv[3])
        elif kind == "syrk":
            f(ch[0], ch[1], iv[0], iv[1], one, A, iv[2], one, Cm, iv[3])
        elif kind == "symm":
            f(ch[0], ch[1], iv[0], iv[1], one, A, iv[2], B, iv[3], one, Cm, iv[4])
        elif kind == "syr2k":
            f(ch[0], ch[1], iv[0], iv[1], one, A, iv[2], B, iv[3], one, Cm, iv[4])
        else:
            raise ValueError(routine)
        return
    kind = routine[len("cblas_") + 1:]
    iv = [C.c_int(v) for v in ints]
    one = ops.one_z if t == "z" else ft(1.0)
    if kind == "gemm":
        f(iv[0], iv[1], iv[2], iv[3], iv[4], iv[5], one, A, iv[6], B, iv[7], one, Cm, iv[8])
    elif kind in ("trsm", "trmm"):
        f(iv[0], iv[1], iv[2], iv[3], iv[4], iv[5], iv[6], one, A, iv[7], B, iv[8])
    elif kind == "syrk":
        f(iv[0], iv[1], iv[2], iv[3], iv[4], one, A, iv[5], one, Cm, iv[6])
    elif kind == "symm":
        f(iv[0], iv[1], iv[2], iv[3], iv[4], one, A, iv[5], B, iv[6], one, Cm, iv[7])
    elif kind == "syr2k":
        f(iv[0], iv[1], iv[2], iv[3], iv[4], one, A, iv[5], B, iv[6], one, Cm, iv[7])
    else:
        raise ValueError(routine)


def record(hook, libs, case_list):
    """[(info, name)] as the hook saw them; (0, "") when xerbla was not called.  `libs` maps a
    routine name to the library that holds it."""
    ops = Operands()
    out = []
    info = C.c_int.in_dll(hook, "hook_info")
    name = (C.c_char * 32).in_dll(hook, "hook_name")
    for routine, args in case_list:
        info.value = 0
        name.value = b""
        call(libs(routine), routine, args, ops)
        out.append((int(info.value), name.value.decode()))
    return out
