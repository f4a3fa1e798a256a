"""Boundary checks that need no GPU: the library loads, exports every symbol the header
declares, decodes arguments like the reference's shims, reports bad arguments through a
caller-supplied xerbla_, and refuses to compute without a device (no CPU fallback)."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

from helpers import ROOT, port

HDR = os.path.join(ROOT, "include", "ulmblas_b200.h")


def declared_symbols():
    text = open(HDR).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\(", text)
    skip = {"defined", "if", "sizeof"}
    funcs = sorted({n for n in names if n not in skip and not n.isupper()})
    data = ["CBLAS_CallFromC", "RowMajorStrg"]
    return funcs, data


def test_library_exports_every_declared_symbol(ulm):
    funcs, data = declared_symbols()
    assert {"dgemm_", "sgemm_", "dtrsm_", "dsyrk_", "xerbla_", "cblas_dgemm", "cblas_sgemm",
            "cblas_dtrsm", "cblas_dsyrk", "cblas_xerbla", "ulmblas_dgemm", "ulmb200_dgemm",
            "ulmb200_sgemm", "ulmb200_dtrsm", "ulmb200_dsyrk", "zgemm_", "cblas_zgemm", "ulmblas_zgemm",
            "ulmb200_zgemm", "cblas_strsm", "cblas_ssyrk", "ulmblas_strsm", "ulmblas_ssyrk"} <= set(funcs)
    for name in funcs:
        assert hasattr(ulm.lib, name), f"{name} is declared in include/ulmblas_b200.h but not exported"
    for name in data:
        C.c_int.in_dll(ulm.lib, name)


def test_symbols_are_plain_c_in_the_dynamic_table(ulm):
    out = subprocess.run(["nm", "-D", "--defined-only", ulm.LIB_PATH], capture_output=True, text=True).stdout
    table = {line.split()[-1]: line.split()[-2] for line in out.splitlines() if len(line.split()) >= 3}
    for name in ("dgemm_", "sgemm_", "dtrsm_", "dsyrk_", "cblas_dgemm", "ulmb200_dgemm"):
        assert table.get(name) == "T"
    # overridable, as the reference's testers require
    assert table.get("xerbla_") == "W" and table.get("cblas_xerbla") == "W"


HOOK_SRC = os.path.join(ROOT, "tests", "cpu", "xerbla_hook.c")

_DRIVER = r"""
import ctypes as C, sys, json
sys.path.insert(0, %(root)r)
hook = C.CDLL(%(hook)r, mode=C.RTLD_GLOBAL)
import ulmblas_b200.api as u
import numpy as np
A = np.zeros((8, 8), order="F"); Z = np.zeros((8, 8), dtype=np.complex128, order="F"); out = []
def rec():
    r = (C.c_int.in_dll(hook, "hook_info").value, C.c_char_p(C.addressof(C.c_char.in_dll(hook, "hook_name"))).value.decode(), u.last_status())
    C.c_int.in_dll(hook, "hook_info").value = 0
    return r
for args in %(gemm)r:
    ta, tb, m, n, k, lda, ldb, ldc = args
    u.dgemm(ta, tb, m, n, k, 1.0, A, A, 0.0, A, lda=lda, ldb=ldb, ldc=ldc); out.append(("dgemm",) + rec())
    u.sgemm(ta, tb, m, n, k, 1.0, A, A, 0.0, A, lda=lda, ldb=ldb, ldc=ldc); out.append(("sgemm",) + rec())
    u.zgemm(ta, tb, m, n, k, 1.0, Z, Z, 0.0, Z, lda=lda, ldb=ldb, ldc=ldc); out.append(("zgemm",) + rec())
for args in %(trsm)r:
    s, ul, t, d, m, n, lda, ldb = args
    u.dtrsm(s, ul, t, d, m, n, 1.0, A, A, lda=lda, ldb=ldb); out.append(("dtrsm",) + rec())
for args in %(syrk)r:
    ul, t, n, k, lda, ldc = args
    u.dsyrk(ul, t, n, k, 1.0, A, 0.0, A, lda=lda, ldc=ldc); out.append(("dsyrk",) + rec())
p = A.ctypes.data_as(C.c_void_p)
for args in %(cgemm)r:
    u.lib.cblas_dgemm(*args[:6], 1.0, p, args[6], p, args[7], 0.0, p, args[8]); out.append(("cblas_dgemm",) + rec())
print(json.dumps(out))
"""

GEMM_CASES = [("X", "N", 1, 1, 1, 1, 1, 1), ("N", "Q", 1, 1, 1, 1, 1, 1), ("N", "N", -1, 1, 1, 1, 1, 1),
              ("N", "N", 1, -1, 1, 1, 1, 1), ("N", "N", 1, 1, -1, 1, 1, 1), ("N", "N", 4, 1, 1, 3, 1, 4),
              ("t", "N", 4, 1, 7, 6, 7, 4), ("N", "N", 4, 1, 7, 4, 6, 4), ("N", "c", 4, 9, 7, 4, 8, 4),
              ("N", "N", 4, 1, 7, 4, 7, 3)]
TRSM_CASES = [("X", "L", "N", "N", 1, 1, 1, 1), ("L", "X", "N", "N", 1, 1, 1, 1), ("L", "L", "X", "N", 1, 1, 1, 1),
              ("L", "L", "N", "X", 1, 1, 1, 1), ("L", "L", "N", "N", -1, 1, 1, 1), ("L", "L", "N", "N", 1, -1, 1, 1),
              ("L", "L", "N", "N", 3, 1, 2, 3), ("R", "L", "N", "N", 3, 5, 4, 3), ("L", "L", "N", "N", 3, 1, 3, 2)]
SYRK_CASES = [("X", "N", 1, 1, 1, 1), ("U", "X", 1, 1, 1, 1), ("U", "N", -1, 1, 1, 1), ("U", "N", 1, -1, 1, 1),
              ("U", "N", 3, 1, 2, 3), ("U", "T", 3, 5, 4, 3), ("U", "N", 3, 1, 3, 2)]
# (order, transA, transB, m, n, k, lda, ldb, ldc) -> expected code, interfaces/blas/C/gemm.cc:426-466
CGEMM_CASES = [((7, 111, 111, 1, 1, 1, 1, 1, 1), 1), ((102, 5, 111, 1, 1, 1, 1, 1, 1), 2),
               ((102, 111, 5, 1, 1, 1, 1, 1, 1), 3), ((102, 111, 111, -1, 1, 1, 1, 1, 1), 4),
               ((101, 111, 111, -1, 1, 1, 1, 1, 1), 5), ((101, 111, 111, 1, -1, 1, 1, 1, 1), 4),
               ((102, 111, 111, 4, 1, 1, 3, 1, 4), 9), ((101, 111, 111, 4, 2, 3, 2, 2, 2), 11),
               ((101, 111, 111, 4, 2, 3, 3, 1, 2), 9), ((102, 111, 111, 4, 1, 7, 4, 7, 3), 14),
               ((101, 111, 111, 4, 5, 7, 7, 5, 4), 14)]


def test_bad_arguments_reach_a_caller_supplied_xerbla(ulm, tmp_path):
    """Runs in a child process so the hook library is loaded before the product library."""
    import json
    hook = str(tmp_path / "libxerbla_hook.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-o", hook, HOOK_SRC], check=True)
    code = _DRIVER % dict(root=ROOT, hook=hook, gemm=GEMM_CASES, trsm=TRSM_CASES, syrk=SYRK_CASES,
                          cgemm=[c for c, _ in CGEMM_CASES])
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    got = json.loads(r.stdout.strip().splitlines()[-1])
    P = port()
    it = iter(got)
    for a in GEMM_CASES:
        want = P.gemm_info(*a)
        for routine, nm in (("dgemm", "DGEMM "), ("sgemm", "SGEMM "), ("zgemm", "ZGEMM ")):
            r_, info, name, status = next(it)
            assert (r_, info, name, status) == (routine, want, nm, ulm.BAD_ARGUMENT), (a, info, name)
    for a in TRSM_CASES:
        r_, info, name, status = next(it)
        assert (info, name, status) == (P.trsm_info(*a), "DTRSM ", ulm.BAD_ARGUMENT), a
    for a in SYRK_CASES:
        r_, info, name, status = next(it)
        assert (info, name, status) == (P.syrk_info(*a), "DSYRK ", ulm.BAD_ARGUMENT), a
    for a, want in CGEMM_CASES:
        r_, info, name, status = next(it)
        assert (info, name) == (want, "cblas_dgemm"), (a, info)


_GOLDEN_DRIVER = r"""
import ctypes as C, json, sys
sys.path.insert(0, %(tests)r); sys.path.insert(0, %(root)r)
hook = C.CDLL(%(hook)r, mode=C.RTLD_GLOBAL)
import ulmblas_b200.api as u, xerbla_cases as X
rows = json.load(open(%(golden)r))
cs = [(r["routine"], tuple(r["args"])) for r in rows]
got = X.record(hook, lambda r: u.lib, cs)
print(json.dumps(got))
"""


def test_error_exits_match_the_reference_case_by_case(ulm, tmp_path):
    """Every Level-3 entry point, Fortran ABI and CBLAS in both storage orders, called with one bad
    argument at a time (the reference tester's DCHKE procedure, test/F77/dblat3.f:1801,
    test/C/c_d3chke.c): routine name and argument index reported to a caller-supplied xerbla must
    equal what the compiled reference reported for the same call (tests/golden/xerbla_codes.json,
    recorded by tests/golden/make_golden_errors.py from interfaces/blas/F77/*.cc and
    interfaces/blas/C/*.cc -- e.g. trsm.cc:410-443, syrk.cc:232-249 of the C interface)."""
    import json
    golden = os.path.join(ROOT, "tests", "golden", "xerbla_codes.json")
    rows = json.load(open(golden))
    assert len(rows) > 700 and all(r["info"] > 0 for r in rows)
    routines = {r["routine"] for r in rows}
    assert {"dgemm_", "sgemm_", "zgemm_", "dtrsm_", "strsm_", "dtrmm_", "dsyrk_", "ssyrk_", "dsymm_", "dsyr2k_",
            "cblas_dgemm", "cblas_sgemm", "cblas_zgemm", "cblas_dtrsm", "cblas_dtrmm", "cblas_dsyrk",
            "cblas_dsymm", "cblas_dsyr2k", "cblas_strsm", "cblas_ssyrk"} <= routines
    hook = str(tmp_path / "libxerbla_hook.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-o", hook, HOOK_SRC], check=True)
    code = _GOLDEN_DRIVER % dict(tests=os.path.join(ROOT, "tests"), root=ROOT, hook=hook, golden=golden)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    got = json.loads(r.stdout.strip().splitlines()[-1])
    wrong = [(row["routine"], row["args"], (row["info"], row["name"]), tuple(g))
             for row, g in zip(rows, got) if (row["info"], row["name"]) != tuple(g)]
    assert not wrong, wrong[:10]


def test_ulmblas_xerbla_is_exported_and_overridable(ulm):
    """interfaces/blas/C/xerbla.cc:7-11 exports ULMBLAS(xerbla) beside CBLAS(xerbla)."""
    out = subprocess.run(["nm", "-D", "--defined-only", ulm.LIB_PATH], capture_output=True, text=True).stdout
    table = {line.split()[-1]: line.split()[-2] for line in out.splitlines() if len(line.split()) >= 3}
    assert table.get("ulmblas_xerbla") == "W"


def test_product_library_exports_no_bench_helpers(ulm):
    """Generator, probes and self tests live in libulmb200_benchsupport.so, which declares them in
    its own header and exports each of them."""
    out = subprocess.run(["nm", "-D", "--defined-only", ulm.LIB_PATH], capture_output=True, text=True).stdout
    names = {line.split()[-1] for line in out.splitlines() if line.split()}
    for helper in ("ulmb200_peak_probe", "ulmb200_fill_f64", "ulmb200_host_fill_f64", "ulmb200_abs_f64",
                   "ulmb200_selftest_wait_timeout"):
        assert helper not in names
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "ulmb200_benchsupport.h")).read(), flags=re.S)
    funcs = sorted({n for n in re.findall(r"\b(ulmb200_[A-Za-z0-9_]*)\s*\(", text)})
    assert len(funcs) >= 8
    for name in funcs:
        assert hasattr(ulm.sup, name), name


def test_no_multicast_in_any_kernel_source():
    """No TMA or bulk load with cluster multicast anywhere in the library's sources: every CTA issues its
    own plain loads and relies on L2 for reuse, so the same code runs on one GPU and on several."""
    csrc = os.path.join(ROOT, "ulmblas_b200", "csrc")
    hits = []
    for base, _, files in os.walk(csrc):
        for f in files:
            if f.endswith((".cu", ".h", ".cuh")):
                for i, line in enumerate(open(os.path.join(base, f), errors="replace"), 1):
                    if "multicast" in line.lower():
                        hits.append(f"{f}:{i}")
    assert not hits, hits


def test_work_schedule_model(tmp_path):
    """CPU model of how the persistent DGEMM kernel shares the last tiles among its CTAs."""
    exe = str(tmp_path / "schedule_model")
    subprocess.run(["g++", "-O1", "-std=c++17", "-o", exe, os.path.join(ROOT, "tests", "cpu", "schedule_model.cpp")],
                   check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.strip().endswith("OK"), r.stdout


def test_inplace_leaf_protocol_model(tmp_path):
    """CPU model of the in-place triangular leaf: units in the kernel's order on few or many CTAs of uneven
    speed; no block is overwritten before its readers are through, nothing waits in a cycle."""
    exe = str(tmp_path / "leaf_model")
    subprocess.run(["g++", "-O1", "-std=c++17", "-o", exe, os.path.join(ROOT, "tests", "cpu", "leaf_model.cpp")], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.strip().startswith("OK"), r.stdout


def test_buffered_piece_protocol_model(tmp_path):
    """CPU model of shared tiles leaving piece by piece through each CTA's single tile buffer: pieces reach C in
    order of k, nothing waits for a buffer or a flag for ever, flags end at zero."""
    exe = str(tmp_path / "piece_model")
    subprocess.run(["g++", "-O1", "-std=c++17", "-o", exe, os.path.join(ROOT, "tests", "cpu", "piece_model.cpp")], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.strip().startswith("OK"), r.stdout


def test_trace_and_environment_reload(ulm, monkeypatch, capfd):
    """ULMB200_TRACE=1 prints one line per call; the environment is read once and again on request."""
    A = np.ones((4, 4), order="F")
    monkeypatch.setenv("ULMB200_TRACE", "1")
    ulm.reload_env()
    ulm.dgemm("N", "T", 0, 4, 4, 1.0, A, A, 0.0, A)          # m == 0: returns before any device work
    err = capfd.readouterr().err
    assert "ulmb200: dgemm NT m=0 n=4 k=4" in err, err
    monkeypatch.delenv("ULMB200_TRACE")
    ulm.reload_env()
    ulm.dgemm("N", "T", 0, 4, 4, 1.0, A, A, 0.0, A)
    assert "ulmb200:" not in capfd.readouterr().err


def test_quick_returns_need_no_device(ulm):
    A = np.ones((4, 4), order="F")
    Cm = np.full((4, 4), 3.0, order="F")
    assert ulm.dgemm("N", "N", 0, 4, 4, 1.0, A, A, 0.0, Cm) == ulm.OK     # m == 0: nothing to do
    assert ulm.dgemm("N", "N", 4, 0, 4, 1.0, A, A, 0.0, Cm) == ulm.OK
    assert np.all(Cm == 3.0)


def test_no_cpu_fallback_without_a_device(ulm):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    A = np.ones((4, 4), order="F")
    Cm = np.full((4, 4), 3.0, order="F")
    st = ulm.dgemm("N", "N", 4, 4, 4, 1.0, A, A, 0.0, Cm)
    assert st == ulm.NO_DEVICE and np.all(Cm == 3.0), "the library computed something without a GPU"
    assert ulm.dsyrk("U", "N", 4, 4, 1.0, A, 0.0, Cm) == ulm.NO_DEVICE
    assert ulm.dtrsm("L", "L", "N", "N", 4, 4, 1.0, A, Cm) == ulm.NO_DEVICE
    assert ulm.launch_count() == 0
    assert ulm.alloc_count() == 0 and ulm.workspace_bytes() == 0
    assert ulm.check_device_error() == ulm.NO_DEVICE


def test_host_generator_is_deterministic_and_blockwise_consistent(ulm):
    a, _ = ulm.fmat(37, 23, 40)
    ulm.host_fill(a, 42, 1)
    b, _ = ulm.fmat(10, 5)
    ulm.host_fill(b, 42, 1, row0=20, col0=11)
    assert np.array_equal(a[20:30, 11:16], b)
    assert a.min() >= -1.0 and a.max() < 1.0 and abs(a.mean()) < 0.1
    c, _ = ulm.fmat(37, 23)
    ulm.host_fill(c, 43, 1)
    assert not np.array_equal(a, c)
    t, _ = ulm.fmat(9, 9)
    ulm.host_fill(t, 3, 0, dist=1, scale=1.0 / 9)
    d = np.diag(t)
    assert d.min() >= 1.0 and d.max() < 2.0 and np.abs(t - np.diag(d)).max() <= 1.0 / 9


def test_layout_model(tmp_path):
    """CPU model of the kernel's shared-memory layout, fragment addressing and MMA lane maps."""
    exe = str(tmp_path / "layout_model")
    subprocess.run(["g++", "-O1", "-std=c++17", "-o", exe, os.path.join(ROOT, "tests", "cpu", "layout_model.cpp")],
                   check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.strip().endswith("OK"), r.stdout
