"""Records what the compiled reference reports for every bad-argument case of
tests/xerbla_cases.py into tests/golden/xerbla_codes.json.

    python tests/golden/make_golden_errors.py        (needs oracle/_ref, i.e. the ulmBLAS sources)

The reference's shims are loaded from builds that leave out its own xerbla objects
(oracle/_ref/libulmref_nox.so, libulmref_cblas_nox.so), so their calls to xerbla_ / cblas_xerbla
bind to the recording hook tests/cpu/xerbla_hook.c, loaded first -- the way the reference's testers
link their own XERBLA in front of the library (test/F77/dblat3.f:2768-2809, test/C/c_xerbla.c).
Runs in a child process: the reference computes after reporting.
"""
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

CHILD = r"""
import ctypes as C, json, sys
sys.path.insert(0, %(tests)r); sys.path.insert(0, %(root)r)
hook = C.CDLL(%(hook)r, mode=C.RTLD_GLOBAL)
import oracle, xerbla_cases as X
f77 = C.CDLL(oracle.ref_path("nox")); cb = C.CDLL(oracle.ref_path("cblas_nox"))
cs = X.cases()
got = X.record(hook, lambda r: cb if r.startswith("cblas_") else f77, cs)
print(json.dumps([{"routine": r, "args": list(a), "info": i, "name": n} for (r, a), (i, n) in zip(cs, got)]))
"""


def main():
    sys.path.insert(0, ROOT)
    import oracle
    oracle.build(ref=True)
    with tempfile.TemporaryDirectory() as tmp:
        hook = os.path.join(tmp, "libxerbla_hook.so")
        subprocess.run(["gcc", "-shared", "-fPIC", "-o", hook, os.path.join(ROOT, "tests", "cpu", "xerbla_hook.c")], check=True)
        code = CHILD % dict(tests=os.path.join(ROOT, "tests"), root=ROOT, hook=hook)
        r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
        if r.returncode != 0:
            sys.exit(r.stderr)
    rows = json.loads(r.stdout.strip().splitlines()[-1])
    with open(os.path.join(HERE, "xerbla_codes.json"), "w") as f:
        f.write("[\n" + ",\n".join(json.dumps(x) for x in rows) + "\n]\n")
    flagged = sum(1 for x in rows if x["info"])
    print(f"{len(rows)} cases, {flagged} reported by the reference")


if __name__ == "__main__":
    main()
