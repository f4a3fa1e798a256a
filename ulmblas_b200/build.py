"""Builds the libraries in-tree with nvcc for sm_100a (no JIT, no torch extension).

    python -m ulmblas_b200.build [--force] [--verbose]

Every .cu under csrc/ is compiled to an object (in parallel) and linked into
libulmblas_b200.so, the product: the BLAS symbols and the ulmb200_* device ABI
(include/ulmblas_b200.h).  The .cu files under csrc/support/ go into
libulmb200_benchsupport.so (include/ulmb200_benchsupport.h): matrix generator, throughput
probes and failure-path self tests for the bench and the tests, linked against the product.
"""
import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libulmblas_b200.so")
SUPPORT_LIB = os.path.join(HERE, "libulmb200_benchsupport.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=default", "--expt-relaxed-constexpr",
]


def _nvcc():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libulmblas_b200.so cannot be built")
    return nvcc


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def support_sources():
    d = os.path.join(CSRC, "support")
    return sorted(os.path.join("support", f) for f in os.listdir(d) if f.endswith(".cu"))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".h")]
    headers += [os.path.join(CSRC, "support", f) for f in os.listdir(os.path.join(CSRC, "support")) if f.endswith(".h")]
    headers.append(os.path.join(HERE, "..", "include", "ulmblas_b200.h"))
    headers.append(os.path.join(HERE, "..", "include", "ulmb200_benchsupport.h"))
    jobs = []
    objs, sobjs = [], []
    for src in sources() + support_sources():
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        (sobjs if src.startswith("support") else objs).append(o)
        if force or _stale(o, [s] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed on " + cmd[-3])
    arch = ["-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
    links = [(LIB, objs, []),
             (SUPPORT_LIB, sobjs, ["-L" + HERE, "-lulmblas_b200", "-Xlinker", "-rpath=$ORIGIN"])]
    for lib, obs, extra in links:
        if force or jobs or _stale(lib, obs):
            tmp = lib + ".tmp"
            r = subprocess.run([nvcc, "-shared", "-o", tmp] + obs + arch + extra, capture_output=True, text=True)
            if r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
                raise RuntimeError("link failed: " + lib)
            os.replace(tmp, lib)       # a reader never sees a half-written library
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
