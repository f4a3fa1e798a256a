"""Device-resident timings of every routine of the library on one GPU, as a table.

    python -m ulmblas_b200.perf_report [--quick]
    python -m ulmblas_b200.perf_report --modes 4096     # one DGEMM per transposition mode
    python -m ulmblas_b200.perf_report --lu 2048        # two LU factorisations: the run to put under a profiler
    python -m ulmblas_b200.perf_report --c4 8192        # DTRSM LLNN n x n and DSYRK UN n x n/2, twice each
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m ulmblas_b200.perf_report --sharded-trsm 8192  # DTRSM LLNN split over N GPUs

CUDA events on the launching stream, 2 warm-ups, median of 5 (3 for the largest cases).  Rates
are algorithmic flops / time: GEMM 2mnk (complex 8mnk), SYRK n(n+1)k, SYR2K 2n(n+1)k, SYMM 2m^2n, TRSM/TRMM m^2n
(left), LU 2n^3/3.
"""
import statistics
import sys

import torch

from . import api as u


def _time(fn, reps):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


def _buf(rows, cols, dtype, seed, mat, dist=0, scale=1.0):
    t = torch.empty((max(cols, 1), max(rows, 1)), dtype=dtype, device="cuda")
    if dtype == torch.float64:
        u.dev_fill_f64(t.data_ptr(), rows, rows, cols, seed, mat, dist=dist, scale=scale)
    else:
        u.dev_fill_f32(t.data_ptr(), rows, rows, cols, seed, mat)
    return t


def modes(sz):
    """One DGEMM per transposition mode (NN, TN, NT, TT) at sz^3: the run to put under a profiler."""
    s = torch.cuda.current_stream().cuda_stream
    A = _buf(sz, sz, torch.float64, 1, 0); B = _buf(sz, sz, torch.float64, 1, 1); C = _buf(sz, sz, torch.float64, 1, 2)
    for ta, tb in ((0, 0), (1, 0), (0, 1), (1, 1)):
        ms = _time(lambda: u.dev_dgemm(ta, tb, sz, sz, sz, 1.0, A.data_ptr(), sz, B.data_ptr(), sz, 0.0,
                                       C.data_ptr(), sz, stream=s), 1)
        print(f"dgemm {'NT'[ta]}{'NT'[tb]} {sz}^3: {ms:.3f} ms {2.0 * sz ** 3 / ms * 1e-9:.2f} TFLOP/s")


def lu_only(m):
    """Two blocked LU factorisations of an m x m matrix (warm-up + one more), timed with CUDA events."""
    s = torch.cuda.current_stream().cuda_stream
    A0 = _buf(m, m, torch.float64, 5, 0)
    W = A0.clone()
    piv = torch.zeros(m + 1, dtype=torch.int32, device="cuda")
    for it in range(2):
        W.copy_(A0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        u.lib.ulmb200_dgetrf(s, m, m, W.data_ptr(), m, piv.data_ptr(), piv.data_ptr() + 4 * m)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    print(f"dgetrf n={m}: {ms:.3f} ms {2.0 * m ** 3 / 3.0 / ms * 1e-9:.2f} TFLOP/s, info = {int(piv[m].item())}")


def config4(n):
    """DTRSM side=L uplo=L trans=N diag=N (n x n) and DSYRK uplo=U trans=N (n, k = n/2): warm-up + one."""
    s = torch.cuda.current_stream().cuda_stream
    k = n // 2
    T = _buf(n, n, torch.float64, 3, 0, dist=1, scale=1.0 / n)
    B = _buf(n, n, torch.float64, 3, 1)
    A = _buf(n, k, torch.float64, 3, 0)
    C = _buf(n, n, torch.float64, 3, 2)
    for name, flops, fn in (("dtrsm LLNN", float(n) ** 3, lambda: u.dev_dtrsm(0, 1, 0, 0, n, n, 1.0, T.data_ptr(), n, B.data_ptr(), n, stream=s)),
                            ("dsyrk UN", float(n) * (n + 1) * k, lambda: u.dev_dsyrk(0, 0, n, k, 1.0, A.data_ptr(), n, 0.5, C.data_ptr(), n, stream=s))):
        ms = None
        for it in range(2):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
        print(f"{name} n={n}: {ms:.3f} ms {flops / ms * 1e-9:.2f} TFLOP/s")


def sharded_trsm(m):
    """DTRSM left/lower/no-trans/non-unit, m x m, B split by column blocks over the ranks of the
    job; A starts on rank 0 only.  Prints the whole-job rate (m^2 n / max-over-ranks device time)
    and each rank's largest deviation from the one-call solve of its block."""
    import os
    import torch.distributed as dist
    from .sharded import ShardedDtrsm
    os.environ.setdefault("NCCL_MAX_CTAS", "8")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if "RANK" in os.environ:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    op = ShardedDtrsm(False, True, False, False, m, m)
    j0, j1 = op.block
    nr = j1 - j0
    A = torch.zeros((m, m), dtype=torch.float64, device="cuda")
    if rank == 0:
        u.dev_fill_f64(A.data_ptr(), m, m, m, 3, 0, dist=1, scale=1.0 / m)
    B0 = torch.empty((max(nr, 1), m), dtype=torch.float64, device="cuda")
    u.dev_fill_f64(B0.data_ptr(), m, m, nr, 3, 1, col0=j0)
    X = B0.clone()
    ts = []
    for it in range(5):
        X.copy_(B0)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        op.run(1.0, A, X)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if it >= 2:
            ts.append(float(t.item()))
    ref = B0.clone()                                      # A has arrived on every rank by now
    u.dev_dtrsm(0, 1, 0, 0, m, nr, 1.0, A.data_ptr(), m, ref.data_ptr(), m,
                stream=torch.cuda.current_stream().cuda_stream)
    dev = torch.tensor([float((X - ref).abs().max().item()) if nr else 0.0], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(dev, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = statistics.median(ts)
        print(f"dtrsm LLNN m=n={m} on {world} GPU(s): {ms:.3f} ms {float(m) ** 3 / ms * 1e-9:.2f} TFLOP/s "
              f"(whole job, A broadcast inside the timed region), max |X - X_one_call| = {dev.item():.3e}")
    if dist.is_initialized():
        dist.destroy_process_group()


def main():
    if "--sharded-trsm" in sys.argv:
        return sharded_trsm(int(sys.argv[sys.argv.index("--sharded-trsm") + 1]))
    if "--c4" in sys.argv:
        return config4(int(sys.argv[sys.argv.index("--c4") + 1]))
    if "--lu" in sys.argv:
        return lu_only(int(sys.argv[sys.argv.index("--lu") + 1]))
    if "--modes" in sys.argv:
        return modes(int(sys.argv[sys.argv.index("--modes") + 1]))
    quick = "--quick" in sys.argv
    s = torch.cuda.current_stream().cuda_stream
    rows = []
    peaks = {"fp64 dmma": u.peak_probe(2, 20000)[0], "fp32 ffma": u.peak_probe(5, 20000)[0]}

    def add(name, flops, ms, peak):
        rows.append((name, ms, flops / ms * 1e-9, flops / ms * 1e-9 / peaks[peak]))

    for (m, n, k) in [(1024, 1024, 1024), (4096, 4096, 4096), (16384, 16384, 16384)][: 2 if quick else 3]:
        for ta, tb in ((0, 0), (1, 0)) if m > 1024 else ((0, 0),):
            A = _buf(k if ta else m, m if ta else k, torch.float64, 1, 0)
            B = _buf(n if tb else k, k if tb else n, torch.float64, 1, 1)
            C = _buf(m, n, torch.float64, 1, 2)
            ms = _time(lambda: u.dev_dgemm(ta, tb, m, n, k, 1.5, A.data_ptr(), k if ta else m, B.data_ptr(),
                                           n if tb else k, 0.5, C.data_ptr(), m, stream=s), 3 if m > 8192 else 5)
            add(f"dgemm {'T' if ta else 'N'}{'T' if tb else 'N'} {m}x{n}x{k}", 2.0 * m * n * k, ms, "fp64 dmma")
            del A, B, C
    m, n, k = 3001, 2047, 513
    A = _buf(3072, k, torch.float64, 11, 0); B = _buf(640, n, torch.float64, 11, 1); C = _buf(3008, n, torch.float64, 11, 2)
    ms = _time(lambda: u.dev_dgemm(0, 0, m, n, k, -0.7, A.data_ptr(), 3072, B.data_ptr(), 640, 1.3, C.data_ptr(), 3008, stream=s), 5)
    add("dgemm NN 3001x2047x513 (padded ld)", 2.0 * m * n * k, ms, "fp64 dmma")
    zs = 2048 if quick else 4096
    A = _buf(2 * zs, zs, torch.float64, 13, 0); B = _buf(2 * zs, zs, torch.float64, 13, 1); C = _buf(2 * zs, zs, torch.float64, 13, 2)
    for ta, ca, nm in ((0, 0, "NN"), (1, 1, "CN")):
        ms = _time(lambda: u.dev_zgemm(ta, ca, 0, 0, zs, zs, zs, 0.7 - 0.3j, A.data_ptr(), zs, B.data_ptr(), zs, 1.3 + 0.2j,
                                       C.data_ptr(), zs, stream=s), 5)
        add(f"zgemm {nm} {zs}^3 (8mnk flops)", 8.0 * zs ** 3, ms, "fp64 dmma")
    del A, B, C
    for mode, name in ((0, "fp32"), (1, "3xtf32")):
        for sz in (4096,) if quick else (4096, 8192):
            A = _buf(sz, sz, torch.float32, 7, 0); B = _buf(sz, sz, torch.float32, 7, 1); C = _buf(sz, sz, torch.float32, 7, 2)
            ms = _time(lambda: u.dev_sgemm(mode, 1, 0, sz, sz, sz, 1.0, A.data_ptr(), sz, B.data_ptr(), sz, 0.0,
                                           C.data_ptr(), sz, stream=s), 5)
            add(f"sgemm TN {sz}^3 {name}", 2.0 * sz ** 3, ms, "fp32 ffma")
            del A, B, C
    n, k = (4096, 2048) if quick else (8192, 4096)
    A = _buf(n, k, torch.float64, 3, 0); C = _buf(n, n, torch.float64, 3, 2); B = _buf(n, k, torch.float64, 3, 1)
    ms = _time(lambda: u.dev_dsyrk(0, 0, n, k, 1.0, A.data_ptr(), n, 0.5, C.data_ptr(), n, stream=s), 5)
    add(f"dsyrk UN n={n} k={k}", float(n) * (n + 1) * k, ms, "fp64 dmma")
    st = u.lib.ulmb200_dsyr2k(s, 0, 0, n, k, 1.0, A.data_ptr(), n, B.data_ptr(), n, 0.5, C.data_ptr(), n)
    ms = _time(lambda: u.lib.ulmb200_dsyr2k(s, 0, 0, n, k, 1.0, A.data_ptr(), n, B.data_ptr(), n, 0.5, C.data_ptr(), n), 5)
    add(f"dsyr2k UN n={n} k={k}", 2.0 * n * (n + 1) * k, ms, "fp64 dmma")
    del A, B, C
    m = 4096 if quick else 8192
    T = _buf(m, m, torch.float64, 3, 0, dist=1, scale=1.0 / m); B = _buf(m, m, torch.float64, 3, 1); C = _buf(m, m, torch.float64, 3, 2)
    ms = _time(lambda: u.dev_dtrsm(0, 1, 0, 0, m, m, 1.0, T.data_ptr(), m, B.data_ptr(), m, stream=s), 5)
    add(f"dtrsm LLNN m=n={m}", float(m) * m * m, ms, "fp64 dmma")
    ms = _time(lambda: u.lib.ulmb200_dtrmm(s, 0, 1, 0, 0, m, m, 1.0, T.data_ptr(), m, B.data_ptr(), m), 5)
    add(f"dtrmm LLNN m=n={m}", float(m) * m * m, ms, "fp64 dmma")
    ms = _time(lambda: u.lib.ulmb200_dsymm(s, 0, 1, m, m, 1.0, T.data_ptr(), m, B.data_ptr(), m, 0.0, C.data_ptr(), m), 5)
    add(f"dsymm LL m=n={m}", 2.0 * m * m * m, ms, "fp64 dmma")
    piv = torch.zeros(m + 1, dtype=torch.int32, device="cuda")
    A0 = _buf(m, m, torch.float64, 5, 0); W = A0.clone()

    def lu():
        W.copy_(A0)
        u.lib.ulmb200_dgetrf(s, m, m, W.data_ptr(), m, piv.data_ptr(), piv.data_ptr() + 4 * m)
    t_copy = _time(lambda: W.copy_(A0), 5)
    ms = _time(lu, 3) - t_copy
    add(f"dgetrf n={m}", 2.0 * m ** 3 / 3.0, ms, "fp64 dmma")

    print(f"measured peaks: FP64 DMMA {peaks['fp64 dmma']:.2f} TFLOP/s, FP32 FFMA {peaks['fp32 ffma']:.2f} TFLOP/s")
    print(f"{'routine':44s} {'ms':>10s} {'TFLOP/s':>9s} {'of peak':>8s}")
    for name, ms, tf, frac in rows:
        print(f"{name:44s} {ms:10.3f} {tf:9.2f} {frac:8.3f}")


if __name__ == "__main__":
    main()
