#!/usr/bin/env python
"""Headline benchmark: DGEMM GFLOP/s (2mnk/t) on 1/2/4/8 B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Workload (the largest configuration of the reference's path that the metric is quoted on):
C = 1*A*B + 0*C, m = n = 65536, k = 16384, fp64, no transposes, entries uniform[-1,1) from seed
99 (synthetic, generated on the device by the library's counter-based generator).  C and B are
split by column blocks over the ranks, A starts on rank 0 and is broadcast by NCCL inside the
timed region.  One step = one full product.  Strong scaling: the problem is fixed, N varies.

Prints ONE JSON line on rank 0.  `--impl reference` times ulmBLAS's own CPU dgemm_
(oracle/_ref, built from the reference's sources) on a bounded sample of the same product.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED = 99
DRAM_BYTES_PER_FLOP = 67.398e9 / (2.0 * 16384 ** 3)     # measured, see profiles/dgemm_tma_kernel_dram_16384.md
UNIT = "GFLOP/s"
METRIC = "DGEMM GFLOP/s (2mnk/t)"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=65536)
    ap.add_argument("--n", type=int, default=65536)
    ap.add_argument("--k", type=int, default=16384)
    ap.add_argument("--kp", type=int, default=4096, help="K-panel of the A broadcast (N > 1)")
    ap.add_argument("--kp-first", type=int, default=1024, help="short first panel (N > 1)")
    ap.add_argument("--nccl-ctas", type=int, default=8, help="CTAs NCCL may use = SMs the GEMM leaves free")
    ap.add_argument("--reserve-panels", type=int, default=2)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--extra", action="store_true", help="also time 16384^3 on one GPU (N = 1)")
    return ap.parse_args()


def workload_name(a):
    return f"dgemm NN m={a.m} n={a.n} k={a.k} alpha=1 beta=0 seed={SEED}, C/B by column blocks, A broadcast"


# ----------------------------------------------------------------------------------------------
# clocks: sampled with nvidia-smi while the timed region runs (read-only query)
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_ids):
        self.ids = ",".join(str(i) for i in gpu_ids)
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.ids, f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()          # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); pw.append(float(f[3]))
            except ValueError:
                continue
            for nm, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------------
# CPU side: the reference's own dgemm_ on a bounded sample of the workload
# ----------------------------------------------------------------------------------------------
def cpu_reference_sample(a, ms, ns, repeats=1):
    """Times C[0:ms, 0:ns] = A[0:ms, :] * B[:, 0:ns] (full k) with ulmBLAS's dgemm_ on one host
    thread (the library has no threading).  Returns (GFLOP/s, kind, seconds per call)."""
    import numpy as np
    import oracle
    import ulmblas_b200.api as ulm
    if oracle.have_ref(""):
        impl, kind = oracle.Ref(""), "reference"
    else:
        impl, kind = oracle.Port(), "port"
    A, _ = ulm.fmat(ms, a.k); B, _ = ulm.fmat(a.k, ns)
    ulm.host_fill(A, SEED, 0); ulm.host_fill(B, SEED, 1)
    Cm = np.zeros((ms, ns), order="F")
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        impl.dgemm("N", "N", ms, ns, a.k, 1.0, A, B, 0.0, Cm)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return 2.0 * ms * ns * a.k / best * 1e-9, kind, best


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ms, ns = min(a.m, 8192), min(a.n, 128)
    vals = []
    for i in range(a.warmup + a.steps):
        # warm-up steps are kept short: the reference's rate is flat above ~1000^3
        gf, kind, dt = cpu_reference_sample(a, ms if i >= a.warmup else min(ms, 2048), ns)
        if i >= a.warmup:
            vals.append((gf, dt))
    gf = sum(v for v, _ in vals) / len(vals)
    ms_step = 1e3 * sum(d for _, d in vals) / len(vals)
    sample = f"rows 0..{ms - 1} x cols 0..{ns - 1} of C, full k={a.k} ({2.0 * ms * ns * a.k:.3g} flop per step)"
    line = {"impl": "reference", "metric": METRIC, "value": gf, "unit": UNIT, "n_gpus": a.gpus,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": workload_name(a), "sample": sample},
            "cpu_baseline": {"value": gf, "unit": UNIT, "cores": 1, "kind": kind, "sample": sample},
            "e2e": {"value": gf, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# GPU side
# ----------------------------------------------------------------------------------------------
def main():
    a = parse()
    if a.impl == "reference":
        return run_reference(a)

    import numpy as np
    import torch
    import torch.distributed as dist
    import ulmblas_b200.api as ulm
    from ulmblas_b200.sharded import ShardedDgemm, column_block

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200; there is no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # keep NCCL's kernels small: they run beside a GEMM grid that leaves them exactly this room
        os.environ.setdefault("NCCL_MAX_CTAS", str(a.nccl_ctas))
        os.environ.setdefault("NCCL_MIN_CTAS", "1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")   # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=dev)
    if a.gpus != world and rank == 0:
        print(f"note: --gpus {a.gpus} but WORLD_SIZE={world}; using {world}", file=sys.stderr)

    m, n, k = a.m, a.n, a.k
    j0, j1 = column_block(n, world, rank)
    nr = j1 - j0
    A = torch.empty((k, m), dtype=torch.float64, device=dev)        # column-major m x k
    Br = torch.empty((max(nr, 1), k), dtype=torch.float64, device=dev)
    Cr = torch.empty((max(nr, 1), m), dtype=torch.float64, device=dev)
    s0 = torch.cuda.current_stream().cuda_stream
    if rank == 0:
        ulm.dev_fill_f64(A.data_ptr(), m, m, k, SEED, 0, stream=s0)
    else:
        A.zero_()
    ulm.dev_fill_f64(Br.data_ptr(), k, k, nr, SEED, 1, col0=j0, stream=s0)
    ulm.dev_fill_f64(Cr.data_ptr(), m, m, nr, SEED, 2, col0=j0, stream=s0)
    torch.cuda.synchronize()

    # roofline denominator: FP64 tensor-pipe throughput measured on this GPU, register operands only
    peak_tf = None
    if rank == 0:
        peak_tf = max(ulm.peak_probe(2, 4000)[0], ulm.peak_probe(2, 20000)[0])

    eng = ShardedDgemm(m, n, k, kp=a.kp, first=a.kp_first, reserve_sms=a.nccl_ctas,
                       reserve_panels=a.reserve_panels)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        eng.run(1.0, A, Br, 0.0, Cr)   # beta = 0 overwrites C; A reaches ranks > 0 by broadcast each step

    for _ in range(a.warmup):
        step()
    barrier()
    sampler = ClockSampler(range(world)) if rank == 0 else None
    if sampler:
        sampler.start()
    launches0 = ulm.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kev = []
    eng.kernel_events = kev
    e0.record()
    for _ in range(a.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    eng.kernel_events = None
    t_ms = e0.elapsed_time(e1)
    launches = ulm.launch_count() - launches0
    if world > 1:
        tt = torch.tensor([t_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        t_ms = float(tt.item())
        lt = torch.tensor([launches], dtype=torch.int64, device=dev)
        dist.all_reduce(lt, op=dist.ReduceOp.SUM)
        launches = int(lt.item())
    barrier()
    clocks = sampler.stop() if sampler else None
    status = ulm.lib.ulmb200_last_status()

    flops_step = 2.0 * m * n * k
    value = flops_step * a.steps / (t_ms * 1e-3) * 1e-9

    # dominant kernel: average launch duration from CUDA events on the launching stream
    kdur = [s.elapsed_time(e) for (s, e, _) in kev]
    kflops = [f for (_, _, f) in kev]
    ach_tf = (sum(kflops) / (sum(kdur) * 1e-3)) * 1e-12 if kdur else None

    # parity on sampled rows x columns of this rank's block against the CPU oracle
    parity = None
    if nr > 0:
        parity = sampled_parity(ulm, np, torch, m, k, j0, nr, Cr)
    if world > 1:
        pt = torch.tensor([parity if parity is not None else 0.0], dtype=torch.float64, device=dev)
        dist.all_reduce(pt, op=dist.ReduceOp.MAX)
        parity = float(pt.item())

    e2e = None
    if not a.no_e2e:
        e2e = run_e2e(a, ulm, torch, dist, np, rank, world, dev, m, n, k, j0, nr, A, Br, Cr, eng)

    extra = None
    if a.extra and world == 1:
        extra = time_square(ulm, torch, 16384, peak_tf)

    cpu = None
    if rank == 0 and world == 1 and not a.no_cpu:
        gf, kind, dt = cpu_reference_sample(a, min(m, 16384), min(n, 256))
        cpu = {"value": gf, "unit": UNIT, "cores": 1, "kind": kind,
               "sample": f"rows 0..{min(m, 16384) - 1} x cols 0..{min(n, 256) - 1} of C, full k={k}, one call, {dt:.1f} s"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": t_ms / a.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": workload_name(a), "m": m, "n": n, "k": k, "k_panels": [l1 - l0 for (l0, l1) in eng.plan.panels],
                       "parallelism": f"column blocks x{world}", "l2": "operands (>= 8 GB per GPU) exceed L2"},
            "roofline": {"bound": "tensor", "achieved": ach_tf, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": (ach_tf / peak_tf) if (ach_tf and peak_tf) else None,
                         # dram__bytes_read+write of one launch, ncu capture at 16384^3 (67.40 GB for
                         # 8.796 TFLOP, profiles/dgemm_tma_kernel_dram_16384.md) scaled by flops: the
                         # traffic is (waves x panels per wave), proportional to m*n*k
                         "traffic": DRAM_BYTES_PER_FLOP * (sum(kflops) / max(len(kflops), 1)) if kflops else None,
                         "traffic_unit": "bytes per launch (scaled from a smaller ncu capture)",
                         "algorithmic_bytes": 8.0 * (m * k + k * nr + m * nr) if world == 1 else None,
                         "peak_source": "FP64 DMMA (mma.sync m16n8k8.f64) register-only probe run on this GPU "
                                        "just before the timed region; MEASURED_PEAKS.json holds no FP64 figure",
                         "kernel": "dgemm_tma_kernel<128,128>", "launches_timed": len(kdur),
                         "launch_ms_first_step": [round(x, 3) for x in kdur[:len(eng.plan.panels)]]},
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": launches,
            "clocks": clocks,
            "parity": {"max_error_over_bound": parity, "bound": "2*k*eps*(|alpha||A||B|+|beta||C|)",
                       "checked": "64 sampled rows x 64 sampled columns per rank against the CPU oracle"},
            "status": status,
        }
        if extra:
            line["extra"] = extra
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def sampled_parity(ulm, np, torch, m, k, j0, nr, Cr):
    """C[rows, cols] of this rank against ulmBLAS's arithmetic on the same rows of A and columns
    of B, regenerated on the host (every element of C depends only on its own row and column)."""
    from tests.helpers import EPS64, bound_ratio, gemm_gauge
    import oracle
    rng = np.random.default_rng(1234 + j0)
    rows = np.sort(rng.choice(m, min(64, m), replace=False))
    cols = np.sort(rng.choice(nr, min(64, nr), replace=False))
    As = np.empty((len(rows), k), order="F")
    Bs = np.empty((k, len(cols)), order="F")
    for i, r in enumerate(rows):
        ulm.host_fill(As[i:i + 1, :], SEED, 0, row0=int(r))
    for j, c in enumerate(cols):
        ulm.host_fill(Bs[:, j:j + 1], SEED, 1, col0=int(j0 + c))
    want = np.zeros((len(rows), len(cols)), order="F")
    chk = oracle.Ref("") if oracle.have_ref("") else oracle.Port()
    chk.dgemm("N", "N", len(rows), len(cols), k, 1.0, As, Bs, 0.0, want)
    if not np.isfinite(want).all():
        alt = np.zeros_like(want, order="F")
        oracle.Port().dgemm("N", "N", len(rows), len(cols), k, 1.0, As, Bs, 0.0, alt)
        bad = ~np.isfinite(want)
        want[bad] = alt[bad]
    idx_c = torch.from_numpy(cols).to(Cr.device)
    idx_r = torch.from_numpy(rows).to(Cr.device)
    got = Cr[idx_c][:, idx_r].cpu().numpy().T
    return bound_ratio(got, want, gemm_gauge(1.0, As, Bs, 0.0, want), k, EPS64)


def time_square(ulm, torch, sz, peak_tf):
    dA = torch.empty((sz, sz), dtype=torch.float64, device="cuda")
    dB = torch.empty((sz, sz), dtype=torch.float64, device="cuda")
    dC = torch.empty((sz, sz), dtype=torch.float64, device="cuda")
    ulm.dev_fill_f64(dA.data_ptr(), sz, sz, sz, 42, 0)
    ulm.dev_fill_f64(dB.data_ptr(), sz, sz, sz, 42, 1)
    s = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        ulm.dev_dgemm(0, 0, sz, sz, sz, 1.0, dA.data_ptr(), sz, dB.data_ptr(), sz, 0.0, dC.data_ptr(), sz, stream=s)
    torch.cuda.synchronize()
    ts = []
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ulm.dev_dgemm(0, 0, sz, sz, sz, 1.0, dA.data_ptr(), sz, dB.data_ptr(), sz, 0.0, dC.data_ptr(), sz, stream=s)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    tf = 2.0 * sz ** 3 / (statistics.median(ts) * 1e-3) * 1e-12
    return {"workload": f"dgemm NN {sz}^3 device-resident", "ms": statistics.median(ts), "tflops": tf,
            "frac_of_measured_fp64_tensor_peak": tf / peak_tf if peak_tf else None}


def run_e2e(a, ulm, torch, dist, np, rank, world, dev, m, n, k, j0, nr, A, Br, Cr, eng):
    """The same product through the reference-facing entry point with HOST buffers: every step
    copies its inputs host->device from pinned memory and brings C back.  One GPU: the Fortran-ABI
    symbol dgemm_ itself.  Several GPUs: each rank stages its own column block, the root stages A."""
    steps, warm = max(1, min(a.steps, 2)), 1
    try:
        hB = torch.empty((max(nr, 1), k), dtype=torch.float64, pin_memory=True)
        hC = torch.empty((max(nr, 1), m), dtype=torch.float64, pin_memory=True)
        hA = torch.empty((k, m), dtype=torch.float64, pin_memory=True) if rank == 0 else None
    except RuntimeError as exc:
        return {"value": None, "unit": UNIT, "unavailable": f"pinned host allocation failed: {exc}"}
    # columns of this rank's block as the device-resident run left them, to check the e2e result against
    rows = torch.linspace(0, max(nr, 1) - 1, steps=min(max(nr, 1), 48)).long()
    want_rows = Cr[rows.to(dev)].clone() if nr > 0 else None
    hB.copy_(Br); hC.zero_()
    if rank == 0:
        hA.copy_(A)
    torch.cuda.synchronize()
    h2d = (m * k * 8 if rank == 0 else 0) + k * nr * 8
    d2h = m * nr * 8

    def one():
        if world == 1:
            st = ulm.dgemm("N", "N", m, n, k, 1.0, hA.numpy().T, hB.numpy().T, 0.0, hC.numpy().T,
                           lda=m, ldb=k, ldc=m)
            if st != ulm.OK:
                raise RuntimeError(ulm.status_string(st))
        else:
            # host staging inside the sharded call: A panel by panel ahead of its broadcast, this rank's
            # block of B in, its block of C out piece by piece behind the last panel's product
            eng.run(1.0, A, Br, 0.0, Cr, host=(hA, hB, hC))
            torch.cuda.synchronize()

    for _ in range(warm):
        one()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    if world > 1:
        tt = torch.tensor([dt, float(h2d), float(d2h)], dtype=torch.float64, device=dev)
        mx = tt.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(tt, op=dist.ReduceOp.SUM)
        dt, h2d, d2h = float(mx[0].item()), int(tt[1].item()), int(tt[2].item())
    # spot check: the e2e result really is the product.  Cr still holds this rank's block from the
    # device-resident run (same inputs, beta = 0); the two differ only by the order of the K panels.
    ok = bool(torch.isfinite(hC[:4, :4]).all().item())
    if nr > 0:
        diff = float((hC[rows].to(dev) - want_rows).abs().max().item())
        ok = ok and diff <= 2.0 * k * 2.220446049250313e-16 * k      # 2 k eps (|A||B|), |entries| <= 1
    if world > 1:
        okt = torch.tensor([1.0 if ok else 0.0], dtype=torch.float64, device=dev)
        dist.all_reduce(okt, op=dist.ReduceOp.MIN)
        ok = bool(okt.item() > 0.5)
    return {"value": 2.0 * m * n * k * steps / dt * 1e-9, "unit": UNIT, "h2d_bytes_per_step": int(h2d),
            "d2h_bytes_per_step": int(d2h), "steps": steps, "ms_per_step": 1e3 * dt / steps,
            "api": "dgemm_ (Fortran ABI, host pointers)" if world == 1 else "ShardedDgemm.run(host=...) : pinned host buffers, staging pipelined with the panels",
            "timer": "host wall clock around blocking calls (the call returns when C is back in host memory)",
            "finite": ok, "checked": "48 sampled columns per rank equal the device-resident result within 2 k eps |A||B|"}


if __name__ == "__main__":
    main()
