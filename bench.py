#!/usr/bin/env python
"""Headline benchmark: DGEMM GFLOP/s (2mnk/t) on 1/2/4/8 B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Workload (the largest configuration of the reference's path that the metric is quoted on):
C = 1*A*B + 0*C, m = n = 65536, k = 16384, fp64, no transposes, entries uniform[-1,1) from seed
99 (synthetic, generated on the device by the counter-based generator).  C and B are split by
column blocks over the ranks, A starts on rank 0 and is broadcast by NCCL inside the timed
region.  One step = one full product.  Strong scaling: the problem is fixed, N varies.

Prints ONE JSON line on rank 0.  On one GPU the line also carries `extra`: every other
configuration of the path (1024^3, SGEMM 4096^3 in both arithmetic modes, the ragged product in
all four transpositions, DTRSM and DSYRK at 8192, DGEMM 16384^3), each timed device-resident
after the headline region and checked against the CPU reference on sampled entries, and the
end-to-end rate of dgemm_ on pageable host memory.

`--impl reference` times ulmBLAS's own CPU dgemm_ (oracle/_ref, built from the reference's
sources) on a bounded sample of the same product.

Tables and single-routine runs (one GPU):
    python bench.py --report [--quick]      every routine, device-resident
    python bench.py --modes 4096            one DGEMM per transposition mode
    python bench.py --small                 DGEMM on small and ragged shapes
    python bench.py --sgemm 4096            SGEMM TN in both arithmetic modes
    python bench.py --lu 2048               two LU factorisations
    python bench.py --c4 8192               DTRSM LLNN n x n and DSYRK UN n x n/2, twice each
    torchrun ... bench.py --sharded-trsm 8192   DTRSM LLNN split over the ranks
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
# dram__bytes_read + dram__bytes_write of one 16384^3 launch under ncu: 69.16 GB for 8.796 TFLOP.
# The traffic is (waves x operand panels per wave), proportional to m*n*k, so it scales by flops.
DRAM_BYTES_PER_FLOP = 69.16e9 / (2.0 * 16384 ** 3)
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
    ap.add_argument("--kp", type=int, default=4096, help="largest K-panel of the A broadcast (N > 1)")
    ap.add_argument("--kp-first", type=int, default=1024, help="first K-panel (N > 1); panels double from here up to --kp")
    ap.add_argument("--nccl-ctas", type=int, default=8, help="CTAs NCCL may use = SMs the GEMM leaves free while panels travel")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the other configurations (N = 1)")
    ap.add_argument("--report", action="store_true")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--modes", type=int)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--sgemm", type=int)
    ap.add_argument("--lu", type=int)
    ap.add_argument("--c4", type=int)
    ap.add_argument("--sharded-trsm", type=int)
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
# CPU side: the reference's own routines (oracle/ is the checker and the CPU baseline; nothing of
# the product is loaded here -- inputs come from the numpy twin of the generator)
# ----------------------------------------------------------------------------------------------
def checker():
    import oracle
    if oracle.have_ref(""):
        return oracle.Ref(""), "reference"
    return oracle.Port(), "port"


def finite_or_port(want, redo):
    """The reference's SSE build can emit NaN on finite inputs (an uninitialised stack tile in its
    buffered micro-kernel); such entries take the value of the bit-identical C restatement."""
    import numpy as np
    import oracle
    if not np.isfinite(want).all():
        alt = redo(oracle.Port())
        bad = ~np.isfinite(want)
        want[bad] = alt[bad]
    return want


def cpu_reference_sample(a, ms, ns, repeats=1):
    """Times C[0:ms, 0:ns] = A[0:ms, :] * B[:, 0:ns] (full k) with ulmBLAS's dgemm_ on one host
    thread (the library has no threading).  Returns (GFLOP/s, kind, seconds per call)."""
    import numpy as np
    from oracle.inputs import gen_uniform
    impl, kind = checker()
    A = gen_uniform(SEED, 0, ms, a.k)
    B = gen_uniform(SEED, 1, a.k, ns)
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
    if a.report or a.modes or a.small or a.sgemm or a.lu or a.c4 or a.sharded_trsm:
        return tables(a)

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
    # (every rank probes its own GPU; rank 0's figure is the line's roofline.peak)
    peak_tf = max(ulm.peak_probe(2, 4000)[0], ulm.peak_probe(2, 20000)[0])

    eng = ShardedDgemm(m, n, k, first=a.kp_first, reserve_sms=a.nccl_ctas)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        eng.run(1.0, A, Br, 0.0, Cr)   # beta = 0 overwrites C; A reaches ranks > 0 by broadcast each step

    for _ in range(a.warmup):
        step()
    # the sampler's child process is started before the barrier: forking a process with a CUDA context takes
    # rank 0 (the root of every broadcast) some 20 ms, which the other ranks would spend inside their timed region
    sampler = ClockSampler(range(world)) if rank == 0 else None
    if sampler:
        sampler.start()
    barrier()
    launches0 = ulm.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    eng.profile(True)            # CUDA events around every product, on the stream it is launched on
    e0.record()
    for _ in range(a.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    eng.profile(False)
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
    status = ulm.check_device_error()

    flops_step = 2.0 * m * n * k
    value = flops_step * a.steps / (t_ms * 1e-3) * 1e-9

    # dominant kernel: launch durations of the last timed step, from the library's CUDA events on
    # the launching (compute) stream; one launch per K panel
    widths, reserve, rate_dev, _ = eng.last_plan()
    kdur = eng.last_gemm_ms()
    kflops = [2.0 * m * nr * w for w in widths][:len(kdur)]
    ach_tf = (sum(kflops) / (sum(kdur) * 1e-3)) * 1e-12 if kdur and sum(kdur) > 0 else None
    # every rank's kernel time and pipe probe: the step ends with the slowest GPU
    rank_ms, rank_peak = [round(sum(kdur), 3)], [round(peak_tf, 2) if peak_tf else None]
    rank_start, rank_gap = None, None
    if world > 1:
        starts = eng.last_gemm_start_ms()
        gap = eng.last_step_gap_ms() if a.steps > 1 else None
        both = torch.tensor([sum(kdur), peak_tf or 0.0, starts[0] if starts else -1.0, gap if gap is not None else -1.0],
                            dtype=torch.float64, device=dev)
        gathered = [torch.zeros_like(both) for _ in range(world)]
        dist.all_gather(gathered, both)
        rank_ms = [round(float(g[0].item()), 3) for g in gathered]
        rank_peak = [round(float(g[1].item()), 2) for g in gathered]
        # where a step's time goes besides the kernels: the wait for the first panel, and the time between the end
        # of a rank's last product and the start of the next step's transfers (all ranks must have finished)
        rank_start = [round(float(g[2].item()), 3) for g in gathered]
        rank_gap = [round(float(g[3].item()), 3) for g in gathered]

    # parity on sampled rows x columns of this rank's block against the CPU oracle
    parity = None
    if nr > 0:
        parity = sampled_parity(np, torch, m, k, j0, nr, Cr)
    if world > 1:
        pt = torch.tensor([parity if parity is not None else 0.0], dtype=torch.float64, device=dev)
        dist.all_reduce(pt, op=dist.ReduceOp.MAX)
        parity = float(pt.item())

    e2e = None
    if not a.no_e2e:
        e2e = run_e2e(a, ulm, torch, dist, np, rank, world, dev, m, n, k, j0, nr, A, Br, Cr, eng)

    del A, Br, Cr
    torch.cuda.empty_cache()
    extra = None
    if world == 1 and not a.no_extra:
        ulm.release_workspace()                      # the end-to-end call left ~50 GB of staging buffers
        extra = other_configurations(ulm, torch, np, peak_tf)

    cpu = None
    if rank == 0 and world == 1 and not a.no_cpu:
        gf, kind, dt = cpu_reference_sample(a, min(m, 16384), min(n, 256))
        cpu = {"value": gf, "unit": UNIT, "cores": 1, "kind": kind,
               "sample": f"rows 0..{min(m, 16384) - 1} x cols 0..{min(n, 256) - 1} of C, full k={k}, one call, {dt:.1f} s"}

    if rank == 0:
        npan = max(len(widths), 1)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": t_ms / a.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": workload_name(a), "m": m, "n": n, "k": k, "k_panels": widths,
                       "panels_leaving_sms_to_nccl": reserve, "measured_transport_gbs": round(rate_dev, 1),
                       "parallelism": f"column blocks x{world}", "l2": "operands (>= 8 GB per GPU) exceed L2",
                       "api": "ulmb200_mg_dgemm (C ABI)"},
            "roofline": {"bound": "tensor", "achieved": ach_tf, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": (ach_tf / peak_tf) if (ach_tf and peak_tf) else None,
                         "traffic": DRAM_BYTES_PER_FLOP * (sum(kflops) / max(len(kflops), 1)) if kflops else None,
                         "traffic_unit": "bytes per launch (scaled by flops from an ncu capture of a 16384^3 launch)",
                         # what one rank's launches of one step must read and write: all of A, its blocks of B and C
                         "algorithmic_bytes": 8.0 * (m * k + k * nr + m * nr) / max(npan, 1),
                         "algorithmic_bytes_unit": f"bytes per launch on rank 0 ({npan} launch(es) per step)",
                         "peak_source": "FP64 DMMA (mma.sync m16n8k8.f64) register-only probe run on this GPU "
                                        "just before the timed region; MEASURED_PEAKS.json holds no FP64 figure",
                         "kernel": "dgemm_tma_kernel<128,128>", "launches_timed": len(kdur),
                         "launch_ms_last_step": [round(x, 3) for x in kdur],
                         "launch_start_ms_last_step": [round(x, 3) for x in eng.last_gemm_start_ms()] if world > 1 else None,
                         "kernel_ms_last_step_by_rank": rank_ms, "peak_by_rank": rank_peak,
                         "first_launch_start_ms_by_rank": rank_start, "ms_between_steps_by_rank": rank_gap},
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


def sampled_parity(np, torch, m, k, j0, nr, Cr, seed=SEED, alpha=1.0):
    """C[rows, cols] of this rank against ulmBLAS's arithmetic on the same rows of A and columns
    of B, regenerated on the host (every element of C depends only on its own row and column)."""
    from oracle.inputs import EPS64, bound_ratio, gemm_gauge, gen_uniform
    rng = np.random.default_rng(1234 + j0)
    rows = np.sort(rng.choice(m, min(64, m), replace=False))
    cols = np.sort(rng.choice(nr, min(64, nr), replace=False))
    As = np.empty((len(rows), k), order="F")
    Bs = np.empty((k, len(cols)), order="F")
    for i, r in enumerate(rows):
        As[i:i + 1, :] = gen_uniform(seed, 0, 1, k, row0=int(r))
    for j, c in enumerate(cols):
        Bs[:, j:j + 1] = gen_uniform(seed, 1, k, 1, col0=int(j0 + c))
    want = np.zeros((len(rows), len(cols)), order="F")
    chk, _ = checker()
    chk.dgemm("N", "N", len(rows), len(cols), k, alpha, As, Bs, 0.0, want)

    def redo(P):
        alt = np.zeros_like(want, order="F")
        P.dgemm("N", "N", len(rows), len(cols), k, alpha, As, Bs, 0.0, alt)
        return alt
    want = finite_or_port(want, redo)
    idx_c = torch.from_numpy(cols).to(Cr.device)
    idx_r = torch.from_numpy(rows).to(Cr.device)
    got = Cr[idx_c][:, idx_r].cpu().numpy().T
    return bound_ratio(got, want, gemm_gauge(alpha, As, Bs, 0.0, want), k, EPS64)


# ----------------------------------------------------------------------------------------------
# the other configurations of the path, one GPU, device-resident (CUDA events, L2 flushed between
# repeats of the small ones by a 256 MB fill)
# ----------------------------------------------------------------------------------------------
class Dev:
    """Column-major device matrices filled by the generator, and event timing."""

    def __init__(self, ulm, torch):
        self.ulm, self.torch = ulm, torch
        self.s = torch.cuda.current_stream().cuda_stream
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")     # 2 x L2

    def buf(self, rows, cols, dtype, seed, mat, ld=None, dist=0, scale=1.0, row0=0, col0=0):
        torch, u = self.torch, self.ulm
        ld = ld or max(rows, 1)
        t = torch.empty((max(cols, 1), ld), dtype=dtype, device="cuda")
        if ld != rows:
            t.fill_(-1e10)
        if dtype == torch.float64:
            u.dev_fill_f64(t.data_ptr(), ld, rows, cols, seed, mat, row0=row0, col0=col0, dist=dist, scale=scale)
        else:
            u.dev_fill_f32(t.data_ptr(), ld, rows, cols, seed, mat, row0=row0, col0=col0)
        return t

    def time(self, fn, reps=5, warm=3, flush=True, setup=None):
        torch = self.torch
        for _ in range(warm):
            if setup:
                setup()
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            if setup:
                setup()
            if flush:
                self.flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)


def normal_matrix(np, seed, rows, cols):
    return np.asfortranarray(np.random.default_rng(seed).standard_normal((rows, cols)))


def other_configurations(ulm, torch, np, peak64):
    from oracle.inputs import EPS32, EPS64, bound_ratio, gemm_gauge, gen_uniform
    D = Dev(ulm, torch)
    s = D.s
    chk, kind = checker()
    peak32 = max(ulm.peak_probe(5, 20000)[0], ulm.peak_probe(7, 20000)[0])
    out = []

    def row(name, flops, ms, peak, parity, note=None):
        tf = flops / ms * 1e-9
        r = {"workload": name, "ms": round(ms, 4), "tflops": round(tf, 3), "frac": round(tf / peak, 4),
             "peak_tflops": round(peak, 2), "parity_max_error_over_bound": parity}
        if note:
            r["note"] = note
        out.append(r)

    f64, f32 = torch.float64, torch.float32
    # --- config 1: DGEMM 1024^3, alpha 1.5 beta 0.5, seed 42 (full comparison) ---------------
    m = n = k = 1024
    A, B, C0 = D.buf(m, k, f64, 42, 0), D.buf(k, n, f64, 42, 1), D.buf(m, n, f64, 42, 2)
    C = C0.clone()
    call = lambda: ulm.dev_dgemm(0, 0, m, n, k, 1.5, A.data_ptr(), m, B.data_ptr(), k, 0.5, C.data_ptr(), m, stream=s)  # noqa: E731
    C.copy_(C0); call(); torch.cuda.synchronize()
    hA, hB, hC = gen_uniform(42, 0, m, k), gen_uniform(42, 1, k, n), gen_uniform(42, 2, m, n)
    want = hC.copy(order="F")
    chk.dgemm("N", "N", m, n, k, 1.5, hA, hB, 0.5, want)

    def redo1(P):
        alt = hC.copy(order="F")
        P.dgemm("N", "N", m, n, k, 1.5, hA, hB, 0.5, alt)
        return alt
    want = finite_or_port(want, redo1)
    par = bound_ratio(C.cpu().numpy().T, want, gemm_gauge(1.5, hA, hB, 0.5, hC), k, EPS64)
    row("config 1: dgemm NN 1024^3 alpha=1.5 beta=0.5 seed 42", 2.0 * m * n * k, D.time(call), peak64, par)
    del A, B, C, C0

    # --- config 2: SGEMM 4096^3 TN, alpha 1 beta 0, seed 7, both arithmetic modes -------------
    m = n = k = 4096
    A, B, C = D.buf(k, m, f32, 7, 0), D.buf(k, n, f32, 7, 1), torch.zeros((n, m), dtype=f32, device="cuda")
    cols = np.sort(np.random.default_rng(0).choice(n, 128, replace=False))
    hA = gen_uniform(7, 0, k, m, dtype=np.float32)
    hBs = np.asfortranarray(np.concatenate([gen_uniform(7, 1, k, 1, col0=int(c), dtype=np.float32) for c in cols], axis=1))
    want = np.zeros((m, len(cols)), np.float32, order="F")
    chk.sgemm("T", "N", m, len(cols), k, 1.0, hA, hBs, 0.0, want)

    def redo2(P):
        alt = np.zeros((m, len(cols)), np.float32, order="F")
        P.sgemm("T", "N", m, len(cols), k, 1.0, hA, hBs, 0.0, alt)
        return alt
    want = finite_or_port(want, redo2)
    gauge = gemm_gauge(1.0, hA.T, hBs, 0.0, want)
    for mode, name in ((0, "FP32 FMA"), (1, "3xTF32 tcgen05")):
        call = lambda: ulm.dev_sgemm(mode, 1, 0, m, n, k, 1.0, A.data_ptr(), k, B.data_ptr(), k, 0.0, C.data_ptr(), m, stream=s)  # noqa: E731
        ms = D.time(call)
        got = C[torch.from_numpy(cols).cuda()].cpu().numpy().T
        row(f"config 2: sgemm TN 4096^3 alpha=1 beta=0 seed 7, {name}", 2.0 * m * n * k, ms, peak32,
            bound_ratio(got, want, gauge, k, EPS32), "frac is of the FP32 FMA pipe probe; 128 sampled columns checked")
    del A, B, C

    # --- config 3: DGEMM 3001 x 2047 x 513, padded ld, alpha -0.7 beta 1.3, normal(0,1) seed 11 --
    m, n, k = 3001, 2047, 513
    for ta, tb in ((0, 0), (0, 1), (1, 0), (1, 1)):
        ra, ca = (k, m) if ta else (m, k)
        rb, cb = (n, k) if tb else (k, n)
        lda, ldb, ldc = 3072, (2048 if tb else 640), 3008
        hA, hB, hC = normal_matrix(np, 11, ra, ca), normal_matrix(np, 12, rb, cb), normal_matrix(np, 13, m, n)

        def padded(h, ld):
            t = torch.full((h.shape[1], ld), -1e10, dtype=f64, device="cuda")
            t[:, :h.shape[0]] = torch.from_numpy(np.ascontiguousarray(h.T)).cuda()
            return t
        A, B, C0 = padded(hA, lda), padded(hB, ldb), padded(hC, ldc)
        C = C0.clone()
        call = lambda: ulm.dev_dgemm(ta, tb, m, n, k, -0.7, A.data_ptr(), lda, B.data_ptr(), ldb, 1.3, C.data_ptr(), ldc, stream=s)  # noqa: E731
        call(); torch.cuda.synchronize()
        got = C.cpu().numpy().T
        pad_ok = bool((got[m:, :] == -1e10).all())
        cols = np.sort(np.random.default_rng(3).choice(n, 256, replace=False))
        Bs = np.asfortranarray(hB[cols, :] if tb else hB[:, cols])
        Cs = np.asfortranarray(hC[:, cols])
        want = Cs.copy(order="F")
        chk.dgemm("NT"[ta], "NT"[tb], m, len(cols), k, -0.7, hA, Bs, 1.3, want)

        def redo3(P):
            alt = Cs.copy(order="F")
            P.dgemm("NT"[ta], "NT"[tb], m, len(cols), k, -0.7, hA, Bs, 1.3, alt)
            return alt
        want = finite_or_port(want, redo3)
        oa, ob = (hA.T if ta else hA), (Bs.T if tb else Bs)
        par = bound_ratio(got[:m, cols], want, gemm_gauge(-0.7, oa, ob, 1.3, Cs), k, EPS64)
        ms = D.time(call)
        row(f"config 3: dgemm {'NT'[ta]}{'NT'[tb]} 3001x2047x513 ld {lda}/{ldb}/{ldc} alpha=-0.7 beta=1.3 seed 11",
            2.0 * m * n * k, ms, peak64, par if pad_ok else float("inf"), "256 sampled columns checked; padding rows untouched")
        del A, B, C, C0

    # --- config 4: DTRSM LLNN 8192^2 and DSYRK UN 8192 x 4096, seed 3 -------------------------
    m = n = 8192
    T = D.buf(m, m, f64, 3, 0, dist=1, scale=1.0 / m)
    upper = torch.triu(torch.ones((m, m), dtype=torch.bool, device="cuda"), 1).T
    T[upper] = -1e10                                     # the unreferenced triangle must not be read
    del upper
    B0 = D.buf(m, n, f64, 3, 1)
    X = B0.clone()
    call = lambda: ulm.dev_dtrsm(0, 1, 0, 0, m, n, 1.0, T.data_ptr(), m, X.data_ptr(), m, stream=s)  # noqa: E731
    ms = D.time(call, reps=3, warm=2, flush=False, setup=lambda: X.copy_(B0))
    cols = np.sort(np.random.default_rng(1).choice(n, 32, replace=False))
    hT = gen_uniform(3, 0, m, m, dist=1, scale=1.0 / m)
    hB = np.asfortranarray(np.concatenate([gen_uniform(3, 1, m, 1, col0=int(c)) for c in cols], axis=1))
    want = hB.copy(order="F")
    chk.dtrsm("L", "L", "N", "N", m, len(cols), 1.0, hT, want)

    def redo4(P):
        alt = hB.copy(order="F")
        P.dtrsm("L", "L", "N", "N", m, len(cols), 1.0, hT, alt)
        return alt
    want = finite_or_port(want, redo4)
    got = X[torch.from_numpy(cols).cuda()].cpu().numpy().T
    L = np.tril(hT)
    resid = bound_ratio(L @ got, hB, np.abs(L) @ np.abs(got) + np.abs(hB), m, EPS64)
    direct = float(np.abs(got - want).max())
    row("config 4: dtrsm LLNN m=n=8192 seed 3", float(m) * m * n, ms, peak64, resid,
        f"multiply-back bound 2 m eps (|A||X| + |B|) on 32 sampled columns; max |X - X_ref| = {direct:.2e}")
    del T, B0, X, hT
    n, k = 8192, 4096
    A, C0 = D.buf(n, k, f64, 3, 0), D.buf(n, n, f64, 3, 2)
    C = C0.clone()
    call = lambda: ulm.dev_dsyrk(0, 0, n, k, 1.0, A.data_ptr(), n, 0.5, C.data_ptr(), n, stream=s)  # noqa: E731
    C.copy_(C0); call(); torch.cuda.synchronize()
    low = torch.tril(torch.ones((n, n), dtype=torch.bool, device="cuda"), -1).T
    tri_ok = bool(torch.equal(C[low], C0[low]))
    del low
    nb, par = 256, 0.0
    for (bi, bj) in [(0, 0), (31, 31), (0, 31), (5, 17)]:
        Ai, Aj = gen_uniform(3, 0, nb, k, row0=bi * nb), gen_uniform(3, 0, nb, k, row0=bj * nb)
        Cij = gen_uniform(3, 2, nb, nb, row0=bi * nb, col0=bj * nb)
        want = Cij.copy(order="F")
        if bi == bj:
            chk.dsyrk("U", "N", nb, k, 1.0, Ai, 0.5, want)
        else:
            chk.dgemm("N", "T", nb, nb, k, 1.0, Ai, Aj, 0.5, want)

        def redo5(P):
            alt = Cij.copy(order="F")
            if bi == bj:
                P.dsyrk("U", "N", nb, k, 1.0, Ai, 0.5, alt)
            else:
                P.dgemm("N", "T", nb, nb, k, 1.0, Ai, Aj, 0.5, alt)
            return alt
        want = finite_or_port(want, redo5)
        got = C[bj * nb:(bj + 1) * nb, bi * nb:(bi + 1) * nb].cpu().numpy().T
        mask = np.triu(np.ones((nb, nb), bool)) if bi == bj else np.ones((nb, nb), bool)
        par = max(par, bound_ratio(np.where(mask, got, 0), np.where(mask, want, 0), gemm_gauge(1.0, Ai, Aj.T, 0.5, Cij), k, EPS64))
    ms = D.time(call, reps=3, warm=2, flush=False)
    row("config 4: dsyrk UN n=8192 k=4096 alpha=1 beta=0.5 seed 3", float(n) * (n + 1) * k, ms, peak64,
        par if tri_ok else float("inf"), "diagonal and off-diagonal 256-blocks checked; strictly lower triangle untouched")
    del A, C, C0

    # --- the one-GPU target shape: DGEMM 16384^3 ------------------------------------------------
    sz = 16384
    A, B, C = D.buf(sz, sz, f64, 42, 0), D.buf(sz, sz, f64, 42, 1), torch.empty((sz, sz), dtype=f64, device="cuda")
    call = lambda: ulm.dev_dgemm(0, 0, sz, sz, sz, 1.0, A.data_ptr(), sz, B.data_ptr(), sz, 0.0, C.data_ptr(), sz, stream=s)  # noqa: E731
    ms = D.time(call, reps=3, warm=2, flush=False)
    par = sampled_parity(np, torch, sz, sz, 0, sz, C, seed=42)
    row("dgemm NN 16384^3 alpha=1 beta=0 seed 42", 2.0 * sz ** 3, ms, peak64, par, "64 x 64 sampled entries checked")

    # --- the same product through dgemm_ with pageable host memory (what a caller of the reference
    # hands over: plain malloc'ed arrays), with and without page-locking them for the call
    e2e = []
    try:
        hA, hB, hC = np.empty((sz, sz), order="F"), np.empty((sz, sz), order="F"), np.zeros((sz, sz), order="F")
        hA[...] = A.cpu().numpy().T
        hB[...] = B.cpu().numpy().T
        want_cols = C[:8].cpu().numpy().T
        del A, B, C
        torch.cuda.empty_cache()
        for pin in (0, 1):
            ulm.lib.ulmb200_set_pin_host(pin)
            ts = []
            for it in range(2):
                hC[:, :8] = 0.0
                t0 = time.perf_counter()
                st = ulm.dgemm("N", "N", sz, sz, sz, 1.0, hA, hB, 0.0, hC)
                ts.append(time.perf_counter() - t0)
                if st != ulm.OK:
                    raise RuntimeError(ulm.status_string(st))
            ok = bool(np.abs(hC[:, :8] - want_cols).max() <= 2.0 * sz * EPS64 * sz)
            e2e.append({"workload": f"dgemm_ 16384^3, pageable host arrays, ulmb200_set_pin_host({pin})",
                        "ms": round(1e3 * ts[-1], 2), "tflops": round(2.0 * sz ** 3 / ts[-1] * 1e-12, 3),
                        "h2d_bytes": 2 * 8 * sz * sz, "d2h_bytes": 8 * sz * sz, "result_checked": ok,
                        "timer": "host wall clock around the blocking call, second of two calls"})
        ulm.lib.ulmb200_set_pin_host(0)
        ulm.release_workspace()
    except (MemoryError, RuntimeError) as exc:
        e2e.append({"workload": "dgemm_ 16384^3 pageable", "unavailable": str(exc)})
    try:
        e2e.append(config1_e2e(ulm, np))
    except Exception as exc:      # noqa: BLE001 - an extra figure must not take the bench line down
        e2e.append({"workload": "dgemm_ 1024^3 pageable", "unavailable": str(exc)})
    return {"device_resident": out, "e2e_pageable": e2e, "checker": kind,
            "fp32_fma_peak_tflops": round(peak32, 2)}


def config1_e2e(ulm, np):
    """dgemm_ on config 1's shape with plain (pageable) host arrays: what a caller of the reference sees for a
    small product, copies and launch included.  Best of five blocking calls, result checked in full."""
    from oracle.inputs import EPS64
    n = 1024
    rng = np.random.default_rng(42)
    A, B, C0 = (np.asfortranarray(rng.uniform(-1.0, 1.0, (n, n))) for _ in range(3))
    want = 1.5 * (A @ B) + 0.5 * C0
    gauge = 1.5 * (np.abs(A) @ np.abs(B)) + 0.5 * np.abs(C0)
    ts, ok = [], True
    for _ in range(6):
        Cm = C0.copy(order="F")
        t0 = time.perf_counter()
        st = ulm.dgemm("N", "N", n, n, n, 1.5, A, B, 0.5, Cm)
        ts.append(time.perf_counter() - t0)
        if st != ulm.OK:
            raise RuntimeError(ulm.status_string(st))
        ok = ok and bool((np.abs(Cm - want) <= 2.0 * n * EPS64 * gauge).all())
    best = min(ts[1:])
    return {"workload": "dgemm_ 1024^3 (config 1 shape) alpha=1.5 beta=0.5, pageable host arrays, ulmb200_set_pin_host(0)",
            "ms": round(1e3 * best, 3), "tflops": round(2.0 * n ** 3 / best * 1e-12, 3),
            "h2d_bytes": 3 * 8 * n * n, "d2h_bytes": 8 * n * n, "result_checked": ok,
            "timer": "host wall clock around the blocking call, best of five after one warm-up"}


class SharedHostMatrix:
    """rows x cols float64 in a shared-memory file that every rank of the box maps and page-locks."""

    def __init__(self, torch, np, dist, rank, rows, cols):
        self.ok, self.tensor, self.path, self.ptr, self.torch, self.rank = False, None, None, None, torch, rank
        box = [f"/dev/shm/ulmb200_bench_{os.getpid()}.bin" if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        self.path = box[0]
        good = 1.0
        try:
            if rank == 0:
                with open(self.path, "wb") as f:
                    f.truncate(rows * cols * 8)
            dist.barrier()
            self.map = np.memmap(self.path, dtype=np.float64, mode="r+", shape=(rows, cols))
            self.tensor = torch.from_numpy(self.map)
            self.ptr = self.tensor.data_ptr()
            if rank == 0:
                self.map[...] = 0.0                 # touch every page before it is locked
            dist.barrier()
            rc = torch.cuda.cudart().cudaHostRegister(self.ptr, rows * cols * 8, 0)
            if int(rc) != 0:
                self.ptr, good = None, 0.0
        except (OSError, RuntimeError, ValueError):
            good = 0.0
        t = torch.tensor([good], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        self.ok = bool(t.item() > 0.5)
        if not self.ok:
            self.close()

    def close(self):
        torch = self.torch
        if self.ptr is not None:
            torch.cuda.synchronize()
            torch.cuda.cudart().cudaHostUnregister(self.ptr)
            self.ptr = None
        self.tensor = None
        if self.rank == 0 and self.path and os.path.exists(self.path):
            os.remove(self.path)


def run_e2e(a, ulm, torch, dist, np, rank, world, dev, m, n, k, j0, nr, A, Br, Cr, eng):
    """The same product through the reference-facing entry point with HOST buffers: every step
    copies its inputs host->device from pinned memory and brings C back.  One GPU: the Fortran-ABI
    symbol dgemm_ itself.  Several GPUs: each rank stages its own column block, the root stages A
    (the reference has no entry point that spans devices; ShardedDgemm is this library's)."""
    steps, warm = max(1, min(a.steps, 2)), (1 if world == 1 else 2)
    shared = None
    try:
        hB = torch.empty((max(nr, 1), k), dtype=torch.float64, pin_memory=True)
        hC = torch.empty((max(nr, 1), m), dtype=torch.float64, pin_memory=True)
        if world > 1:
            # A in one page-locked host segment that every rank maps: each rank can then bring its share
            # of every panel over its own PCIe link
            shared = SharedHostMatrix(torch, np, dist, rank, k, m)
        hA = shared.tensor if (shared and shared.ok) else (torch.empty((k, m), dtype=torch.float64, pin_memory=True) if rank == 0 else None)
    except RuntimeError as exc:
        return {"value": None, "unit": UNIT, "unavailable": f"pinned host allocation failed: {exc}"}
    every = bool(shared and shared.ok)
    # columns of this rank's block as the device-resident run left them, to check the e2e result against
    rows = torch.linspace(0, max(nr, 1) - 1, steps=min(max(nr, 1), 48)).long()
    want_rows = Cr[rows.to(dev)].clone() if nr > 0 else None
    hB.copy_(Br); hC.zero_()
    if rank == 0:
        hA.copy_(A)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
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
            eng.run(1.0, A, Br, 0.0, Cr, host=(hA, hB, hC), every_rank_has_a=every)
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
    plan = eng.last_plan() if world > 1 else None
    if shared:
        shared.close()
    return {"value": 2.0 * m * n * k * steps / dt * 1e-9, "unit": UNIT, "h2d_bytes_per_step": int(h2d),
            "d2h_bytes_per_step": int(d2h), "steps": steps, "ms_per_step": 1e3 * dt / steps,
            "api": ("dgemm_ (Fortran ABI) on page-locked host arrays (cudaHostAlloc); the pageable case is in extra.e2e_pageable"
                    if world == 1 else
                    "ulmb200_mg_dgemm_host (C ABI) on page-locked host buffers, staging pipelined with the panels; "
                    + ("A in a host segment every rank maps, each rank bringing its share of a panel over its own PCIe link"
                       if every else "A pushed by the root alone")
                    + " (no entry point of the reference spans devices)"),
            "k_panels": plan[0] if plan else None, "measured_transport_gbs": round(plan[3], 1) if plan else None,
            "timer": "host wall clock around blocking calls (the call returns when C is back in host memory)",
            "finite": ok, "checked": "48 sampled columns per rank equal the device-resident result within 2 k eps |A||B|"}


# ----------------------------------------------------------------------------------------------
# tables and single-routine runs
# ----------------------------------------------------------------------------------------------
def tables(a):
    import torch
    import ulmblas_b200.api as u
    if a.sharded_trsm:
        return sharded_trsm(a.sharded_trsm, torch, u)
    D = Dev(u, torch)
    s = D.s
    f64, f32 = torch.float64, torch.float32
    peak64 = max(u.peak_probe(2, 20000)[0], u.peak_probe(2, 4000)[0])
    peak32 = max(u.peak_probe(5, 20000)[0], u.peak_probe(7, 20000)[0])
    rows = []

    def add(name, flops, ms, peak):
        rows.append((name, ms, flops / ms * 1e-9, flops / ms * 1e-9 / peak))

    def show():
        print(f"measured peaks: FP64 DMMA {peak64:.2f} TFLOP/s, FP32 FMA {peak32:.2f} TFLOP/s")
        print(f"{'routine':52s} {'ms':>10s} {'TFLOP/s':>9s} {'of peak':>8s}")
        for name, ms, tf, frac in rows:
            print(f"{name:52s} {ms:10.4f} {tf:9.2f} {frac:8.3f}")

    def dgemm_row(ta, tb, m, n, k, lda=None, ldb=None, ldc=None, alpha=1.5, beta=0.5, reps=5, tag=""):
        ra, ca = (k, m) if ta else (m, k)
        rb, cb = (n, k) if tb else (k, n)
        A, B, C = D.buf(ra, ca, f64, 1, 0, ld=lda), D.buf(rb, cb, f64, 1, 1, ld=ldb), D.buf(m, n, f64, 1, 2, ld=ldc)
        ms = D.time(lambda: u.dev_dgemm(ta, tb, m, n, k, alpha, A.data_ptr(), lda or ra, B.data_ptr(), ldb or rb, beta,
                                        C.data_ptr(), ldc or m, stream=s), reps, flush=m * n * k < 8192 ** 3)
        add(f"dgemm {'NT'[ta]}{'NT'[tb]} {m}x{n}x{k}{tag}", 2.0 * m * n * k, ms, peak64)

    if a.modes:
        for ta, tb in ((0, 0), (1, 0), (0, 1), (1, 1)):
            dgemm_row(ta, tb, a.modes, a.modes, a.modes, reps=1)
        return show()
    if a.small:
        for (m, n, k) in [(256, 256, 256), (512, 512, 512), (768, 768, 768), (1024, 1024, 1024), (1536, 1536, 1536),
                          (2048, 2048, 2048), (1024, 1024, 128), (1024, 1024, 4096), (4096, 4096, 256), (768, 768, 8192),
                          (200, 3000, 1000), (8192, 256, 256), (256, 8192, 256)]:
            dgemm_row(0, 0, m, n, k)
        for ta, tb in ((0, 0), (0, 1), (1, 0), (1, 1)):
            dgemm_row(ta, tb, 3001, 2047, 513, lda=3072, ldb=2048 if tb else 640, ldc=3008, alpha=-0.7, beta=1.3, tag=" padded ld")
        return show()
    if a.sgemm:
        sz = a.sgemm
        A, B, C = D.buf(sz, sz, f32, 7, 0), D.buf(sz, sz, f32, 7, 1), D.buf(sz, sz, f32, 7, 2)
        for mode, name, tt in ((0, "fp32", ((1, 0), (0, 0), (0, 1), (1, 1))), (1, "3xtf32", ((1, 0),))):
            for ta, tb in tt:
                ms = D.time(lambda: u.dev_sgemm(mode, ta, tb, sz, sz, sz, 1.0, A.data_ptr(), sz, B.data_ptr(), sz, 0.0,
                                                C.data_ptr(), sz, stream=s), 3, warm=2)
                add(f"sgemm {'NT'[ta]}{'NT'[tb]} {sz}^3 {name}", 2.0 * sz ** 3, ms, peak32)
        return show()
    if a.lu:
        m = a.lu
        A0 = D.buf(m, m, f64, 5, 0)
        W = A0.clone()
        piv = torch.zeros(m + 1, dtype=torch.int32, device="cuda")
        ms = D.time(lambda: u.lib.ulmb200_dgetrf(s, m, m, W.data_ptr(), m, piv.data_ptr(), piv.data_ptr() + 4 * m),
                    1, warm=1, flush=False, setup=lambda: W.copy_(A0))
        add(f"dgetrf n={m} (info {int(piv[m].item())})", 2.0 * m ** 3 / 3.0, ms, peak64)
        return show()
    if a.c4:
        n = a.c4
        k = n // 2
        T, B0 = D.buf(n, n, f64, 3, 0, dist=1, scale=1.0 / n), D.buf(n, n, f64, 3, 1)
        B = B0.clone()
        ms = D.time(lambda: u.dev_dtrsm(0, 1, 0, 0, n, n, 1.0, T.data_ptr(), n, B.data_ptr(), n, stream=s), 1, warm=1,
                    flush=False, setup=lambda: B.copy_(B0))
        add(f"dtrsm LLNN n={n}", float(n) ** 3, ms, peak64)
        A, C = D.buf(n, k, f64, 3, 0), D.buf(n, n, f64, 3, 2)
        ms = D.time(lambda: u.dev_dsyrk(0, 0, n, k, 1.0, A.data_ptr(), n, 0.5, C.data_ptr(), n, stream=s), 1, warm=1, flush=False)
        add(f"dsyrk UN n={n} k={k}", float(n) * (n + 1) * k, ms, peak64)
        return show()

    # --report: every routine
    quick = a.quick
    for (m, n, k) in [(1024, 1024, 1024), (4096, 4096, 4096), (16384, 16384, 16384)][: 2 if quick else 3]:
        for ta, tb in ((0, 0), (1, 0)) if m > 1024 else ((0, 0),):
            dgemm_row(ta, tb, m, n, k, reps=3 if m > 8192 else 5)
    dgemm_row(0, 0, 3001, 2047, 513, lda=3072, ldb=640, ldc=3008, alpha=-0.7, beta=1.3, tag=" padded ld")
    zs = 2048 if quick else 4096
    A = D.buf(2 * zs, zs, f64, 13, 0); B = D.buf(2 * zs, zs, f64, 13, 1); C = D.buf(2 * zs, zs, f64, 13, 2)
    for ta, ca, nm in ((0, 0, "NN"), (1, 1, "CN")):
        ms = D.time(lambda: u.dev_zgemm(ta, ca, 0, 0, zs, zs, zs, 0.7 - 0.3j, A.data_ptr(), zs, B.data_ptr(), zs, 1.3 + 0.2j,
                                        C.data_ptr(), zs, stream=s), 5)
        add(f"zgemm {nm} {zs}^3 (8mnk flops)", 8.0 * zs ** 3, ms, peak64)
    del A, B, C
    for mode, name in ((0, "fp32"), (1, "3xtf32")):
        for sz in (4096,) if quick else (4096, 8192):
            A = D.buf(sz, sz, f32, 7, 0); B = D.buf(sz, sz, f32, 7, 1); C = D.buf(sz, sz, f32, 7, 2)
            ms = D.time(lambda: u.dev_sgemm(mode, 1, 0, sz, sz, sz, 1.0, A.data_ptr(), sz, B.data_ptr(), sz, 0.0,
                                            C.data_ptr(), sz, stream=s), 5)
            add(f"sgemm TN {sz}^3 {name}", 2.0 * sz ** 3, ms, peak32)
            del A, B, C
    n, k = (4096, 2048) if quick else (8192, 4096)
    A = D.buf(n, k, f64, 3, 0); C = D.buf(n, n, f64, 3, 2); B = D.buf(n, k, f64, 3, 1)
    ms = D.time(lambda: u.dev_dsyrk(0, 0, n, k, 1.0, A.data_ptr(), n, 0.5, C.data_ptr(), n, stream=s), 5, flush=False)
    add(f"dsyrk UN n={n} k={k}", float(n) * (n + 1) * k, ms, peak64)
    ms = D.time(lambda: u.lib.ulmb200_dsyr2k(s, 0, 0, n, k, 1.0, A.data_ptr(), n, B.data_ptr(), n, 0.5, C.data_ptr(), n), 5, flush=False)
    add(f"dsyr2k UN n={n} k={k}", 2.0 * n * (n + 1) * k, ms, peak64)
    del A, B, C
    m = 4096 if quick else 8192
    T = D.buf(m, m, f64, 3, 0, dist=1, scale=1.0 / m); B0 = D.buf(m, m, f64, 3, 1); C = D.buf(m, m, f64, 3, 2)
    B = B0.clone()
    restore = lambda: B.copy_(B0)  # noqa: E731
    ms = D.time(lambda: u.dev_dtrsm(0, 1, 0, 0, m, m, 1.0, T.data_ptr(), m, B.data_ptr(), m, stream=s), 5, flush=False, setup=restore)
    add(f"dtrsm LLNN m=n={m}", float(m) * m * m, ms, peak64)
    ms = D.time(lambda: u.lib.ulmb200_dtrmm(s, 0, 1, 0, 0, m, m, 1.0, T.data_ptr(), m, B.data_ptr(), m), 5, flush=False, setup=restore)
    add(f"dtrmm LLNN m=n={m}", float(m) * m * m, ms, peak64)
    ms = D.time(lambda: u.lib.ulmb200_dsymm(s, 0, 1, m, m, 1.0, T.data_ptr(), m, B.data_ptr(), m, 0.0, C.data_ptr(), m), 5, flush=False)
    add(f"dsymm LL m=n={m}", 2.0 * m * m * m, ms, peak64)
    piv = torch.zeros(m + 1, dtype=torch.int32, device="cuda")
    A0 = D.buf(m, m, f64, 5, 0); W = A0.clone()
    ms = D.time(lambda: u.lib.ulmb200_dgetrf(s, m, m, W.data_ptr(), m, piv.data_ptr(), piv.data_ptr() + 4 * m), 3,
                flush=False, setup=lambda: W.copy_(A0))
    add(f"dgetrf n={m}", 2.0 * m ** 3 / 3.0, ms, peak64)
    show()


def sharded_trsm(m, torch, u):
    """DTRSM left/lower/no-trans/non-unit, m x m, B split by column blocks over the ranks of the
    job; A starts on rank 0 only.  Prints the whole-job rate (m^2 n / max-over-ranks device time)
    and each rank's largest deviation from the one-call solve of its block."""
    import torch.distributed as dist
    from ulmblas_b200.sharded import ShardedDtrsm
    os.environ.setdefault("NCCL_MAX_CTAS", "8")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if "RANK" in os.environ:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
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


if __name__ == "__main__":
    main()
