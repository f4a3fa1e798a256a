"""The sharded product behind the C ABI (ulmb200_mg_dgemm, ulmb200_mg_dgemm_host).

On one GPU the communicator has a single rank: the device-resident call is one product, the
host-resident call pipelines the copy of A in K panels against the products and returns C in
column pieces -- both against the reference.  With two or more GPUs visible the same calls run as
child processes, one rank per GPU, with NCCL's in-switch reduction off (plain peer transport):
device-resident (broadcast of A), host-resident with A pushed by the root, and host-resident with
every rank bringing its share of A."""
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import EPS64, ROOT, bound_ratio, det_uniform, gemm_gauge
from test_gpu_dgemm import reference_dgemm

pytestmark = pytest.mark.gpu


def _dev(torch, M):
    return torch.from_numpy(np.ascontiguousarray(M.T)).cuda()


def test_single_rank_device_and_host_calls(ulm, torch_cuda):
    torch = torch_cuda
    from ulmblas_b200.sharded import ShardedDgemm
    m, n, k = 700, 520, 2300
    A, B, C0 = det_uniform(51, m, k), det_uniform(52, k, n), det_uniform(53, m, n)
    want = reference_dgemm("N", "N", m, n, k, 1.5, A, B, 0.5, C0, m)
    gauge = gemm_gauge(1.5, A, B, 0.5, C0)
    eng = ShardedDgemm(m, n, k)
    assert eng.plan.cols == (0, n) and eng.plan.panels == [(0, k)]
    dA, dB, dC = _dev(torch, A), _dev(torch, B), _dev(torch, C0)
    eng.profile(True)
    eng.run(1.5, dA, dB, 0.5, dC)
    torch.cuda.synchronize()
    assert eng.wait(10000) == ulm.OK
    assert len(eng.last_gemm_ms()) == 1 and eng.last_gemm_ms()[0] > 0.0
    assert bound_ratio(dC.cpu().numpy().T, want, gauge, k, EPS64) <= 1.0
    # host-resident: page-locked copies of the operands, device buffers as work space
    hA, hB, hC = (torch.from_numpy(np.ascontiguousarray(X.T)).pin_memory() for X in (A, B, C0))
    wA, wB, wC = torch.zeros_like(dA), torch.zeros_like(dB), torch.zeros_like(dC)
    eng.run(1.5, wA, wB, 0.5, wC, host=(hA, hB, hC))
    torch.cuda.synchronize()
    assert ulm.check_device_error() == ulm.OK
    assert bound_ratio(hC.numpy().T, want, gauge, k, EPS64) <= 1.0
    assert np.array_equal(hA.numpy().T, A) and np.array_equal(hB.numpy().T, B), "an input operand was modified"
    eng.close()


_RANK = r"""
import os, sys
sys.path.insert(0, %(root)r); sys.path.insert(0, os.path.join(%(root)r, "tests"))
rank, world, port = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port, RANK=str(rank), WORLD_SIZE=str(world),
                  NCCL_NVLS_ENABLE="0", NCCL_MAX_CTAS="8")
import numpy as np, torch, torch.distributed as dist
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
import ulmblas_b200.api as ulm
from ulmblas_b200.sharded import ShardedDgemm
from helpers import EPS64, bound_ratio, det_uniform, gemm_gauge
from test_gpu_dgemm import reference_dgemm
m, n, k = 1300, 1100, 5000
A, B, C0 = det_uniform(61, m, k), det_uniform(62, k, n), det_uniform(63, m, n)


def agree(ok, what):
    # Every rank learns whether all ranks passed this step (a tiny all-reduce between steps, nothing else in
    # flight); if one did not, all leave together instead of one leaving its peers inside a collective.
    t = torch.tensor([1.0 if ok else 0.0], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if t.item() < 0.5:
        if not ok:
            print("FAILED on rank %%d: %%s" %% (rank, what), flush=True)
        dist.destroy_process_group()
        sys.exit(1 if not ok else 0)


eng = ShardedDgemm(m, n, k, first=256)
j0, j1 = eng.plan.cols
nr = j1 - j0
want = reference_dgemm("N", "N", m, nr, k, -0.7, A, np.asfortranarray(B[:, j0:j1]), 1.3, np.asfortranarray(C0[:, j0:j1]), m)
gauge = gemm_gauge(-0.7, A, B[:, j0:j1], 1.3, C0[:, j0:j1])
dev = lambda M: torch.from_numpy(np.ascontiguousarray(M.T)).cuda()
pin = lambda M: torch.from_numpy(np.ascontiguousarray(M.T)).pin_memory()
# 1. device-resident: A only on the root
dA = dev(A) if rank == 0 else torch.zeros((k, m), dtype=torch.float64, device="cuda")
dB, dC = dev(B[:, j0:j1]), dev(C0[:, j0:j1])
for rep in range(2):                     # the second call plans with the measured transport rate
    dC.copy_(dev(C0[:, j0:j1]))
    eng.run(-0.7, dA, dB, 1.3, dC)
    torch.cuda.synchronize()
agree(eng.wait(20000) == ulm.OK, "a kernel gave up on a bounded wait (device-resident)")
widths, reserve, rate, _ = eng.last_plan()
agree(sum(widths) == k and reserve[-1] == 0 and rate > 0.0, "plan %%s %%s %%s" %% (widths, reserve, rate))


def where_off(got):
    bad = np.argwhere(np.abs(got - want) > 2 * k * EPS64 * gauge)
    if len(bad) == 0:
        return ""
    tiles = sorted(set((int(r) // 128, int(c) // 128) for r, c in bad))
    return "; %%d entries off in %%d tiles %%s, rows %%d..%%d, first %%s, got/want %%s" %% (
        len(bad), len(tiles), tiles[:16], bad[:, 0].min(), bad[:, 0].max(), bad[:4].tolist(),
        [(float(got[r, c]), float(want[r, c])) for r, c in bad[:3]])


got = dC.cpu().numpy().T
ratio = bound_ratio(got, want, gauge, k, EPS64)
agree(ratio <= 1.0, "device-resident block wrong: error / bound = %%g, plan %%s%%s" %% (ratio, widths, where_off(got)))
agree(rank == 0 or np.array_equal(dA.cpu().numpy().T, A), "A did not arrive intact")
# 2. host-resident, A pushed by the root; 3. every rank holds A and brings its share
for every in (False, True):
    hA = pin(A) if (rank == 0 or every) else None
    hB, hC = pin(B[:, j0:j1]), pin(C0[:, j0:j1])
    wA = torch.zeros((k, m), dtype=torch.float64, device="cuda")
    wB, wC = torch.zeros_like(dB), torch.zeros_like(dC)
    eng.run(-0.7, wA, wB, 1.3, wC, host=(hA, hB, hC), every_rank_has_a=every)
    torch.cuda.synchronize()
    agree(eng.wait(20000) == ulm.OK, "a kernel gave up on a bounded wait (host-resident, every=%%s)" %% every)
    got = hC.numpy().T
    ratio = bound_ratio(got, want, gauge, k, EPS64)
    where = where_off(got) if ratio > 1.0 else ""
    agree(ratio <= 1.0, "host-resident block wrong (every=%%s): error / bound = %%g, plan %%s%%s" %% (every, ratio, eng.last_plan()[0], where))
    agree(np.array_equal(wA.cpu().numpy().T, A), "A did not arrive intact (every=%%s)" %% every)
dist.barrier()
eng.close()
if rank == 0:
    print("OK")
dist.destroy_process_group()
"""


def test_ranks_on_several_gpus(torch_cuda, tmp_path):
    torch = torch_cuda
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("one GPU visible: the multi-rank path needs at least two")
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    script = tmp_path / "rank.py"
    script.write_text(_RANK % dict(root=ROOT))
    logs = [open(tmp_path / f"rank{r}.log", "w+") for r in range(world)]
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(world), str(port)], stdout=logs[r],
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    # A rank that fails an assertion leaves its peers waiting in their next collective: as soon as one rank
    # has exited with an error (or after five minutes) the others are stopped, by PID, and the first failure
    # is reported.
    import time
    deadline = time.time() + 300
    failed = None
    while any(p.poll() is None for p in procs) and time.time() < deadline and failed is None:
        for r, p in enumerate(procs):
            if p.poll() not in (None, 0):
                failed = r
        time.sleep(0.5)
    for p in procs:
        if p.poll() is None:
            if failed is None and time.time() < deadline:
                continue
            p.kill()
    for p in procs:
        p.wait()

    def log(r):
        logs[r].seek(0)
        return logs[r].read()[-3000:]
    if failed is None:
        failed = next((r for r, p in enumerate(procs) if p.returncode != 0), None)
    assert failed is None, f"rank {failed} failed:\n" + log(failed)
    assert "OK" in log(0)
