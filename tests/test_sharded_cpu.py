"""Host logic of the multi-GPU path on CPU: the column-block partition, the K-panel schedule,
and the broadcast/compute ordering run as two gloo ranks.  The arithmetic is a test double
(numpy) injected where the product passes its device GEMM -- the library itself has no CPU path."""
import os
import sys

import numpy as np
import pytest

from helpers import ROOT, det_uniform

from ulmblas_b200.sharded import PanelPlan, column_block, k_panels, run_panels


def test_column_blocks_tile_the_matrix():
    for n in (0, 1, 127, 128, 129, 1000, 65536, 65537):
        for world in (1, 2, 3, 4, 8):
            blocks = [column_block(n, world, r) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == n
            for (a0, a1), (b0, b1) in zip(blocks, blocks[1:]):
                assert a1 == b0 and a0 <= a1
            for j0, j1 in blocks:
                assert j0 % 128 == 0 or j0 == n
            widths = [j1 - j0 for j0, j1 in blocks]
            assert max(widths) - min(widths) <= 255
    assert column_block(65536, 8, 3) == (3 * 8192, 4 * 8192)
    with pytest.raises(ValueError):
        column_block(10, 2, 2)


def test_k_panels():
    assert k_panels(0, 4) == []
    assert k_panels(10, 4) == [(0, 4), (4, 8), (8, 10)]
    assert k_panels(8, 100) == [(0, 8)]
    assert PanelPlan(4, 4, 16384, 1, 0, 2048).panels == [(0, 16384)]          # one GPU: one piece
    assert len(PanelPlan(4, 4, 16384, 8, 0, 2048).panels) == 8
    assert PanelPlan(4, 4, 16384, 8, 0, 4096, 1024).panels == [(0, 1024), (1024, 5120), (5120, 9216), (9216, 13312), (13312, 16384)]


def test_run_panels_orders_beta_and_waits():
    plan = PanelPlan(m=6, n=300, k=10, world=2, rank=1, kp=4)
    log = []

    class W:
        def __init__(self, tag): self.tag = tag
        def wait(self): log.append(("wait", self.tag))

    def recv(h, l0, l1):
        log.append(("bcast", l0, l1))
        return W((l0, l1))

    def gemm(h, l0, l1, beta_l, w):
        w.wait()
        log.append(("gemm", l0, l1, beta_l))

    j0, j1 = run_panels(plan, 2.0, 0.5, lambda l0, l1: (l0, l1), recv, gemm)
    assert (j0, j1) == (256, 300)
    # every broadcast is queued before the first product; beta applies to the first panel only
    assert log[:3] == [("bcast", 0, 4), ("bcast", 4, 8), ("bcast", 8, 10)]
    assert [e for e in log if e[0] == "gemm"] == [("gemm", 0, 4, 0.5), ("gemm", 4, 8, 1.0), ("gemm", 8, 10, 1.0)]


_WORKER = r"""
import os, sys
sys.path.insert(0, %(root)r); sys.path.insert(0, os.path.join(%(root)r, "tests"))
import numpy as np, torch, torch.distributed as dist
from helpers import det_uniform
from ulmblas_b200.sharded import PanelPlan, run_panels
rank, world = int(sys.argv[1]), int(sys.argv[2])
os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=sys.argv[3], RANK=str(rank), WORLD_SIZE=str(world))
dist.init_process_group("gloo", rank=rank, world_size=world)
m, n, k, kp = 70, 300, 50, 16
A_full, B_full, C_full = det_uniform(1, m, k), det_uniform(2, k, n), det_uniform(3, m, n)
plan = PanelPlan(m, n, k, world, rank, kp)
j0, j1 = plan.cols
A = torch.from_numpy(np.ascontiguousarray(A_full.T)) if rank == 0 else torch.zeros((k, m), dtype=torch.float64)
Br, Cr = B_full[:, j0:j1].copy(), C_full[:, j0:j1].copy()
def A_panel(l0, l1): return A[l0:l1, :]
def recv(h, l0, l1): return dist.broadcast(h, src=0, async_op=True)
def gemm(h, l0, l1, beta_l, w):
    w.wait()
    Cr[...] = 1.5 * (h.numpy().T @ Br[l0:l1, :]) + beta_l * Cr       # test double for the device GEMM
run_panels(plan, 1.5, 0.5, A_panel, recv, gemm)
want = 1.5 * A_full @ B_full[:, j0:j1] + 0.5 * C_full[:, j0:j1]
assert np.allclose(Cr, want, rtol=1e-13, atol=1e-13), "rank %%d block wrong" %% rank
assert rank == 0 or np.array_equal(A.numpy().T, A_full), "A did not arrive intact"
out = [None] * world
dist.all_gather_object(out, (j0, j1))
if rank == 0:
    assert out[0][0] == 0 and out[-1][1] == n and all(a[1] == b[0] for a, b in zip(out, out[1:]))
    print("OK")
dist.destroy_process_group()
"""


def test_two_gloo_ranks_compute_their_column_blocks(tmp_path):
    import socket
    import subprocess
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    script = tmp_path / "worker.py"
    script.write_text(_WORKER % dict(root=ROOT))
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "2", str(port)], stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, e[-2000:]
    assert "OK" in outs[0][0]
