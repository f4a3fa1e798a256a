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


def test_the_library_plans_the_k_panels(ulm):
    """ulmb200_mg_plan_panels (csrc/mg_plan.h): a short first panel whose transfer nothing hides, a second
    one just long enough for the rest of A to arrive behind its product, and a last panel with the
    remaining K that needs no SMs left free because nothing travels any more."""
    from ulmblas_b200.sharded import planned_panels
    m = n = 65536
    k = 16384
    for world in (2, 4, 8):
        nb = n // world
        for rate in (40.0, 100.0, 150.0, 250.0, 400.0, 700.0):
            pans, reserve = planned_panels(m, nb, k, world, 1024, rate, 35.0)
            assert pans[0] == (0, 1024) and pans[-1][1] == k
            assert all(a[1] == b[0] for a, b in zip(pans, pans[1:])) and 2 <= len(pans) <= 3
            assert reserve[-1] == 0 and all(r == 1 for r in reserve[:-1])
            assert all((l1 - l0) % 256 == 0 for l0, l1 in pans[:-1])
            # all of A has arrived (at the assumed rate) before the last panel's product starts
            arrive = 8.0 * m * k / (rate * 1e9)
            start_last = 1024 * 8.0 * m / (rate * 1e9) + 2.0 * m * nb * pans[-1][0] / 35e12
            assert start_last >= arrive or len(pans) == 3 and pans[1][1] - pans[1][0] >= 256, (world, rate, pans)
            # the panels that leave SMs free are a small part of the work once the transport is fast
            if rate >= 250.0:
                assert pans[-1][0] <= 2048 * (8 // world if world < 8 else 1) + 1024, (world, rate, pans)
    assert planned_panels(m, n, k, 1)[0] == [(0, k)]                      # one GPU: one piece, nothing reserved
    assert planned_panels(m, n, k, 1)[1] == [0]
    assert planned_panels(100, 100, 300, 4)[0] == [(0, 256), (256, 300)] or planned_panels(100, 100, 300, 4)[0] == [(0, 300)]
    assert planned_panels(100, 100, 200, 4)[0] == [(0, 200)]             # shorter than a first panel
    # a slow transport makes the middle panel longer, never the reserved share larger than needed
    slow = planned_panels(m, 8192, k, 8, 1024, 40.0, 35.0)[0]
    fast = planned_panels(m, 8192, k, 8, 1024, 400.0, 35.0)[0]
    assert slow[-1][0] > fast[-1][0]
    assert PanelPlan(m, n, k, 8, 3).panels[0] == (0, 1024)               # kp = None: the library's plan


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


# ---------------------------------------------------------------------------
# sharded triangular solve
# ---------------------------------------------------------------------------
from ulmblas_b200.sharded import run_trsm_panels, trsm_panel_widths, trsm_steps  # noqa: E402


def _triangle(rng, na, lower, unit):
    """(the triangle the solve means, what is stored: other triangle rogue, diagonal kept)."""
    full = rng.uniform(-1, 1, (na, na)) / na + np.diag(rng.uniform(1, 2, na))
    T = np.tril(full) if lower else np.triu(full)
    rogue = np.triu(np.full((na, na), 7e9), 1) if lower else np.tril(np.full((na, na), 7e9), -1)
    stored = T + rogue
    if unit:
        T = T.copy()
        np.fill_diagonal(T, 1.0)
    return T, stored


def _numpy_doubles(X, stored, right, lower, trans, unit):
    """Test doubles for the device TRSM / GEMM calls of one rank, acting on X in place."""
    def solve(h, s, w):
        if w is not None:
            w.wait()
        J = slice(s.j0, s.j1)
        D = np.tril(stored[J, J]) if lower else np.triu(stored[J, J])
        if unit:
            D = D.copy()
            np.fill_diagonal(D, 1.0)
        Dop = D.T if trans else D
        if right:
            X[:, J] = np.linalg.solve(Dop.T, X[:, J].T).T
        else:
            X[J, :] = np.linalg.solve(Dop, X[J, :])

    def update(h, s, w):
        if w is not None:
            w.wait()
        J, R = slice(s.j0, s.j1), slice(s.r0, s.r1)
        Ar = stored[R, J]
        if not right and not trans:
            X[R, :] -= Ar @ X[J, :]
        elif not right:
            X[J, :] -= Ar.T @ X[R, :]
        elif not trans:
            X[:, J] -= X[:, R] @ Ar
        else:
            X[:, R] -= X[:, J] @ Ar.T
    return solve, update


def test_trsm_steps_order_and_ranges():
    # left, lower, no trans: forward, rest below the block, solve first
    st = trsm_steps(False, True, False, 10, 4)
    assert [(s.j0, s.j1, s.r0, s.r1, s.update_first) for s in st] == [
        (0, 4, 4, 10, False), (4, 8, 8, 10, False), (8, 10, 10, 10, False)]
    # left, lower, trans: effectively upper -> backward, update first
    st = trsm_steps(False, True, True, 10, 4)
    assert [(s.j0, s.j1, s.r0, s.r1, s.update_first) for s in st] == [
        (8, 10, 10, 10, True), (4, 8, 8, 10, True), (0, 4, 4, 10, True)]
    # right, upper, no trans: forward, rest above, update first
    st = trsm_steps(True, False, False, 10, 4)
    assert [(s.j0, s.j1, s.r0, s.r1, s.update_first) for s in st] == [
        (0, 4, 0, 0, True), (4, 8, 0, 4, True), (8, 10, 0, 8, True)]
    # growing panels, measured from the end the walk starts at
    assert trsm_panel_widths(20, 2, grow=True) == [2, 2, 4, 8, 4]
    assert trsm_panel_widths(5, 2) == [2, 2, 1]
    st = trsm_steps(False, False, False, 20, 2, grow=True)          # left, upper: backward
    assert [(s.j0, s.j1) for s in st] == [(18, 20), (16, 18), (12, 16), (4, 12), (0, 4)]
    st = trsm_steps(False, False, False, 21, 2, grow=True)          # ragged piece first
    assert [(s.j0, s.j1) for s in st] == [(20, 21), (18, 20), (16, 18), (12, 16), (4, 12), (0, 4)]
    assert all((s.r0, s.r1) == (0, s.j0) for s in st)
    assert trsm_steps(False, True, False, 0, 4) == []
    assert len(trsm_steps(True, True, True, 5, 100)) == 1


def test_trsm_panel_walk_all_sixteen_cases():
    rng = np.random.default_rng(5)
    for right in (False, True):
        for lower in (False, True):
            for trans in (False, True):
                for unit in (False, True):
                    na, other, kp = 37, 11, 8
                    T, stored = _triangle(rng, na, lower, unit)
                    op = T.T if trans else T
                    B = rng.uniform(-1, 1, (other, na)) if right else rng.uniform(-1, 1, (na, other))
                    X = B.copy()
                    solve, update = _numpy_doubles(X, stored, right, lower, trans, unit)
                    run_trsm_panels(trsm_steps(right, lower, trans, na, kp, grow=unit), 1, lambda a, b: None, None, solve, update)
                    want = np.linalg.solve(op.T, B.T).T if right else np.linalg.solve(op, B)
                    assert np.abs(X - want).max() < 1e-12, (right, lower, trans, unit)


_TRSM_WORKER = r"""
import os, sys
sys.path.insert(0, %(root)r); sys.path.insert(0, os.path.join(%(root)r, "tests"))
import numpy as np, torch, torch.distributed as dist
from ulmblas_b200.sharded import column_block, row_block, run_trsm_panels, trsm_steps
from test_sharded_cpu import _triangle, _numpy_doubles
rank, world = int(sys.argv[1]), int(sys.argv[2])
os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=sys.argv[3], RANK=str(rank), WORLD_SIZE=str(world))
dist.init_process_group("gloo", rank=rank, world_size=world)
na, other, kp = 150, 300, 64
for right, lower, trans, unit in ((False, True, False, False), (False, False, True, True), (True, False, False, False), (True, True, True, False)):
    rng = np.random.default_rng(11)                       # same stream on both ranks
    T, stored = _triangle(rng, na, lower, unit)
    op = T.T if trans else T
    B = rng.uniform(-1, 1, (other, na)) if right else rng.uniform(-1, 1, (na, other))
    b0, b1 = (row_block if right else column_block)(other, world, rank)
    X = (B[b0:b1, :] if right else B[:, b0:b1]).copy()
    # column-major A as a (na, na) tensor whose row j is column j; only rank 0 holds data at first
    A = torch.from_numpy(np.ascontiguousarray(stored.T)) if rank == 0 else torch.zeros((na, na), dtype=torch.float64)
    order = []
    def A_panel(j0, j1): return A[j0:j1, :]
    def recv(h, j0, j1):
        order.append((j0, j1))
        return dist.broadcast(h, src=0, async_op=True)
    local = A.numpy().T                                    # view: fills in as panels arrive
    solve, update = _numpy_doubles(X, local, right, lower, trans, unit)
    steps = trsm_steps(right, lower, trans, na, 16, grow=True)
    run_trsm_panels(steps, world, A_panel, recv, solve, update)
    assert order == [(s.j0, s.j1) for s in steps]
    want = np.linalg.solve(op.T, B.T).T if right else np.linalg.solve(op, B)
    want = want[b0:b1, :] if right else want[:, b0:b1]
    assert np.abs(X - want).max() < 1e-11, ("rank %%d" %% rank, right, lower, trans, unit)
    assert np.array_equal(A.numpy().T, stored), "A did not arrive intact"
if rank == 0:
    print("OK")
dist.destroy_process_group()
"""


def test_two_gloo_ranks_solve_their_blocks(tmp_path):
    import socket
    import subprocess
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    script = tmp_path / "trsm_worker.py"
    script.write_text(_TRSM_WORKER % dict(root=ROOT))
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "2", str(port)], stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, e[-2000:]
    assert "OK" in outs[0][0]
