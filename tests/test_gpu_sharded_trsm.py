"""The panelled triangular solve of the multi-GPU path, run on one GPU with the panel walk forced:
every side/uplo/trans/diag case against the reference's solution of the same system."""
import itertools

import numpy as np
import pytest

from helpers import ROGUE, det_uniform, port, ref, repair_nonfinite
from test_gpu_level3 import tri_matrix

pytestmark = pytest.mark.gpu


def reference_dtrsm(side, uplo, tr, diag, m, n, alpha, A, B0):
    want = B0.copy(order="F")
    R = ref("")
    if R is not None:
        R.dtrsm(side, uplo, tr, diag, m, n, alpha, A, want)
    if R is None or not np.isfinite(want).all():
        alt = B0.copy(order="F")
        port().dtrsm(side, uplo, tr, diag, m, n, alpha, A, alt)
        if R is None:
            want = alt
        else:
            repair_nonfinite(want, alt)
    return want


@pytest.mark.parametrize("side", "LR")
def test_forced_panel_walk_matches_reference(ulm, torch_cuda, side):
    torch = torch_cuda
    from ulmblas_b200.sharded import ShardedDtrsm
    seed = 41000
    for uplo, tr, diag in itertools.product("UL", "NT", "NU"):
        for (na, other, kp, alpha) in [(300, 70, 128, 0.7), (257, 129, 64, 1.0)]:
            seed += 2
            m, n = (na, other) if side == "L" else (other, na)
            A = tri_matrix(seed, na, uplo)                       # the other triangle holds rogue values
            B0 = np.asfortranarray(det_uniform(seed + 1, m, n))
            want = reference_dtrsm(side, uplo, tr, diag, m, n, alpha, A, B0)
            dA = torch.from_numpy(np.ascontiguousarray(A.T)).cuda()
            dB = torch.from_numpy(np.ascontiguousarray(B0.T)).cuda()
            op = ShardedDtrsm(side == "R", uplo == "L", tr == "T", diag == "U", m, n, kp=kp, grow=(diag == "U"), force_panels=True)
            assert len(op.steps) >= 3 and sum(st.j1 - st.j0 for st in op.steps) == na
            b0, b1 = op.run(alpha, dA, dB)
            torch.cuda.synchronize()
            assert (b0, b1) == (0, other)
            X = dB.cpu().numpy().T
            assert np.isfinite(X).all(), "the unreferenced (rogue) triangle of A leaked into the result"
            assert np.abs(X - want).max() <= 1e-10, (side, uplo, tr, diag, na, other)
            assert np.array_equal(dA.cpu().numpy().T, A)


def test_one_gpu_solves_in_one_call(ulm, torch_cuda):
    torch = torch_cuda
    from ulmblas_b200.sharded import ShardedDtrsm
    m, n = 200, 90
    A = tri_matrix(777, m, "L")
    B0 = np.asfortranarray(det_uniform(778, m, n))
    want = reference_dtrsm("L", "L", "N", "N", m, n, 1.0, A, B0)
    dA = torch.from_numpy(np.ascontiguousarray(A.T)).cuda()
    dB = torch.from_numpy(np.ascontiguousarray(B0.T)).cuda()
    op = ShardedDtrsm(False, True, False, False, m, n)
    assert op.steps == [] and not op.panelled
    op.run(1.0, dA, dB)
    torch.cuda.synchronize()
    assert np.abs(dB.cpu().numpy().T - want).max() <= 1e-10
