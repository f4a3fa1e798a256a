"""ulmb200_dtrsm_noalloc -- the triangular solve for callers that cannot allocate device memory
(real-time loops, plug-ins with a fixed memory budget, processes whose device memory is already
committed).  It must give what ulmb200_dtrsm gives, call after call, although every call reuses
one fixed work area inside the library that still holds the previous call's contents.

Collected last on purpose (file name): a run that stops at the first failure has then already
run every other GPU test.  Passes alone in a fresh process and after the rest of the suite."""
import numpy as np
import pytest

from helpers import ROGUE, det_uniform, port

pytestmark = pytest.mark.gpu


def _tri(seed, na, lower):
    A = det_uniform(seed, na, na)
    d = np.diag(A).copy()
    A = np.asfortranarray(A / na)
    A[np.arange(na), np.arange(na)] = 1.5 + 0.25 * d
    other = np.triu(np.ones((na, na), bool), 1) if lower else np.tril(np.ones((na, na), bool), -1)
    A[other] = ROGUE                       # the unreferenced triangle must never be read
    return A


def _to_dev(torch, M):
    return torch.from_numpy(np.ascontiguousarray(M.T)).cuda()       # column-major M == row-major M.T


def _solve_both(ulm, torch, side, lower, trans, unit, m, n, alpha, seed):
    na = m if side == 0 else n
    dA = _to_dev(torch, _tri(seed, na, lower))
    B = det_uniform(seed + 1, m, n)
    d_ref, d_new = _to_dev(torch, B), _to_dev(torch, B)
    s = torch.cuda.current_stream().cuda_stream
    ulm.dev_dtrsm(side, lower, trans, unit, m, n, alpha, dA.data_ptr(), na, d_ref.data_ptr(), m, stream=s)
    torch.cuda.synchronize()
    # The property in the name: across the call no device memory is allocated, neither by the
    # library (its own count of cudaMalloc calls) nor by anything else (free bytes of the device).
    # The driver loads a kernel's code on its first launch, which takes device memory once per
    # kernel; so the free bytes are compared across a repeat of the same call.
    allocs = ulm.alloc_count()
    d_warm = d_new.clone()
    st = ulm.dev_dtrsm_noalloc(side, lower, trans, unit, m, n, alpha, dA.data_ptr(), na, d_warm.data_ptr(), m, stream=s)
    assert st == ulm.OK, ulm.status_string(st)
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    st = ulm.dev_dtrsm_noalloc(side, lower, trans, unit, m, n, alpha, dA.data_ptr(), na, d_new.data_ptr(), m, stream=s)
    assert st == ulm.OK, ulm.status_string(st)
    assert ulm.check_device_error(s) == ulm.OK
    assert ulm.alloc_count() == allocs, "ulmb200_dtrsm_noalloc allocated device memory"
    assert torch.cuda.mem_get_info()[0] == free0, "free device memory changed across ulmb200_dtrsm_noalloc"
    assert torch.equal(d_warm, d_new), "two calls in a row on the same inputs differ"
    ref, new = d_ref.cpu().numpy().T, d_new.cpu().numpy().T
    assert np.isfinite(new).all()
    # the same solver on the same inputs (the allocating entry point uses 256-wide diagonal blocks
    # for larger triangles, this one 128-wide): the tolerance of the TRSM parity tests
    assert np.abs(new - ref).max() <= 1e-10, (side, lower, trans, unit, m, n)
    if m * n <= 300 * 1000:
        # and against the CPU restatement of the reference's own solver
        A = dA.cpu().numpy().T
        want = np.asfortranarray(B.copy())
        port().dtrsm("LR"[side], "UL"[lower], "NT"[trans], "NU"[unit], m, n, alpha, np.asfortranarray(A), want)
        assert np.abs(new - want).max() <= 1e-10, ("oracle", side, lower, trans, unit, m, n)
    return new


def test_noalloc_matches_dtrsm_on_consecutive_calls(ulm, torch_cuda):
    torch = torch_cuda
    # two calls in a row with different shapes and variants: the second finds the first one's
    # block inverses and leaf tile in the shared work area and must not be affected by them
    first = _solve_both(ulm, torch, 0, 1, 0, 0, 700, 333, 1.0, 31000)
    second = _solve_both(ulm, torch, 0, 1, 0, 0, 300, 129, 0.7, 31010)
    assert first.shape == (700, 333) and second.shape == (300, 129)
    # and the remaining families: upper / transposed / unit diagonal / right side
    _solve_both(ulm, torch, 0, 0, 1, 1, 257, 64, 1.0, 31020)
    _solve_both(ulm, torch, 1, 0, 0, 0, 200, 385, -0.5, 31030)
    _solve_both(ulm, torch, 1, 1, 1, 1, 130, 300, 1.0, 31040)
    # the first shape again: identical to the first answer despite everything that ran in between
    again = _solve_both(ulm, torch, 0, 1, 0, 0, 700, 333, 1.0, 31000)
    assert np.array_equal(again, first)


def test_noalloc_on_a_shape_that_splits_k_in_the_allocating_path(ulm, torch_cuda):
    """768 x 768 at k up to 768: few tiles per update, where ulmb200_dtrsm's products share tiles
    through scheduler words from the library's cache; this entry point must not reach for them."""
    _solve_both(ulm, torch_cuda, 0, 1, 0, 0, 768, 768, 1.0, 31200)
    _solve_both(ulm, torch_cuda, 1, 0, 1, 0, 768, 768, 0.5, 31210)


def test_a_fault_in_a_noalloc_solve_is_reported(ulm, torch_cuda):
    """The work area has its own error word; ulmb200_check_device_error reads it (a plain copy, no
    allocation).  Provoked with a wait that nothing satisfies and that gives up after about a
    millisecond -- no fault, no trap, no hang -- written into that word."""
    torch = torch_cuda
    _solve_both(ulm, torch, 0, 1, 0, 0, 200, 100, 1.0, 31300)             # the word exists from here on
    assert ulm.sup.ulmb200_selftest_wait_timeout_noalloc_word() == ulm.OK
    allocs = ulm.alloc_count()
    assert ulm.check_device_error() == ulm.KERNEL_FAULT
    assert ulm.check_device_error() == ulm.OK, "the record is cleared by the check that reports it"
    assert ulm.alloc_count() == allocs
    _solve_both(ulm, torch, 0, 1, 0, 0, 200, 100, 1.0, 31300)             # and the next solve is right


def test_noalloc_refuses_sizes_beyond_its_fixed_work_area(ulm, torch_cuda):
    torch = torch_cuda
    d = torch.zeros(16, dtype=torch.float64, device="cuda")
    launches = ulm.launch_count()
    assert ulm.dev_dtrsm_noalloc(0, 1, 0, 0, 2049, 8, 1.0, d.data_ptr(), 2049, d.data_ptr(), 2049) == ulm.TOO_LARGE
    assert ulm.dev_dtrsm_noalloc(0, 1, 0, 0, 8, 4097, 1.0, d.data_ptr(), 8, d.data_ptr(), 8) == ulm.TOO_LARGE
    assert ulm.dev_dtrsm_noalloc(1, 1, 0, 0, 4097, 8, 1.0, d.data_ptr(), 8, d.data_ptr(), 4097) == ulm.TOO_LARGE
    assert ulm.launch_count() == launches, "a refused call launched a kernel"
    assert ulm.dev_dtrsm_noalloc(0, 1, 0, 0, -1, 8, 1.0, d.data_ptr(), 1, d.data_ptr(), 1) == ulm.BAD_ARGUMENT


def test_noalloc_at_its_size_limit(ulm, torch_cuda):
    torch = torch_cuda
    _solve_both(ulm, torch, 0, 1, 0, 0, 2048, 4096, 1.0, 31100)
