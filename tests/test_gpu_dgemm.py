"""DGEMM parity on the GPU: libulmblas_b200's dgemm_ / ulmb200_dgemm against the reference
(compiled ulmBLAS when oracle/_ref is present, its C restatement otherwise), under the
componentwise bound  |C - Cref| <= 2*k*eps*(|alpha||A||B| + |beta||C|)."""
import itertools
import os

import numpy as np
import pytest

from helpers import (EPS64, ROGUE, bound_ratio, det_uniform, gemm_gauge, golden_inputs, load_golden,
                     padded, port, ref, repair_nonfinite)

pytestmark = pytest.mark.gpu


def reference_dgemm(ta, tb, m, n, k, alpha, A, B, beta, C0, ldc):
    """Reference result on a copy of C0's allocation; NaN entries the SSE build emits on
    finite inputs are replaced by the (bit-identical elsewhere) restatement."""
    R = ref("")
    want = C0.copy(order="F")
    if R is not None:
        R.dgemm(ta, tb, m, n, k, alpha, A, B, beta, want[:m, :n], ldc=ldc)
        if not np.isfinite(want[:m, :n]).all():
            alt = C0.copy(order="F")
            port().dgemm(ta, tb, m, n, k, alpha, A, B, beta, alt[:m, :n], ldc=ldc)
            repair_nonfinite(want, alt)
    else:
        port().dgemm(ta, tb, m, n, k, alpha, A, B, beta, want[:m, :n], ldc=ldc)
    return want


def op(M, t):
    return M.T if t in "TC" else M


def check_case(ulm, ta, tb, m, n, k, alpha, beta, seed, lda=None, ldb=None, ldc=None, gen=None):
    ra, ca = (m, k) if ta == "N" else (k, m)
    rb, cb = (k, n) if tb == "N" else (n, k)
    gen = gen or det_uniform
    A, Ab = padded(gen(seed, ra, ca), lda or ra)
    B, Bb = padded(gen(seed + 1, rb, cb), ldb or rb)
    C0v, C0b = padded(gen(seed + 2, m, n), ldc or m)
    ldc_ = C0b.shape[0]
    Ab0, Bb0 = Ab.copy(order="F"), Bb.copy(order="F")
    want = reference_dgemm(ta, tb, m, n, k, alpha, A, B, beta, C0b, ldc_)
    got = C0b.copy(order="F")
    st = ulm.dgemm(ta, tb, m, n, k, alpha, A, B, beta, got[:m, :n], lda=Ab.shape[0], ldb=Bb.shape[0], ldc=ldc_)
    assert st == ulm.OK, ulm.status_string(st)
    assert np.array_equal(Ab, Ab0) and np.array_equal(Bb, Bb0), "an input operand was modified"
    assert np.array_equal(got[m:, :], C0b[m:, :]), "padding rows of C were written"
    ratio = bound_ratio(got[:m, :n], want[:m, :n], gemm_gauge(alpha, op(A, ta), op(B, tb), beta, C0v), k, EPS64)
    assert ratio <= 1.0, f"{ta}{tb} {m}x{n}x{k} alpha={alpha} beta={beta}: error/bound = {ratio:.3g}"
    return ratio


def test_config1_dgemm_1024(ulm):
    """DGEMM C = 1.5*A*B + 0.5*C, m=n=k=1024, seed 42, through dgemm_ with host pointers."""
    m = n = k = 1024
    A, _ = ulm.fmat(m, k); B, _ = ulm.fmat(k, n); C0, _ = ulm.fmat(m, n)
    ulm.host_fill(A, 42, 0); ulm.host_fill(B, 42, 1); ulm.host_fill(C0, 42, 2)
    want = reference_dgemm("N", "N", m, n, k, 1.5, A, B, 0.5, C0, m)
    got = C0.copy(order="F")
    before = ulm.launch_count()
    assert ulm.dgemm("N", "N", m, n, k, 1.5, A, B, 0.5, got) == ulm.OK
    assert ulm.launch_count() > before, "no kernel of this library was launched"
    ratio = bound_ratio(got, want, gemm_gauge(1.5, A, B, 0.5, C0), k, EPS64)
    assert ratio <= 1.0, ratio


def _normal(seed, r, c, dtype=np.float64):
    rng = np.random.default_rng(seed)
    return np.asfortranarray(rng.standard_normal((r, c)).astype(dtype))


@pytest.mark.parametrize("ta,tb", list(itertools.product("NT", "NT")))
def test_config3_ragged_padded(ulm, ta, tb):
    """m=3001 n=2047 k=513, padded leading dimensions, alpha=-0.7 beta=1.3, normal(0,1), seed 11.
    ldb is 640 only where that is a legal argument (B stored 513 x 2047); for B^T the stored
    matrix has 2047 rows and ldb = 2048."""
    check_case(ulm, ta, tb, 3001, 2047, 513, -0.7, 1.3, 11, lda=3072, ldb=640 if tb == "N" else 2048,
               ldc=3008, gen=_normal)


def test_tester_grid_small_shapes(ulm):
    """Sizes, alphas, betas and the ld = dim+1 rule of the reference's Level-3 tester
    (test/F77/dblat3.dat:9-14): odd leading dimensions exercise the non-TMA kernel."""
    sizes = [0, 1, 2, 3, 7, 12, 31]
    seed = 1000
    count = 0
    for (m, n, k) in [(1, 1, 1), (2, 3, 1), (7, 12, 31), (31, 7, 12), (12, 31, 7), (31, 31, 31), (3, 0, 7),
                      (0, 3, 7), (7, 3, 0), (1, 31, 2)]:
        assert m in sizes and n in sizes and k in sizes
        for ta, tb in itertools.product("NT", "NT"):
            for alpha, beta in itertools.product([0.0, 1.0, 0.7], [0.0, 1.0, 1.3]):
                seed += 3
                ra = (m if ta == "N" else k) + 1
                rb = (k if tb == "N" else n) + 1
                check_case(ulm, ta, tb, m, n, k, alpha, beta, seed, lda=ra, ldb=rb, ldc=m + 1)
                count += 1
    assert count == 360


@pytest.mark.parametrize("tile,path", [("64", ""), ("128", ""), ("12864", ""), ("64", "ldg"), ("128", "ldg")])
def test_every_kernel_variant(ulm, tile, path, monkeypatch):
    """Force each tile shape (64 x 64, 128 x 128, 128 x 64) on each load path (TMA / plain loads) over all
    four transpositions, on shapes with ragged edges in m, n and k."""
    monkeypatch.setenv("ULMB200_DGEMM_TILE", tile)
    if path:
        monkeypatch.setenv("ULMB200_DGEMM_PATH", path)
    ulm.reload_env()
    seed = 5000
    for (m, n, k) in [(300, 260, 100), (129, 65, 17), (64, 64, 16), (200, 1, 33), (1100, 1300, 270)]:
        for ta, tb in itertools.product("NT", "NT"):
            seed += 3
            ra = (m if ta == "N" else k)
            rb = (k if tb == "N" else n)
            check_case(ulm, ta, tb, m, n, k, 1.25, -0.5, seed, lda=ra + (ra % 2), ldb=rb + (rb % 2), ldc=m + 4)


@pytest.mark.parametrize("tile", ["128", "12864"])
def test_device_c_without_tensor_map(ulm, torch_cuda, tile, monkeypatch):
    """Device-resident operands whose C has an odd leading dimension, or starts 8 bytes off a 16-byte
    boundary: TMA can feed A and B but cannot address C, so the consumers write the tiles themselves
    instead of sending them out through shared memory.  Padding rows of C stay as they were."""
    torch = torch_cuda
    monkeypatch.setenv("ULMB200_DGEMM_TILE", tile)
    ulm.reload_env()
    m, n, k = 700, 900, 150
    A, B = det_uniform(77, m, k), det_uniform(78, k, n)
    dA, dB = torch.from_numpy(A.T.copy()).cuda(), torch.from_numpy(B.T.copy()).cuda()      # column-major on the device
    for ldc, off in [(m + 1, 0), (m + 2, 1)]:
        C0 = det_uniform(79 + ldc, ldc, n + 1)
        want = reference_dgemm("N", "N", m, n, k, -0.7, A, B, 1.3, np.asfortranarray(C0[off:off + m, :n]), m)
        dC = torch.from_numpy(C0.T.copy()).cuda()
        ulm.dev_dgemm(0, 0, m, n, k, -0.7, dA.data_ptr(), m, dB.data_ptr(), k, 1.3, dC.data_ptr() + 8 * off, ldc)
        torch.cuda.synchronize()
        assert ulm.check_device_error() == 0
        got = dC.cpu().numpy().T
        assert np.array_equal(got[off + m:, :], C0[off + m:, :]) and np.array_equal(got[:off, :], C0[:off, :])
        assert np.array_equal(got[:, n:], C0[:, n:])
        ratio = bound_ratio(got[off:off + m, :n], want[:m, :n], gemm_gauge(-0.7, A, B, 1.3, C0[off:off + m, :n]), k, EPS64)
        assert ratio <= 1.0, (tile, ldc, off, ratio)


@pytest.mark.parametrize("tile", ["", "128", "12864"])
def test_device_padding_below_an_odd_number_of_rows(ulm, torch_cuda, tile, monkeypatch):
    """Device-resident C with an odd number of rows and padding rows below them, operands TMA can address:
    whole tiles leave through shared memory and a TMA store, which clips rows in units of 16 bytes, so the
    last row needs its own care.  Padding rows (rogue values, also in A and B) stay bit for bit."""
    torch = torch_cuda
    if tile:
        monkeypatch.setenv("ULMB200_DGEMM_TILE", tile)
    ulm.reload_env()
    seed = 300
    for (m, n, k, ta, tb, beta) in [(1025, 700, 130, "N", "N", 1.3), (1025, 700, 130, "T", "T", 0.0), (3001, 2047, 65, "N", "T", 1.3),
                                    (257, 129, 513, "T", "N", 0.0), (1, 300, 40, "N", "N", 0.5)]:
        seed += 5
        ra, ca = (m, k) if ta == "N" else (k, m)
        rb, cb = (k, n) if tb == "N" else (n, k)
        lda, ldb, ldc = ra + 2 + (ra % 2), rb + 4 + (rb % 2), m + 7
        A, B, C0 = det_uniform(seed, ra, ca), det_uniform(seed + 1, rb, cb), det_uniform(seed + 2, m, n)

        def dev(h, ld):
            t = torch.full((h.shape[1], ld), ROGUE, dtype=torch.float64, device="cuda")
            t[:, :h.shape[0]] = torch.from_numpy(np.ascontiguousarray(h.T)).cuda()
            return t
        dA, dB, dC = dev(A, lda), dev(B, ldb), dev(C0, ldc)
        ulm.dev_dgemm(ta == "T", tb == "T", m, n, k, -0.7, dA.data_ptr(), lda, dB.data_ptr(), ldb, beta, dC.data_ptr(), ldc)
        torch.cuda.synchronize()
        assert ulm.check_device_error() == 0
        got = dC.cpu().numpy().T
        assert (got[m:, :] == ROGUE).all(), (tile, m, n, k, ta, tb, "padding rows of C were written")
        want = reference_dgemm(ta, tb, m, n, k, -0.7, A, B, beta, C0, m)
        ratio = bound_ratio(got[:m, :], want, gemm_gauge(-0.7, op(A, ta), op(B, tb), beta, C0), k, EPS64)
        assert ratio <= 1.0, (tile, m, n, k, ta, tb, beta, ratio)


def test_shared_tile_pieces_with_an_odd_number_of_rows(ulm, torch_cuda, monkeypatch):
    """Tiles shared among CTAs leave through the tile buffer piece by piece: the head is stored, the later
    pieces are added to C by bulk tensor reductions in order of k.  With an odd number of rows the last row
    of each piece is stored (or added) by the output warp's lanes.  Device-resident C with padding rows,
    sharing forced on: full comparison, padding bit for bit, and bit-identical repeats."""
    torch = torch_cuda
    monkeypatch.setenv("ULMB200_DGEMM_TILE", "128")
    monkeypatch.setenv("ULMB200_DGEMM_SPLITK", "2")
    ulm.reload_env()
    seed = 700
    for (m, n, k, ta, tb, beta) in [(3001, 2047, 513, "N", "N", 1.3), (1001, 1001, 1001, "T", "N", 0.5), (1601, 1500, 520, "T", "T", 0.0),
                                    (769, 641, 4099, "N", "T", 1.0), (129, 1100, 3000, "N", "N", -0.5)]:
        seed += 5
        ra, ca = (m, k) if ta == "N" else (k, m)
        rb, cb = (k, n) if tb == "N" else (n, k)
        lda, ldb, ldc = ra + (ra % 2), rb + 2 + (rb % 2), m + 3
        A, B, C0 = det_uniform(seed, ra, ca), det_uniform(seed + 1, rb, cb), det_uniform(seed + 2, m, n)

        def dev(h, ld):
            t = torch.full((h.shape[1], ld), ROGUE, dtype=torch.float64, device="cuda")
            t[:, :h.shape[0]] = torch.from_numpy(np.ascontiguousarray(h.T)).cuda()
            return t
        dA, dB, dC0 = dev(A, lda), dev(B, ldb), dev(C0, ldc)
        want = reference_dgemm(ta, tb, m, n, k, -0.7, A, B, beta, C0, m)
        gauge = gemm_gauge(-0.7, op(A, ta), op(B, tb), beta, C0)
        first = None
        for rep in range(3):
            dC = dC0.clone()
            ulm.dev_dgemm(ta == "T", tb == "T", m, n, k, -0.7, dA.data_ptr(), lda, dB.data_ptr(), ldb, beta, dC.data_ptr(), ldc)
            torch.cuda.synchronize()
            assert ulm.check_device_error() == 0
            got = dC.cpu().numpy().T
            assert (got[m:, :] == ROGUE).all(), (m, n, k, ta, tb, "padding rows of C were written")
            if first is None:
                first = got
                ratio = bound_ratio(got[:m, :], want, gauge, k, EPS64)
                assert ratio <= 1.0, (m, n, k, ta, tb, beta, ratio)
            else:
                assert np.array_equal(got, first), (m, n, k, rep, "results of identical calls differ")


def test_golden_fixture_cases_on_gpu(ulm):
    """The committed outputs of the compiled reference, reproduced on the GPU within the bound."""
    for name, c in load_golden().items():
        if c["kind"] != "dgemm":
            continue
        A, B, C0 = golden_inputs(c)
        got = C0.copy(order="F")
        assert ulm.dgemm(c["ta"], c["tb"], c["m"], c["n"], c["k"], c["alpha"], A, B, c["beta"], got) == ulm.OK
        ratio = bound_ratio(got, c["C"], gemm_gauge(c["alpha"], op(A, c["ta"]), op(B, c["tb"]), c["beta"], C0),
                            c["k"], EPS64)
        assert ratio <= 1.0, (name, ratio)


def test_device_pointer_path_and_beta_zero_ignores_c(ulm, torch_cuda):
    """Device-resident operands through ulmb200_dgemm; with beta == 0, NaN in C must not propagate
    (BLAS semantics; the reference's SSE kernel differs here on full tiles)."""
    torch = torch_cuda
    m, n, k = 777, 513, 260
    A = det_uniform(1, m, k); B = det_uniform(2, k, n)
    dA = torch.from_numpy(np.ascontiguousarray(A.T)).cuda()      # column-major m x k == row-major k x m
    dB = torch.from_numpy(np.ascontiguousarray(B.T)).cuda()
    dC = torch.full((n, m), float("nan"), dtype=torch.float64, device="cuda")
    ulm.dev_dgemm(0, 0, m, n, k, 2.0, dA.data_ptr(), m, dB.data_ptr(), k, 0.0, dC.data_ptr(), m,
                  stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    got = dC.cpu().numpy().T
    want = np.zeros((m, n), order="F")
    port().dgemm("N", "N", m, n, k, 2.0, A, B, 0.0, want)
    assert np.isfinite(got).all()
    assert bound_ratio(got, want, gemm_gauge(2.0, A, B, 0.0, want), k, EPS64) <= 1.0


def test_cblas_row_major(ulm):
    """cblas_dgemm row-major = the column-major product with operands swapped
    (interfaces/blas/C/gemm.cc:478-484); checked against numpy."""
    m, n, k = 50, 70, 33
    rng = np.random.default_rng(3)
    A = rng.uniform(-1, 1, (m, k)); B = rng.uniform(-1, 1, (n, k)); C0 = rng.uniform(-1, 1, (m, n))
    got = C0.copy()
    ulm.lib.cblas_dgemm(ulm.CblasRowMajor, ulm.CblasNoTrans, ulm.CblasTrans, m, n, k, 0.5,
                        A.ctypes.data, k, B.ctypes.data, k, 2.0, got.ctypes.data, n)
    assert ulm.last_status() == ulm.OK
    want = 0.5 * A @ B.T + 2.0 * C0
    assert bound_ratio(got, want, 0.5 * np.abs(A) @ np.abs(B.T) + 2.0 * np.abs(C0), k, EPS64) <= 1.0


def test_device_fill_matches_host_fill(ulm, torch_cuda):
    torch = torch_cuda
    rows, cols, ld = 301, 77, 304
    d = torch.zeros((cols, ld), dtype=torch.float64, device="cuda")
    ulm.dev_fill_f64(d.data_ptr(), ld, rows, cols, 99, 2, row0=5, col0=1000)
    torch.cuda.synchronize()
    h, _ = ulm.fmat(rows, cols)
    ulm.host_fill(h, 99, 2, row0=5, col0=1000)
    assert np.array_equal(d.cpu().numpy().T[:rows, :], h)
    f = torch.zeros((cols, ld), dtype=torch.float32, device="cuda")
    ulm.dev_fill_f32(f.data_ptr(), ld, rows, cols, 7, 0)
    torch.cuda.synchronize()
    hf, _ = ulm.fmat(rows, cols, dtype=np.float32)
    ulm.host_fill(hf, 7, 0)
    assert np.array_equal(f.cpu().numpy().T[:rows, :], hf)


def test_bounded_wait_reports_and_context_survives(ulm):
    """Every mbarrier wait in the kernels is bounded; when one runs out the kernel records it and
    returns.  Provoked here with a wait nothing can satisfy (no fault, no trap, no hang): the call
    must report KERNEL_FAULT and the very next product must still be right."""
    assert ulm.sup.ulmb200_selftest_wait_timeout() == ulm.KERNEL_FAULT
    assert ulm.last_status() == ulm.KERNEL_FAULT
    check_case(ulm, "N", "T", 150, 140, 70, 1.0, 0.0, 777)


def test_calls_from_several_host_threads(ulm):
    """The reference is re-entrant (its scratch pool is mutex-guarded); so are the BLAS entry points
    here: four threads calling dgemm_/dtrsm_ at once on their own data all get the right answer."""
    import threading
    errors = []

    def worker(i):
        try:
            for rep in range(3):
                check_case(ulm, "NT"[i % 2], "N", 300 + 17 * i, 200 + 5 * i, 150 + rep, 1.0 + i, 0.5, 9000 + 10 * i + rep)
        except Exception as exc:        # noqa: BLE001 - reported below
            errors.append((i, repr(exc)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors


def test_random_shapes_property(ulm):
    """Randomised sweep (seeded): any shape up to 400, any transposition, any legal padding of the
    leading dimensions (odd ones take the plain-load kernel, even ones the TMA kernel), random
    alpha/beta including 0 and 1 -- always inside the bound, padding and inputs untouched."""
    rng = np.random.default_rng(20261125)
    for it in range(80):
        m, n, k = (int(x) for x in rng.integers(1, 400, 3))
        ta, tb = "NT"[rng.integers(2)], "NT"[rng.integers(2)]
        alpha = float(rng.choice([0.0, 1.0, -1.0, 0.37, 2.5]))
        beta = float(rng.choice([0.0, 1.0, -0.5, 1.3]))
        ra, rb = (m if ta == "N" else k), (k if tb == "N" else n)
        check_case(ulm, ta, tb, m, n, k, alpha, beta, 30000 + 3 * it, lda=ra + int(rng.integers(0, 5)),
                   ldb=rb + int(rng.integers(0, 5)), ldc=m + int(rng.integers(0, 5)))


def test_tail_split_tiles_shared_by_several_ctas(ulm):
    """Tile counts a little above a multiple of the SM count: the last few 128x128 tiles are shared by
    2-8 CTAs, one K range each, added in a fixed order.  Full comparison against the reference (the
    split tiles are the last columns), all four transpositions once, and bit-identical repeats."""
    # 13 x 12 = 156 tiles on 148 SMs: 8 left over
    for i, (ta, tb, m, n, k, alpha, beta) in enumerate([("N", "N", 1664, 1536, 2100, 1.0, 0.0),
                                                        ("T", "N", 1600, 1530, 700, -0.7, 1.3),
                                                        ("N", "T", 1664, 1536, 1030, 1.5, 0.5),
                                                        ("T", "T", 1601, 1500, 520, 1.0, 1.0)]):
        check_case(ulm, ta, tb, m, n, k, alpha, beta, 88000 + 10 * i)
    ra, rb = det_uniform(1, 1664, 2100), det_uniform(2, 2100, 1536)
    c1, c2 = np.zeros((1664, 1536), order="F"), np.zeros((1664, 1536), order="F")
    assert ulm.dgemm("N", "N", 1664, 1536, 2100, 1.0, ra, rb, 0.0, c1) == ulm.OK
    assert ulm.dgemm("N", "N", 1664, 1536, 2100, 1.0, ra, rb, 0.0, c2) == ulm.OK
    assert np.array_equal(c1, c2), "the split must not make results depend on timing"


@pytest.mark.parametrize("mode", ["2", "0"])
def test_shared_tiles_forced_on_and_off(ulm, mode, monkeypatch):
    """ULMB200_DGEMM_SPLITK=2 shares the tiles beyond the last full wave among all CTAs whenever the
    schedule allows it (also where it would not pay), =0 never does.  Either way every result is
    inside the bound; shapes cover one tile, a few tiles, a wave and a bit, ragged edges, short and
    long inner dimensions, all four transpositions."""
    monkeypatch.setenv("ULMB200_DGEMM_SPLITK", mode)
    monkeypatch.setenv("ULMB200_DGEMM_TILE", "128")
    ulm.reload_env()
    seed = 91000
    shapes = [(128, 128, 64), (100, 90, 33), (1024, 1024, 1024), (300, 260, 100), (1664, 1536, 50), (2000, 1300, 513),
              (129, 4000, 700), (2304, 2304, 16), (640, 384, 4099)]
    for i, (m, n, k) in enumerate(shapes):
        for ta, tb in ([("N", "N"), ("T", "N"), ("N", "T"), ("T", "T")] if i % 3 == 0 else [("NT"[i % 2], "NT"[(i // 2) % 2])]):
            seed += 3
            check_case(ulm, ta, tb, m, n, k, -0.7, 1.3, seed)
    A, B = det_uniform(7, 1024, 1024), det_uniform(8, 1024, 1024)
    c1, c2 = np.zeros((1024, 1024), order="F"), np.zeros((1024, 1024), order="F")
    assert ulm.dgemm("N", "N", 1024, 1024, 1024, 1.0, A, B, 0.0, c1) == ulm.OK
    assert ulm.dgemm("N", "N", 1024, 1024, 1024, 1.0, A, B, 0.0, c2) == ulm.OK
    assert np.array_equal(c1, c2), "sharing tiles must not make results depend on timing"


def test_shared_tiles_second_piece_per_cta_is_repeatable(ulm, torch_cuda, monkeypatch):
    """Products whose last tiles are shared so that most CTAs take two pieces (the head of one tile, then the
    tail of the tile before it), repeated while another stream keeps the SMs busy.  Two things went wrong here
    once and are pinned by this test: a CTA's release of a pipeline stage overtaking its own shared loads (the
    TMA refill for the second piece changed the stage under them: wrong values of a few k in one 16-row block,
    in up to two launches out of three), and old values of C read from a stale L1 line when the columns of C do
    not start on 128-byte boundaries (ldc = 1300).  Every result must equal the first bit for bit and lie
    inside the bound."""
    torch = torch_cuda
    monkeypatch.setenv("ULMB200_DGEMM_TILE", "128")
    monkeypatch.setenv("ULMB200_DGEMM_SPLITK", "2")
    ulm.reload_env()
    side = torch.cuda.Stream()
    X = torch.rand(2048, 2048, device="cuda")
    Y = torch.empty_like(X)
    for (m, n, k, reps) in [(1280, 640, 4744, 40), (1300, 550, 3976, 25), (2100, 900, 700, 12)]:
        A, B, C0 = det_uniform(400 + m, m, k), det_uniform(401 + m, k, n), det_uniform(402 + m, m, n)
        want = reference_dgemm("N", "N", m, n, k, -0.7, A, B, 1.0, C0, m)
        gauge = gemm_gauge(-0.7, A, B, 1.0, C0)
        dA, dB = (torch.from_numpy(np.ascontiguousarray(X_.T)).cuda() for X_ in (A, B))
        dC0 = torch.from_numpy(np.ascontiguousarray(C0.T)).cuda()
        first = None
        for rep in range(reps):
            dC = dC0.clone()
            torch.cuda.synchronize()
            with torch.cuda.stream(side):
                for _ in range(3):
                    torch.mm(X, X, out=Y)
            ulm.dev_dgemm(0, 0, m, n, k, -0.7, dA.data_ptr(), m, dB.data_ptr(), k, 1.0, dC.data_ptr(), m)
            torch.cuda.synchronize()
            got = dC.cpu().numpy().T
            if first is None:
                first = got
                assert bound_ratio(got, want, gauge, k, EPS64) <= 1.0, (m, n, k)
            else:
                assert np.array_equal(got, first), (m, n, k, rep, "results of identical calls differ")
    assert ulm.check_device_error() == 0


def test_launches_on_two_streams_do_not_disturb_each_other(ulm, torch_cuda):
    """One large product on stream A while 160 small ones go out on stream B: the persistent kernels'
    tile counters and fold flags belong to the stream, so neither side can advance or reset the
    other's.  The large result is checked on sampled columns, every small one in full."""
    torch = torch_cuda
    m, n, k = 4096, 4224, 2048                      # 33 x 33 tiles = 1089 = 7 waves + 53 shared tiles
    A, B = det_uniform(61, m, k), det_uniform(62, k, n)
    dA = torch.from_numpy(np.ascontiguousarray(A.T)).cuda()
    dB = torch.from_numpy(np.ascontiguousarray(B.T)).cuda()
    dC = torch.zeros((n, m), dtype=torch.float64, device="cuda")
    sm, sn, sk = 256, 192, 96
    a = det_uniform(63, sm, sk); b = det_uniform(64, sk, sn)
    da = torch.from_numpy(np.ascontiguousarray(a.T)).cuda()
    db = torch.from_numpy(np.ascontiguousarray(b.T)).cuda()
    nsmall = 160
    dc = torch.zeros((nsmall, sn, sm), dtype=torch.float64, device="cuda")
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    for rep in range(2):
        ulm.dev_dgemm(0, 0, m, n, k, 1.0, dA.data_ptr(), m, dB.data_ptr(), k, 0.0, dC.data_ptr(), m, stream=s1.cuda_stream)
        for i in range(nsmall):
            ulm.dev_dgemm(0, 0, sm, sn, sk, 1.0 + i, da.data_ptr(), sm, db.data_ptr(), sk, 0.0, dc[i].data_ptr(), sm,
                          stream=s2.cuda_stream)
    torch.cuda.synchronize()
    assert ulm.check_device_error() == ulm.OK
    cols = np.sort(np.random.default_rng(5).choice(n, 48, replace=False))
    Bs = np.asfortranarray(B[:, cols])
    want = reference_dgemm("N", "N", m, len(cols), k, 1.0, A, Bs, 0.0, np.zeros((m, len(cols)), order="F"), m)
    got = dC[torch.from_numpy(cols).cuda()].cpu().numpy().T
    assert bound_ratio(got, want, gemm_gauge(1.0, A, Bs, 0.0, want), k, EPS64) <= 1.0
    small = dc.cpu().numpy()
    base = a @ b
    gauge = np.abs(a) @ np.abs(b)
    for i in range(nsmall):
        assert bound_ratio(small[i].T, (1.0 + i) * base, (1.0 + i) * gauge, sk, EPS64) <= 1.0, i


def test_workspace_can_be_released_and_capped(ulm, monkeypatch):
    """Host-pointer calls stage through cached device buffers; the cache can be given back, and
    ULMB200_WORKSPACE_CAP_MB bounds it (a request beyond the bound fails cleanly, C untouched)."""
    check_case(ulm, "N", "N", 600, 500, 300, 1.0, 0.5, 92000)
    assert ulm.workspace_bytes() > 0
    assert ulm.release_workspace() == ulm.OK and ulm.workspace_bytes() == 0
    check_case(ulm, "T", "N", 600, 500, 300, 1.0, 0.5, 92010)          # the cache grows again on demand
    assert ulm.release_workspace() == ulm.OK
    monkeypatch.setenv("ULMB200_WORKSPACE_CAP_MB", "1")
    ulm.reload_env()
    A, B = det_uniform(1, 600, 300), det_uniform(2, 300, 500)
    Cm = np.full((600, 500), 3.0, order="F")
    assert ulm.dgemm("N", "N", 600, 500, 300, 1.0, A, B, 0.0, Cm) == ulm.CUDA_ERROR
    assert np.all(Cm == 3.0)
    monkeypatch.delenv("ULMB200_WORKSPACE_CAP_MB")
    ulm.reload_env()
    check_case(ulm, "N", "T", 600, 500, 300, 1.0, 0.5, 92020)


def test_few_tiles_long_k_every_tile_split(ulm):
    """A product of tall, narrow operands (few 128x128 tiles, long inner dimension): every tile is cut
    along K over several CTAs.  All four transpositions, alpha/beta != trivial, bit-identical repeats."""
    for i, (ta, tb) in enumerate(itertools.product("NT", "NT")):
        check_case(ulm, ta, tb, 700, 500, 4100, -0.7, 1.3, 89000 + 10 * i)
    A, B = det_uniform(5, 640, 8192), det_uniform(6, 8192, 384)
    c1, c2 = np.zeros((640, 384), order="F"), np.zeros((640, 384), order="F")
    assert ulm.dgemm("N", "N", 640, 384, 8192, 1.0, A, B, 0.0, c1) == ulm.OK
    assert ulm.dgemm("N", "N", 640, 384, 8192, 1.0, A, B, 0.0, c2) == ulm.OK
    assert np.array_equal(c1, c2)
