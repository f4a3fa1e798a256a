"""Large DGEMM (and, further down, DTRSM) split over the GPUs of one box by column blocks of C.

    C[:, J_r] <- alpha * A * B[:, J_r] + beta * C[:, J_r]        on rank r

One process per GPU.  Rank r owns the column block J_r of B and C for good; A lives on the root
rank and reaches the others by NCCL broadcast over NVLink, cut into K panels A[:, l0:l1]
(contiguous in column-major storage).  The broadcasts are queued ahead on a communication
stream; the product of panel l is queued on the compute stream behind "panel l has arrived".
There is no reduction and no other exchange: columns of C are independent.

The DGEMM driver itself is C++ behind the library's C ABI (``ulmb200_mg_*`` in
include/ulmblas_b200.h, csrc/mg_dgemm.cu): partition, K-panel plan, transport and products.
``ShardedDgemm`` is its binding for torch buffers; ``torch.distributed`` only carries the NCCL
unique id to the ranks.  ``PanelPlan`` / ``run_panels`` state the same schedule with the
transport and the arithmetic injected, so that the ordering can be exercised by CPU ranks
(gloo) in the tests; the triangular solve further down is driven from Python.

The reference has no multi-device path (it is single-threaded CPU code); the partition follows
its own loop order, which already walks C by column blocks (ulmblas/level3/gemm.tcc:60).
"""
import ctypes as C
from dataclasses import dataclass

ALIGN = 128          # column blocks start on CTA-tile boundaries


def column_block(n, world, rank, align=ALIGN):
    """[j0, j1) of rank `rank`: near-equal blocks whose starts are multiples of `align`
    (the library's ulmb200_mg_column_block for the default alignment)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    if align == ALIGN:
        from . import api
        return api.mg_column_block(n, world, rank)
    units = (n + align - 1) // align
    base, extra = divmod(units, world)
    u0 = rank * base + min(rank, extra)
    u1 = u0 + base + (1 if rank < extra else 0)
    return min(u0 * align, n), min(u1 * align, n)


def k_panels(k, kp, first=None):
    """[(l0, l1)] covering [0, k): an optional short first panel, then panels of kp (the last may
    be short).  The fixed-width walk of the triangular solve and of the tests."""
    if k <= 0:
        return []
    kp = max(1, min(kp, k))
    out, l0 = [], 0
    if first is not None and 0 < first < kp and first < k:
        out.append((0, first))
        l0 = first
    while l0 < k:
        out.append((l0, min(l0 + kp, k)))
        l0 += kp
    return out


def planned_panels(m, n_block, k, world, first=1024, transport_gbs=150.0, gemm_tflops=35.0):
    """The library's K-panel plan as ([(l0, l1)], [reserve flags]) -- ulmb200_mg_plan_panels."""
    from . import api
    widths, reserve = api.mg_plan_panels(m, n_block, k, world, first, transport_gbs, gemm_tflops)
    out, l0 = [], 0
    for w in widths:
        out.append((l0, l0 + w))
        l0 += w
    return out, reserve


@dataclass
class PanelPlan:
    m: int
    n: int
    k: int
    world: int
    rank: int
    kp: int = None          # None: the library's plan; a number: fixed-width panels (tests)
    first: int = None

    @property
    def cols(self):
        return column_block(self.n, self.world, self.rank)

    @property
    def panels(self):
        # one GPU needs no transport, so it multiplies in one piece
        if self.world == 1:
            return k_panels(self.k, self.k)
        if self.kp is None:
            nb = max(column_block(self.n, self.world, r)[1] - column_block(self.n, self.world, r)[0] for r in range(self.world))
            return planned_panels(self.m, nb, self.k, self.world, self.first or 1024)[0]
        return k_panels(self.k, self.kp, self.first)


def run_panels(plan, alpha, beta, A_panel, recv_panel, gemm):
    """Drive one sharded product (the schedule csrc/mg_dgemm.cu implements, with everything injected).

    A_panel(l0, l1)      -> handle of the local buffer that holds / will hold A[:, l0:l1]
    recv_panel(h, l0, l1)-> makes that panel present on this rank (broadcast from the root);
                            returns a waitable or None
    gemm(h, l0, l1, beta_l, waitable) -> queues C_r <- alpha*A[:, l0:l1]*B_r[l0:l1, :] + beta_l*C_r
    """
    j0, j1 = plan.cols
    pending = []
    for (l0, l1) in plan.panels:
        h = A_panel(l0, l1)
        w = recv_panel(h, l0, l1) if plan.world > 1 else None
        pending.append((h, l0, l1, w))
    first = True
    for (h, l0, l1, w) in pending:
        if j1 > j0:
            gemm(h, l0, l1, beta if first else 1.0, w)
        elif w is not None and hasattr(w, "wait"):
            w.wait()
        first = False
    return j0, j1


class ShardedDgemm:
    """ulmb200_mg_dgemm / ulmb200_mg_dgemm_host on torch buffers (column-major, as the BLAS sees them).

    A  : torch.float64 CUDA tensor of shape (k, m) on every rank (column-major m x k, ld = m);
         only the root's copy needs to hold data before ``run``.
    Br : (nr, k)  this rank's column block of B  (column-major k x nr, ld = k)
    Cr : (nr, m)  this rank's column block of C  (column-major m x nr, ld = m)
    """

    def __init__(self, m, n, k, first=1024, group=None, root=0, reserve_sms=8, **_ignored):
        import torch
        import torch.distributed as dist
        from . import api
        self.torch, self.dist, self.api = torch, dist, api
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.group, self.root = group, root
        self.m, self.n, self.k = m, n, k
        self.plan = PanelPlan(m, n, k, self.world, self.rank, None, first)
        ident = None
        if self.world > 1:
            box = [None]
            if self.rank == root:
                buf = C.create_string_buffer(128)
                api._check(api.lib.ulmb200_mg_unique_id(buf), "ulmb200_mg_unique_id")
                box = [buf.raw]
            dist.broadcast_object_list(box, src=root, group=group)
            ident = box[0]
        import os
        os.environ.setdefault("ULMB200_MG_RESERVE_SMS", str(reserve_sms))
        os.environ.setdefault("ULMB200_MG_FIRST_PANEL", str(first))
        self.handle = C.c_void_p()
        api._check(api.lib.ulmb200_mg_init(ident, self.rank, self.world, C.byref(self.handle)), "ulmb200_mg_init")

    def close(self):
        if getattr(self, "handle", None):
            self.api.lib.ulmb200_mg_finalize(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:      # noqa: BLE001 - interpreter shutdown
            pass

    def profile(self, on=True):
        self.api.lib.ulmb200_mg_profile(self.handle, 1 if on else 0)

    def last_gemm_ms(self):
        ms = (C.c_double * 32)()
        n = self.api.lib.ulmb200_mg_last_gemm_ms(self.handle, ms, 32)
        return [float(ms[i]) for i in range(max(n, 0))]

    def last_gemm_start_ms(self):
        """Start of each product of the last call, in ms after its first transfer was queued (world > 1)."""
        ms = (C.c_double * 32)()
        n = self.api.lib.ulmb200_mg_last_gemm_start_ms(self.handle, ms, 32)
        return [float(ms[i]) for i in range(max(n, 0))]

    def last_step_gap_ms(self):
        """ms between the end of the previous call's last product and the start of the last call's transfers
        (None unless the two latest calls were device-resident, profiled and on more than one rank)."""
        ms = (C.c_double * 1)()
        return float(ms[0]) if self.api.lib.ulmb200_mg_last_step_gap_ms(self.handle, ms) == 0 else None

    def last_plan(self):
        """(widths, reserve flags, measured device transport GB/s, measured host transport GB/s) of the last call."""
        w, r = (C.c_int64 * 32)(), (C.c_int * 32)()
        dr, hr = C.c_double(0.0), C.c_double(0.0)
        n = self.api.lib.ulmb200_mg_last_plan(self.handle, w, r, 32, C.byref(dr), C.byref(hr))
        return [int(w[i]) for i in range(max(n, 0))], [int(r[i]) for i in range(max(n, 0))], dr.value, hr.value

    def wait(self, timeout_ms=-1):
        return self.api.lib.ulmb200_mg_wait(self.handle, int(timeout_ms))

    def run(self, alpha, A, Br, beta, Cr, host=None, every_rank_has_a=False):
        """One sharded product, queued behind the current torch stream, which continues after it.

        host = (hA, hB, hC): page-locked host tensors shaped like A (required on the root; on the other
        ranks too when every_rank_has_a), Br and Cr.  It makes the call end to end: A goes host -> device
        panel by panel ahead of its transport, this rank's block of B with it, and the block of C
        returns in column pieces while the last panel is still being multiplied."""
        torch, api = self.torch, self.api
        j0, j1 = self.plan.cols
        s = torch.cuda.current_stream().cuda_stream
        m, n, k = self.m, self.n, self.k
        if host is None:
            st = api.lib.ulmb200_mg_dgemm(self.handle, s, m, n, k, alpha, A.data_ptr(), m, Br.data_ptr(), k, beta,
                                          Cr.data_ptr(), m, self.root)
        else:
            hA, hB, hC = host
            st = api.lib.ulmb200_mg_dgemm_host(self.handle, s, m, n, k, alpha, hA.data_ptr() if hA is not None else None, m,
                                               hB.data_ptr(), k, beta, hC.data_ptr(), m, A.data_ptr(), Br.data_ptr(), k,
                                               Cr.data_ptr(), m, self.root, 1 if every_rank_has_a else 0)
        api._check(st, "ulmb200_mg_dgemm")
        return j0, j1


# ---------------------------------------------------------------------------
# Triangular solve split over the GPUs
# ---------------------------------------------------------------------------
# op(A) X = alpha B (left) has independent columns of B, X op(A) = alpha B (right) independent
# rows: rank r keeps a column block (left) or a row block (right) of B and overwrites it with
# its part of X.  Only A travels.  The solve walks A by column panels J -- contiguous in
# column-major storage, so each is one broadcast -- and every one of the eight
# side/uplo/trans cases needs exactly column panel J at step J:
#
#   left,  no trans   solve X_J with A[J,J];  then  B[rest,:] -= A[rest,J]   X_J      (right-looking)
#   left,  trans      B[J,:] -= A[rest,J]^T X_rest;  then solve X_J with A[J,J]^T     (left-looking)
#   right, no trans   B[:,J] -= X_rest A[rest,J];    then solve X_J with A[J,J]       (left-looking)
#   right, trans      solve X_J with A[J,J]^T; then B[:,rest] -= X_J A[rest,J]^T      (right-looking)
#
# with rest = the rows of the panel below J when A is stored lower, above J when stored upper.
# The reference reaches the same eight cases by swapping strides in front of two drivers
# (interfaces/blas/F77/trsm.cc:183-227) and blocks each by MC (ulmblas/level3/trlsm.tcc:66-88).

@dataclass
class TrsmStep:
    j0: int
    j1: int
    r0: int            # rest = [r0, r1)
    r1: int
    update_first: bool  # left-looking: the update precedes the solve of the block


def trsm_panel_widths(na, kp, grow=False):
    """Widths of the panels in the order they are processed.  With `grow` the walk starts with two
    panels of kp and doubles from there (kp, kp, 2kp, 4kp, ...): the first panel, whose transfer
    nothing can hide, stays small, while later steps are large enough to run at full rate."""
    out, left, w, count = [], na, max(1, kp), 0
    while left > 0:
        take = min(w, left)
        out.append(take)
        left -= take
        count += 1
        if grow and count >= 2:
            w *= 2
    return out


def trsm_steps(right, lower, trans, na, kp, grow=False):
    """Ordered steps of the panelled solve with a triangle of order `na` and first panel width `kp`."""
    if na <= 0:
        return []
    eff_lower = bool(lower) != bool(trans)
    forward = eff_lower if not right else (not eff_lower)
    update_first = bool(trans) if not right else (not bool(trans))
    out, pos = [], (0 if forward else na)
    kp = max(1, min(kp, na))
    widths = trsm_panel_widths(na, kp, grow)
    if not forward and na % kp:
        # a backward walk takes the ragged piece first, so that every boundary stays a multiple of kp
        widths = [na % kp] + trsm_panel_widths(na - na % kp, kp, grow)
    for w in widths:
        j0, j1 = (pos, pos + w) if forward else (pos - w, pos)
        pos = j1 if forward else j0
        r0, r1 = (j1, na) if lower else (0, j0)
        out.append(TrsmStep(j0, j1, r0, r1, update_first))
    return out


def row_block(m, world, rank, align=ALIGN):
    """Row blocks of the right-side solve: same cut as the column blocks."""
    return column_block(m, world, rank, align)


def run_trsm_panels(steps, world, A_panel, recv_panel, solve, update):
    """Drive one sharded solve.

    A_panel(j0, j1)        -> handle of the local buffer that holds / will hold A[:, j0:j1]
    recv_panel(h, j0, j1)  -> makes that panel present on this rank; returns a waitable or None
    solve(h, step, waitable)   -> queues the solve of block J with the panel's diagonal block
    update(h, step, waitable)  -> queues the update that uses A[rest, J]   (skipped when rest is empty)
    The first of the two that a step queues gets the panel's waitable, the second gets None.
    All broadcasts are queued before the first arithmetic, in the order the steps need them.
    """
    pending = []
    for s in steps:
        h = A_panel(s.j0, s.j1)
        w = recv_panel(h, s.j0, s.j1) if world > 1 else None
        pending.append((h, s, w))
    for (h, s, w) in pending:
        have_rest = s.r1 > s.r0
        if s.update_first and have_rest:
            update(h, s, w)
            solve(h, s, None)
        else:
            solve(h, s, w)
            if have_rest:
                update(h, s, None)


class ShardedDtrsm:
    """Device-resident sharded DTRSM on torch CUDA buffers (column-major, as the BLAS sees them).

    A  : torch.float64 tensor of shape (na, na) on every rank (column-major, ld = na; element
         (i, j) at A[j, i]); only the root's copy needs to hold data before ``run``.
    Bl : left  side: (nr, m) this rank's column block of B (column-major m x nr, ld = m)
         right side: (n, mr) this rank's row block of B    (column-major mr x n, ld = mr)
    """

    def __init__(self, right, lower, trans, unit, m, n, kp=512, grow=True, group=None, root=0,
                 reserve_sms=8, force_panels=False):
        import torch
        import torch.distributed as dist
        from . import api
        self.torch, self.dist, self.api = torch, dist, api
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.group, self.root = group, root
        self.right, self.lower, self.trans, self.unit = bool(right), bool(lower), bool(trans), bool(unit)
        self.m, self.n = m, n
        self.na = n if right else m
        self.block = row_block(m, self.world, self.rank) if right else column_block(n, self.world, self.rank)
        # one GPU has nothing to wait for: one call, unless a test asks for the panelled walk
        self.panelled = self.world > 1 or force_panels
        self.steps = trsm_steps(right, lower, trans, self.na, kp, grow) if self.panelled else []
        self.compute = torch.cuda.Stream()
        self.comm = torch.cuda.Stream()
        self.reserve_sms = reserve_sms if self.world > 1 else 0

    def run(self, alpha, A, Bl):
        torch, dist, api = self.torch, self.dist, self.api
        b0, b1 = self.block
        nb = b1 - b0                                  # my columns (left) or rows (right)
        na = self.na
        ldb = na if not self.right else max(nb, 1)
        cur = torch.cuda.current_stream()
        self.compute.wait_stream(cur)
        self.comm.wait_stream(cur)
        cs = self.compute.cuda_stream
        pB = Bl.data_ptr()
        side = 1 if self.right else 0

        if not self.panelled:
            if nb > 0:
                with torch.cuda.stream(self.compute):
                    if self.right:
                        api.dev_dtrsm(1, self.lower, self.trans, self.unit, nb, na, alpha, A.data_ptr(), na, pB, ldb, stream=cs)
                    else:
                        api.dev_dtrsm(0, self.lower, self.trans, self.unit, na, nb, alpha, A.data_ptr(), na, pB, ldb, stream=cs)
            cur.wait_stream(self.compute)
            return b0, b1

        if nb > 0 and alpha != 1.0:
            # B <- alpha B once, then every step works with alpha = 1 (a product with k = 0 only scales)
            rows, cols = (nb, na) if self.right else (na, nb)
            with torch.cuda.stream(self.compute):
                api.dev_dgemm(0, 0, rows, cols, 0, 0.0, pB, max(rows, 1), pB, 1, alpha, pB, ldb, stream=cs)

        def A_panel(j0, j1):
            return A[j0:j1, :]

        def recv_panel(h, j0, j1):
            with torch.cuda.stream(self.comm):
                return dist.broadcast(h, src=self.root, group=self.group, async_op=True)

        done = [0]
        nsteps = len(self.steps)

        def reserve():
            # leave SMs to the transport while panels are still on their way (first half of the walk)
            api.set_sm_reserve(self.reserve_sms if 2 * done[0] < nsteps else 0)

        def el(i, j, base, ld):                        # address of element (i, j)
            return base + 8 * (i + j * ld)

        pA = A.data_ptr()

        def solve(h, s, w):
            with torch.cuda.stream(self.compute):
                if w is not None:
                    w.wait()
                if nb == 0:
                    return
                reserve()
                jb = s.j1 - s.j0
                if self.right:
                    api.dev_dtrsm(1, self.lower, self.trans, self.unit, nb, jb, 1.0, el(s.j0, s.j0, pA, na), na,
                                  el(0, s.j0, pB, ldb), ldb, stream=cs)
                else:
                    api.dev_dtrsm(0, self.lower, self.trans, self.unit, jb, nb, 1.0, el(s.j0, s.j0, pA, na), na,
                                  el(s.j0, 0, pB, ldb), ldb, stream=cs)
                done[0] += 1

        def update(h, s, w):
            with torch.cuda.stream(self.compute):
                if w is not None:
                    w.wait()
                if nb == 0:
                    return
                reserve()
                jb, nrest = s.j1 - s.j0, s.r1 - s.r0
                a_rest = el(s.r0, s.j0, pA, na)                     # A[rest, J]
                if not self.right and not self.trans:               # B[rest,:] -= A[rest,J] B[J,:]
                    api.dev_dgemm(0, 0, nrest, nb, jb, -1.0, a_rest, na, el(s.j0, 0, pB, ldb), ldb, 1.0,
                                  el(s.r0, 0, pB, ldb), ldb, stream=cs)
                elif not self.right:                                # B[J,:] -= A[rest,J]^T B[rest,:]
                    api.dev_dgemm(1, 0, jb, nb, nrest, -1.0, a_rest, na, el(s.r0, 0, pB, ldb), ldb, 1.0,
                                  el(s.j0, 0, pB, ldb), ldb, stream=cs)
                elif not self.trans:                                # B[:,J] -= B[:,rest] A[rest,J]
                    api.dev_dgemm(0, 0, nb, jb, nrest, -1.0, el(0, s.r0, pB, ldb), ldb, a_rest, na, 1.0,
                                  el(0, s.j0, pB, ldb), ldb, stream=cs)
                else:                                               # B[:,rest] -= B[:,J] A[rest,J]^T
                    api.dev_dgemm(0, 1, nb, nrest, jb, -1.0, el(0, s.j0, pB, ldb), ldb, a_rest, na, 1.0,
                                  el(0, s.r0, pB, ldb), ldb, stream=cs)

        run_trsm_panels(self.steps, self.world, A_panel, recv_panel, solve, update)
        api.set_sm_reserve(0)
        cur.wait_stream(self.compute)
        cur.wait_stream(self.comm)
        return b0, b1
