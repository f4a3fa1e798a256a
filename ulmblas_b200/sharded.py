"""Large DGEMM (and, further down, DTRSM) split over the GPUs of one box by column blocks of C.

    C[:, J_r] <- alpha * A * B[:, J_r] + beta * C[:, J_r]        on rank r

One process per GPU (``torch.distributed``, NCCL).  Rank r owns the column block J_r of B
and C for good; A lives on the root rank and reaches the others by NCCL broadcast over
NVLink, cut into K-panels A[:, l*kp:(l+1)*kp] (contiguous in column-major storage).  The
broadcasts are queued ahead on NCCL's stream; the product of panel l is queued on the
compute stream behind "panel l has arrived", so panel l+1 travels while panel l
multiplies.  There is no reduction and no other exchange: columns of C are independent.

The reference has no multi-device path (it is single-threaded CPU code); the partition
follows its own loop order, which already walks C by column blocks
(ulmblas/level3/gemm.tcc:60).

The arithmetic is injected (``gemm`` callable) so that the partitioning and the panel
schedule can be exercised on CPU ranks with the gloo backend by the tests; the product
path always passes the library's device GEMM.
"""
from dataclasses import dataclass

ALIGN = 128          # column blocks start on CTA-tile boundaries


def column_block(n, world, rank, align=ALIGN):
    """[j0, j1) of rank `rank`: near-equal blocks whose starts are multiples of `align`."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad world/rank")
    units = (n + align - 1) // align
    base, extra = divmod(units, world)
    u0 = rank * base + min(rank, extra)
    u1 = u0 + base + (1 if rank < extra else 0)
    return min(u0 * align, n), min(u1 * align, n)


def k_panels(k, kp, first=None):
    """[(l0, l1)] covering [0, k): an optional short first panel (so the first product can start
    early), then panels of kp (the last may be short)."""
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


def two_phase_plan(panels, k, nr, npieces=8, align=ALIGN):
    """(number of leading panels applied to the whole column block, [(c0, cn)] column pieces that take the
    remaining panels one piece at a time).  The first phase covers the first quarter to third of K --
    about the time the root needs to bring A in -- and always leaves at least one panel for the second."""
    covered, n1 = 0, 0
    while n1 < len(panels) - 1 and covered * 4 < k:
        covered += panels[n1][1] - panels[n1][0]
        n1 += 1
    q = max(align, ((nr + npieces - 1) // npieces + align - 1) // align * align)
    pieces = [(c0, min(q, nr - c0)) for c0 in range(0, nr, q)]
    return n1, pieces


@dataclass
class PanelPlan:
    m: int
    n: int
    k: int
    world: int
    rank: int
    kp: int
    first: int = None

    @property
    def cols(self):
        return column_block(self.n, self.world, self.rank)

    @property
    def panels(self):
        # one GPU needs no transport, so it multiplies in one piece
        if self.world == 1:
            return k_panels(self.k, self.k)
        return k_panels(self.k, self.kp, self.first)


def run_panels(plan, alpha, beta, A_panel, recv_panel, gemm):
    """Drive one sharded product.

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
    """Device-resident sharded DGEMM on torch CUDA buffers (column-major, as the BLAS sees them).

    A  : torch.float64 tensor of shape (k, m) on every rank (column-major m x k, ld = m);
         only the root's copy needs to hold data before ``run``.
    Br : (nr, k)  this rank's column block of B  (column-major k x nr, ld = k)
    Cr : (nr, m)  this rank's column block of C  (column-major m x nr, ld = m)
    """

    def __init__(self, m, n, k, kp=4096, first=1024, group=None, root=0, reserve_sms=8, reserve_panels=2):
        import torch
        import torch.distributed as dist
        from . import api
        self.torch, self.dist, self.api = torch, dist, api
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.group, self.root = group, root
        self.plan = PanelPlan(m, n, k, self.world, self.rank, kp, first)
        self.compute = torch.cuda.Stream()
        self.comm = torch.cuda.Stream()
        # when set to a list, run() appends (start_event, end_event, flops) per GEMM launch,
        # recorded on the launching stream
        self.kernel_events = None
        # While panels are still travelling, the GEMMs leave a few SMs free so that NCCL's
        # kernels can always be scheduled next to the persistent grid (bench.py caps NCCL at
        # the same number of CTAs); later GEMMs take the whole GPU again.
        self.reserve_sms = reserve_sms if self.world > 1 else 0
        self.reserve_panels = reserve_panels

    def run(self, alpha, A, Br, beta, Cr, host=None):
        """One sharded product on device buffers.

        host = (hA, hB, hC), pinned host tensors shaped like A (root only, else None), Br and Cr, makes it
        an end-to-end call: the root's A goes host -> device panel by panel, each panel broadcast as soon
        as it has landed (the first product waits for one panel, not for all of A); every rank copies its
        own block of B in (and of C, when beta != 0), and its block of C back out in four column pieces,
        each as soon as the last panel's product of that piece is done.  Returns when the device work
        is queued; the caller synchronises."""
        torch, dist, api, p = self.torch, self.dist, self.api, self.plan
        j0, j1 = p.cols
        nr = j1 - j0
        cur = torch.cuda.current_stream()
        self.compute.wait_stream(cur)
        self.comm.wait_stream(cur)
        hA = hB = hC = None
        if host is not None:
            hA, hB, hC = host
            if not hasattr(self, "h2d"):
                self.h2d, self.d2h = torch.cuda.Stream(), torch.cuda.Stream()
            self.h2d.wait_stream(cur)
            self.d2h.wait_stream(cur)
            with torch.cuda.stream(self.h2d):
                if nr > 0:
                    Br.copy_(hB, non_blocking=True)
                    if beta != 0.0:
                        Cr.copy_(hC, non_blocking=True)
            self.compute.wait_stream(self.h2d)       # B (and C) of this rank before its first product

        def A_panel(l0, l1):
            return A[l0:l1, :]                      # rows of the (k, m) tensor = columns l0..l1 of A

        def stage_panel(h, l0, l1):
            if hA is not None and self.rank == self.root:
                with torch.cuda.stream(self.h2d):
                    h.copy_(hA[l0:l1, :], non_blocking=True)
                self.comm.wait_stream(self.h2d)      # the broadcast (or the product) follows the copy

        def recv_panel(h, l0, l1):
            stage_panel(h, l0, l1)
            with torch.cuda.stream(self.comm):
                return dist.broadcast(h, src=self.root, group=self.group, async_op=True)

        launched = [0]
        npanels = len(p.panels)

        def gemm(h, l0, l1, beta_l, w):
            api.set_sm_reserve(self.reserve_sms if launched[0] < self.reserve_panels else 0)
            launched[0] += 1
            last = launched[0] == npanels
            with torch.cuda.stream(self.compute):
                if w is not None:
                    w.wait()                         # compute stream waits for the panel, host does not
                ev = None
                if self.kernel_events is not None:
                    ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                    ev[0].record(self.compute)
                # the last panel's product goes by column pieces when C returns to the host, so that
                # each piece can leave while the next is still being multiplied
                pieces = [(0, nr)]
                if last and hC is not None and nr >= 4 * ALIGN:
                    q = ((nr + 3) // 4 + ALIGN - 1) // ALIGN * ALIGN
                    pieces = [(c0, min(q, nr - c0)) for c0 in range(0, nr, q)]
                for (c0, cn) in pieces:
                    api.dev_dgemm(0, 0, p.m, cn, l1 - l0, alpha, h.data_ptr(), p.m,
                                  Br.data_ptr() + 8 * (l0 + c0 * p.k), p.k, beta_l, Cr.data_ptr() + 8 * c0 * p.m, p.m,
                                  stream=self.compute.cuda_stream)
                    if last and hC is not None:
                        done = torch.cuda.Event()
                        done.record(self.compute)
                        self.d2h.wait_event(done)
                        with torch.cuda.stream(self.d2h):
                            hC[c0:c0 + cn, :].copy_(Cr[c0:c0 + cn, :], non_blocking=True)
                if ev is not None:
                    ev[1].record(self.compute)
                    self.kernel_events.append((ev[0], ev[1], 2.0 * p.m * nr * (l1 - l0)))

        if self.world == 1:
            # one piece (or, with host staging, the same panels as the copy of A)
            if hA is None:
                run_panels(p, alpha, beta, A_panel, recv_panel, gemm)
            else:
                pans = k_panels(p.k, p.kp, p.first)
                npanels = len(pans)
                for i, (l0, l1) in enumerate(pans):
                    h = A_panel(l0, l1)
                    stage_panel(h, l0, l1)
                    self.compute.wait_stream(self.h2d)
                    if nr > 0:
                        gemm(h, l0, l1, beta if i == 0 else 1.0, None)
        elif hC is None or nr < 8 * ALIGN or len(p.panels) < 3:
            run_panels(p, alpha, beta, A_panel, recv_panel, gemm)
        else:
            self._run_host_two_phase(alpha, beta, A, Br, Cr, hC, A_panel, recv_panel)
        api.set_sm_reserve(0)
        cur.wait_stream(self.compute)
        cur.wait_stream(self.comm)
        if host is not None:
            cur.wait_stream(self.h2d)
            cur.wait_stream(self.d2h)
        return j0, j1


    def _run_host_two_phase(self, alpha, beta, A, Br, Cr, hC, A_panel, recv_panel):
        """End-to-end order of the products when C has to go back to the host.

        Panel by panel, C is complete only after the last panel, so its copy back could overlap nothing
        but that last product.  Here the first panels (about the time A needs to arrive) are still
        applied to the whole block, and the remaining ones column piece by column piece: piece j is
        complete -- and leaves for the host -- after (j+1)/J of that second phase, so the copies spread
        over most of the run."""
        torch, api, p = self.torch, self.api, self.plan
        j0, j1 = p.cols
        nr = j1 - j0
        pans = list(p.panels)
        pending = []
        for (l0, l1) in pans:
            h = A_panel(l0, l1)
            pending.append((h, l0, l1, recv_panel(h, l0, l1)))
        n1, pieces = two_phase_plan(pans, p.k, nr)
        cs = self.compute.cuda_stream

        def product(h, l0, l1, c0, cn, beta_l):
            api.dev_dgemm(0, 0, p.m, cn, l1 - l0, alpha, h.data_ptr(), p.m, Br.data_ptr() + 8 * (l0 + c0 * p.k), p.k,
                          beta_l, Cr.data_ptr() + 8 * c0 * p.m, p.m, stream=cs)

        with torch.cuda.stream(self.compute):
            for i, (h, l0, l1, w) in enumerate(pending[:n1]):
                api.set_sm_reserve(self.reserve_sms if i < self.reserve_panels else 0)
                if w is not None:
                    w.wait()
                product(h, l0, l1, 0, nr, beta if i == 0 else 1.0)
            api.set_sm_reserve(0)
            for (h, l0, l1, w) in pending[n1:]:
                if w is not None:
                    w.wait()                      # all of A is here before the second phase starts
            for (c0, cn) in pieces:
                for (h, l0, l1, w) in pending[n1:]:
                    product(h, l0, l1, c0, cn, 1.0)
                done = torch.cuda.Event()
                done.record(self.compute)
                self.d2h.wait_event(done)
                with torch.cuda.stream(self.d2h):
                    hC[c0:c0 + cn, :].copy_(Cr[c0:c0 + cn, :], non_blocking=True)


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
