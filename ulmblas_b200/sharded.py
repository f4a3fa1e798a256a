"""Large DGEMM split over the GPUs of one box by column blocks of C.

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

    def run(self, alpha, A, Br, beta, Cr):
        torch, dist, api, p = self.torch, self.dist, self.api, self.plan
        j0, j1 = p.cols
        nr = j1 - j0
        cur = torch.cuda.current_stream()
        self.compute.wait_stream(cur)
        self.comm.wait_stream(cur)

        def A_panel(l0, l1):
            return A[l0:l1, :]                      # rows of the (k, m) tensor = columns l0..l1 of A

        def recv_panel(h, l0, l1):
            with torch.cuda.stream(self.comm):
                return dist.broadcast(h, src=self.root, group=self.group, async_op=True)

        launched = [0]

        def gemm(h, l0, l1, beta_l, w):
            api.set_sm_reserve(self.reserve_sms if launched[0] < self.reserve_panels else 0)
            launched[0] += 1
            with torch.cuda.stream(self.compute):
                if w is not None:
                    w.wait()                         # compute stream waits for the panel, host does not
                ev = None
                if self.kernel_events is not None:
                    ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                    ev[0].record(self.compute)
                api.dev_dgemm(0, 0, p.m, nr, l1 - l0, alpha, h.data_ptr(), p.m,
                              Br.data_ptr() + 8 * l0, p.k, beta_l, Cr.data_ptr(), p.m,
                              stream=self.compute.cuda_stream)
                if ev is not None:
                    ev[1].record(self.compute)
                    self.kernel_events.append((ev[0], ev[1], 2.0 * p.m * nr * (l1 - l0)))

        run_panels(p, alpha, beta, A_panel, recv_panel, gemm)
        api.set_sm_reserve(0)
        cur.wait_stream(self.compute)
        cur.wait_stream(self.comm)
        return j0, j1
