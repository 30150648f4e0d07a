"""Sharding of the two configurations of the path that partition across the GPUs of one box.

The reference engine is single-GPU; these are the partitionings of its two workloads that shard across GPUs:

* 27B-class FFN, tensor parallel: gate/up column-parallel (a rank owns a slice of gate rows AND the matching up
  rows, so the SwiGLU epilogue stays local), down row-parallel with f32 partial products, one all-reduce (sum)
  before the single rounding and the residual add.
* MoE block, expert parallel: experts partitioned contiguously, token rows data-parallel; the token rows of every
  routed (row, slot) pair travel to the rank that owns the pair's expert (all-to-all), are sorted and multiplied
  there, and the expert outputs travel back (all-to-all) to be combined in slot order at home.

One process per GPU; the plumbing is torch.distributed (NCCL on GPUs; the same code runs on gloo with CPU tensors
for the host-logic tests). Every kernel reads and writes only its own GPU's memory: remote rows land in local
buffers through the collective before any kernel touches them.

The arithmetic is behind a small backend object so that the sharding and exchange logic here is the same code in
production (GpuBackend: the CUDA kernels through the C ABI) and in the CPU tests (a backend the tests supply).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

OUT_BF16, OUT_F32, OUT_RESIDUAL, OUT_SWIGLU = range(4)


# --------------------------------------------------------------------------- tensor-parallel FFN

def shard_gate_up(wgu: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """[gate(inter) | up(inter)] rows -> this rank's [gate slice | up slice] (column-parallel)."""
    inter = wgu.shape[0] // 2
    assert inter % world == 0, "intermediate size must divide by the number of ranks"
    ip = inter // world
    return torch.cat([wgu[rank * ip : (rank + 1) * ip], wgu[inter + rank * ip : inter + (rank + 1) * ip]], dim=0).contiguous()


def shard_down(wd: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Wdown [h][inter] -> this rank's K slice as its own contiguous [h][inter/world] matrix (row-parallel)."""
    inter = wd.shape[1]
    assert inter % world == 0
    ip = inter // world
    return wd[:, rank * ip : (rank + 1) * ip].contiguous()


def tp_ffn(backend, x, wgu_local, wd_local, y, group=None):
    """y = bf16(y + bf16(sum over ranks of H_r . Wd_r^T)), H_r = swiglu(x . Wgu_r^T). x is replicated."""
    h_local = backend.gemm(x, wgu_local, OUT_SWIGLU)
    acc = backend.gemm(h_local, wd_local, OUT_F32)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=group)
    backend.epilogue(acc, y, OUT_RESIDUAL)
    return y


# --------------------------------------------------------------------------- expert-parallel MoE

def exchange_rows(send: torch.Tensor, send_counts, recv_counts, group=None) -> torch.Tensor:
    """Variable all-to-all of rows: chunk d of `send` (send_counts[d] rows) goes to rank d; the result holds the
    chunks received from ranks 0..P-1 in rank order."""
    world = dist.get_world_size(group)
    if send.dtype == torch.bfloat16 and dist.get_backend(group) != "nccl":
        return exchange_rows(send.view(torch.int16), send_counts, recv_counts, group).view(torch.bfloat16)
    recv = send.new_empty((int(sum(recv_counts)),) + tuple(send.shape[1:]))
    if dist.get_backend(group) == "nccl":
        dist.all_to_all_single(recv, send, output_split_sizes=[int(c) for c in recv_counts], input_split_sizes=[int(c) for c in send_counts], group=group)
        return recv
    # gloo has no all-to-all: pairwise sends in a fixed schedule
    rank = dist.get_rank(group)
    s_off = [0]
    r_off = [0]
    for d in range(world):
        s_off.append(s_off[-1] + int(send_counts[d]))
        r_off.append(r_off[-1] + int(recv_counts[d]))
    recv[r_off[rank] : r_off[rank + 1]] = send[s_off[rank] : s_off[rank + 1]]
    ops = []
    for d in range(world):
        if d == rank:
            continue
        if send_counts[d]:
            ops.append(dist.P2POp(dist.isend, send[s_off[d] : s_off[d + 1]].contiguous(), d, group))
        if recv_counts[d]:
            ops.append(dist.P2POp(dist.irecv, recv[r_off[d] : r_off[d + 1]], d, group))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    return recv


def exchange_counts(send_counts: torch.Tensor, group=None) -> torch.Tensor:
    """Every rank tells every other how many rows it will send it (a small all-gather)."""
    world = dist.get_world_size(group)
    allc = [torch.empty_like(send_counts) for _ in range(world)]
    dist.all_gather(allc, send_counts, group=group)
    rank = dist.get_rank(group)
    return torch.stack([c[rank] for c in allc])


def ep_moe(backend, x_local, scores_local, wgu_local, wd_local, experts: int, top_k: int, mi: int, bm: int, group=None, debug=None):
    """The sparse block for this rank's token rows. wgu_local / wd_local hold this rank's experts
    [rank*E/P, (rank+1)*E/P). Returns out_local [rows_local][h]."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    assert experts % world == 0
    epr = experts // world
    rows, h = x_local.shape
    route = backend.route(scores_local, top_k)  # [rows][2*top_k]: experts ascending, then weight bits
    # destination rank of every (row, slot) pair; pairs grouped by destination in pair order = a stable counting
    # sort with the destination as the "expert" (the same sort kernel)
    dest = route.clone()
    dest[:, :top_k] = torch.div(route[:, :top_k], epr, rounding_mode="floor")
    send_order, _ = backend.sort(dest, world, top_k, 16)  # list of local pair ids
    send_counts = torch.bincount(dest[:, :top_k].reshape(-1).long(), minlength=world).to(torch.int64)
    if world > 1:
        recv_counts = exchange_counts(send_counts, group)
    else:
        recv_counts = send_counts.clone()
    send_counts_l, recv_counts_l = send_counts.tolist(), recv_counts.tolist()
    # rows and their (local) expert ids, packed in send order
    send_rows = backend.gather(x_local, send_order, top_k)  # [pairs][h]: X[pair // top_k]
    pair_expert = route[:, :top_k].reshape(-1)
    send_expert = (pair_expert[send_order.long()] % epr).to(torch.int32).reshape(-1, 1).contiguous()
    if world > 1:
        recv_rows = exchange_rows(send_rows, send_counts_l, recv_counts_l, group)
        recv_expert = exchange_rows(send_expert, send_counts_l, recv_counts_l, group)
    else:
        recv_rows, recv_expert = send_rows, send_expert
    n_recv = recv_rows.shape[0]
    if n_recv:
        # every received pair is a one-slot row of a local route: [expert | weight unused]
        local_route = torch.zeros((n_recv, 2), dtype=route.dtype, device=route.device)
        local_route[:, 0] = recv_expert.reshape(-1).to(route.dtype)
        lst, tiles = backend.sort(local_route, epr, 1, bm)
        ey_recv = backend.expert_ffn(recv_rows, wgu_local, wd_local, lst, tiles, epr, mi, h, bm)  # rows in receive order
    else:
        lst = torch.zeros(0, dtype=route.dtype, device=route.device)
        ey_recv = recv_rows.new_zeros((0, h))
    if debug is not None:
        debug.update(route=route, send_order=send_order, recv_expert=recv_expert, local_list=lst, send_counts=send_counts_l, recv_counts=recv_counts_l)
    if world > 1:
        ey_back = exchange_rows(ey_recv, recv_counts_l, send_counts_l, group)  # in this rank's send order
    else:
        ey_back = ey_recv
    # EY[pair] = ey_back[position of pair in the send order]
    inv = torch.empty_like(send_order)
    inv[send_order.long()] = torch.arange(send_order.numel(), dtype=send_order.dtype, device=send_order.device)
    ey = backend.gather(ey_back, inv, 1)  # [pairs][h] indexed by pair = row*top_k + slot
    return backend.combine(ey, route, top_k)


# --------------------------------------------------------------------------- the CUDA backend

class GpuBackend:
    """The backend that runs the CUDA kernels of libhb200.so on torch CUDA tensors (device memory and stream
    plumbing only). `hb` is the loaded binding module, `ctx` its Context bound to torch's current stream."""

    def __init__(self, hb, ctx, rows_max: int = 2048):
        self.hb, self.ctx, self.rows_max = hb, ctx, rows_max

    def _w(self, t):
        assert t.is_cuda and t.is_contiguous()
        return self.ctx.wrap(t.data_ptr(), max(t.numel() * t.element_size(), 1))

    def gemm(self, x, w, out, y=None):
        m, k = x.shape
        n = w.shape[0]
        if y is None:
            y = torch.empty((m, n // 2 if out == OUT_SWIGLU else n), device=x.device, dtype=torch.float32 if out == OUT_F32 else torch.bfloat16)
        self.ctx.gemm(k, n, out, rows_max=max(m, self.rows_max))(m, self._w(w), self._w(x), self._w(y))
        return y

    def epilogue(self, acc, y, out):
        m, n = acc.shape
        self.ctx.epilogue(n, out)(m, self._w(acc), self._w(y))
        return y

    def route(self, scores, top_k):
        m, e = scores.shape
        route = torch.empty((m, 2 * top_k), device=scores.device, dtype=torch.int32)
        self.ctx.route(e, top_k)(m, self._w(scores), self._w(route))
        return route

    def sort(self, route, experts, top_k, bm):
        m = route.shape[0]
        lst = torch.empty(m * top_k, device=route.device, dtype=torch.int32)
        tiles = torch.zeros(1 + 3 * self.hb.lib().hb_moe_tiles(m, top_k, experts, bm), device=route.device, dtype=torch.int32)
        rows_max = 1 << max(m - 1, 0).bit_length()  # kernels are named by their capacity: round it up so few are made
        self.ctx.moe_sort(experts, top_k, rows_max, bm)(m, self._w(route.contiguous()), self._w(lst), self._w(tiles))
        return lst, tiles

    def gather(self, x, lst, top_k):
        pairs, h = lst.numel(), x.shape[1]
        xs = torch.empty((pairs, h), device=x.device, dtype=x.dtype)
        if pairs:
            self.ctx.moe_gather(h, top_k)(pairs // top_k, self._w(x), self._w(lst), self._w(xs))
        return xs

    def expert_ffn(self, rows, wgu, wd, lst, tiles, experts, mi, h, bm):
        n = rows.shape[0]
        kw = dict(rows_max=max(n, self.rows_max), top_k=1, experts=experts, bm=bm, merge_runs=1)
        ehb = torch.empty((n, mi), device=rows.device, dtype=torch.bfloat16)
        ey = torch.empty((n, h), device=rows.device, dtype=torch.bfloat16)
        self.ctx.gemm(h, 2 * mi, OUT_SWIGLU, rows_mode=self.hb.ROWS_GATHER, **kw)(n, self._w(wgu), self._w(rows), self._w(ehb), self._w(lst), self._w(tiles))
        self.ctx.gemm(mi, h, OUT_BF16, rows_mode=self.hb.ROWS_SCATTER, **kw)(n, self._w(wd), self._w(ehb), self._w(ey), self._w(lst), self._w(tiles))
        return ey

    def combine(self, ey, route, top_k):
        m, h = route.shape[0], ey.shape[1]
        out = torch.empty((m, h), device=ey.device, dtype=torch.bfloat16)
        self.ctx.moe_combine(h, top_k)(m, self._w(ey), self._w(route), self._w(out))
        return out


# --------------------------------------------------------------------------- expert-parallel MoE over peer memory
#
# The same block as ep_moe with the exchange done by the library's own kernels through NVLink (include/hb200.h,
# "expert-parallel exchange over peer memory"): nothing is read back to the host, no variable-size collective.
# Per rank and call, in the plain form: route, sort by global expert (+ offsets), all-gather of the offsets (1 KB per
# rank), dispatch (stores into the owners' receive buffers), barrier, plan + gate/up + down on the received rows,
# barrier, return (loads from the owners' output buffers), combine. In the default form (EpPeer below) the all-gather
# and both barrier kernels are gone: seven kernels.

def ep_positions_np(offs_all, rank: int, epr: int, region: int = 0):
    """Host mirror of the dispatch / return index arithmetic: for every sorted position p of `rank`, the
    destination rank and the row in that rank's receive buffer. offs_all: int array [world][experts + 1].
    region > 0: the direct form, every source's rows from row source * region of every buffer."""
    import numpy as np

    offs_all = np.asarray(offs_all, dtype=np.int64)
    world = offs_all.shape[0]
    pairs = int(offs_all[rank, -1])
    first = np.array([offs_all[rank, d * epr] for d in range(world)] + [pairs])
    base = np.array([rank * region if region else sum(int(offs_all[s, (d + 1) * epr] - offs_all[s, d * epr]) for s in range(rank)) for d in range(world)])
    p = np.arange(pairs)
    d = np.searchsorted(first[1:], p, side="right")
    return d, base[d] + p - first[d]


def ep_plan_np(offs_all, rank: int, epr: int, bm: int, region: int = 0):
    """Host mirror of the plan kernel: (list, tiles) of `rank`'s experts over its receive buffer (region > 0: the
    direct form, source s's rows from row s * region)."""
    import numpy as np

    offs_all = np.asarray(offs_all, dtype=np.int64)
    world = offs_all.shape[0]
    e0 = rank * epr
    n_from = [int(offs_all[s, e0 + epr] - offs_all[s, e0]) for s in range(world)]
    recvbase = np.arange(world + 1) * region if region else np.concatenate([[0], np.cumsum(n_from)])
    lst, tiles = [], []
    for e in range(epr):
        start = len(lst)
        for s in range(world):
            lo, hi = int(offs_all[s, e0 + e]), int(offs_all[s, e0 + e + 1])
            src0 = int(recvbase[s]) + lo - int(offs_all[s, e0])
            lst.extend(range(src0, src0 + hi - lo))
        total = len(lst) - start
        for j in range(0, total, bm):
            tiles.append((e, start + j, min(bm, total - j)))
    flat = [len(tiles)] + [v for t in tiles for v in t]
    return np.array(lst, dtype=np.uint32), np.array(flat, dtype=np.uint32)


def _view(buf, shape, typestr: str, device) -> torch.Tensor:
    """A torch tensor over a library allocation (no copy)."""
    class _Holder:
        pass

    h = _Holder()
    h.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (buf.ptr, False), "version": 3}
    return torch.as_tensor(h, device=device)


def _launch_now(kernel, m, *ranges):
    kernel(m, *ranges)


class _Recorded:
    """The kernel calls of one step of a peer-memory block, taken down instead of launched, then replayed as one
    recorded sequence (hb_graph_record): a step is 6 to 13 short kernels, and enqueueing them one by one from the
    host takes longer than the GPU needs to run them."""

    def __init__(self, ctx, *emitters, overlap: bool = False):
        # overlap: the sequence is recorded with overlapped launches (hb_set_launch_overlap): every kernel of it must
        # then be one that waits for its predecessor itself before it touches that kernel's outputs
        self.ctx, self.emitters, self.graphs, self.overlap = ctx, emitters, {}, overlap

    def run(self, key, step):
        """step() makes the kernel calls of the step through the emitters; the first time a key is seen they are
        recorded, afterwards (and then too) the recording is launched."""
        if key not in self.graphs:
            ops = []
            for e in self.emitters:
                e.emit = lambda kernel, m, *ranges: ops.append((kernel, m, *ranges))
            try:
                step()
            finally:
                for e in self.emitters:
                    e.emit = _launch_now
            if self.overlap:
                self.ctx.set_launch_overlap(True)
            try:
                self.graphs[key] = self.ctx.record(ops)
            finally:
                if self.overlap:
                    self.ctx.set_launch_overlap(False)
            for e in self.emitters:
                e.kernels_per_step = len(ops)
        else:
            step(replay=True)
        self.graphs[key].launch()

    def close(self):
        for g in self.graphs.values():
            g.free()
        self.graphs = {}


class PeerBuffers:
    """Named buffers of this rank that the other ranks of the node read and write, with the device tables
    (u64[world], one address per rank) the kernels take. A flag array for the barrier kernel is always there."""

    def __init__(self, ctx, rank: int, world: int, sizes: dict, device):
        self.ctx, self.rank, self.world, self.device = ctx, rank, world, device
        self.sizes = dict(sizes, flags=256)
        self.local = {name: ctx.alloc(size) for name, size in self.sizes.items()}
        self.tables = {name: torch.zeros(world, device=device, dtype=torch.int64) for name in self.sizes}
        self.opened = []
        self.emulated = True
        self.emit = _launch_now  # what a kernel call does: launch it, or (while a step is recorded) note it

    def handles(self) -> dict:
        return {name: self.ctx.ipc_export(buf) for name, buf in self.local.items()}

    def connect(self, all_handles=None, local_peers=None) -> None:
        """all_handles: handles() of every rank (other processes); local_peers: the PeerBuffers of every rank when
        all ranks live in this process on this GPU (the tests' emulation: no barrier kernel may run then)."""
        self.emulated = all_handles is None
        for name in self.sizes:
            ptrs = []
            for r in range(self.world):
                if r == self.rank:
                    ptrs.append(self.local[name].ptr)
                elif local_peers is not None:
                    ptrs.append(local_peers[r].local[name].ptr)
                else:
                    b = self.ctx.ipc_open(all_handles[r][name], self.sizes[name])
                    self.opened.append(b)
                    ptrs.append(b.ptr)
            self.tables[name].copy_(torch.tensor(ptrs, dtype=torch.int64))

    def connect_group(self, group=None) -> None:
        if self.world == 1:
            self.connect(local_peers=[self])
            return
        gathered = [None] * self.world
        dist.all_gather_object(gathered, self.handles(), group=group)
        self.connect(all_handles=gathered)
        dist.barrier(group=group)  # every rank has mapped every buffer before the first kernel touches one

    def table(self, name: str):
        t = self.tables[name]
        return self.ctx.wrap(t.data_ptr(), t.numel() * 8)

    def barrier(self) -> None:
        """The barrier kernel on the stream (nothing on one rank or in the emulation)."""
        if self.world == 1 or self.emulated:
            return
        if not hasattr(self, "_k_barrier"):
            self._k_barrier = self.ctx.peer_sync(0, self.world, self.rank)
        self.emit(self._k_barrier, 1, self.table("flags"))  # (the barrier numbers itself)

    def allgather(self, payload: torch.Tensor, name: str) -> None:
        """payload (int32 words) -> slot `rank` of buffer `name` on every rank, then the barrier."""
        words = payload.numel()
        if not hasattr(self, "_k_gather"):
            self._k_gather = {}
        if words not in self._k_gather:
            self._k_gather[words] = self.ctx.peer_sync(words, self.world, self.rank)
        self.emit(self._k_gather[words], 1, self.table("flags"), self.ctx.wrap(payload.data_ptr(), words * 4), self.table(name))

    def close(self) -> None:
        for b in self.opened:
            self.ctx.ipc_close(b)
        self.opened = []


class EpPeer:
    """One rank of the peer-memory MoE block: its buffers, kernels and the four phases between the barriers.

    `ctx` must launch on torch's current stream (Context.set_stream) so that the phases and any collective are
    ordered. `cap` is the number of rows the receive and output buffers hold; the default, every pair of every
    rank, can never overflow.

    fused (the default): the dispatch notes where every pair's output row will be and tells the other ranks when its
    rows have landed; the plan waits for that itself (no barrier kernel between dispatch and expert GEMMs); the return
    and the combine are one kernel that reads every slot's output row from its owner (no EY written and re-read).
    direct (the default with fused, when cap divides by the number of ranks): every source owns a fixed region of every
    receive buffer, so nobody needs anybody's counts to place rows and the all-gather of the offsets before the dispatch
    falls away (the dispatch delivers the offsets itself): route, sort, dispatch, plan, two GEMMs, and a combine that
    carries the barrier "every rank's outputs are complete" itself when every rank is a process of its own.
    fused = False: all-gather, dispatch, barrier, plan, GEMMs, barrier, return into EY, combine.
    With one rank there is nothing to exchange and the step is the plain block (route, sort, the expert GEMMs gathering
    from X and scattering into EY, combine) unless plain_when_alone is False (the exchange kernels with one rank, as the
    tests run them).
    """

    def __init__(self, hb, ctx, rank: int, world: int, rows: int, h: int, mi: int, experts: int, top_k: int, bm: int = 64, cap: int | None = None,
                 device=None, fused: bool = True, plain_when_alone: bool = True, direct: bool | None = None, overlap: bool = False):
        # overlap: record the step with overlapped launches (its kernels wait for their predecessors themselves);
        # measured no faster than plain launches for this block on one B200 (326 us either way), so off unless asked for
        assert experts % world == 0
        self.hb, self.ctx, self.rank, self.world = hb, ctx, rank, world
        self.rows, self.h, self.mi, self.experts, self.top_k, self.bm = rows, h, mi, experts, top_k, bm
        self.epr = experts // world
        self.pairs = rows * top_k
        self.plain = world == 1 and plain_when_alone
        self.fused = fused and not self.plain
        self.cap = cap if cap is not None else self.pairs * world
        self.direct = self.fused and self.cap % world == 0 if direct is None else bool(direct) and self.fused
        dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        i32 = dict(device=dev, dtype=torch.int32)
        # shared with the peers: the rows this rank receives and the outputs of its experts, both [cap][h] bf16, and
        # two copies of the offsets of all ranks (calls alternate: a peer may write the next while this one is read)
        offs_bytes = world * (experts + 1) * 4
        sizes = {"offs0": offs_bytes, "offs1": offs_bytes}
        if not self.plain:
            sizes.update(recv=self.cap * h * 2, ey=self.cap * h * 2)
        if self.fused:
            sizes["landed"] = 256
            sizes["done"] = 256
        self.pb = PeerBuffers(ctx, rank, world, sizes, dev)
        self.offs_both = [_view(self.pb.local[n], (world, experts + 1), "<i4", dev) for n in ("offs0", "offs1")]
        self.parity = 0
        self.route = torch.zeros(rows, 2 * top_k, **i32)
        self.list = torch.zeros(self.pairs, **i32)
        self.tiles = torch.zeros(1 + 3 * hb.lib().hb_moe_tiles(rows, top_k, experts, bm), **i32)
        self.offs = torch.zeros(experts + 1, **i32)
        self.out = torch.zeros(rows, h, device=dev, dtype=torch.bfloat16)
        self.token = torch.zeros(1, device=dev, dtype=torch.float32)  # operand of the NCCL form of the barrier
        rows_cap = 1 << max(rows - 1, 0).bit_length()
        self.k_route = ctx.route(experts, top_k)
        self.k_sort = ctx.moe_sort(experts, top_k, rows_cap, bm)
        self.k_combine = ctx.moe_combine(h, top_k)
        if self.plain:
            kw = dict(rows_max=rows_cap, top_k=top_k, experts=experts, bm=bm, merge_runs=1)
            self.ehb = torch.zeros(self.pairs, mi, device=dev, dtype=torch.bfloat16)
            self.ey = torch.zeros(self.pairs, h, device=dev, dtype=torch.bfloat16)
            self.k_gate_up = ctx.gemm(h, 2 * mi, OUT_SWIGLU, rows_mode=hb.ROWS_GATHER, **kw)
            self.k_down = ctx.gemm(mi, h, OUT_BF16, rows_mode=hb.ROWS_SCATTER, **kw)
        else:
            self.recv, self.ey_recv = self.pb.local["recv"], self.pb.local["ey"]
            self.rlist = torch.zeros(self.cap, **i32)
            self.rtiles = torch.zeros(1 + 3 * hb.lib().hb_moe_tiles(self.cap, 1, self.epr, bm), **i32)
            self.ehb = torch.zeros(self.cap, mi, device=dev, dtype=torch.bfloat16)
            kw = dict(rows_max=self.cap, top_k=1, experts=self.epr, bm=bm, merge_runs=1)
            self.k_dispatch = ctx.ep_dispatch(h, top_k, experts, world, rank, self.cap, direct=self.direct)
            self.k_plan = ctx.ep_plan(experts, world, rank, bm, self.cap, direct=self.direct)
            self.k_gate_up = ctx.gemm(h, 2 * mi, OUT_SWIGLU, rows_mode=hb.ROWS_GATHER, **kw)
            self.k_down = ctx.gemm(mi, h, OUT_BF16, rows_mode=hb.ROWS_SCATTER, **kw)
            if self.fused:
                self.where = torch.zeros(self.pairs, **i32)
                self.ctl = ctx.alloc(256)  # zeroed: step 0
                self.ctl_done = ctx.alloc(256)
                self.k_ep_combine = ctx.ep_combine(h, top_k, world)
                # the same with the barrier "every rank's outputs are complete" inside (one process per GPU only)
                self.k_ep_combine_sync = ctx.ep_combine(h, top_k, world, sync_rank=rank) if world > 1 else None
            else:
                self.ey = torch.zeros(self.pairs, h, device=dev, dtype=torch.bfloat16)
                self.k_return = ctx.ep_return(h, top_k, experts, world, rank, self.cap)
        self.kernels_per_step = 0
        self.emit = _launch_now
        # (every kernel of the step either waits for its predecessor itself or is launched plainly: the barrier kernels)
        self.recorded = _Recorded(ctx, self, self.pb, overlap=overlap)

    def _w(self, t):
        return self.ctx.wrap(t.data_ptr(), max(t.numel() * t.element_size(), 1))

    @property
    def offs_all(self) -> torch.Tensor:
        """[world][experts + 1]: the offsets of every rank for the call in progress."""
        return self.offs_both[self.parity]

    def connect(self, local_peers) -> None:
        self.pb.connect(local_peers=[p.pb for p in local_peers])

    def close(self) -> None:
        self.recorded.close()
        self.pb.close()

    # ---- the phases
    def phase_sort(self, x, scores) -> None:
        self.x = x
        self.parity ^= 1
        self.emit(self.k_route, self.rows, self._w(scores), self._w(self.route))
        if self.plain:
            self.emit(self.k_sort, self.rows, self._w(self.route), self._w(self.list), self._w(self.tiles))
        else:
            self.emit(self.k_sort, self.rows, self._w(self.route), self._w(self.list), self._w(self.tiles), self._w(self.offs))

    def phase_dispatch(self) -> None:  # offs_all holds every rank's offsets
        if self.plain:
            return
        args = [self._w(self.x), self.pb.table("recv"), self._w(self.list), self._w(self.offs if self.direct else self.offs_all)]
        if self.fused:
            args += [self._w(self.where), self.pb.table("landed"), self.ctl]
        if self.direct:  # the dispatch delivers this rank's offsets into every rank's table itself
            args += [self.pb.table("offs1" if self.parity else "offs0")]
        self.emit(self.k_dispatch, self.rows, *args)

    def phase_experts(self, wgu_local, wd_local) -> None:  # every rank's dispatch has finished (fused: the plan sees to that)
        if self.plain:
            self.emit(self.k_gate_up, self.rows, self._w(wgu_local), self._w(self.x), self._w(self.ehb), self._w(self.list), self._w(self.tiles))
            self.emit(self.k_down, self.rows, self._w(wd_local), self._w(self.ehb), self._w(self.ey), self._w(self.list), self._w(self.tiles))
            return
        args = [self._w(self.offs_all), self._w(self.rlist), self._w(self.rtiles)]
        if self.fused:
            args += [self.pb.local["landed"], self.ctl]
        self.emit(self.k_plan, 1, *args)
        self.emit(self.k_gate_up, self.cap, self._w(wgu_local), self.recv, self._w(self.ehb), self._w(self.rlist), self._w(self.rtiles))
        self.emit(self.k_down, self.cap, self._w(wd_local), self._w(self.ehb), self.ey_recv, self._w(self.rlist), self._w(self.rtiles))

    def phase_return(self, sync: bool = False):
        """Every rank's expert GEMMs have finished; or, fused with sync = True, the combine finds that out itself."""
        if self.fused:
            args = [self.pb.table("ey"), self._w(self.where), self._w(self.route), self._w(self.out)]
            if sync:
                self.emit(self.k_ep_combine_sync, self.rows, *args, self.pb.table("done"), self.pb.local["done"], self.ctl_done)
            else:
                self.emit(self.k_ep_combine, self.rows, *args)
            return self.out
        if not self.plain:
            self.emit(self.k_return, self.rows, self.pb.table("ey"), self._w(self.ey), self._w(self.list), self._w(self.offs_all))
        self.emit(self.k_combine, self.rows, self._w(self.ey), self._w(self.route), self._w(self.out))
        return self.out


def ep_peer_connect(state: EpPeer, group=None) -> None:
    """Exchanges the buffer handles among the processes of the group and maps the peers' buffers."""
    state.pb.connect_group(group)


def ep_moe_peer(state: EpPeer, x_local, scores_local, wgu_local, wd_local, group=None, nccl_sync: bool = False, recorded: bool = False):
    """The sparse block for this rank's token rows with the exchange through peer memory; returns out [rows][h].
    nccl_sync = True orders the steps with NCCL collectives (an all-gather and two one-word all-reduces) instead
    of the library's barrier kernel; the data path is the same. recorded = True (several ranks, the library's
    barriers): the step's kernels (7 in the default form) are recorded once per (buffers, parity) and replayed with one call."""
    multi = state.world > 1
    if recorded and multi and not nccl_sync and not state.pb.emulated:
        def step(replay=False):
            if replay:
                state.parity ^= 1  # what phase_sort does: the two offset buffers take turns
                return
            _ep_step(state, x_local, scores_local, wgu_local, wd_local, group, False)
        key = (state.parity ^ 1, x_local.data_ptr(), scores_local.data_ptr(), wgu_local.data_ptr(), wd_local.data_ptr())
        state.recorded.run(key, step)
        return state.out
    return _ep_step(state, x_local, scores_local, wgu_local, wd_local, group, nccl_sync)


def _ep_step(state: EpPeer, x_local, scores_local, wgu_local, wd_local, group, nccl_sync):
    launched = state.ctx.launch_count()
    try:
        return _ep_step_body(state, x_local, scores_local, wgu_local, wd_local, group, nccl_sync)
    finally:
        if state.emit is _launch_now:
            state.kernels_per_step = state.ctx.launch_count() - launched


def _ep_step_body(state: EpPeer, x_local, scores_local, wgu_local, wd_local, group, nccl_sync):
    multi = state.world > 1
    state.phase_sort(x_local, scores_local)
    if state.plain:
        state.phase_experts(wgu_local, wd_local)
        return state.phase_return()
    if state.direct:
        pass  # no all-gather: every source has its own region of the buffers, and the dispatch delivers the offsets
    elif not multi:
        state.offs_all[0].copy_(state.offs)
    elif nccl_sync:
        dist.all_gather_into_tensor(state.offs_all.view(-1), state.offs, group=group)
    else:
        state.pb.allgather(state.offs, "offs1" if state.parity else "offs0")
    state.phase_dispatch()
    if multi and nccl_sync:
        dist.all_reduce(state.token, group=group)
    elif multi and not state.fused:
        state.pb.barrier()  # every rank's rows have landed (fused: the dispatch flags it and the plan waits)
    state.phase_experts(wgu_local, wd_local)
    if multi and state.fused and not nccl_sync and not state.pb.emulated:
        return state.phase_return(sync=True)  # the combine carries the barrier "every rank's outputs are complete"
    if multi:
        dist.all_reduce(state.token, group=group) if nccl_sync else state.pb.barrier()  # every rank's outputs are complete
    return state.phase_return()


# --------------------------------------------------------------------------- tensor-parallel FFN over peer memory
#
# The same FFN as tp_ffn with the all-reduce replaced by the library's tp_reduce kernel: every rank's down GEMM
# leaves its f32 partial in a buffer the peers can read; after a barrier each rank sums its slice of rows from all
# partials (rank order), rounds, adds the residual and writes the bf16 rows into every rank's Y; a second barrier
# closes the step. Per rank (P-1)/P of one f32 [m/P][h] slice per peer crosses NVLink instead of an all-reduce of
# the whole f32 matrix, and the output mode needs no pass of its own.

TP_GROUP_ROWS, TP_MAX_GROUPS, TP_CTL_WORDS = 256, 64, 128  # the CTA pair's row tile; HB_TP_MAX_GROUPS; HB_TP_CTL_WORDS


def pair_tile_n(ctx, m: int, k: int, n: int, out: int, w, x, y) -> int:
    """The CTA-pair tile's columns, 256 or 192, whichever is faster on these very operands (plain output into y, which
    is scratch here): 2048 x 5120 is 160 tiles of 256 x 256 for 74 pairs, 2.2 waves run as 3, and 216 tiles of
    256 x 192, 2.9 waves of three quarters the length; but the narrower tile moves more bytes into the SMs per FLOP,
    so where the waves do not decide, it loses (K = 2176: 50 against 60 us; K = 8704: no difference; the gate/up GEMM
    at 2048 x 5120 x 17408: 285 against 253 us). Timed, not modelled: three rounds of five launches, the median."""
    wrap = lambda t: ctx.wrap(t.data_ptr(), t.numel() * t.element_size())
    best, best_t = 256, None
    for bn in (256, 192):
        kern = ctx.gemm(k, n, out, rows_max=m, cta_pair=1, tile_n=bn)
        op = (kern, m, wrap(w), wrap(x), wrap(y))
        ctx.time([op], 2)
        t = sorted(ctx.time([op], 5) for _ in range(3))[1]
        if best_t is None or t < 0.97 * best_t:  # the narrower tile has to win by a margin
            best, best_t = bn, t
    return best


class TpPeer:
    """One rank of the peer-memory FFN: the partial-product buffer, the output Y and their peer tables.

    Forms of the exchange, the same bits from each (the f32 partials are summed in rank order by one rank per row):

    "push" (the default): contiguous blocks of rows, one per rank; the down GEMM pushes its partial into the staging of
      the rank that sums the block; tp_sum sums, rounds, stores Y to every rank and carries the step's two barriers itself
      (hb_tp_sum_sync_get: three kernels per step), or, with fold_barriers=False, sits between two barrier kernels.
    "pull": the partial stays local; a barrier kernel, tp_reduce pulls the blocks it sums from the peers, a barrier.
    "pushsync": the rows are dealt in groups of 256 (the down GEMM's row tile) and every rank sums 256 / world rows of
      every group; the sum is hb_tp_sum_stream_get's kernel with both barriers inside (sync = 2). Three kernels.
    "stream": as pushsync, and the down GEMM flags a group when its last tile is out; the summing kernel starts beside
      the GEMM, takes the groups as they complete and closes the step with a handshake of its own. Three kernels.
      The slowest as measured: a flag needs a fence behind a tile's remote stores, and with NVLink as the bound a
      fence is expensive.
    Measured for the 27B-class FFN (2048 rows), step replayed, on two / four / eight B200s: push 436-452 / 258-282 /
    200-203 us, pushsync 445 / 263 / 207, pull 470 / 298 / 248, stream 465 / 317 / 279. (The pushed stores leave as whole
    128-byte row segments: one 16-byte piece per lane took 537 us on two and 437 us on eight.)"""

    def __init__(self, hb, ctx, rank: int, world: int, m: int, h: int, out: int = OUT_RESIDUAL, device=None, push: bool | None = None, mode: str | None = None,
                 tune_tiles: bool = True, fold_barriers: bool = True):
        self.hb, self.ctx, self.rank, self.world, self.m, self.h, self.out = hb, ctx, rank, world, m, h, out
        self.tune_tiles, self.tile_n = tune_tiles, (256, 256)
        dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        if mode is None:
            mode = ("push" if push else "pull") if push is not None else "push"
        if world == 1:
            mode = "pull"
        assert mode in ("stream", "push", "pull", "pushsync")
        self.mode = mode
        self.push = mode == "push"
        self.grouped = mode in ("stream", "pushsync")  # rows dealt in groups of 256, the streaming sum kernel
        self.rows_per = (m + world - 1) // world
        self.groups = (m + TP_GROUP_ROWS - 1) // TP_GROUP_ROWS
        self.group_part = TP_GROUP_ROWS // world
        # acc: the whole partial [m][h] (pull), the staging [world][rows_per][h] of the blocks this rank sums (push), or the
        # staging [world][groups][256 / world][h] of its slices of every group (stream)
        acc_rows = {"pull": m, "push": max(m, world * self.rows_per)}.get(mode, world * self.groups * self.group_part)
        sizes = {"acc": acc_rows * h * 4, "y": m * h * 2}
        if self.grouped:
            assert self.groups <= TP_MAX_GROUPS
            sizes.update(gflags=world * TP_MAX_GROUPS * 4, done=256)
            self.ctl = ctx.alloc(TP_CTL_WORDS * 4)  # zeroed: step 0
        # push: tp_sum can carry the step's two barriers itself (one process per GPU): flags on every rank, its own counters
        self.fold_barriers = self.push and world > 1 and fold_barriers
        if self.fold_barriers:
            sizes.update(done=256)
            self.ctl = ctx.alloc(TP_CTL_WORDS * 4)
        self.pb = PeerBuffers(ctx, rank, world, sizes, dev)
        self.acc, self.y = self.pb.local["acc"], self.pb.local["y"]
        self._yv = _view(self.y, (m, h), "<i2", dev).view(torch.bfloat16)
        self.token = torch.zeros(1, device=dev, dtype=torch.float32)
        self.k_reduce = None if self.grouped else ctx.tp_sum(h, out, world, rank) if self.push else ctx.tp_reduce(h, out, world, rank)
        self.k_reduce_sync = ctx.tp_sum(h, out, world, rank, sync=True) if self.fold_barriers else None
        self._k_stream = {}
        self.push_table = torch.zeros(world, device=dev, dtype=torch.int64)  # where this rank's block for owner d goes
        self.kernels = {}
        self.kernels_per_step = 0
        self.emit = _launch_now
        self.recorded = _Recorded(ctx, self, self.pb)

    def describe(self) -> str:
        return {
            "stream": "rows dealt in groups of 256, each rank sums 256/P rows of every group: the down GEMM's epilogue stores its f32 partial tile by tile into the "
                      "summing ranks' staging (NVLink, under the GEMM) and flags each finished group; tp_sum_stream runs beside the GEMM (programmatic launch), sums "
                      "the groups as they complete in rank order, rounds once, adds the residual, stores bf16 Y to every rank and ends with its own handshake "
                      "(3 kernels per step, no barrier kernel, no NCCL call)",
            "pushsync": "rows dealt in groups of 256, each rank sums 256/P rows of every group: the down GEMM's epilogue stores its f32 partial tile by tile into "
                        "the summing ranks' staging (NVLink, under the GEMM); tp_sum_stream with both barriers inside (its first block says that this rank's "
                        "partial is out, every block waits for all ranks; the last block closes the step with a handshake): 3 kernels per step, no NCCL call",
            "push": "down GEMM epilogue stores its f32 partial block by block into the summing ranks' memory (NVLink, under the GEMM); tp_sum: rank-order sum, one "
                    "rounding, residual, peer stores of bf16 Y; " + ("the step's two barriers inside tp_sum: 3 kernels" if self.fold_barriers else "2 barrier kernels") +
                    " (no NCCL call in the step)",
            "pull": "f32 partial stays local; tp_reduce pulls the blocks it sums through NVLink loads, rank-order sum, one rounding, residual, peer stores of bf16 Y; "
                    "2 barrier kernels (no NCCL call in the step)",
        }[self.mode]

    def _w(self, t):
        return self.ctx.wrap(t.data_ptr(), max(t.numel() * t.element_size(), 1))

    def connect(self, local_peers) -> None:
        self.pb.connect(local_peers=[p.pb for p in local_peers])
        self._after_connect()

    def _after_connect(self) -> None:
        # slot `rank` of every owner's staging buffer
        slot = self.rank * (self.groups * self.group_part if self.grouped else self.rows_per) * self.h * 4
        self.push_table.copy_(self.pb.tables["acc"] + slot)

    def close(self) -> None:
        self.recorded.close()
        self.pb.close()

    def set_y(self, y: torch.Tensor) -> None:
        """Loads the residual stream (replicated: the same on every rank) into the shared Y."""
        self._yv.copy_(y)

    def y_view(self) -> torch.Tensor:
        """Y as a torch tensor over the library's allocation (no copy)."""
        return self._yv

    def phase_gemms(self, x, wgu_local, wd_local) -> None:
        m, h = x.shape
        ip = wgu_local.shape[0] // 2
        key = (h, ip)
        if key not in self.kernels:
            hmid = torch.empty((self.m, ip), device=x.device, dtype=torch.bfloat16)
            form = {"pull": {}, "push": dict(y_shards=self.world), "pushsync": dict(y_shards=self.world, y_group_rows=TP_GROUP_ROWS),
                    "stream": dict(y_shards=self.world, y_group_rows=TP_GROUP_ROWS, y_signal=self.rank + 1)}[self.mode]
            # the tile width of each GEMM is chosen by timing both on these operands (plain local outputs: nothing of a
            # peer's is touched)
            tn_gu = pair_tile_n(self.ctx, self.m, h, 2 * ip, OUT_SWIGLU, wgu_local, x[: self.m], hmid) if self.tune_tiles else 256
            tmp = torch.empty((self.m, h), device=x.device, dtype=torch.float32) if self.tune_tiles else None
            tn_dn = pair_tile_n(self.ctx, self.m, ip, h, OUT_F32, wd_local, hmid, tmp) if self.tune_tiles else 256
            del tmp
            self.tile_n = (tn_gu, tn_dn)
            self.kernels[key] = (self.ctx.gemm(h, 2 * ip, OUT_SWIGLU, rows_max=self.m, cta_pair=1, tile_n=tn_gu),
                                 self.ctx.gemm(ip, h, OUT_F32, rows_max=self.m, cta_pair=1, tile_n=tn_dn, **form), hmid)
        k_gu, k_down, hmid = self.kernels[key]
        self.emit(k_gu, m, self._w(wgu_local), self._w(x), self._w(hmid))
        if self.mode == "stream":
            self.emit(k_down, m, self._w(wd_local), self._w(hmid), self._w(self.push_table), self.pb.table("gflags"), self.ctl)
        else:
            self.emit(k_down, m, self._w(wd_local), self._w(hmid), self._w(self.push_table) if self.mode != "pull" else self.acc)

    def phase_reduce(self, sync: bool = False) -> None:
        """pull / push: every rank's partial is complete (push: has arrived). stream / pushsync with sync: right behind
        this rank's GEMMs, the kernel orders itself against the other ranks; without: as for push."""
        if self.grouped:
            sync = (1 if self.mode == "stream" else 2) if sync else 0
            if sync not in self._k_stream:
                self._k_stream[sync] = self.ctx.tp_sum_stream(self.h, self.out, self.world, self.rank, TP_GROUP_ROWS, sync)
            self.emit(self._k_stream[sync], self.m, self.acc, self.pb.table("y"), self.pb.local["gflags"], self.pb.table("done"), self.ctl)
        elif sync and self.fold_barriers:
            self.emit(self.k_reduce_sync, self.m, self.acc, self.pb.table("y"), self.pb.table("done"), self.ctl)
        else:
            self.emit(self.k_reduce, self.m, self.acc if self.push else self.pb.table("acc"), self.pb.table("y"))


def tp_peer_connect(state: TpPeer, group=None) -> None:
    state.pb.connect_group(group)
    state._after_connect()


def tp_ffn_peer(state: TpPeer, x, wgu_local, wd_local, group=None, nccl_sync: bool = False, recorded: bool = False):
    """state.y <- bf16(state.y + bf16(sum over ranks of H_r . Wd_r^T)) on every rank; returns the view of Y.
    recorded = True (several ranks, the library's barriers): the step is recorded once per set of buffers and replayed."""
    multi = state.world > 1
    if recorded and multi and not nccl_sync and not state.pb.emulated:
        def step(replay=False):
            if not replay:
                _tp_step(state, x, wgu_local, wd_local, group, False)
        state.recorded.run((x.data_ptr(), wgu_local.data_ptr(), wd_local.data_ptr()), step)
        return state.y_view()
    return _tp_step(state, x, wgu_local, wd_local, group, nccl_sync)


def _tp_step(state: TpPeer, x, wgu_local, wd_local, group, nccl_sync):
    launched = state.ctx.launch_count()
    try:
        return _tp_step_body(state, x, wgu_local, wd_local, group, nccl_sync)
    finally:
        if state.emit is _launch_now:
            state.kernels_per_step = state.ctx.launch_count() - launched


def _tp_step_body(state: TpPeer, x, wgu_local, wd_local, group, nccl_sync):
    multi = state.world > 1
    state.phase_gemms(x, wgu_local, wd_local)
    if (state.grouped or state.fold_barriers) and multi and not nccl_sync and not state.pb.emulated:
        state.phase_reduce(sync=True)  # the kernel orders itself against the other ranks: no barrier before or after
        return state.y_view()
    if multi:
        dist.all_reduce(state.token, group=group) if nccl_sync else state.pb.barrier()  # every rank's partial is complete
    state.phase_reduce()
    if multi:
        dist.all_reduce(state.token, group=group) if nccl_sync else state.pb.barrier()  # every rank's Y is complete
    return state.y_view()
