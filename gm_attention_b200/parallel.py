"""Latitude-band sharding of the sphere across the GPUs of one node.

The reference has no distributed code (it runs one process per GPU on
independent runs); this module is new.  Neighbourhoods only join lattice rows
with ``|row_i - row_j| <= w`` (every geodesic distance is at least the
colatitude difference), so the sphere splits into contiguous bands of target
rows, one per rank, with ONE exchange per direction:

* forward: every rank receives the ``w`` rows either side of its band
  (the *halo*) of the key and value fields from the ranks that own them;
* backward: the key / value gradients a rank accumulated for its halo rows are
  sent back to their owners and added there.

Bands are balanced by edge count, not by row count: polar rows carry hundreds
to thousands of neighbours per node, equatorial rows a few dozen.  A band
narrower than ``w`` rows makes a rank's halo reach past its direct neighbour,
so the exchange is written for arbitrary overlaps of "rows I need" with "rows
you own".

Two exchangers share one interface.  :class:`NativeHaloExchanger` (GPUs) hands an
exchange to the library as a list of (peer, direction, pointer, bytes) operations that
become ONE NCCL group on the current stream: sends read the field's slabs in place,
receives land in the halo rows themselves -- no staging copies, no per-operation
interpreter work, nothing blocks the host.  :class:`HaloExchanger` goes through
``torch.distributed`` point-to-point (gloo on CPU for the tests, NCCL on GPUs) with
staging buffers; every wait of it has a timeout and raises :class:`HaloTimeout`.
Received halos land in the rank's own memory; kernels never read a peer's memory.
"""

from __future__ import annotations

import ctypes
import datetime
from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch import Tensor


class HaloTimeout(RuntimeError):
    """A halo message did not arrive in time (a peer never posted its side of the exchange)."""


def balanced_cuts(row_cost: list[int] | list[float], parts: int) -> list[int]:
    """Cut ``len(row_cost)`` rows into ``parts`` contiguous non-empty bands minimising the
    largest band cost (exact: binary search on the bottleneck + greedy feasibility, then
    the cuts are placed as evenly as the bottleneck allows)."""
    n = len(row_cost)
    if not 1 <= parts <= n:
        raise ValueError(f"cannot cut {n} rows into {parts} bands")
    prefix = [0.0]
    for c in row_cost:
        prefix.append(prefix[-1] + float(c))

    def cuts_for(limit: float) -> list[int] | None:
        cuts, start = [0], 0
        for p in range(parts):
            remaining = parts - p - 1
            end = start
            while end < n - remaining and prefix[end + 1] - prefix[start] <= limit:
                end += 1
            if end == start:
                return None
            cuts.append(end)
            start = end
        return cuts if start == n else None

    lo, hi = max(row_cost), prefix[-1]
    for _ in range(64):
        mid = 0.5 * (lo + hi)
        if cuts_for(mid) is None:
            lo = mid
        else:
            hi = mid
    cuts = cuts_for(hi)
    assert cuts is not None
    return cuts


@dataclass(frozen=True)
class BandPlan:
    """Which lattice rows each rank owns and which it must hold."""

    nlat: int
    nlon: int
    halo: int  # w
    cuts: tuple[int, ...]  # world + 1 row indices, cuts[r] .. cuts[r + 1] owned by rank r

    @property
    def world(self) -> int:
        return len(self.cuts) - 1

    def owned(self, rank: int) -> tuple[int, int]:
        return self.cuts[rank], self.cuts[rank + 1]

    def extended(self, rank: int) -> tuple[int, int]:
        lo, hi = self.owned(rank)
        return max(0, lo - self.halo), min(self.nlat, hi + self.halo)

    def needs(self, rank: int, other: int) -> tuple[int, int] | None:
        """Rows ``rank`` holds as halo that ``other`` owns (global row range), or None."""
        if rank == other:
            return None
        elo, ehi = self.extended(rank)
        olo, ohi = self.owned(other)
        lo, hi = max(elo, olo), min(ehi, ohi)
        return (lo, hi) if lo < hi else None

    @staticmethod
    def balanced(nlat: int, nlon: int, halo: int, row_degree: list[int] | list[float], world: int) -> BandPlan:
        """Bands of (nearly) equal total ``row_degree`` -- edges per node of each row, or any per-row cost."""
        return BandPlan(nlat, nlon, halo, tuple(balanced_cuts([d * nlon for d in row_degree], world)))

    def load(self, row_degree: list[int]) -> list[int]:
        return [sum(row_degree[self.cuts[r]:self.cuts[r + 1]]) * self.nlon for r in range(self.world)]


class HaloExchanger:
    """Moves halo rows of fields laid out ``(batch, extended rows, nlon, D)``.

    The peers and row ranges are fixed by the band plan, so the staging buffers of every (field shape, dtype) are
    allocated once and reused: an exchange is a few slice copies, one batched send / receive and the landing copies."""

    def __init__(self, plan: BandPlan, rank: int, group: dist.ProcessGroup | None = None, timeout: float = 60.0) -> None:
        """``timeout``: seconds a wait for a message may take before :class:`HaloTimeout` is raised (host-side waits of
        CPU process groups; on NCCL a wait only orders streams, and the process group's own timeout covers a dead peer)."""
        self.plan, self.rank, self.group, self.timeout = plan, rank, group, timeout
        self.elo, self.ehi = plan.extended(rank)
        self.lo, self.hi = plan.owned(rank)
        #: (peer, rows the peer needs from me, rows I need from the peer): global row ranges or None
        self.peers = [(other, plan.needs(other, rank), plan.needs(rank, other)) for other in range(plan.world)
                      if other != rank and (plan.needs(other, rank) is not None or plan.needs(rank, other) is not None)]
        self._buffers: dict = {}

    def _local(self, rows: tuple[int, int]) -> slice:
        return slice(rows[0] - self.elo, rows[1] - self.elo)

    def _staging(self, like: Tensor, count: int, peer: int, rows: tuple[int, int], kind: str) -> Tensor:
        """One buffer per (peer, direction) for ALL fields of an exchange: (count, batch, rows, nlon, D)."""
        key = (kind, count, peer, rows, tuple(like.shape), like.dtype, like.device)
        buf = self._buffers.get(key)
        if buf is None:
            buf = torch.empty((count, like.shape[0], rows[1] - rows[0], *like.shape[2:]), dtype=like.dtype, device=like.device)
            self._buffers[key] = buf
        return buf

    def _post(self, sends: list[tuple[int, Tensor]], recvs: list[tuple[int, Tensor]]) -> list:
        if not sends and not recvs:
            return []
        ops = [dist.P2POp(dist.isend, t, peer, self.group) for peer, t in sends]
        ops += [dist.P2POp(dist.irecv, t, peer, self.group) for peer, t in recvs]
        return dist.batch_isend_irecv(ops)

    def start_fill(self, *fields: Tensor):
        """Forward exchange, first half: stage the rows the neighbours need and enqueue the messages.  Work that does
        not read the halo rows can be launched before :meth:`finish_fill` and runs while the messages travel."""
        sends, recvs = [], []
        for other, theirs, mine in self.peers:
            if theirs is not None:
                out = self._staging(fields[0], len(fields), other, theirs, "send")
                for slot, f in enumerate(fields):
                    out[slot].copy_(f[:, self._local(theirs)])
                sends.append((other, out))
            if mine is not None:
                recvs.append((other, self._staging(fields[0], len(fields), other, mine, "recv")))
        return self._post(sends, recvs), fields

    def _wait(self, works: list, what: str) -> None:
        for work in works:
            try:
                done = work.wait(datetime.timedelta(seconds=self.timeout))
            except RuntimeError as exc:  # gloo reports an expired wait as a RuntimeError
                raise HaloTimeout(f"rank {self.rank}: {what} did not complete within {self.timeout} s: {exc}") from exc
            if done is False:
                raise HaloTimeout(f"rank {self.rank}: {what} did not complete within {self.timeout} s")

    def finish_fill(self, handle) -> None:
        """Second half: wait for the messages and copy the owners' rows into this rank's halo rows."""
        works, fields = handle
        self._wait(works, "the halo fill")
        for other, theirs, mine in self.peers:
            if mine is not None:
                buf = self._staging(fields[0], len(fields), other, mine, "recv")
                for slot, f in enumerate(fields):
                    f[:, self._local(mine)].copy_(buf[slot])

    def fill_halos(self, *fields: Tensor) -> None:
        """Forward exchange: copy the owners' rows into this rank's halo rows of every field (one message per peer
        and direction carries all fields)."""
        self.finish_fill(self.start_fill(*fields))

    def start_reduce(self, *grads: Tensor):
        """Backward exchange, first half: send the gradient rows accumulated for other ranks' nodes (they must be
        final) to their owners.  The rank's own rows may still be written until :meth:`finish_reduce`."""
        sends, recvs = [], []
        for other, theirs, mine in self.peers:
            if mine is not None:  # halo rows I computed partial sums for: they belong to `other`
                out = self._staging(grads[0], len(grads), other, mine, "send")
                for slot, g in enumerate(grads):
                    out[slot].copy_(g[:, self._local(mine)])
                sends.append((other, out))
            if theirs is not None:  # rows of mine `other` computed partial sums for
                recvs.append((other, self._staging(grads[0], len(grads), other, theirs, "recv")))
        return self._post(sends, recvs), grads

    def finish_reduce(self, handle) -> None:
        """Second half: add what the others accumulated for this rank's nodes, and zero the halo rows."""
        works, grads = handle
        self._wait(works, "the halo reduction")
        for other, theirs, mine in self.peers:
            if theirs is not None:
                buf = self._staging(grads[0], len(grads), other, theirs, "recv")
                for slot, g in enumerate(grads):
                    g[:, self._local(theirs)].add_(buf[slot])
        for g in grads:
            g[:, : self.lo - self.elo].zero_()
            g[:, self.hi - self.elo:].zero_()

    def reduce_halos(self, *grads: Tensor) -> None:
        """Backward exchange: send the gradient rows accumulated for other ranks' nodes to their
        owners, add what the others accumulated for this rank's nodes, and zero the halo rows."""
        self.finish_reduce(self.start_reduce(*grads))


class NativeHaloExchanger:
    """The halo exchange through the library's own NCCL path (``gm_halo_*``): same interface as :class:`HaloExchanger`.

    The communicator is created collectively over ``group`` (default: the world): rank 0's NCCL id travels through
    ``torch.distributed``.  An exchange is: one launch per neighbour packing the rows it needs (all fields, all samples)
    into one buffer, ONE NCCL group of one message per neighbour and direction, one launch per neighbour unpacking
    (forward) or adding (backward) what arrived -- all enqueued on the CURRENT stream (or, for the split calls, on a side
    stream ordered against it with events); nothing waits on the host.  ``packed=False`` sends every (field, sample)
    slab as its own message straight out of field memory instead: no packing launches, many more NCCL operations."""

    def __init__(self, plan: BandPlan, rank: int, device: torch.device, group: dist.ProcessGroup | None = None, packed: bool = True) -> None:
        from gm_attention_b200 import _lib

        self._lib = _lib
        self.plan, self.rank, self.device, self.packed = plan, rank, device, packed
        self.elo, self.ehi = plan.extended(rank)
        self.lo, self.hi = plan.owned(rank)
        self.peers = [(other, plan.needs(other, rank), plan.needs(rank, other)) for other in range(plan.world)
                      if other != rank and (plan.needs(other, rank) is not None or plan.needs(rank, other) is not None)]
        ident = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            raw = (ctypes.c_ubyte * 128)()
            _lib.call("gm_halo_unique_id", ctypes.addressof(raw))
            ident = torch.tensor(list(raw), dtype=torch.uint8)
        ident = ident.to(device)
        dist.broadcast(ident, 0, group=group)
        raw = (ctypes.c_ubyte * 128)(*ident.cpu().tolist())
        comm = ctypes.c_void_p()
        with torch.cuda.device(device):
            _lib.call("gm_halo_comm_create", ctypes.addressof(raw), rank, plan.world, ctypes.byref(comm))
        self.comm = comm
        self.side = torch.cuda.Stream(device)
        self._buffers: dict = {}
        self._plans: dict = {}

    def close(self) -> None:
        if self.comm:
            torch.cuda.synchronize(self.device)
            self._lib.call("gm_halo_comm_destroy", self.comm)
            self.comm = ctypes.c_void_p()

    def _local(self, rows: tuple[int, int]) -> tuple[int, int]:
        return rows[0] - self.elo, rows[1] - self.elo

    def _buffer(self, kind: str, like: Tensor, count: int, other: int, rows: tuple[int, int]) -> Tensor:
        """One packed buffer per (direction, peer) for all fields of an exchange: (count, batch, rows, nlon, D)."""
        key = (kind, count, other, rows, tuple(like.shape), like.dtype)
        buf = self._buffers.get(key)
        if buf is None:
            buf = torch.empty((count, like.shape[0], rows[1] - rows[0], *like.shape[2:]), dtype=like.dtype, device=like.device)
            self._buffers[key] = buf
        return buf

    @staticmethod
    def _slabs(field: Tensor, r0: int, r1: int):
        """(address, bytes) of the rows r0 .. r1 - 1 of every sample of a (batch, rows, nlon, D) field: contiguous each."""
        row_bytes = field.shape[2] * field.shape[3] * field.element_size()
        sample_bytes = field.shape[1] * row_bytes
        base = field.data_ptr()
        return [(base + b * sample_bytes + r0 * row_bytes, (r1 - r0) * row_bytes) for b in range(field.shape[0])]

    def _plan(self, kind: str, fields: tuple[Tensor, ...]) -> tuple:
        """ctypes arguments of an exchange, cached by the fields' addresses and shape: (moves before, messages, moves
        after).  A move is the argument tuple of ``gm_halo_move`` up to the stream; the messages are the arrays of
        ``gm_halo_exchange``.  ``kind``: "fill" sends the rows neighbours need of MY rows and receives my halo rows;
        "reduce" sends my halo rows' sums and receives, into buffers, the sums neighbours formed for my rows."""
        key = (kind, self.packed, *(f.data_ptr() for f in fields), tuple(fields[0].shape), fields[0].dtype)
        hit = self._plans.get(key)
        if hit is not None:
            return hit
        like, count = fields[0], len(fields)
        row_bytes = like.shape[2] * like.shape[3] * like.element_size()
        sample_bytes = like.shape[1] * row_bytes
        code = self._lib.dtype_code(like.dtype) if like.dtype in (torch.float32, torch.bfloat16) else 0

        def move(mode: int, rows: tuple[int, int], buf: Tensor) -> tuple:
            r0, r1 = self._local(rows)
            bases = (ctypes.c_void_p * count)(*[f.data_ptr() + r0 * row_bytes for f in fields])
            return (mode, bases, count, like.shape[0], (r1 - r0) * row_bytes, sample_bytes, buf.data_ptr(), code)

        before, after, ops = [], [], []
        for other, theirs, mine in self.peers:
            outgoing, incoming = (theirs, mine) if kind == "fill" else (mine, theirs)
            if outgoing is not None:
                if self.packed:
                    buf = self._buffer("send", like, count, other, outgoing)
                    before.append(move(0, outgoing, buf))
                    ops.append((other, 1, buf.data_ptr(), buf.numel() * buf.element_size()))
                else:
                    for f in fields:
                        ops += [(other, 1, ptr, n) for ptr, n in self._slabs(f, *self._local(outgoing))]
            if incoming is not None:
                if self.packed or kind == "reduce":
                    buf = self._buffer("recv", like, count, other, incoming)
                    after.append(move(1 if kind == "fill" else 2, incoming, buf))
                if self.packed:
                    ops.append((other, 0, buf.data_ptr(), buf.numel() * buf.element_size()))
                elif kind == "fill":
                    for f in fields:
                        ops += [(other, 0, ptr, n) for ptr, n in self._slabs(f, *self._local(incoming))]
                else:
                    slab = buf[0, 0].numel() * buf.element_size()
                    ops += [(other, 0, buf[slot, b].data_ptr(), slab) for slot in range(count) for b in range(buf.shape[1])]
        n = len(ops)
        messages = (n, (ctypes.c_int * n)(*[o[0] for o in ops]), (ctypes.c_int * n)(*[o[1] for o in ops]),
                    (ctypes.c_void_p * n)(*[o[2] for o in ops]), (ctypes.c_int64 * n)(*[o[3] for o in ops]))
        if len(self._plans) > 64:
            self._plans.clear()
        hit = self._plans[key] = (before, messages, after)
        return hit

    def _check(self, fields: tuple[Tensor, ...]) -> None:
        if len(fields) > 4:
            raise RuntimeError("at most four fields per halo exchange")
        for f in fields:
            if not f.is_contiguous() or f.shape != fields[0].shape or f.dtype != fields[0].dtype:
                raise RuntimeError("halo exchange needs contiguous (batch, rows, nlon, D) fields of one shape and dtype")

    def _send(self, plan: tuple, stream: torch.cuda.Stream) -> None:
        before, (n, peers, sends, pointers, nbytes), _ = plan
        with torch.cuda.device(self.device):
            for args in before:
                self._lib.call("gm_halo_move", *args, stream.cuda_stream)
            self._lib.call("gm_halo_exchange", self.comm, n, peers, sends, pointers, nbytes, stream.cuda_stream)

    def _land(self, plan: tuple, stream: torch.cuda.Stream) -> None:
        with torch.cuda.device(self.device):
            for args in plan[2]:
                self._lib.call("gm_halo_move", *args, stream.cuda_stream)

    def _zero_halo(self, grads: tuple[Tensor, ...], stream: torch.cuda.Stream) -> None:
        with torch.cuda.stream(stream):
            for g in grads:
                if self.lo > self.elo:
                    g[:, : self.lo - self.elo].zero_()
                if self.ehi > self.hi:
                    g[:, self.hi - self.elo:].zero_()

    def fill_halos(self, *fields: Tensor, stream: torch.cuda.Stream | None = None) -> None:
        """Forward exchange on the current stream: every field's halo rows receive the owners' rows."""
        self._check(fields)
        stream = stream or torch.cuda.current_stream(self.device)
        plan = self._plan("fill", fields)
        self._send(plan, stream)
        self._land(plan, stream)

    def start_fill(self, *fields: Tensor):
        """The forward exchange on a side stream: work that does not read the halo rows can be launched on the current
        stream before :meth:`finish_fill` and runs while the rows travel."""
        self.side.wait_stream(torch.cuda.current_stream(self.device))
        self.fill_halos(*fields, stream=self.side)
        done = torch.cuda.Event()
        done.record(self.side)
        return done

    def finish_fill(self, done) -> None:
        torch.cuda.current_stream(self.device).wait_event(done)

    def reduce_halos(self, *grads: Tensor, zero_halo: bool = True) -> None:
        """Backward exchange on the current stream: the partial sums this rank formed for other ranks' rows go to
        their owners, the sums others formed for this rank's rows are added in, the halo rows are zeroed."""
        self._check(grads)
        stream = torch.cuda.current_stream(self.device)
        plan = self._plan("reduce", grads)
        self._send(plan, stream)
        self._land(plan, stream)
        if zero_halo:
            self._zero_halo(grads, stream)

    def start_reduce(self, *grads: Tensor):
        """The backward exchange on a side stream.  The halo rows' sums must be final on the current stream; the rank's
        own rows may still be written until :meth:`finish_reduce`, which adds the received sums on the current stream."""
        self._check(grads)
        self.side.wait_stream(torch.cuda.current_stream(self.device))
        plan = self._plan("reduce", grads)
        self._send(plan, self.side)
        done = torch.cuda.Event()
        done.record(self.side)
        return done, grads, plan

    def finish_reduce(self, handle, zero_halo: bool = True) -> None:
        done, grads, plan = handle
        stream = torch.cuda.current_stream(self.device)
        stream.wait_event(done)
        self._land(plan, stream)
        if zero_halo:
            self._zero_halo(grads, stream)


class PeerHaloExchanger:
    """The halo exchange through peer memory (``gm_peer_*``): same interface as :class:`HaloExchanger`.

    Every rank owns one device block with a receive buffer per (neighbour, kind of exchange) and the flag words of the
    protocol; neighbours map each other's blocks through CUDA IPC.  A send is ONE kernel (for both sides of the band) that stores
    the rows straight into the neighbours' buffers over NVLink and raises a flag in each; a landing is ONE kernel that waits
    for its flags (bounded) and unpacks (forward) or adds (backward).  Needs GPUs that can map each other's memory: construction raises ``RuntimeError``
    on every rank when any rank could not map a neighbour (use :class:`NativeHaloExchanger` then).  The blocks are sized at
    the first exchange for that call's field shape, dtype and field count (at most four fields); later calls must match."""

    KINDS = ("fill", "reduce")
    WORD = 128  # bytes between flag words: one per cache line

    def __init__(self, plan: BandPlan, rank: int, device: torch.device, group: dist.ProcessGroup | None = None) -> None:
        from gm_attention_b200 import _lib

        self._lib = _lib
        self.plan, self.rank, self.device, self.group = plan, rank, device, group
        self.elo, self.ehi = plan.extended(rank)
        self.lo, self.hi = plan.owned(rank)
        self.peers = [(other, plan.needs(other, rank), plan.needs(rank, other)) for other in range(plan.world)
                      if other != rank and (plan.needs(other, rank) is not None or plan.needs(rank, other) is not None)]
        self.side = torch.cuda.Stream(device)
        self.block = ctypes.c_void_p()
        self.mapped: dict[int, ctypes.c_void_p] = {}
        self.layout: dict | None = None
        self.remote: dict[int, dict] = {}
        self.steps = {(other, kind): 0 for other, _, _ in self.peers for kind in self.KINDS}
        self._shape = None

    # ---- set-up (collective, at the first exchange)
    def _setup(self, like: Tensor, count: int) -> None:
        row_bytes = like.shape[2] * like.shape[3] * like.element_size()
        batch = like.shape[0]
        layout: dict = {}
        cursor = 0

        def take(nbytes: int) -> int:
            nonlocal cursor
            at = cursor
            cursor += -(-nbytes // 256) * 256
            return at

        for other, theirs, mine in self.peers:
            # what I RECEIVE from `other`: in a fill my halo rows `mine`, in a reduce the sums for my rows `theirs`
            for kind, rows in (("fill", mine), ("reduce", theirs)):
                layout[(other, kind)] = {"buffer": take(count * batch * (rows[1] - rows[0]) * row_bytes) if rows is not None else None,
                                         "data": take(self.WORD), "ack": take(self.WORD), "send_ticket": take(self.WORD),
                                         "land_ticket": take(self.WORD)}
        handle = (ctypes.c_ubyte * 64)()
        status, message = 0, ""
        try:
            with torch.cuda.device(self.device):
                self._lib.call("gm_peer_alloc", max(cursor, 256), ctypes.byref(self.block), ctypes.addressof(handle))
        except RuntimeError as exc:
            status, message = 1, str(exc)
        mine_info = {"rank": self.rank, "handle": bytes(handle), "layout": layout, "status": status}
        everyone: list = [None] * self.plan.world
        dist.all_gather_object(everyone, mine_info, group=self.group)
        by_rank = {info["rank"]: info for info in everyone}
        if status == 0:
            for other, _, _ in self.peers:
                if by_rank[other]["status"]:
                    continue
                mapped = ctypes.c_void_p()
                theirs_handle = (ctypes.c_ubyte * 64).from_buffer_copy(by_rank[other]["handle"])  # kept alive across the call
                try:
                    with torch.cuda.device(self.device):
                        self._lib.call("gm_peer_open", ctypes.addressof(theirs_handle), ctypes.byref(mapped))
                    self.mapped[other] = mapped
                    self.remote[other] = by_rank[other]["layout"]
                except RuntimeError as exc:
                    status, message = 1, str(exc)
        verdict = torch.tensor([status], device=self.device, dtype=torch.int32)
        dist.all_reduce(verdict, op=dist.ReduceOp.MAX, group=self.group)
        if int(verdict.item()) or any(info["status"] for info in everyone):
            self.close()
            raise RuntimeError(f"peer-memory halo exchange is not available on this machine ({message or 'another rank could not map its neighbour'})")
        self.layout = layout
        self._shape = (tuple(like.shape), like.dtype, count)

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            for mapped in self.mapped.values():
                self._lib.call("gm_peer_close", mapped)
            self.mapped = {}
            if self.block:
                self._lib.call("gm_peer_free", self.block)
                self.block = ctypes.c_void_p()

    def error(self) -> int:
        """0, or which bounded wait ran out on this device (1: a send's acknowledgement, 2: a landing's data)."""
        code = ctypes.c_int(0)
        with torch.cuda.device(self.device):
            self._lib.call("gm_peer_error", ctypes.byref(code))
        return code.value

    # ---- one exchange
    def _check(self, fields: tuple[Tensor, ...]) -> None:
        if len(fields) > 4:
            raise RuntimeError("at most four fields per halo exchange")
        for f in fields:
            if not f.is_contiguous() or f.shape != fields[0].shape or f.dtype != fields[0].dtype:
                raise RuntimeError("halo exchange needs contiguous (batch, rows, nlon, D) fields of one shape and dtype")
        if self.layout is None:
            self._setup(fields[0], len(fields))
        elif self._shape != (tuple(fields[0].shape), fields[0].dtype, len(fields)):
            raise RuntimeError("this exchanger's buffers were sized for another field shape, dtype or field count")

    def _launch(self, entry: str, lanes: list[dict], fields: tuple[Tensor, ...], extra: tuple, stream: torch.cuda.Stream) -> None:
        """One launch per pair of neighbours: both sides of a band travel at the same time."""
        like = fields[0]
        row_bytes = like.shape[2] * like.shape[3] * like.element_size()
        count = len(fields)
        with torch.cuda.device(self.device):
            for first in range(0, len(lanes), 2):
                group = lanes[first:first + 2]
                n = len(group)
                bases = (ctypes.c_void_p * (n * count))(*[f.data_ptr() + (lane["rows"][0] - self.elo) * row_bytes for lane in group for f in fields])
                slabs = (ctypes.c_int64 * n)(*[(lane["rows"][1] - lane["rows"][0]) * row_bytes for lane in group])
                pointers = lambda key: (ctypes.c_void_p * n)(*[lane[key] for lane in group])
                steps = (ctypes.c_uint32 * n)(*[lane["step"] for lane in group])
                self._lib.call(entry, n, bases, count, like.shape[0], slabs, like.shape[1] * row_bytes, pointers("buffer"), *extra,
                               pointers("wait"), pointers("ticket"), pointers("signal"), steps, stream.cuda_stream)

    def _send(self, kind: str, fields: tuple[Tensor, ...], stream: torch.cuda.Stream) -> None:
        lanes = []
        for other, theirs, mine in self.peers:
            rows = theirs if kind == "fill" else mine  # rows of MY extended band that go to `other`
            if rows is None:
                continue
            self.steps[(other, kind)] += 1  # one counter per (neighbour, kind): its send and its landing advance together
            there, here = self.remote[other][(self.rank, kind)], self.layout[(other, kind)]
            base = self.mapped[other].value
            lanes.append({"rows": rows, "step": self.steps[(other, kind)], "buffer": base + there["buffer"], "wait": self.block.value + here["ack"],
                          "ticket": self.block.value + here["send_ticket"], "signal": base + there["data"]})
        if lanes:
            self._launch("gm_peer_send_many", lanes, fields, (), stream)

    def _land(self, kind: str, fields: tuple[Tensor, ...], stream: torch.cuda.Stream) -> None:
        code = self._lib.dtype_code(fields[0].dtype) if fields[0].dtype in (torch.float32, torch.bfloat16) else 0
        lanes = []
        for other, theirs, mine in self.peers:
            rows = mine if kind == "fill" else theirs  # rows of MY extended band that `other` sent
            if rows is None:
                continue
            # the landing of the step whose send has just been counted; when this rank sends nothing to `other` in this
            # kind of exchange the counter advances here
            if (theirs if kind == "fill" else mine) is None:
                self.steps[(other, kind)] += 1
            there, here = self.remote[other][(self.rank, kind)], self.layout[(other, kind)]
            base = self.mapped[other].value
            lanes.append({"rows": rows, "step": self.steps[(other, kind)], "buffer": self.block.value + here["buffer"],
                          "wait": self.block.value + here["data"], "ticket": self.block.value + here["land_ticket"], "signal": base + there["ack"]})
        if lanes:
            self._launch("gm_peer_land_many", lanes, fields, (int(kind == "reduce"), code), stream)

    def _zero_halo(self, grads: tuple[Tensor, ...], stream: torch.cuda.Stream) -> None:
        with torch.cuda.stream(stream):
            for g in grads:
                if self.lo > self.elo:
                    g[:, : self.lo - self.elo].zero_()
                if self.ehi > self.hi:
                    g[:, self.hi - self.elo:].zero_()

    def fill_halos(self, *fields: Tensor, stream: torch.cuda.Stream | None = None) -> None:
        """Forward exchange on the current stream: every field's halo rows receive the owners' rows."""
        self._check(fields)
        stream = stream or torch.cuda.current_stream(self.device)
        self._send("fill", fields, stream)
        self._land("fill", fields, stream)

    def start_fill(self, *fields: Tensor):
        self.side.wait_stream(torch.cuda.current_stream(self.device))
        self.fill_halos(*fields, stream=self.side)
        done = torch.cuda.Event()
        done.record(self.side)
        return done

    def finish_fill(self, done) -> None:
        torch.cuda.current_stream(self.device).wait_event(done)

    def reduce_halos(self, *grads: Tensor, zero_halo: bool = True) -> None:
        """Backward exchange on the current stream: halo rows' partial sums go to their owners and are added there."""
        self._check(grads)
        stream = torch.cuda.current_stream(self.device)
        self._send("reduce", grads, stream)
        self._land("reduce", grads, stream)
        if zero_halo:
            self._zero_halo(grads, stream)

    def start_reduce(self, *grads: Tensor):
        self._check(grads)
        self.side.wait_stream(torch.cuda.current_stream(self.device))
        self._send("reduce", grads, self.side)
        done = torch.cuda.Event()
        done.record(self.side)
        return done, grads

    def finish_reduce(self, handle, zero_halo: bool = True) -> None:
        done, grads = handle
        stream = torch.cuda.current_stream(self.device)
        stream.wait_event(done)
        self._land("reduce", grads, stream)
        if zero_halo:
            self._zero_halo(grads, stream)


@dataclass(frozen=True)
class OverlapTables:
    """Row subsets of a rank's lattice tables for running the layer around the halo exchange."""

    full: object           # all owned target rows, all sources (as built)
    interior: object       # target rows whose neighbour rows are all owned: need no halo
    boundary: object       # the other target rows
    halo_sources: object   # source-major pass over the halo rows only (their dk, dv are what the owners are sent)
    owned_sources: object  # source-major pass over the rank's own rows


def overlap_tables(tables, plan: BandPlan, rank: int) -> OverlapTables:
    """Split the row lists of ``tables`` (built by :func:`band_geometry` + ``build_lattice_tables`` for ``rank``) so that
    the forward of the interior rows can run while the K / V halos travel and the source-major backward of the rank's own
    rows while the dK / dV halo sums travel."""
    import dataclasses

    lo, hi = plan.owned(rank)
    elo, ehi = plan.extended(rank)
    a, b, w = lo - elo, hi - elo, plan.halo  # owned rows in extended-row indices
    device = tables.row_order.device

    def pick(rows: Tensor, keep) -> Tensor:
        values = rows.cpu().tolist()
        return torch.tensor([r for r in values if keep(r)], dtype=rows.dtype, device=device)

    def is_interior(r: int) -> bool:
        return (elo == lo or r - w >= a) and (ehi == hi or r + w < b)

    def is_halo(r: int) -> bool:
        return r < a or r >= b

    return OverlapTables(
        full=tables,
        interior=dataclasses.replace(tables, row_order=pick(tables.row_order, is_interior)),
        boundary=dataclasses.replace(tables, row_order=pick(tables.row_order, lambda r: not is_interior(r))),
        halo_sources=dataclasses.replace(tables, t_row_order=pick(tables.t_row_order, is_halo)),
        owned_sources=dataclasses.replace(tables, t_row_order=pick(tables.t_row_order, lambda r: not is_halo(r))),
    )


def band_geometry(lattice, plan: BandPlan, rank: int, radius: float, *, max_frequency: int = 4, dtype: torch.dtype = torch.float32):
    """The neighbourhood geometry one rank keeps resident: nodes = its extended rows (band + halo),
    edges = those whose TARGET lies in the band (halo rows examine no candidates and get degree 0),
    node indices relative to the extended rows.  Built on the rank's own device."""
    from gm_attention_b200.geometry import SphericalLattice, compute_edge_geometry

    nlon = lattice.nlon
    lo, hi = plan.owned(rank)
    elo, ehi = plan.extended(rank)
    rows_ext = ehi - elo
    sel = slice(elo * nlon, ehi * nlon)
    sub = SphericalLattice(rows_ext, nlon, lattice.theta[elo:ehi], lattice.nodes[sel].contiguous(),
                           lattice.quadrature_weights[sel].contiguous(), lattice.frames[sel].contiguous())
    c_lo, c_hi = lattice.candidate_ranges(radius)
    c_lo = (c_lo[sel] - elo * nlon).clamp_min(0)
    c_hi = (c_hi[sel] - elo * nlon).clamp_max(rows_ext * nlon)
    owned = torch.zeros(rows_ext, dtype=torch.bool, device=lattice.nodes.device)
    owned[lo - elo: hi - elo] = True
    c_hi = torch.where(owned.repeat_interleave(nlon), c_hi, c_lo)
    return compute_edge_geometry(sub, sub.frames, radius, max_frequency=max_frequency, dtype=dtype, candidates=(c_lo.contiguous(), c_hi.contiguous()))


def row_degrees(lattice, radius: float) -> list[int]:
    """Neighbours per node of every lattice row (independent of longitude), from a count-only pass."""
    from gm_attention_b200 import _lib

    device = lattice.nodes.device
    n = lattice.n_nodes
    lo, hi = lattice.candidate_ranges(radius)
    degree = torch.empty(n, dtype=torch.int64, device=device)
    with torch.cuda.device(device):
        _lib.call("gm_geometry_count", _lib.ptr(lattice.nodes), n, _lib.ptr(lo), _lib.ptr(hi), float(radius), _lib.ptr(degree), _lib.stream(device))
    return degree.reshape(lattice.nlat, lattice.nlon)[:, 0].tolist()


def row_pair_counts(lattice, radius: float) -> Tensor:
    """``(nlat, 2 W + 1)``: neighbours a node of row ``i`` has in row ``i + dj`` (0 where the row does not exist),
    from count-only passes restricted to one source row each."""
    from gm_attention_b200 import _lib

    device = lattice.nodes.device
    nlat, nlon, w = lattice.nlat, lattice.nlon, lattice.band(radius)
    rows = torch.arange(nlat, device=device)
    counts = torch.zeros(nlat, 2 * w + 1, dtype=torch.int64, device=device)
    degree = torch.empty(nlat * nlon, dtype=torch.int64, device=device)
    with torch.cuda.device(device):
        for dj in range(-w, w + 1):
            src = rows + dj
            ok = (src >= 0) & (src < nlat)
            lo = (src.clamp(0, nlat - 1) * nlon)
            hi = torch.where(ok, lo + nlon, lo)
            lo_n, hi_n = lo.repeat_interleave(nlon).contiguous(), hi.repeat_interleave(nlon).contiguous()
            _lib.call("gm_geometry_count", _lib.ptr(lattice.nodes), nlat * nlon, _lib.ptr(lo_n), _lib.ptr(hi_n), float(radius),
                      _lib.ptr(degree), _lib.stream(device))
            counts[:, dj + w] = degree.reshape(nlat, nlon)[:, 0]
    return counts


def tensor_core_row_cost(pair_counts: Tensor) -> list[float]:
    """Relative cost of one lattice row under the tensor-core lattice kernels (forward + both backward passes).
    A warp owns 8 consecutive owners and walks, for every neighbour row, the 7 + cnt positions their windows cover in
    steps of 16; a CTA stages the neighbour row in chunks and pays a fixed cost per owner tile.  The weights are a
    fit to measured times of row groups from the pole to the equator of a 256 x 512 lattice (within 15 % for every
    group; the bands of an 8-way split, each timed alone, come out within 3 % of one another).  Narrow equatorial
    windows cost several times more PER EDGE than whole-row polar windows, which an edge-count balance ignores.  The constant
    per row was re-fitted on a 4-way split (bands [0, 40), [40, 128) and their mirror images timed side by side: with the
    constant at 10 the equatorial bands took 4.08 ms against 3.90 ms for the polar ones)."""
    cnt = pair_counts.to(torch.float64)
    present = cnt > 0
    steps = torch.ceil((7 + cnt) / 16)
    chunks = torch.ceil((63 + cnt) / 80) + torch.ceil((31 + cnt) / 80)
    cost = torch.where(present, 7.1 * steps + 2.9 * chunks, torch.zeros_like(cnt))
    return (14.5 + cost.sum(1)).tolist()
