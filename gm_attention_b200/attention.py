"""The fully fused gauge-attention layer as one differentiable op.

``out_i = sum_e softmax_e(scale <q_i, tau(e) k_j> + bias_e) tau(e) v_j`` per
head: the composition of the reference's ``Softmax`` op
(``nn/fused_attention.py:371-397``) with its eager value path (transport the
gathered values, weight by alpha, segment-sum per target;
``nn/kernels.py:156-189``, ``nn/_scatter.py:36-46``).  Neither alpha nor any
per-edge field is materialised; the backward recomputes the logits from the
saved per-(node, head) log-sum-exp.

The geometry describes one sample; ``q, k, v`` are ``(batch * n_nodes, D)`` and
every sample shares the tables.  Node fields may be float32, float64 or
bfloat16 (bf16 storage, fp32 arithmetic; the tables are then float32).
"""

from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Any

import torch
from torch import Tensor

from gm_attention_b200 import _lib


@dataclass(frozen=True)
class AttentionTables:
    """Resident per-edge constants of one edge set (device tensors) plus the
    head layout in host memory."""

    transport: Tensor  # (E, orders, 2) fp32 / fp64
    bias: Tensor  # (E,)
    inside: Tensor  # (E,) uint8
    row_ptr: Tensor  # (N + 1,) int64
    source: Tensor  # (E,) int64
    rows: tuple[tuple[int, int, int, int, int], ...]  # descriptor rows (n, a_n, offset, coeff offset, dim)
    heads: int
    scale: float

    @property
    def n_nodes(self) -> int:
        return self.row_ptr.shape[0] - 1

    @property
    def n_edges(self) -> int:
        return self.source.shape[0]

    def host_descriptor(self) -> Any:
        flat = [x for row in self.rows for x in row]
        return (ctypes.c_int64 * len(flat))(*flat)


def _table_dtype(dtype: torch.dtype) -> torch.dtype:
    return torch.float64 if dtype == torch.float64 else torch.float32


def _check(q: Tensor, k: Tensor, v: Tensor, t: AttentionTables) -> tuple[torch.device, int]:
    device = _lib.require_cuda(q, k, v, t.transport, t.bias, t.inside, t.row_ptr, t.source)
    if not (q.dim() == 2 and q.shape == k.shape == v.shape and q.dtype == k.dtype == v.dtype):
        raise RuntimeError("q, k and v must be (batch * n_nodes, D) tensors of one dtype")
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        raise RuntimeError("q, k and v must be contiguous")
    if t.n_nodes == 0 or q.shape[0] % t.n_nodes:
        raise RuntimeError(f"the node fields hold {q.shape[0]} rows, not a multiple of the geometry's {t.n_nodes} nodes")
    want = _table_dtype(q.dtype)
    if t.transport.dtype != want or t.bias.dtype != want:
        raise RuntimeError(f"tables must be {want} for {q.dtype} node fields")
    if t.inside.dtype != torch.uint8 or t.row_ptr.dtype != torch.int64 or t.source.dtype != torch.int64:
        raise RuntimeError("inside must be uint8; row_ptr and source int64")
    return device, q.shape[0] // t.n_nodes


def attention_forward(q: Tensor, k: Tensor, v: Tensor, t: AttentionTables) -> tuple[Tensor, Tensor]:
    """``(out, lse)``: the layer's output ``(batch * n_nodes, D)`` and each row's log-sum-exp ``(batch * n_nodes, H)``."""
    device, batch = _check(q, k, v, t)
    out = torch.empty_like(q)
    lse = torch.empty((q.shape[0], t.heads), dtype=_table_dtype(q.dtype), device=device)
    desc = t.host_descriptor()
    with torch.cuda.device(device):
        _lib.call("gm_attention_forward", _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(t.transport), _lib.ptr(t.bias),
                  _lib.ptr(t.inside), ctypes.addressof(desc), _lib.ptr(t.row_ptr), _lib.ptr(t.source), t.n_nodes, t.n_edges, batch,
                  q.shape[1], len(t.rows), t.transport.shape[1], t.heads, float(t.scale), _lib.dtype_code(q.dtype), _lib.ptr(out),
                  _lib.ptr(lse), _lib.stream(device))
    return out, lse


def attention_backward(dout: Tensor, q: Tensor, k: Tensor, v: Tensor, out: Tensor, lse: Tensor,
                       t: AttentionTables) -> tuple[Tensor, Tensor, Tensor]:
    device, batch = _check(q, k, v, t)
    dout = dout.contiguous()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    code = _lib.dtype_code(q.dtype)
    need = _lib.lib().gm_attention_backward_scratch_bytes(t.n_nodes, batch, q.shape[1], code)
    scratch = torch.empty(need, dtype=torch.uint8, device=device) if need else None
    desc = t.host_descriptor()
    with torch.cuda.device(device):
        _lib.call("gm_attention_backward", _lib.ptr(dout), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(lse),
                  _lib.ptr(t.transport), _lib.ptr(t.bias), _lib.ptr(t.inside), ctypes.addressof(desc), _lib.ptr(t.row_ptr),
                  _lib.ptr(t.source), t.n_nodes, t.n_edges, batch, q.shape[1], len(t.rows), t.transport.shape[1], t.heads,
                  float(t.scale), code, _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(scratch), _lib.stream(device))
    return dq, dk, dv


class GaugeAttention(torch.autograd.Function):
    """``GaugeAttention.apply(q, k, v, tables) -> out`` with ``tables`` an
    :class:`AttentionTables` (any graph) or a :class:`LatticeTables` (equiangular lattice fast path)."""

    @staticmethod
    def forward(ctx: Any, q: Tensor, k: Tensor, v: Tensor, tables: Any) -> Tensor:
        forward = lattice_attention_forward if isinstance(tables, LatticeTables) else attention_forward
        with torch.profiler.record_function("gm::attention/fused"):
            out, lse = forward(q.contiguous(), k.contiguous(), v.contiguous(), tables)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.tables = tables
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx: Any, grad_out: Tensor) -> tuple:  # type: ignore[override]
        q, k, v, out, lse = ctx.saved_tensors
        backward = lattice_attention_backward if isinstance(ctx.tables, LatticeTables) else attention_backward
        with torch.profiler.record_function("gm::attention/fused_backward"):
            dq, dk, dv = backward(grad_out, q.contiguous(), k.contiguous(), v.contiguous(), out, lse, ctx.tables)
        return dq, dk, dv, None


# ----------------------------------------------------------------------------- equiangular lattices

@dataclass(frozen=True)
class LatticeTables:
    """Compact per-(target row, source row, longitude offset) tables of a lattice
    with longitude-equivariant frames, forward and transposed (see
    ``gm_lattice_attention_forward`` in ``include/gm_b200.h``)."""

    rows: int
    nlon: int
    halo: int  # W
    entry_stride: int  # ES
    orders: int  # NORD
    win_cnt: Tensor
    win_lo: Tensor
    win_off: Tensor
    entries: Tensor
    row_order: Tensor
    t_win_cnt: Tensor
    t_win_lo: Tensor
    t_win_off: Tensor
    t_entries: Tensor
    t_row_order: Tensor
    desc_rows: tuple[tuple[int, int, int, int, int], ...]
    heads: int
    scale: float
    n_edges: int  # edges of one sample
    # the tensor-core kernels' own copy of the entries (12 or 20 words per offset, padded per row pair; see
    # ``tensor_core_entries``) with the window offsets into it, forward and transposed; None when the orders exceed 3
    tc_entries: Tensor | None = None
    tc_win_off: Tensor | None = None
    t_tc_entries: Tensor | None = None
    t_tc_win_off: Tensor | None = None
    # where the entries came from: the per-edge index (an edge of the target in column 0) of every entry, and the forward
    # entry of every transposed entry
    entry_edge: Tensor | None = None
    t_entry: Tensor | None = None

    def host_descriptor(self) -> Any:
        flat = [x for row in self.desc_rows for x in row]
        return (ctypes.c_int64 * len(flat))(*flat)


TC_PAD_BEFORE, TC_PAD_AFTER = 8, 24


def tensor_core_entry_words(norders: int) -> int:
    """32-bit words per entry of the tensor-core table: an odd multiple of 16 bytes."""
    return 20 if norders == 3 else 12


def tensor_core_entries(entries: Any, win_cnt: Any, win_off: Any, norders: int) -> tuple[Any, Any]:
    """The entry table in the layout the tensor-core lattice kernels read (numpy in, numpy out).

    Per longitude offset ``x`` of a row pair 12 words (orders <= 2) or 20 (order 3): ``[0..3]`` fp32 cos, sin of orders
    1, 2; ``[4..7]`` the same rounded to bf16 and packed in pairs (entry ``x`` in the low half, entry ``x - 1`` in the
    high half: the two accumulator elements a thread holds side by side); ``[8]`` bias * log2(e); with order 3 also
    ``[9..10]`` its cos, sin and ``[12..13]`` their packed pairs.  Every row pair's run is preceded by 8 and followed
    by 24 padding entries with bias ``-inf``: a 16 x 8 tile of (position, owner) pairs reads the entry of every pair
    without a bounds test, and pairs outside an owner's window come out with logit ``-inf``.  Returns ``(table,
    win_off)`` with ``win_off`` pointing at each run's first real entry."""
    import numpy as np

    log2e = 1.4426950408889634
    flat_cnt, flat_off = win_cnt.reshape(-1), win_off.reshape(-1)
    present = np.flatnonzero(flat_cnt > 0)
    lengths = flat_cnt[present].astype(np.int64)
    starts = np.zeros(present.shape[0], np.int64)
    if present.size:
        starts[1:] = np.cumsum(lengths + TC_PAD_BEFORE + TC_PAD_AFTER)[:-1]
    starts += TC_PAD_BEFORE
    total = int((lengths + TC_PAD_BEFORE + TC_PAD_AFTER).sum()) + 1
    phases = np.zeros((total, 6), np.float32)
    bias = np.full(total, -np.inf, np.float32)
    if present.size:
        within = np.arange(int(lengths.sum())) - np.repeat(np.cumsum(lengths) - lengths, lengths)
        src = np.repeat(flat_off[present].astype(np.int64), lengths) + within
        dst = np.repeat(starts, lengths) + within
        phases[dst, :2 * norders] = entries[src, :2 * norders]
        bias[dst] = entries[src, 2 * norders] * np.float32(log2e)
    bits = phases.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint32)  # bf16, round to nearest even
    previous = np.vstack([np.zeros((1, 6), np.uint32), rounded[:-1]])
    packed = np.ascontiguousarray((rounded | (previous << 16)).astype(np.uint32)).view(np.float32)
    table = np.zeros((total, tensor_core_entry_words(norders)), np.float32)
    table[:, 0:4] = phases[:, 0:4]
    table[:, 4:8] = packed[:, 0:4]
    table[:, 8] = bias
    if norders == 3:
        table[:, 9:11] = phases[:, 4:6]
        table[:, 12:14] = packed[:, 4:6]
    new_off = np.zeros_like(flat_off)
    new_off[present] = starts.astype(flat_off.dtype)
    return table, new_off.reshape(win_off.shape)


def lattice_layout_supported(rows: tuple[tuple[int, int, int, int, int], ...]) -> bool:
    """Head layouts the lattice kernels serve: at most one scalar row, at most four
    complex frequencies, all with the same multiplicity, runs of at most 4 copies per lane."""
    complex_mult = {a for n, a, *_ in rows if n > 0}
    scalar = [a for n, a, *_ in rows if n == 0]
    n_cf = sum(1 for n, *_ in rows if n > 0)
    if len(scalar) > 1 or len(complex_mult) > 1 or n_cf > 4:
        return False
    for lanes in (4, 8):
        nr = -(-(scalar[0] if scalar else 0) // lanes)
        uc = -(-(next(iter(complex_mult)) if complex_mult else 0) // lanes)
        fits = any(nr <= a and n_cf <= b and uc <= c for a, b, c in ((1, 2, 1), (2, 2, 2), (2, 3, 2), (4, 2, 4), (4, 4, 4)))
        if not fits:
            return False
    return True


def window_is_hard(geometry: Any, e0: Tensor, o0: Tensor, e1: Tensor) -> bool:
    """Whether a disagreement of the `inside` flags of two columns is a real asymmetry: under a hard window every
    in-window weight is far from zero, under a smooth one a weight that underflows in one column only is rounding."""
    differ = (geometry.inside[e0][o0] > 0) != (geometry.inside[e1] > 0)
    weights = torch.exp(torch.maximum(geometry.bias[e0][o0], geometry.bias[e1])[differ].double())
    return bool((weights > 1e-12 * torch.exp(geometry.bias[e0].double()).max()).any())


def build_lattice_tables(geometry: Any, rows: int, nlon: int, desc_rows: tuple[tuple[int, int, int, int, int], ...], heads: int,
                         scale: float) -> LatticeTables:
    """Collapse per-edge tables (``transport``, ``bias``, ``inside``, ``row_ptr``, ``source`` of a
    :class:`gm_attention_b200.nn.fused_attention.Geometry` or :class:`AttentionTables`) of a
    ``rows x nlon`` lattice into compact ones, reading the edges of the targets in column 0.
    Raises ``ValueError`` when a neighbourhood is not a cyclic run of longitudes per source row
    (the lattice / frames are then not longitude-symmetric: use the general kernels)."""
    import numpy as np

    device = geometry.row_ptr.device
    if nlon % 2:
        raise ValueError("the lattice path needs an even number of longitudes")
    row_ptr = geometry.row_ptr.reshape(-1)
    if row_ptr.numel() != rows * nlon + 1:
        raise ValueError(f"row_ptr describes {row_ptr.numel() - 1} nodes, not a {rows} x {nlon} lattice")
    per_node = (row_ptr[1:] - row_ptr[:-1]).reshape(rows, nlon)
    if not bool((per_node == per_node[:, :1]).all()):
        raise ValueError("the degree varies along a lattice row: not a longitude-symmetric lattice")
    # the tables below are read off column 0; a second column must hold the same runs shifted by its longitude
    # (frames that are not longitude-equivariant give the same edge set but different transport phases)
    probe = max(1, nlon // 3) if nlon > 1 else 0
    if probe:
        a0, b0 = row_ptr[torch.arange(rows, device=device) * nlon], row_ptr[torch.arange(rows, device=device) * nlon + probe]
        deg = per_node[:, 0]
        within = torch.arange(int(deg.sum()), device=device) - torch.repeat_interleave(torch.cumsum(deg, 0) - deg, deg)
        e0 = torch.repeat_interleave(a0, deg) + within
        e1 = torch.repeat_interleave(b0, deg) + within
        s0, s1 = geometry.source[e0], geometry.source[e1]
        key0 = (s0 // nlon) * nlon + (s0 % nlon + probe) % nlon  # column 0's sources moved to the probe column ...
        owner = torch.repeat_interleave(torch.arange(rows, device=device), deg)
        o0 = torch.argsort(owner * (rows * nlon) + key0)            # ... in the probe column's (sorted-source) order
        if not torch.equal(key0[o0], s1):
            raise ValueError("neighbourhoods are not the same longitude offsets in every column: not a longitude-symmetric lattice")
        n_ord = max((n for n, *_ in desc_rows), default=0)
        tau_gap = (geometry.transport[e0][o0][:, 1:n_ord + 1] - geometry.transport[e1][:, 1:n_ord + 1]).abs().max() if n_ord and e0.numel() else 0.0
        inside0 = geometry.inside[e0][o0] > 0
        # compare the weights exp(bias), not the logarithms: near the edge of a smooth window the logarithm of a vanishing
        # weight moves by O(1) under the rounding of the distance
        both = inside0 & (geometry.inside[e1] > 0)
        w0, w1 = torch.exp(geometry.bias[e0][o0][both].double()), torch.exp(geometry.bias[e1][both].double())
        bias_gap = ((w0 - w1).abs().max() / w0.abs().max().clamp_min(1e-300)) if bool(both.any()) else 0.0
        if float(tau_gap) > 1e-3 or float(bias_gap) > 1e-3 or int((inside0 != (geometry.inside[e1] > 0)).sum()) > 0 and window_is_hard(geometry, e0, o0, e1):
            raise ValueError("transport phases / bias differ between columns: the frames are not longitude-equivariant; use the general kernels")
    col0 = torch.arange(rows, device=device) * nlon
    starts, stops = row_ptr[col0].cpu().numpy(), row_ptr[col0 + 1].cpu().numpy()
    degree = stops - starts
    index = np.concatenate([np.arange(a, b) for a, b in zip(starts, stops)]) if degree.sum() else np.zeros(0, np.int64)
    index_t = torch.from_numpy(index).to(device)
    source = geometry.source.index_select(0, index_t).cpu().numpy()
    norders = max((n for n, *_ in desc_rows), default=0)
    if geometry.transport.shape[1] <= norders:
        raise ValueError(f"the transport table holds orders < {geometry.transport.shape[1]}, the heads need {norders}")
    tau = geometry.transport.index_select(0, index_t)[:, 1:norders + 1].float().cpu().numpy()  # (n, NORD, 2)
    bias = geometry.bias.index_select(0, index_t).float().cpu().numpy()
    inside = geometry.inside.index_select(0, index_t).cpu().numpy()
    bias = np.where(inside > 0, bias, -np.inf).astype(np.float32)
    owner_row = np.repeat(np.arange(rows), degree)
    src_row, src_lon = source // nlon, source % nlon
    dlon = np.where(src_lon < nlon // 2, src_lon, src_lon - nlon)
    drow = src_row - owner_row
    halo = int(np.abs(drow).max()) if drow.size else 0
    stride = 8 if 2 * norders + 1 <= 8 else 16
    width = 2 * halo + 1
    order = np.lexsort((dlon, drow, owner_row))
    owner_row, drow, dlon, tau, bias = owner_row[order], drow[order], dlon[order], tau[order], bias[order]
    entry_edge = index[order]
    win_cnt = np.zeros((rows, width), np.int32)
    win_lo = np.zeros((rows, width), np.int32)
    win_off = np.zeros((rows, width), np.int32)
    key = owner_row * width + (drow + halo)
    boundaries = np.flatnonzero(np.diff(key, prepend=-1)) if key.size else np.zeros(0, np.int64)
    ends = np.append(boundaries[1:], key.size)
    for a, b in zip(boundaries, ends):
        run = dlon[a:b]
        if not np.array_equal(run, np.arange(run[0], run[0] + (b - a))):
            raise ValueError("a neighbourhood is not a contiguous run of longitude offsets: not a longitude-symmetric lattice")
        i, c = divmod(int(key[a]), width)
        win_cnt[i, c], win_lo[i, c], win_off[i, c] = b - a, run[0], a
    entries = np.zeros((key.size, stride), np.float32)
    entries[:, :2 * norders] = tau.reshape(key.size, 2 * norders)
    entries[:, 2 * norders] = bias
    # transposed: owner = source row j, neighbours = targets in row i = j + di that see it; offsets negate, entries reverse
    t_cnt = np.zeros_like(win_cnt)
    t_lo = np.zeros_like(win_lo)
    t_off = np.zeros_like(win_off)
    t_entries = np.zeros_like(entries)
    t_entry = np.zeros(key.size, np.int64)
    cursor = 0
    for j in range(rows):
        for c in range(width):
            i = j + (c - halo)
            if not 0 <= i < rows:
                continue
            cc = (j - i) + halo
            n = int(win_cnt[i, cc])
            if n == 0:
                continue
            a = int(win_off[i, cc])
            t_cnt[j, c], t_lo[j, c], t_off[j, c] = n, -(int(win_lo[i, cc]) + n - 1), cursor
            t_entries[cursor:cursor + n] = entries[a:a + n][::-1]
            t_entry[cursor:cursor + n] = np.arange(a + n - 1, a - 1, -1)
            cursor += n
    cost = win_cnt.sum(1)
    t_cost = t_cnt.sum(1)
    row_order = np.array([r for r in np.argsort(-cost, kind="stable") if cost[r] > 0], np.int32)
    t_row_order = np.array([r for r in np.argsort(-t_cost, kind="stable") if t_cost[r] > 0], np.int32)
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(device)
    tc = (None, None, None, None)
    if 1 <= norders <= 3:
        tc_e, tc_o = tensor_core_entries(entries, win_cnt, win_off, norders)
        t_tc_e, t_tc_o = tensor_core_entries(t_entries, t_cnt, t_off, norders)
        tc = (dev(tc_e), dev(tc_o), dev(t_tc_e), dev(t_tc_o))
    return LatticeTables(rows, nlon, halo, stride, norders, dev(win_cnt), dev(win_lo), dev(win_off), dev(entries), dev(row_order),
                         dev(t_cnt), dev(t_lo), dev(t_off), dev(t_entries), dev(t_row_order), tuple(tuple(int(x) for x in r) for r in desc_rows),
                         heads, float(scale), int(geometry.source.shape[0]), *tc, dev(entry_edge.astype(np.int64)), dev(t_entry))


def _check_lattice(q: Tensor, k: Tensor, v: Tensor, t: LatticeTables) -> tuple[torch.device, int]:
    device = _lib.require_cuda(q, k, v, t.entries)
    if not (q.dim() == 2 and q.shape == k.shape == v.shape and q.dtype == k.dtype == v.dtype):
        raise RuntimeError("q, k and v must be (batch * n_nodes, D) tensors of one dtype")
    if q.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("the lattice kernels take float32 or bfloat16 node fields")
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        raise RuntimeError("q, k and v must be contiguous")
    n = t.rows * t.nlon
    if q.shape[0] % n:
        raise RuntimeError(f"the node fields hold {q.shape[0]} rows, not a multiple of the lattice's {n} nodes")
    return device, q.shape[0] // n


def tensor_core_layout_supported(rows: tuple[tuple[int, int, int, int, int], ...]) -> bool:
    """Head layouts of the tensor-core lattice kernels: an optional scalar block of <= 16 copies and one
    to three complex frequencies of orders 1, 2, 3 sharing a multiplicity <= 16 (the instantiated combinations)."""
    scalar = [a for n, a, *_ in rows if n == 0]
    mult = {a for n, a, *_ in rows if n > 0}
    orders = sorted(n for n, *_ in rows if n > 0)
    n_cf = len(orders)
    if len(scalar) > 1 or len(mult) != 1 or (scalar and scalar[0] > 16) or next(iter(mult)) > 16:
        return False
    if orders != list(range(1, n_cf + 1)):
        return False
    ksc = 2 if next(iter(mult)) > 8 else 1
    return (bool(scalar), n_cf, ksc) in {(True, 2, 2), (True, 2, 1), (True, 3, 1), (True, 1, 2), (True, 1, 1), (False, 2, 1)}


def four_head_layout_supported(t: LatticeTables, width: int) -> bool:
    """Head layouts and lattices of the four-heads-per-CTA tensor-core kernels: 4 heads of 16 scalar copies and 16
    complex copies of each of the orders 1 .. n (n <= 3), every block on a 16-byte boundary and inside the row, at most
    32 neighbour rows, at least 40 longitudes, the padded entry table present."""
    if t.heads != 4 or t.tc_entries is None or width % 8 or 2 * t.halo + 1 > 32 or t.nlon < 40:
        return False
    orders = [n for n, *_ in t.desc_rows]
    if orders != list(range(0, len(orders))) or not 2 <= len(orders) <= 4:
        return False
    for n, a_n, off, _, _ in t.desc_rows:
        if a_n != 16 or off % 8 or off + (64 if n == 0 else 128) > width:
            return False
    return True


#: "auto": bf16 node fields take the tensor-core kernels when the head layout allows; "0": never
TENSOR_CORES = os.environ.get("GM_LATTICE_TENSOR_CORES", "auto")
#: "1": the four-heads-per-CTA kernels where the layout allows; "0" (default): the one-head-per-CTA kernels, which
#: measured 6 % faster over the three passes at 256 x 512 x 8 (the four-head forward / target-major passes are on par,
#: its source-major pass spills)
FOUR_HEADS = os.environ.get("GM_LATTICE_FOUR_HEADS", "0")


def lattice_attention_forward(q: Tensor, k: Tensor, v: Tensor, t: LatticeTables, tensor_cores: bool | None = None,
                              out: Tensor | None = None, lse: Tensor | None = None) -> tuple[Tensor, Tensor]:
    """``(out, lse)`` for the target rows in ``t.row_order``.  ``out`` / ``lse`` of an earlier call can be passed in to
    have another set of rows written into the same buffers (rows outside every set keep 0 / -inf)."""
    device, batch = _check_lattice(q, k, v, t)
    if tensor_cores is None:
        tensor_cores = TENSOR_CORES != "0" and q.dtype == torch.bfloat16 and tensor_core_layout_supported(t.desc_rows)
    full = t.row_order.numel() == t.rows
    if out is None:
        out = torch.empty_like(q) if full else torch.zeros_like(q)
    if lse is None:
        lse = torch.empty((q.shape[0], t.heads), dtype=torch.float32, device=device) if full else \
            torch.full((q.shape[0], t.heads), float("-inf"), dtype=torch.float32, device=device)
    if t.row_order.numel() == 0:  # a band too narrow to have rows of this class (e.g. no row clear of the halo)
        return out, lse
    desc = t.host_descriptor()
    four = tensor_cores and FOUR_HEADS == "1" and four_head_layout_supported(t, q.shape[1])
    off, ent, stride = (t.tc_win_off, t.tc_entries, t.tc_entries.shape[1]) if four else (t.win_off, t.entries, t.entry_stride)
    common = (_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(t.win_cnt), _lib.ptr(t.win_lo), _lib.ptr(off), _lib.ptr(ent),
              _lib.ptr(t.row_order), t.row_order.numel(), ctypes.addressof(desc), len(t.desc_rows), t.rows, t.nlon, batch, q.shape[1],
              t.heads, t.halo, stride, t.orders, float(t.scale))
    with torch.cuda.device(device):
        if four:
            _lib.call("gm_lattice_attention_forward_tc4", *common, _lib.ptr(out), _lib.ptr(lse), _lib.stream(device))
        elif tensor_cores:
            _lib.call("gm_lattice_attention_forward_tc", *common, _lib.ptr(out), _lib.ptr(lse), _lib.stream(device))
        else:
            _lib.call("gm_lattice_attention_forward", *common, _lib.dtype_code(q.dtype), _lib.ptr(out), _lib.ptr(lse), _lib.stream(device))
    return out, lse


def lattice_attention_backward(dout: Tensor, q: Tensor, k: Tensor, v: Tensor, out: Tensor, lse: Tensor, t: LatticeTables,
                               tensor_cores: bool | None = None, passes: int = 7, workspace: tuple | None = None) -> tuple[Tensor, Tensor, Tensor]:
    """``(dq, dk, dv)``.  ``passes`` (tensor-core path only) selects Delta (1), the target-major pass (2) and the
    source-major pass (4) for timing them separately; ``workspace = (dq, dk, dv, delta)`` reuses buffers of an earlier call."""
    device, batch = _check_lattice(q, k, v, t)
    if tensor_cores is None:
        tensor_cores = TENSOR_CORES != "0" and q.dtype == torch.bfloat16 and tensor_core_layout_supported(t.desc_rows)
    dout = dout.contiguous()
    alloc = torch.empty_like if t.row_order.numel() == t.rows else torch.zeros_like
    alloc_t = torch.empty_like if t.t_row_order.numel() == t.rows else torch.zeros_like
    if workspace is not None:
        dq, dk, dv, delta = workspace
    else:
        dq, dk, dv = alloc(q), alloc_t(q), alloc_t(q)
        delta = torch.empty((q.shape[0], t.heads), dtype=torch.float32, device=device)
    # passes over an empty row list are dropped (a band too narrow to have rows of that class)
    if t.row_order.numel() == 0:
        passes &= ~3
    if t.t_row_order.numel() == 0:
        passes &= ~4
    if passes == 0 or (t.row_order.numel() == 0 and t.t_row_order.numel() == 0):
        return dq, dk, dv
    desc = t.host_descriptor()
    four = tensor_cores and FOUR_HEADS == "1" and four_head_layout_supported(t, q.shape[1])
    off, ent, t_off, t_ent, stride = (t.tc_win_off, t.tc_entries, t.t_tc_win_off, t.t_tc_entries, t.tc_entries.shape[1]) if four else \
        (t.win_off, t.entries, t.t_win_off, t.t_entries, t.entry_stride)
    # an empty list still needs an address (the entry points refuse null pointers): the other list's, with a count of zero
    rows_ptr = _lib.ptr(t.row_order) or _lib.ptr(t.t_row_order)
    t_rows_ptr = _lib.ptr(t.t_row_order) or _lib.ptr(t.row_order)
    common = (_lib.ptr(dout), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(lse), _lib.ptr(t.win_cnt), _lib.ptr(t.win_lo),
              _lib.ptr(off), _lib.ptr(ent), rows_ptr, t.row_order.numel(), _lib.ptr(t.t_win_cnt),
              _lib.ptr(t.t_win_lo), _lib.ptr(t_off), _lib.ptr(t_ent), t_rows_ptr, t.t_row_order.numel(),
              ctypes.addressof(desc), len(t.desc_rows), t.rows, t.nlon, batch, q.shape[1], t.heads, t.halo, stride, t.orders,
              float(t.scale))
    outputs = (_lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(delta), _lib.stream(device))
    with torch.cuda.device(device):
        if four:
            _lib.call("gm_lattice_attention_backward_tc4_passes", *common, *outputs[:4], int(passes), outputs[4])
        elif tensor_cores:
            _lib.call("gm_lattice_attention_backward_tc_passes", *common, *outputs[:4], int(passes), outputs[4])
        else:
            _lib.call("gm_lattice_attention_backward", *common, _lib.dtype_code(q.dtype), *outputs)
    return dq, dk, dv


# ----------------------------------------------------------------------------- host-resident fields

class HostPipeline:
    """Forward + backward of the fused layer for fields that live in (pinned) HOST memory.

    Samples share the geometry and are otherwise independent, so the batch is cut
    into chunks of samples and three CUDA streams run concurrently: chunk ``i + 1``
    is copied host -> device while chunk ``i`` is computed and the results of chunk
    ``i - 1`` are copied device -> host.  Device staging buffers are allocated once
    (two chunks deep) and reused across calls."""

    def __init__(self, tables: Any, batch: int, width: int, dtype: torch.dtype, device: torch.device, chunk: int = 1,
                 halo: Any = None) -> None:
        """``halo``: a :class:`gm_attention_b200.parallel.HaloExchanger` when the lattice is sharded into latitude
        bands: every chunk's key / value halos are filled before its forward and its dk / dv halo sums are handed
        back after its backward, on the compute stream (all ranks walk the chunks in the same order)."""
        if chunk < 1 or batch % chunk:
            raise ValueError(f"the batch of {batch} samples is not a whole number of chunks of {chunk}")
        self.tables, self.batch, self.chunk, self.device, self.halo = tables, batch, chunk, device, halo
        n = (tables.rows * tables.nlon) if isinstance(tables, LatticeTables) else tables.n_nodes
        self.n_nodes = n
        shape = (chunk * n, width)
        self.inputs = [[torch.empty(shape, dtype=dtype, device=device) for _ in range(4)] for _ in range(2)]
        self.streams = [torch.cuda.Stream(device) for _ in range(3)]  # h2d, compute, d2h
        self.consumed: list[Any] = [None, None]  # per staging slot: the compute that last read it has finished
        self.lattice = isinstance(tables, LatticeTables)
        self.profile = False  # True: every run records when each of the three streams starts and ends its share
        self._marks: list[tuple[Any, Any]] = []

    def run(self, q: Tensor, k: Tensor, v: Tensor, dout: Tensor, out: Tensor, dq: Tensor, dk: Tensor, dv: Tensor,
            wait: bool = True) -> None:
        """All arguments are host tensors ``(batch * n_nodes, D)`` (pinned for overlap); the last four are written.

        ``wait=True``: the caller's current stream waits for the results (they are valid once that stream has
        synchronised).  ``wait=False`` only enqueues: back-to-back calls then overlap (the first copies of one call
        run under the last compute and write-back of the previous one); call :meth:`join` before reading results."""
        fwd = lattice_attention_forward if self.lattice else attention_forward
        bwd = lattice_attention_backward if self.lattice else attention_backward
        h2d, comp, d2h = self.streams
        rows = self.chunk * self.n_nodes
        n_chunks = self.batch // self.chunk
        main = torch.cuda.current_stream(self.device)
        for s in self.streams:
            s.wait_stream(main)
        loaded = [torch.cuda.Event() for _ in range(n_chunks)]
        computed = [torch.cuda.Event() for _ in range(n_chunks)]
        if self.profile:
            self._marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in self.streams]
            for (first, _), st in zip(self._marks, self.streams):
                first.record(st)
        for i in range(n_chunks):
            sl = slice(i * rows, (i + 1) * rows)
            slot = self.inputs[i % 2]
            with torch.cuda.stream(h2d):
                if self.consumed[i % 2] is not None:
                    h2d.wait_event(self.consumed[i % 2])  # the slot's previous occupant (this call's or the last one's) has been consumed
                for dst, src in zip(slot, (q, k, v, dout)):
                    dst.copy_(src[sl], non_blocking=True)
                loaded[i].record(h2d)
            with torch.cuda.stream(comp):
                comp.wait_event(loaded[i])
                if self.halo is not None:
                    banded = (self.chunk, self.tables.rows, self.tables.nlon, slot[1].shape[1])
                    self.halo.fill_halos(slot[1].view(banded), slot[2].view(banded))
                o, lse = fwd(slot[0], slot[1], slot[2], self.tables)
                grads = bwd(slot[3], slot[0], slot[1], slot[2], o, lse, self.tables)
                if self.halo is not None:
                    self.halo.reduce_halos(grads[1].view(banded), grads[2].view(banded))
                computed[i].record(comp)
                self.consumed[i % 2] = computed[i]
            with torch.cuda.stream(d2h):
                d2h.wait_event(computed[i])
                for dst, src in zip((out, dq, dk, dv), (o, *grads)):
                    dst[sl].copy_(src, non_blocking=True)
                    src.record_stream(d2h)
        if self.profile:
            for (_, last), st in zip(self._marks, self.streams):
                last.record(st)
        if wait:
            self.join()

    def phase_ms(self) -> dict[str, float]:
        """Of the last profiled run (after a synchronise): how long each stream was busy or waiting between its first and
        last operation -- host-to-device copies, compute (with the halo exchanges), device-to-host copies.  The three
        overlap; the run takes about as long as the longest."""
        names = ("h2d", "compute", "d2h")
        return {n: first.elapsed_time(last) for n, (first, last) in zip(names, self._marks)}

    def join(self) -> None:
        """Make the caller's current stream wait for everything enqueued so far."""
        main = torch.cuda.current_stream(self.device)
        for s in self.streams:
            main.wait_stream(s)
