"""Depthwise steerable convolution on a longitude-symmetric lattice WITHOUT the per-edge coefficient stream.

The reference evaluates its radial network on every edge and hands the depthwise op ``E x (a_0 + W)`` coefficients
(``nn/depthwise.py:206-238`` ``stacked_coefficients`` -> ``nn/fused_attention.py:309-321`` ``forward_depthwise``):
53 GB in float32 for ONE sample of a 256 x 512 lattice at radius 4 pi / 256, so it has to chunk.  On a lattice whose
frames turn with the longitude, the distance, both phase tables and the aggregation weight of an edge depend on (target
row, source row, longitude offset) only -- 44 920 distinct entries instead of 22 999 040 edges there.  So here

1. the radial network runs on the ENTRIES (:class:`RadialCoefficients`: the reference's Gaussian basis, trunk and two
   read-outs, ``nn/kernels.py:191-240``, ``nn/depthwise.py:60-121``; ordinary PyTorch, ordinary autograd);
2. :func:`fold` turns an entry's coefficients, phases and weight into one real 2 x 2 matrix per complex copy and one
   real factor per scalar channel (``z -> A tau z + w B conj(tau z)`` is a real-linear map of the plane; also ordinary
   tensor algebra, so autograd carries the table's gradient back to the network);
3. :class:`LatticeDepthwise` applies the table (``gm_lattice_conv_apply``) and, backward, forms the field's gradient
   (the same kernel on the transposed windows) and the table's gradient (``gm_lattice_conv_table_grad``).

Results equal the reference's op on the same per-edge coefficients to rounding (tested against its compiled CPU
driver and the C oracle); the table can also be folded from coefficients that came from anywhere else.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Sequence

import numpy as np
import torch
from torch import Tensor, nn

from gm_attention_b200 import _lib
from gm_attention_b200.attention import LatticeTables, build_lattice_tables

OFFSETS_PER_BLOCK = 8  # offsets one CTA of the table-gradient kernel covers


@dataclass(frozen=True)
class ConvTables:
    """Windows of a lattice (forward and transposed) with the per-entry constants the fold needs."""

    lattice: LatticeTables
    rows: tuple[tuple[int, int, int, int, int], ...]  # descriptor rows (n, a_n, flat offset, coefficient offset, dim)
    a_0: int
    complex_width: int
    table_width: int
    items: Tensor  # (n_items, 3) int32: kind, field column, table column
    blocks: Tensor  # (n_blocks, 2) int32: window index, first offset
    distances: Tensor  # (entries,)
    weights: Tensor  # (entries,) aggregation weight of the entry's edges
    tau: Tensor  # (entries, complex frequencies) complex64: transport phase of order n
    omega: Tensor  # (entries, complex frequencies) complex64: (r / cutoff)^{2n} e^{2 i n phi}

    @property
    def n_entries(self) -> int:
        return int(self.distances.shape[0])


def conv_tables(geometry: Any, distances: Tensor, weights: Tensor, rows: Sequence[Sequence[int]], n_rows: int, nlon: int) -> ConvTables:
    """``geometry``: the per-edge constants of the lattice's edge set (:func:`gm_attention_b200.nn.fused_attention.geometry`);
    ``distances`` / ``weights``: per-edge geodesic distance and aggregation weight (window x tangent quadrature weight,
    divided by the target's window mass when the layer normalises); ``rows``: the depthwise plan's descriptor rows."""
    rows = tuple(tuple(int(x) for x in r) for r in rows)
    scalar = [r for r in rows if r[0] == 0]
    a_0 = scalar[0][1] if scalar else 0
    if a_0 % 2:
        raise ValueError("the lattice depthwise kernels pair the scalar channels: their number must be even")
    lat = build_lattice_tables(geometry, n_rows, nlon, rows, 1, 1.0)
    edge = lat.entry_edge
    complex_rows = [r for r in rows if r[0] > 0]
    padded = -(-a_0 // 4) * 4
    items, column = [], padded
    for p in range(a_0 // 2):
        items.append((1, scalar[0][2] + 2 * p, 2 * p))
    for n, copies, flat, _, _ in complex_rows:
        for c in range(copies):
            items.append((0, flat + 2 * c, column))
            column += 4
    device = edge.device
    cnt = lat.win_cnt.cpu().numpy().reshape(-1)
    blocks = [(w, d) for w in np.flatnonzero(cnt > 0) for d in range(0, int(cnt[w]), OFFSETS_PER_BLOCK)]
    blocks.sort(key=lambda wd: -min(OFFSETS_PER_BLOCK, int(cnt[wd[0]]) - wd[1]))  # full blocks first
    rho = geometry.rho.index_select(0, edge).float()
    tau = [torch.view_as_complex(geometry.transport.index_select(0, edge)[:, n].float().contiguous()) for n, *_ in complex_rows]
    omega = []
    for n, *_ in complex_rows:
        power = torch.ones_like(rho)
        for _ in range(2 * n):  # repeated multiplication, as the reference forms it (attention.h:137-142)
            power = power * rho
        omega.append(power * torch.view_as_complex(geometry.angular.index_select(0, edge)[:, 2 * n].float().contiguous()))
    stack = lambda xs: torch.stack(xs, 1) if xs else torch.zeros((edge.shape[0], 0), dtype=torch.complex64, device=device)
    return ConvTables(lat, rows, a_0, sum(4 * r[1] for r in complex_rows), column,
                      torch.tensor(items, dtype=torch.int32, device=device).reshape(-1, 3),
                      torch.tensor(blocks, dtype=torch.int32, device=device).reshape(-1, 2),
                      distances.index_select(0, edge).float(), weights.index_select(0, edge).float(), stack(tau), stack(omega))


def fold(real_coefficients: Tensor | None, complex_coefficients: Tensor | None, t: ConvTables) -> Tensor:
    """Per-entry coefficients ``(entries, a_0)`` / ``(entries, W)`` in the reference's layout (per frequency ``A (a_n, 2)``
    then ``B (a_n, 2)``, ``nn/depthwise.py:176-186``) -> the table ``(entries, table_width)`` the kernels read: the scalar
    factors times the weight, then per complex copy the matrix ``[[a, b], [c, d]]`` of
    ``z -> w_e (A tau z + omega B conj(tau z))`` acting on ``(re z, im z)``.  Differentiable."""
    weight = t.weights.unsqueeze(1)
    parts = []
    if t.a_0:
        scaled = real_coefficients.float() * weight
        pad = -t.a_0 % 4
        parts.append(torch.nn.functional.pad(scaled, (0, pad)) if pad else scaled)
    index = 0
    for n, copies, _, offset, _ in t.rows:
        if n == 0:
            continue
        block = complex_coefficients[:, offset:offset + 4 * copies].float().reshape(-1, 2, copies, 2)
        linear = torch.view_as_complex(block[:, 0].contiguous())
        antilinear = torch.view_as_complex(block[:, 1].contiguous())
        tau, omega = t.tau[:, index:index + 1], t.omega[:, index:index + 1]
        a = weight * tau * linear
        b = weight * (omega * tau.conj()) * antilinear
        parts.append(torch.stack([a.real + b.real, b.imag - a.imag, a.imag + b.imag, a.real - b.real], -1).reshape(-1, 4 * copies))
        index += 1
    return torch.cat(parts, 1).contiguous()


def _apply(x: Tensor, table: Tensor, t: ConvTables, transposed: bool) -> Tensor:
    lat = t.lattice
    device = _lib.require_cuda(x, table)
    nodes = lat.rows * lat.nlon
    if x.dim() != 2 or x.shape[0] % nodes or not x.is_contiguous():
        raise RuntimeError(f"the field must be a contiguous (batch * {nodes}, D) tensor")
    if table.shape != (t.n_entries, t.table_width) or table.dtype != torch.float32 or not table.is_contiguous():
        raise RuntimeError(f"the table must be a contiguous float32 ({t.n_entries}, {t.table_width}) tensor")
    y = torch.empty_like(x)
    cnt, lo, off, order = (lat.t_win_cnt, lat.t_win_lo, lat.t_win_off, lat.t_row_order) if transposed else \
        (lat.win_cnt, lat.win_lo, lat.win_off, lat.row_order)
    if order.numel() != lat.rows:
        y.zero_()
    with torch.cuda.device(device):
        _lib.call("gm_lattice_conv_apply", _lib.ptr(x), _lib.ptr(table), _lib.ptr(t.items), t.items.shape[0], _lib.ptr(cnt), _lib.ptr(lo),
                  _lib.ptr(off), _lib.ptr(order), order.numel(), lat.rows, lat.nlon, x.shape[0] // nodes, x.shape[1], lat.halo,
                  t.table_width, int(transposed), _lib.dtype_code(x.dtype), _lib.ptr(y), _lib.stream(device))
    return y


def _table_gradient(grad: Tensor, x: Tensor, t: ConvTables) -> Tensor:
    lat = t.lattice
    device = _lib.require_cuda(grad, x)
    out = torch.zeros((t.n_entries, t.table_width), dtype=torch.float32, device=device)
    with torch.cuda.device(device):
        _lib.call("gm_lattice_conv_table_grad", _lib.ptr(grad), _lib.ptr(x), _lib.ptr(t.items), t.items.shape[0], _lib.ptr(lat.win_cnt),
                  _lib.ptr(lat.win_lo), _lib.ptr(lat.win_off), _lib.ptr(t.blocks), t.blocks.shape[0], lat.rows, lat.nlon,
                  x.shape[0] // (lat.rows * lat.nlon), x.shape[1], lat.halo, t.table_width, _lib.dtype_code(x.dtype), _lib.ptr(out),
                  _lib.stream(device))
    return out


class LatticeDepthwise(torch.autograd.Function):
    """``y = table applied to v`` on the lattice, differentiable in ``v`` and in the table."""

    @staticmethod
    def forward(ctx: Any, v: Tensor, table: Tensor, tables: ConvTables) -> Tensor:
        ctx.save_for_backward(v, table)
        ctx.tables = tables
        return _apply(v, table, tables, False)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx: Any, grad_out: Tensor) -> tuple:  # type: ignore[override]
        v, table = ctx.saved_tensors
        t = ctx.tables
        grad_out = grad_out.contiguous()
        grad_v = _apply(grad_out, table.index_select(0, t.lattice.t_entry), t, True) if ctx.needs_input_grad[0] else None
        grad_table = _table_gradient(grad_out, v, t) if ctx.needs_input_grad[1] else None
        return grad_v, grad_table, None


def lattice_depthwise(v: Tensor, real_coefficients: Tensor | None, complex_coefficients: Tensor | None, tables: ConvTables) -> Tensor:
    """The depthwise convolution of the flat field ``v (batch * nodes, D)`` under per-ENTRY coefficients."""
    return LatticeDepthwise.apply(v.contiguous(), fold(real_coefficients, complex_coefficients, tables), tables)  # type: ignore[no-any-return]


class RadialCoefficients(nn.Module):
    """The reference's radial network of a depthwise kernel, evaluated on distances: Gaussian basis in
    ``s = (r / cutoff)^2`` with centres evenly spaced on [0, 1] and width = their spacing (``nn/kernels.py:191-240``), a
    trunk of ``Linear`` + ``SiLU`` pairs (``:328-343``), and two linear read-outs of widths ``a_0`` and ``W``
    (``nn/depthwise.py:100-121``)."""

    def __init__(self, a_0: int, complex_width: int, cutoff: float, n_radial_basis: int = 8, radial_hidden_features: Sequence[int] = (16,),
                 bias: bool = True, dtype: torch.dtype | None = None, device: Any = None) -> None:
        super().__init__()
        self.cutoff = float(cutoff)
        self.spacing = 1.0 / max(n_radial_basis - 1, 1)
        self.register_buffer("centers", torch.linspace(0.0, 1.0, n_radial_basis, dtype=dtype, device=device))
        widths = [n_radial_basis, *radial_hidden_features]
        layers: list[nn.Module] = []
        for fan_in, fan_out in zip(widths[:-1], widths[1:]):
            layers += [nn.Linear(fan_in, fan_out, bias=bias, dtype=dtype, device=device), nn.SiLU()]
        self.radial_trunk = nn.Sequential(*layers)
        self.real_head = nn.Linear(widths[-1], a_0, bias=bias, dtype=dtype, device=device) if a_0 else None
        self.complex_head = nn.Linear(widths[-1], complex_width, bias=bias, dtype=dtype, device=device) if complex_width else None

    def forward(self, distances: Tensor) -> tuple[Tensor | None, Tensor | None]:
        normalized = distances / self.cutoff
        difference = (normalized * normalized).unsqueeze(-1) - self.centers
        hidden = self.radial_trunk(torch.exp(-0.5 * (difference / self.spacing) ** 2))
        return (None if self.real_head is None else self.real_head(hidden),
                None if self.complex_head is None else self.complex_head(hidden))
