"""Neighbourhood geometry, built once on the device and kept resident.

:func:`compute_edge_geometry` mirrors the reference's function of the same name
(``discretization/edge_geometry.py:320-396``): from a grid (nodes, quadrature
weights, float64 lattice coordinates) and tangent frames it returns the
target-major CSR of all directed pairs within ``coverage_radius`` (bit-exact
with the reference's search) and the per-edge tables, as an
:class:`EdgeGeometry` with the reference's field names.  The search and the
tables run in CUDA kernels (``csrc/geometry.cu``); only the prefix sum of the
degrees uses a torch op.

:func:`midpoint_lattice` builds the equiangular lattice of the benchmark
configurations (colatitudes ``(i + 1/2) pi / nlat``, longitudes
``2 pi j / nlon``) with longitude-equivariant (east, north) frames, for which
every table depends on (target row, source row, longitude offset) only.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

import torch
from torch import Tensor

from gm_attention_b200 import _lib

DEFAULT_MAX_FREQUENCY = 4


@dataclass(frozen=True)
class SphericalLattice:
    """An equiangular lattice: node ``i * nlon + j`` sits at colatitude
    ``theta[i]`` and longitude ``2 pi j / nlon``.  All tensors are float64 on
    ``device``; the object also serves as the ``grid`` of :func:`compute_edge_geometry`."""

    nlat: int
    nlon: int
    theta: Tensor  # (nlat,)
    nodes: Tensor  # (N, 3) float64
    quadrature_weights: Tensor  # (N,)
    frames: Tensor  # (N, 3, 2): columns (east, north)

    @property
    def exact_nodes(self) -> Tensor:
        return self.nodes

    @property
    def n_nodes(self) -> int:
        return self.nlat * self.nlon

    def band(self, radius: float) -> int:
        """Rows ``|i - j| <= band`` can hold a neighbour: every geodesic distance is
        at least the colatitude difference."""
        spacing = float((self.theta[1:] - self.theta[:-1]).min()) if self.nlat > 1 else math.pi
        return min(self.nlat - 1, int(math.ceil(radius / spacing - 1e-9)))

    def candidate_ranges(self, radius: float) -> tuple[Tensor, Tensor]:
        """Per target the index range of the lattice rows within :meth:`band`."""
        w = self.band(radius)
        rows = torch.arange(self.nlat, device=self.nodes.device)
        lo = ((rows - w).clamp_min(0) * self.nlon).repeat_interleave(self.nlon)
        hi = ((rows + w + 1).clamp_max(self.nlat) * self.nlon).repeat_interleave(self.nlon)
        return lo.contiguous(), hi.contiguous()


def midpoint_lattice(nlat: int, nlon: int, device: torch.device | str = "cuda") -> SphericalLattice:
    theta = (torch.arange(nlat, dtype=torch.float64, device=device) + 0.5) * (math.pi / nlat)
    phi = torch.arange(nlon, dtype=torch.float64, device=device) * (2.0 * math.pi / nlon)
    t, p = torch.meshgrid(theta, phi, indexing="ij")
    nodes = torch.stack([t.sin() * p.cos(), t.sin() * p.sin(), t.cos()], -1).reshape(-1, 3)
    weights = (t.sin() * (math.pi / nlat) * (2.0 * math.pi / nlon)).reshape(-1)
    east = torch.stack([-p.sin(), p.cos(), torch.zeros_like(p)], -1).reshape(-1, 3)
    north = torch.stack([-t.cos() * p.cos(), -t.cos() * p.sin(), t.sin()], -1).reshape(-1, 3)
    return SphericalLattice(nlat, nlon, theta, nodes.contiguous(), weights.contiguous(), torch.stack([east, north], -1).contiguous())


@dataclass(frozen=True)
class EdgeGeometry:
    """Directed edges ``i <- j`` in target-major, source-minor order with their
    tables (field names of the reference's ``EdgeGeometry``, ``edge_geometry.py:25-79``)."""

    edge_index: Tensor  # (2, E) int64
    row_ptr: Tensor  # (N + 1,) int64
    log_coordinates: Tensor  # (E, 2)
    distances: Tensor  # (E,)
    polar_angles: Tensor
    transport_angles: Tensor
    tangent_quadrature_weights: Tensor
    angular_phases: Tensor  # (E, K + 1) complex
    transport_phases: Tensor  # (E, K + 1) complex

    @property
    def n_edges(self) -> int:
        return self.edge_index.shape[1]

    @property
    def target_index(self) -> Tensor:
        return self.edge_index[0]

    @property
    def source_index(self) -> Tensor:
        return self.edge_index[1]

    @property
    def max_frequency(self) -> int:
        return self.angular_phases.shape[-1] - 1

    def _harmonic(self, table: Tensor, order: int) -> Tensor:
        if isinstance(order, bool) or not isinstance(order, int):
            raise TypeError(f"order must be an int, got {type(order).__name__}.")
        if abs(order) > self.max_frequency:
            raise ValueError(f"Harmonic order {order} is not tabulated (orders up to {self.max_frequency}).")
        column = table[:, abs(order)]
        return column.conj() if order < 0 else column

    def angular_harmonic(self, order: int) -> Tensor:
        return self._harmonic(self.angular_phases, order)

    def transport_harmonic(self, order: int) -> Tensor:
        return self._harmonic(self.transport_phases, order)

    _PER_EDGE = ("log_coordinates", "distances", "polar_angles", "transport_angles", "tangent_quadrature_weights", "angular_phases",
                 "transport_phases")

    def _with_tables(self, edge_index: Tensor, row_ptr: Tensor, per_edge) -> EdgeGeometry:
        return type(self)(edge_index, row_ptr, *(per_edge(getattr(self, name)) for name in self._PER_EDGE))

    def select(self, selection: Tensor, *, n_nodes: int | None = None) -> EdgeGeometry:
        """The edges picked by a Boolean mask (one entry per edge) or by ascending edge indices, in their present
        order, with a ``row_ptr`` over ``n_nodes`` targets (default: as many as now; a smaller count restricts the
        targets to ``0 .. n_nodes - 1``, which every kept edge must respect).  Reference: ``edge_geometry.py:159-214``."""
        if selection.dim() != 1:
            raise ValueError("Edge selection must be one-dimensional.")
        if selection.dtype == torch.bool:
            if selection.shape[0] != self.n_edges:
                raise ValueError("A Boolean edge mask must have one entry per edge.")
        elif selection.dtype != torch.long:
            raise TypeError("Edge selection must have dtype torch.bool or torch.long.")
        kept = self.edge_index[:, selection].contiguous()
        n = self.row_ptr.shape[0] - 1 if n_nodes is None else int(n_nodes)
        row_ptr = torch.zeros(n + 1, dtype=torch.long, device=kept.device)
        if kept.shape[1]:
            torch.cumsum(torch.bincount(kept[0], minlength=n)[:n], 0, out=row_ptr[1:])
        return self._with_tables(kept, row_ptr, lambda table: table[selection].contiguous())

    def tile(self, count: int, *, n_sources: int) -> EdgeGeometry:
        """``count`` disjoint copies of the edge set as ONE graph: copy ``b`` joins sources ``b * n_sources + j`` to
        targets ``b * n_targets + i`` (the reference's batching, ``edge_geometry.py:216-252``; the kernels of this
        package share one copy across the batch instead, this is for callers that want the union graph)."""
        count = int(count)
        if count < 1:
            raise ValueError(f"count must be at least 1, got {count}.")
        if count == 1:
            return self
        n_targets, n_edges = self.row_ptr.shape[0] - 1, self.n_edges
        copy = torch.arange(count, dtype=torch.long, device=self.edge_index.device)[:, None]
        index = torch.stack([(self.edge_index[0][None] + copy * n_targets).reshape(-1), (self.edge_index[1][None] + copy * int(n_sources)).reshape(-1)])
        row_ptr = torch.cat([self.row_ptr[:1], (self.row_ptr[1:][None] + copy * n_edges).reshape(-1)])
        return self._with_tables(index, row_ptr, lambda table: table.repeat(count, *([1] * (table.dim() - 1))))

    def target_range(self, first: int, last: int) -> tuple[EdgeGeometry, int, int]:
        """The whole neighbourhoods of the targets ``first .. last - 1`` as an edge set of their own, plus the edge
        span ``(e_first, e_last)`` it occupies here -- what ``forward_chunked`` (reference ``nn/attention.py:344-402``)
        selects per chunk and hands to ``fused_attention.register_chunk`` so that the chunk's constants are views."""
        e_first, e_last = int(self.row_ptr[first]), int(self.row_ptr[last])
        return self.select(torch.arange(e_first, e_last, device=self.edge_index.device)), e_first, e_last


def compute_edge_geometry(grid: Any, frames: Tensor, coverage_radius: float, *, max_frequency: int = DEFAULT_MAX_FREQUENCY,
                          dtype: torch.dtype | None = None, candidates: tuple[Tensor, Tensor] | None = None) -> EdgeGeometry:
    """All directed pairs within ``coverage_radius`` and their tables.

    ``grid`` carries ``nodes`` (N, 3), ``quadrature_weights`` (N,) and
    ``exact_nodes`` (float64 lattice coordinates; falls back to ``nodes``).  The
    tables come out in ``dtype`` (default: ``grid.nodes.dtype`` when it is
    float32/float64).  ``candidates = (lo, hi)`` restricts target ``i`` to
    sources in ``[lo[i], hi[i])``; a :class:`SphericalLattice` supplies its row band."""
    radius = float(coverage_radius)
    if not (0.0 < radius < math.pi):
        raise ValueError(f"coverage_radius must lie in (0, pi), got {radius}.")
    exact = getattr(grid, "exact_nodes", None)
    nodes = (grid.nodes if exact is None else exact).to(torch.float64).contiguous()
    device = _lib.require_cuda(nodes)
    if nodes.dim() != 2 or nodes.shape[1] != 3:
        raise ValueError(f"nodes must have shape (n_nodes, 3), got {tuple(nodes.shape)}.")
    n = nodes.shape[0]
    if tuple(frames.shape) != (n, 3, 2):
        raise ValueError(f"frames must have shape (n_nodes, 3, 2), got {tuple(frames.shape)}.")
    weights = grid.quadrature_weights
    if tuple(weights.shape) != (n,):
        raise ValueError(f"spherical_quadrature_weights must have shape ({n},), got {tuple(weights.shape)}.")
    if dtype is None:
        dtype = grid.nodes.dtype if grid.nodes.dtype in (torch.float32, torch.float64) else torch.float32
    frames64 = frames.to(device=device, dtype=torch.float64).contiguous()
    weights64 = weights.to(device=device, dtype=torch.float64).contiguous()
    if candidates is None and isinstance(grid, SphericalLattice):
        candidates = grid.candidate_ranges(radius)
    lo, hi = (None, None) if candidates is None else (candidates[0].contiguous(), candidates[1].contiguous())
    stream = _lib.stream(device)
    with torch.cuda.device(device):
        degree = torch.empty(n, dtype=torch.int64, device=device)
        _lib.call("gm_geometry_count", _lib.ptr(nodes), n, _lib.ptr(lo), _lib.ptr(hi), radius, _lib.ptr(degree), stream)
        row_ptr = torch.zeros(n + 1, dtype=torch.int64, device=device)
        torch.cumsum(degree, 0, out=row_ptr[1:])
        e = int(row_ptr[-1])
        k = max_frequency + 1
        edge_index = torch.empty((2, e), dtype=torch.int64, device=device)
        real = lambda *shape: torch.empty(shape, dtype=dtype, device=device)
        dist, logxy, polar, gamma, tangent = real(e), real(e, 2), real(e), real(e), real(e)
        angular, transport = real(e, k, 2), real(e, k, 2)
        if e:
            _lib.call("gm_geometry_fill", _lib.ptr(nodes), _lib.ptr(frames64), _lib.ptr(weights64), n, _lib.ptr(lo), _lib.ptr(hi),
                      radius, _lib.ptr(row_ptr), max_frequency, _lib.dtype_code(dtype), _lib.ptr(edge_index[0]),
                      _lib.ptr(edge_index[1]), _lib.ptr(dist), _lib.ptr(logxy), _lib.ptr(polar), _lib.ptr(gamma), _lib.ptr(tangent),
                      _lib.ptr(angular), _lib.ptr(transport), stream)
    return EdgeGeometry(edge_index, row_ptr, logxy, dist, polar, gamma, tangent, torch.view_as_complex(angular),
                        torch.view_as_complex(transport))
