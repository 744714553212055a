"""The fused layer's oracle on a SAMPLE of a large lattice.

TEST INFRASTRUCTURE ONLY: imported by ``tests/`` and by the parity self-check of
``bench.py``; the shipped package never imports it.

At 128 x 256 and 256 x 512 the whole layer is minutes of CPU work; the rows of a
few targets are seconds.  The layer is local, so a sample is exact:

* ``out_i`` and ``dq_i`` of a target ``i`` need the complete CSR row of ``i``
  (its own softmax) and nothing else;
* ``dk_s`` and ``dv_s`` of a source ``s`` need the complete rows of every target
  that sees ``s`` (the membership rule is symmetric, so those targets are the
  neighbours of ``s``).

``sample_problem`` cuts exactly those rows out of the lattice: it renumbers the
union of the nodes involved (ascending, so the (target, source) edge order of
``discretization/edge_geometry.py:701-704`` is kept), builds the per-edge tables of
the reduced graph with ``geometry_np.edge_tables`` (the restatement of
``edge_geometry_from_index``, ``edge_geometry.py:506-619``) and the attention
constants of ``nn/fused_attention.py:234-238``.  ``run`` then evaluates the C
oracle (``gm_oracle.c``: reference Softmax op + eager value path and its chain-rule
backward) on the reduced fields; rows of nodes that are not complete targets are
empty there and their results are not looked at.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable

import numpy as np

from oracle import geometry_np as G
from oracle import oracle as O


@dataclass
class Sample:
    nodes: np.ndarray  # (U,) original node indices, ascending
    targets: np.ndarray  # original indices of the targets whose out / dq are complete
    sources: np.ndarray  # original indices of the sources whose dk / dv are complete
    row_ptr: np.ndarray  # reduced graph, (U + 1,)
    source_index: np.ndarray  # reduced numbering
    transport: np.ndarray  # (E, orders, 2)
    bias: np.ndarray
    inside: np.ndarray
    n_edges: int
    # the depthwise op's per-edge constants (nn/fused_attention.py:213-222): geodesic distance, (cos, sin)(k phi) for
    # k <= max_frequency, window value and tangent quadrature weight
    distances: np.ndarray | None = None
    angular: np.ndarray | None = None
    window: np.ndarray | None = None
    quadrature: np.ndarray | None = None

    def position(self, original: np.ndarray) -> np.ndarray:
        return np.searchsorted(self.nodes, original)


def _row_neighbourhood(lat: G.Lattice, radius: float, band: int, row: int) -> tuple[np.ndarray, np.ndarray]:
    """(source rows, longitude offsets) of the target in column 0 of ``row`` (membership rule of
    ``edge_geometry.py:381-383``: float64 geodesic distance <= radius + 1e-10)."""
    nlon = lat.nlon
    lo, hi = max(0, row - band) * nlon, min(lat.nlat, row + band + 1) * nlon
    cand = np.arange(lo, hi, dtype=np.int64)
    d = G.geodesic(np.broadcast_to(lat.nodes[row * nlon], (cand.shape[0], 3)), lat.nodes[cand])
    near = cand[d <= radius + G.EXACT_SLACK]
    return near // nlon, near % nlon


def _window(r: np.ndarray, cutoff: float, kind: str) -> np.ndarray:
    """Hard / quartic aggregation window (``nn/convolution.py:82-89``, ``edge_geometry.py:447-462``)."""
    if kind == "hard":
        return (r <= cutoff + (1e-10 if r.dtype == np.float64 else 1e-5)).astype(r.dtype)
    return (np.maximum(1.0 - (r / r.dtype.type(cutoff)) ** 2, 0) ** 2).astype(r.dtype)


def sample_problem(lat: G.Lattice, radius: float, targets, sources, max_frequency: int, dtype=np.float32,
                   window: str = "hard") -> Sample:
    """Reduced graph holding the complete rows of ``targets`` and of every target that sees one of ``sources``."""
    nlon = lat.nlon
    band = int(math.ceil(radius / (math.pi / lat.nlat) - 1e-9))
    cache: dict[int, tuple[np.ndarray, np.ndarray]] = {}

    def neighbours(node: int) -> np.ndarray:
        row, col = divmod(int(node), nlon)
        if row not in cache:
            cache[row] = _row_neighbourhood(lat, radius, band, row)
        rows, offs = cache[row]
        return np.sort(rows * nlon + (offs + col) % nlon)

    targets = np.unique(np.asarray(targets, np.int64))
    sources = np.unique(np.asarray(sources, np.int64))
    complete = set(int(t) for t in targets)
    for s in sources:
        complete.update(int(t) for t in neighbours(int(s)))
    complete_sorted = np.array(sorted(complete), np.int64)
    rows = {int(t): neighbours(int(t)) for t in complete_sorted}
    nodes = np.unique(np.concatenate([complete_sorted] + list(rows.values()))) if rows else np.zeros(0, np.int64)
    ti = np.concatenate([np.full(rows[int(t)].shape[0], np.searchsorted(nodes, t), np.int64) for t in complete_sorted])
    sj = np.concatenate([np.searchsorted(nodes, rows[int(t)]) for t in complete_sorted])
    e = G.edge_tables(lat.nodes[nodes].astype(dtype), lat.frames[nodes].astype(dtype), lat.weights[nodes].astype(dtype),
                      np.stack([ti, sj], 0), nodes.shape[0], max_frequency)
    tiny = np.finfo(dtype).tiny
    win = _window(e.distances, radius, window)
    bias = (np.log(np.maximum(win, tiny)) + np.log(np.maximum(e.tangent_quadrature_weights, tiny))).astype(dtype)
    transport = np.ascontiguousarray(np.stack([e.transport_phases.real, e.transport_phases.imag], -1).astype(dtype))
    angular = np.ascontiguousarray(np.stack([e.angular_phases.real, e.angular_phases.imag], -1).astype(dtype))
    return Sample(nodes, targets, sources, e.row_ptr, e.source_index.copy(), transport, bias, (win > 0).astype(np.uint8),
                  int(e.n_edges), e.distances.astype(dtype), angular, win.astype(dtype), e.tangent_quadrature_weights.astype(dtype))


def run(sample: Sample, gather: Callable[[np.ndarray], tuple[np.ndarray, np.ndarray, np.ndarray, np.ndarray]], desc: np.ndarray,
        heads: int, scale: float) -> dict[str, np.ndarray]:
    """``gather(nodes) -> (q, k, v, dout)`` rows of ONE sample for the given original node indices (float32 or
    float64 arrays ``(len(nodes), D)``).  Returns ``out`` / ``dq`` on ``sample.targets`` and ``dk`` / ``dv`` on
    ``sample.sources``, in the order of those index arrays."""
    q, k, v, g = (np.ascontiguousarray(x) for x in gather(sample.nodes))
    args = (sample.transport, sample.bias, sample.inside, np.asarray(desc, np.int64), sample.row_ptr, sample.source_index, heads, scale, 1)
    out = O.attention_forward(q, k, v, *args)
    dq, dk, dv = O.attention_backward(g, q, k, v, *args)
    tp, sp = sample.position(sample.targets), sample.position(sample.sources)
    return {"out": out[tp], "dq": dq[tp], "dk": dk[sp], "dv": dv[sp]}


def run_conv(sample: Sample, v: np.ndarray, g: np.ndarray, rc: np.ndarray, cc: np.ndarray, desc: np.ndarray, cutoff: float,
             a0: int, w: int) -> dict[str, np.ndarray]:
    """The depthwise op (``nn/fused/attention.h:174-232, 265-287``) on the reduced graph: ``v`` / ``g`` rows of ONE sample on
    ``sample.nodes``, ``rc (E, a0)`` / ``cc (E, w)`` per reduced edge, aggregation weight = window x tangent quadrature
    weight.  Returns ``out`` on the targets, ``dv`` on the sources and the per-edge ``drc`` / ``dcc`` (edges of complete
    rows only carry meaning; ``g`` must be zero on the rows of incomplete targets for ``dv`` to be exact -- it is, for
    those rows have no edges here)."""
    dt = v.dtype.type
    args = (np.ascontiguousarray(rc[None]), np.ascontiguousarray(cc[None]), sample.transport, sample.angular,
            (sample.distances / dt(cutoff)).astype(dt), (sample.window * sample.quadrature).astype(dt), np.asarray(desc, np.int64),
            sample.row_ptr, sample.source_index, a0, w)
    out = O.conv_forward(np.ascontiguousarray(v), *args)
    dv, drc, dcc = O.conv_backward(np.ascontiguousarray(g), np.ascontiguousarray(v), *args)
    tp, sp = sample.position(sample.targets), sample.position(sample.sources)
    return {"out": out[tp], "dv": dv[sp], "drc": drc.reshape(-1, a0), "dcc": dcc.reshape(-1, w)}


def default_sample_nodes(nlat: int, nlon: int, row_lo: int = 0, row_hi: int | None = None,
                         polar_source_row: int | None = 2) -> tuple[np.ndarray, np.ndarray]:
    """Targets and sources worth checking on rows ``[row_lo, row_hi)`` of a lattice.  Targets: the rows next to a
    pole (whole-row windows), a few rows further in, the equator and the range's own first / last rows, each at the
    two columns of the longitude seam and one in the middle.  Sources (each costs the complete rows of all the targets
    that see it): one near the pole in ``polar_source_row`` (None: left out; row 2 of a 256 x 512 lattice is ~1.5 M
    edges of oracle work), rows 6 and 8, the equator, and the first / last rows of a range that ends inside the lattice, at the seam columns."""
    row_hi = nlat if row_hi is None else row_hi
    inside = lambda rows: sorted({r for r in rows if row_lo <= r < row_hi and 0 <= r < nlat})
    t_rows = inside([0, 1, 3, 8, nlat // 4, nlat // 2, nlat - 1, row_lo, row_hi - 1])
    targets = np.array([r * nlon + c for r in t_rows for c in sorted({0, nlon - 1, nlon // 2 + 1})], np.int64)
    s_nodes = {r * nlon + c for r in inside([6, nlat // 2]) for c in (0, nlon - 1)} | {r * nlon for r in inside([8])}
    if row_lo > 0:  # a band's first / last rows: their sums cross the cut
        s_nodes.add(row_lo * nlon)
    if row_hi < nlat:
        s_nodes.add((row_hi - 1) * nlon + nlon - 1)
    if polar_source_row is not None:
        s_nodes |= {r * nlon + nlon - 1 for r in inside([polar_source_row])}
    return targets, np.array(sorted(s_nodes), np.int64)
