"""Shared builders for the tests: lattices, per-edge constants, seeded inputs.

Geometry comes from the numpy oracle (``oracle/geometry_np.py``), never from
the package under test, so that operator tests and geometry tests fail
independently.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from functools import lru_cache

import numpy as np
import torch

from oracle import geometry_np as G

from gm_attention_b200.fields import FieldType


@dataclass
class Case:
    """One attention problem on a midpoint lattice, as numpy arrays in ``dtype``."""

    nlat: int
    nlon: int
    radius: float
    heads: int
    head_type: FieldType
    full_type: FieldType
    desc: np.ndarray  # (F, 5) int64
    row_ptr: np.ndarray
    source: np.ndarray
    target: np.ndarray
    transport: np.ndarray  # (E, orders, 2)
    angular: np.ndarray
    rho: np.ndarray
    weights: np.ndarray
    bias: np.ndarray
    inside: np.ndarray
    scale: float
    max_degree: int

    @property
    def n_nodes(self) -> int:
        return self.nlat * self.nlon

    @property
    def width(self) -> int:
        return self.full_type.dimension


def descriptor_rows(head_type: FieldType, heads: int) -> np.ndarray:
    full = head_type.scaled(heads)
    starts = {n: s.start for n, s in full.slices().items()}
    rows, coff = [], 0
    for n, a in head_type.items():
        rows.append([n, a, starts[n], 0 if n == 0 else coff, 1 if n == 0 else 2])
        if n:
            coff += 4 * a
    return np.array(rows, np.int64).reshape(-1, 5)


@lru_cache(maxsize=16)
def _edges(nlat: int, nlon: int, radius: float, max_frequency: int, dtype_name: str) -> G.Edges:
    return G.lattice_edges(G.midpoint_lattice(nlat, nlon), radius, max_frequency, np.dtype(dtype_name).type)


def window_values(r: np.ndarray, cutoff: float, kind: str) -> np.ndarray:
    if kind == "hard":
        slack = 1e-10 if r.dtype == np.float64 else 1e-5
        return (r <= cutoff + slack).astype(r.dtype)
    return (np.maximum(1.0 - (r / r.dtype.type(cutoff)) ** 2, 0) ** 2).astype(r.dtype)


def make_case(nlat: int, nlon: int, radius: float, head_type: dict[int, int], heads: int, dtype=np.float32,
              window: str = "hard", max_frequency: int = 4) -> Case:
    e = _edges(nlat, nlon, float(radius), max_frequency, np.dtype(dtype).name)
    attn = FieldType(head_type)
    dt = np.dtype(dtype).type
    tiny = np.finfo(dtype).tiny
    win = window_values(e.distances, radius, window)
    quad = e.tangent_quadrature_weights
    bias = (np.log(np.maximum(win, tiny)) + np.log(np.maximum(quad, tiny))).astype(dtype)
    as_pairs = lambda z: np.ascontiguousarray(np.stack([z.real, z.imag], -1).astype(dtype))
    degree = np.diff(e.row_ptr)
    return Case(nlat, nlon, float(radius), heads, attn, attn.scaled(heads), descriptor_rows(attn, heads), e.row_ptr.copy(),
                e.source_index.copy(), e.target_index.copy(), as_pairs(e.transport_phases), as_pairs(e.angular_phases),
                (e.distances / dt(radius)).astype(dtype), (win * quad).astype(dtype), bias, (win > 0).astype(np.uint8),
                1.0 / math.sqrt(attn.dimension), int(degree.max()))


def seeded(shape: tuple[int, ...], seed: int, dtype=np.float32, count: int = 1) -> list[np.ndarray]:
    """``count`` N(0, 1) arrays drawn in order from one torch CPU generator (fp32 draws, then cast)."""
    gen = torch.Generator().manual_seed(seed)
    return [torch.randn(*shape, generator=gen, dtype=torch.float32).numpy().astype(dtype) for _ in range(count)]


def cuda(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel_err(a, b) -> float:
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def assert_close(actual, expected, rtol: float, atol: float, what: str = "") -> None:
    """``|a - e| <= atol + rtol * |e|`` elementwise, reported with the worst offender."""
    a = np.asarray(actual, np.float64)
    e = np.asarray(expected, np.float64)
    assert a.shape == e.shape, f"{what}: shape {a.shape} vs {e.shape}"
    if a.size == 0:
        return
    excess = np.abs(a - e) - (atol + rtol * np.abs(e))
    worst = int(np.argmax(excess))
    assert excess.flat[worst] <= 0, f"{what}: |{a.flat[worst]} - {e.flat[worst]}| exceeds atol={atol} rtol={rtol} (max abs diff {np.abs(a - e).max():.3e})"


class StandInKernel(torch.nn.Module):
    """A general steerable kernel with the attributes the pair-term driver reads, laid out as the reference lays its
    own out (``nn/kernels.py:328-419``): Gaussian basis in ``s = (r / cutoff)^2`` (centres ``linspace(0, 1, n)``, width
    = spacing), Linear + SiLU trunk, a complex head holding consecutive (n, m, role) ranges of ``2 b_m a_n`` rows and a
    real head of ``b_0 a_0`` rows for the (0, 0) block, radial power ``|m - n|`` (linear) / ``m + n`` (antilinear)."""

    class Basis(torch.nn.Module):
        def __init__(self, n: int, cutoff: float, dtype):
            super().__init__()
            self.cutoff = cutoff
            self.register_buffer("centers", torch.linspace(0, 1, n, dtype=dtype))
            self.width = 1.0 / max(n - 1, 1)

        def forward(self, r):
            s = (r / self.cutoff) ** 2
            return torch.exp(-0.5 * ((s[:, None] - self.centers[None, :]) / self.width) ** 2)

    def __init__(self, field_in: dict[int, int], field_out: dict[int, int], cutoff: float, trunk: int = 8, n_basis: int = 4, bias: bool = True,
                 dtype=torch.float64, seed: int = 0) -> None:
        super().__init__()
        torch.manual_seed(seed)
        self.field_type_in, self.field_type_out = FieldType(field_in), FieldType(field_out)
        self.radial_basis = self.Basis(n_basis, cutoff, dtype)
        self.radial_trunk = torch.nn.Sequential(torch.nn.Linear(n_basis, trunk, bias=bias, dtype=dtype), torch.nn.SiLU())
        self._pair_ranges, self._pair_powers = {}, {}
        offset, real_width = 0, 0
        for n in self.field_type_in.frequencies:
            for m in self.field_type_out.frequencies:
                a, b = self.field_type_in.multiplicity(n), self.field_type_out.multiplicity(m)
                if n == 0 and m == 0:
                    real_width = a * b
                    continue
                roles = [("linear", abs(m - n))] + ([("antilinear", m + n)] if n and m else [])
                for role, power in roles:
                    self._pair_ranges[(n, m, role)] = slice(offset, offset + 2 * a * b)
                    self._pair_powers[(n, m, role)] = power
                    offset += 2 * a * b
        self._max_power = max(self._pair_powers.values(), default=0)
        self.complex_head = torch.nn.Linear(trunk, offset, bias=bias, dtype=dtype) if offset else None
        self.real_head = torch.nn.Linear(trunk, real_width, bias=bias, dtype=dtype) if real_width else None

    def _radial_powers(self, distances):
        rho = distances / self.radial_basis.cutoff
        table = [torch.ones_like(rho)]
        for _ in range(self._max_power):
            table.append(table[-1] * rho)
        return torch.stack(table, -1)

    def pair_loop(self, x, edges):
        """The general kernel's pair loop in plain PyTorch (the arithmetic of ``nn/fused/pairs.h:301-324`` term by term):
        ``out_m += post * scale * f(M (pre u~))`` with ``M = W h + b`` reshaped ``(b_m, a_n)``."""
        hidden = self.radial_basis(edges.distances)
        for layer in self.radial_trunk:
            hidden = layer(hidden)
        powers = self._radial_powers(edges.distances)
        out = {}
        for m in self.field_type_out.frequencies:
            b = self.field_type_out.multiplicity(m)
            acc = None
            for n in self.field_type_in.frequencies:
                a = self.field_type_in.multiplicity(n)
                values = x[n]
                values = values if values.shape[0] == edges.n_edges else values[edges.source_index]
                if n == 0 and m == 0:
                    block = self.real_head(hidden).reshape(-1, b, a)
                    term = torch.einsum("eba,ea->eb", block, values)
                else:
                    u = values.to(torch.complex128 if values.dtype == torch.float64 else torch.complex64) if n == 0 else \
                        edges.transport_harmonic(n)[:, None] * torch.view_as_complex(values.contiguous())
                    term = 0
                    for role in ("linear", "antilinear"):
                        if (n, m, role) not in self._pair_ranges:
                            continue
                        rows = self.complex_head(hidden)[:, self._pair_ranges[(n, m, role)]]
                        block = torch.complex(rows[:, 0::2], rows[:, 1::2]).reshape(-1, b, a)
                        scale = powers[:, self._pair_powers[(n, m, role)]]
                        if n == 0:
                            part = edges.angular_harmonic(m)[:, None] * torch.einsum("eba,ea->eb", block, u)
                        elif m == 0:
                            part = torch.einsum("eba,ea->eb", block, edges.angular_harmonic(n)[:, None] * u.conj()).real
                        elif role == "linear":
                            part = torch.einsum("eba,ea->eb", block, edges.angular_harmonic(m - n)[:, None] * u)
                        else:
                            part = torch.einsum("eba,ea->eb", block, edges.angular_harmonic(m + n)[:, None] * u.conj())
                        term = term + scale[:, None] * part
                acc = term if acc is None else acc + term
            out[m] = acc if m == 0 else torch.view_as_real(acc)
        return out
