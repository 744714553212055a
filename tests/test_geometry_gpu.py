"""The on-device geometry builder against the reference: CSR bit-exact (golden
tables from the reference's compute_edge_geometry, checksums and per-row
degrees for the benchmark lattices), float tables within rounding of the table
dtype, and the numpy oracle on a mid-size lattice."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from oracle import geometry_np as G

from tests.golden.make_golden_checksum import csr_checksum
from tests.helpers import assert_close

pytestmark = pytest.mark.gpu


def build(nlat, nlon, radius, dtype, max_frequency=4):
    from gm_attention_b200.geometry import compute_edge_geometry, midpoint_lattice

    lat = midpoint_lattice(nlat, nlon)
    return compute_edge_geometry(lat, lat.frames, radius, max_frequency=max_frequency, dtype=dtype)


@pytest.mark.parametrize("name,nlat,nlon,dtype", [("geometry_8x16", 8, 16, torch.float64), ("geometry_12x24", 12, 24, torch.float32)])
def test_tables_match_reference_golden(golden_dir, name, nlat, nlon, dtype):
    gold = np.load(golden_dir / f"{name}.npz")
    e = build(nlat, nlon, float(gold["radius"]), dtype)
    assert np.array_equal(e.edge_index.cpu().numpy(), gold["edge_index"])
    assert np.array_equal(e.row_ptr.cpu().numpy(), gold["row_ptr"])
    tol = 1e-12 if dtype == torch.float64 else 2e-6
    assert_close(e.distances.cpu().numpy(), gold["distances"], 0, tol, "distances")
    assert_close(e.tangent_quadrature_weights.cpu().numpy(), gold["tangent_quadrature_weights"], 0, tol, "tangent weights")
    assert_close(e.log_coordinates.cpu().numpy(), gold["log_coordinates"], 0, tol, "log coordinates")
    assert np.abs(e.transport_phases.cpu().numpy() - gold["transport_phases"]).max() < 8 * tol
    off_origin = gold["distances"] > 1e-4
    assert np.abs(e.angular_phases.cpu().numpy() - gold["angular_phases"])[off_origin].max() < 8 * tol
    self_loops = e.edge_index[0] == e.edge_index[1]
    assert int(self_loops.sum()) == nlat * nlon
    assert float(e.distances[self_loops].abs().max()) < 1e-7
    assert float(e.transport_angles[self_loops].abs().max()) < 1e-6


def test_counts_degrees_and_checksums_of_the_benchmark_lattices(golden_dir):
    gold = np.load(golden_dir / "geometry_counts.npz")
    for idx, name in enumerate(gold["names"]):
        nlat, rest = str(name).split("x")
        nlon, mult = rest.split("_r")
        nlat, nlon, mult = int(nlat), int(nlon), int(mult)
        e = build(nlat, nlon, mult * math.pi / nlat, torch.float32, max_frequency=2)
        assert e.n_edges == int(gold["counts"][idx]), name
        deg = (e.row_ptr[1:] - e.row_ptr[:-1]).reshape(nlat, nlon)
        assert bool((deg == deg[:, :1]).all()), "degree must not depend on longitude (whole-shell rule)"
        assert np.array_equal(deg[:, 0].cpu().numpy(), gold["degrees"][idx][:nlat]), name
        assert csr_checksum(e.row_ptr.cpu().numpy(), e.edge_index[1].cpu().numpy()) == int(gold["checksums"][idx]), name
        del e


def test_matches_numpy_oracle_without_candidate_ranges():
    """Arbitrary point set path: every node examines every node."""
    from gm_attention_b200.geometry import compute_edge_geometry, midpoint_lattice
    from types import SimpleNamespace

    lat = midpoint_lattice(16, 32)
    grid = SimpleNamespace(nodes=lat.nodes, quadrature_weights=lat.quadrature_weights, exact_nodes=lat.nodes)
    radius = 2.3 * math.pi / 16
    e = compute_edge_geometry(grid, lat.frames, radius, max_frequency=3, dtype=torch.float64)
    want = G.lattice_edges(G.midpoint_lattice(16, 32), radius, 3, np.float64)
    assert np.array_equal(e.edge_index.cpu().numpy(), want.edge_index)
    assert_close(e.transport_phases.cpu().numpy().view(np.float64), want.transport_phases.view(np.float64), 0, 1e-12, "transport phases")
    assert_close(e.tangent_quadrature_weights.cpu().numpy(), want.tangent_quadrature_weights, 0, 1e-14, "weights")
    assert e.max_frequency == 3
    assert torch.equal(e.transport_harmonic(-2), e.transport_phases[:, 2].conj())
    with pytest.raises(ValueError):
        e.angular_harmonic(4)


def test_fused_attention_driver_geometry_on_device_tables():
    """geometry() of the host driver consumes the on-device EdgeGeometry unchanged."""
    from gm_attention_b200.nn import fused_attention as fa

    e = build(8, 16, 2 * math.pi / 8, torch.float32)
    g = fa.geometry(e, 2 * math.pi / 8, "hard", torch.float32)
    assert g.transport.shape == (e.n_edges, 5, 2) and g.inside.dtype == torch.uint8
    assert g.max_degree == int((e.row_ptr[1:] - e.row_ptr[:-1]).max())
    assert fa.geometry(e, 2 * math.pi / 8, "hard", torch.float32) is g  # cached per edge set
    normalized = g.aggregation_weights(True, 1e-12)
    sums = torch.segment_reduce(normalized, "sum", offsets=e.row_ptr)
    assert torch.allclose(sums, torch.ones_like(sums), atol=1e-5)
