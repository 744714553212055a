"""Edge-set operations of ``EdgeGeometry`` (select, tile, target ranges) and the chunk registry of the attention
driver, on CPU tensors: chunk geometries are views of the parent's cached tables and neither the geometry cache nor
the registry grows (the logic of the reference's ``tests/nn/test_fused_attention.py:345-373``)."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from oracle import geometry_np as G


def cpu_edges(dtype=np.float64):
    from gm_attention_b200.geometry import EdgeGeometry

    e = G.lattice_edges(G.midpoint_lattice(8, 16), 2 * math.pi / 8, 4, dtype)
    t = torch.from_numpy
    return EdgeGeometry(t(e.edge_index), t(e.row_ptr), t(e.log_coordinates), t(e.distances), t(e.polar_angles), t(e.transport_angles),
                        t(e.tangent_quadrature_weights), t(e.angular_phases), t(e.transport_phases))


def test_select_by_mask_and_by_indices():
    edges = cpu_edges()
    mask = edges.distances < 0.4
    by_mask = edges.select(mask)
    by_index = edges.select(torch.nonzero(mask).reshape(-1))
    assert by_mask.n_edges == int(mask.sum()) and torch.equal(by_mask.edge_index, by_index.edge_index)
    assert torch.equal(by_mask.row_ptr, by_index.row_ptr) and by_mask.row_ptr.shape == edges.row_ptr.shape
    degree = torch.bincount(edges.target_index[mask], minlength=edges.row_ptr.shape[0] - 1)
    assert torch.equal(by_mask.row_ptr[1:] - by_mask.row_ptr[:-1], degree)
    assert torch.equal(by_mask.transport_phases, edges.transport_phases[mask]) and by_mask.transport_phases.is_contiguous()
    fewer = edges.select(edges.target_index < 32, n_nodes=32)
    assert fewer.row_ptr.shape[0] == 33 and int(fewer.row_ptr[-1]) == fewer.n_edges
    with pytest.raises(ValueError):
        edges.select(mask[:-1])
    with pytest.raises(TypeError):
        edges.select(torch.zeros(3, dtype=torch.int32))
    with pytest.raises(ValueError):
        edges.select(mask[None])


def test_tile_is_the_disjoint_union():
    edges = cpu_edges()
    n = edges.row_ptr.shape[0] - 1
    assert edges.tile(1, n_sources=n) is edges
    three = edges.tile(3, n_sources=n)
    e = edges.n_edges
    assert three.n_edges == 3 * e and three.row_ptr.shape[0] == 3 * n + 1
    for b in range(3):
        assert torch.equal(three.edge_index[:, b * e:(b + 1) * e], edges.edge_index + b * n)
        assert torch.equal(three.row_ptr[b * n:(b + 1) * n + 1], edges.row_ptr + b * e)
        assert torch.equal(three.angular_phases[b * e:(b + 1) * e], edges.angular_phases)
    with pytest.raises(ValueError):
        edges.tile(0, n_sources=n)


def test_chunk_geometries_are_views_and_nothing_accumulates():
    from gm_attention_b200.nn import fused_attention as fa

    edges = cpu_edges()
    cutoff = 2 * math.pi / 8
    fa._GEOMETRIES.clear()
    fa._CHUNKS.clear()
    parent = fa.geometry(edges, cutoff, "quartic", torch.float64)
    n = edges.row_ptr.shape[0] - 1
    for _ in range(3):  # chunked passes over all targets: every chunk registers, is answered with views, and dies
        for first in range(0, n, 37):
            last = min(n, first + 37)
            chunk, e_first, e_last = edges.target_range(first, last)
            fa.register_chunk(chunk, edges, e_first, e_last)
            g = fa.geometry(chunk, cutoff, "quartic", torch.float64)
            assert g.base is parent and g.span == (e_first, e_last)
            assert g.transport.data_ptr() == parent.transport[e_first:e_last].data_ptr()  # a view, not a copy
            assert g.bias.data_ptr() == parent.bias[e_first:e_last].data_ptr()
            assert g.row_ptr is not parent.row_ptr and int(g.row_ptr[-1]) == e_last - e_first
            assert g.max_degree == int((chunk.row_ptr[1:] - chunk.row_ptr[:-1]).max())
            assert torch.equal(g.source, edges.source_index[e_first:e_last])
            torch.testing.assert_close(g.aggregation_weights(True, 1e-6), parent.aggregation_weights(True, 1e-6)[e_first:e_last])
            del chunk, g
        assert len(fa._GEOMETRIES) == 1  # the parent's entry alone: chunks are never cached
    fa._purge()
    assert len(fa._CHUNKS) == 0  # every chunk has died with its pass
    assert fa.chunk_of(edges) is None
