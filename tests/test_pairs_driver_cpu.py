"""The pair-term driver (``_FusedPairs`` and ``forward_general``) against a plain-PyTorch pair loop, on CPU:
the Python logic of the driver -- term loop, table indexing, in-place accumulation, the blocked readout gradient --
runs here over the REFERENCE's compiled CPU pair driver (oracle/_ref) standing in for the CUDA extension, which
has the same functions and signatures.  float64: values 1e-12, gradients 1e-11 (the bounds of the reference's own
``tests/nn/test_fused_pairs.py:73-93``); the field-type cases are the ones that test uses."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from oracle import geometry_np as G

from tests.helpers import StandInKernel

CASES = [
    ({0: 2, 1: 2, 2: 1}, {0: 1, 1: 2, 2: 2}, True),   # (0,0), (0,m), (n,0), (n,m) with m - n of both signs
    ({0: 2, 1: 2, 2: 1}, {0: 1, 1: 2, 2: 2}, False),  # no bias
    ({0: 3}, {0: 2}, True),                            # real head only
    ({1: 2, 2: 1}, {1: 1, 2: 2}, True),                # complex head only
    ({0: 2, 1: 1}, {1: 2}, True),                      # real input into complex output only
    ({1: 2}, {0: 2}, True),                            # complex input into the real output only
    ({1: 16}, {1: 16}, True),                          # the largest block the kernels take
]


def cpu_edges(dtype=np.float64):
    from gm_attention_b200.geometry import EdgeGeometry

    lat = G.midpoint_lattice(5, 8)
    e = G.lattice_edges(lat, 1.3 * math.pi / 5, 4, dtype)
    t = torch.from_numpy
    return EdgeGeometry(t(e.edge_index), t(e.row_ptr), t(e.log_coordinates), t(e.distances), t(e.polar_angles), t(e.transport_angles),
                        t(e.tangent_quadrature_weights), t(e.angular_phases), t(e.transport_phases)), 1.3 * math.pi / 5


def run(kernel, flat, edges, fused: bool):
    from gm_attention_b200.fields import FeatureField
    from gm_attention_b200.nn import fused_pairs as fp

    flat = flat.detach().clone().requires_grad_(True)
    x = FeatureField.from_flat(kernel.field_type_in, flat)
    if fused:
        out = fp.forward_general(kernel, x, edges).coefficients
    else:
        out = kernel.pair_loop(x, edges)
    loss = sum((out[m] * torch.arange(1, out[m].numel() + 1, dtype=flat.dtype).reshape(out[m].shape) / out[m].numel()).sum() for m in out)
    grads = torch.autograd.grad(loss, [flat, *kernel.parameters()])
    return {m: v.detach() for m, v in out.items()}, [g.detach() for g in grads]


@pytest.mark.parametrize("field_in, field_out, bias", CASES)
def test_driver_matches_the_pair_loop(reference_modules, monkeypatch, field_in, field_out, bias):
    from gm_attention_b200.nn import fused_pairs as fp

    monkeypatch.setattr(fp, "extension", lambda *sizes: reference_modules["gm_fused_pairs_cpu"])
    edges, cutoff = cpu_edges()
    kernel = StandInKernel(field_in, field_out, cutoff, trunk=5, bias=bias)
    gen = torch.Generator().manual_seed(3)
    flat = torch.randn(edges.n_edges, kernel.field_type_in.dimension, generator=gen, dtype=torch.float64)  # an edge-level field
    y_plain, g_plain = run(kernel, flat, edges, False)
    y_fused, g_fused = run(kernel, flat, edges, True)
    for m in y_plain:
        torch.testing.assert_close(y_fused[m], y_plain[m], atol=1e-12, rtol=0.0)
    assert len(g_fused) == len(g_plain)
    for a, b in zip(g_fused, g_plain):
        torch.testing.assert_close(a, b, atol=1e-11, rtol=0.0)


def test_plan_order_and_node_level_fields(reference_modules, monkeypatch):
    """Term order = for every output frequency, for every input frequency (reference ``tests/nn/test_fused_pairs.py:136-147``);
    a node-level field is gathered by the driver itself; the blocked readout gradient equals the plain product."""
    from gm_attention_b200.fields import FeatureField
    from gm_attention_b200.nn import fused_pairs as fp

    monkeypatch.setattr(fp, "extension", lambda *sizes: reference_modules["gm_fused_pairs_cpu"])
    edges, cutoff = cpu_edges()
    kernel = StandInKernel({0: 1, 1: 2}, {0: 2, 1: 1}, cutoff)
    assert [(t.n, t.m, t.role) for t in fp.plan(kernel)] == [(0, 0, "real"), (1, 0, "linear"), (0, 1, "linear"), (1, 1, "linear"), (1, 1, "antilinear")]
    nodes = torch.randn(40, kernel.field_type_in.dimension, dtype=torch.float64, generator=torch.Generator().manual_seed(4))
    x = FeatureField.from_flat(kernel.field_type_in, nodes)
    gathered = FeatureField.from_flat(kernel.field_type_in, nodes[edges.source_index])
    a, b = fp.forward_general(kernel, x, edges), fp.forward_general(kernel, gathered, edges)
    for m in a.field_type.frequencies:
        assert torch.equal(a[m], b[m])
    monkeypatch.setattr(fp, "GRADIENT_BLOCK_ROWS", 7)
    gk, op = torch.randn(6, 40, dtype=torch.float64), torch.randn(40, 5, dtype=torch.float64)
    torch.testing.assert_close(fp._coefficient_product(gk, op), gk @ op, atol=1e-12, rtol=0)
