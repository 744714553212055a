"""Parity of the op-level CUDA kernels (scores + softmax, depthwise convolution;
forward and backward) with the reference's own compiled CPU drivers, through
the extension-shim -> C ABI -> kernel path.

Tolerances: float64 1e-11 relative (summation order only); float32 1e-5
relative / 1e-6 absolute, scaled by the magnitude of the compared tensor for
gradients that sum hundreds of terms."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from oracle import oracle as O

from tests.helpers import assert_close, cuda, make_case, seeded

pytestmark = pytest.mark.gpu

CASES = [
    (8, 16, 2 * math.pi / 8, {0: 3, 1: 2, 2: 1}, 2, "hard"),
    (8, 16, 2.5 * math.pi / 8, {0: 2, 1: 2}, 4, "quartic"),
    (6, 12, 2 * math.pi / 6, {1: 3, 3: 2}, 1, "hard"),
    (16, 32, 2 * math.pi / 16, {0: 4, 1: 4, 2: 4}, 2, "hard"),  # 4 x (m = 0, 1, 2) per head, 2 heads, on a half-size grid
    (12, 24, 3 * math.pi / 12, {0: 5, 1: 3}, 3, "quartic"),  # odd offsets, H = 3
]


def magnitude(a) -> float:
    return max(float(np.abs(a).max()), 1.0) if a.size else 1.0


def tolerances(dtype):
    return (1e-11, 1e-12) if dtype == np.float64 else (1e-5, 1e-6)


@pytest.fixture(scope="module")
def ext():
    from gm_attention_b200.nn import fused_attention as fa

    return fa.extension(True)


def reference_or_oracle_softmax(reference_modules, c, q, k, da):
    t = torch.from_numpy
    ref = reference_modules["gm_fused_attention_cpu"]
    alpha = ref.softmax_forward(t(q), t(k), t(c.transport), t(c.bias), t(c.inside), t(c.desc), t(c.row_ptr), t(c.source), c.heads,
                                c.scale, c.max_degree)
    dq, dk = ref.softmax_backward(t(da), t(q), t(k), t(c.transport), t(c.bias), t(c.inside), t(c.desc), t(c.row_ptr), t(c.source),
                                  alpha, c.heads, c.scale, c.max_degree)
    return alpha.numpy(), dq.numpy(), dk.numpy()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("case", CASES)
def test_softmax_forward_backward(ext, reference_modules, case, dtype):
    c = make_case(*case[:5], dtype=dtype, window=case[5])
    q, k = seeded((c.n_nodes, c.width), 11, dtype, 2)
    da, = seeded((c.source.shape[0], c.heads), 12, dtype)
    alpha_ref, dq_ref, dk_ref = reference_or_oracle_softmax(reference_modules, c, q, k, da)
    tables = [cuda(x) for x in (c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source)]
    alpha = ext.softmax_forward(cuda(q), cuda(k), *tables, c.heads, c.scale, c.max_degree)
    rtol, atol = tolerances(dtype)
    assert_close(alpha.cpu().numpy(), alpha_ref, rtol, atol, "alpha")
    dq, dk = ext.softmax_backward(cuda(da), cuda(q), cuda(k), *tables, cuda(alpha_ref), c.heads, c.scale, c.max_degree)
    scale = magnitude(dk_ref)
    assert_close(dq.cpu().numpy(), dq_ref, rtol, atol * scale * 10, "dq")
    assert_close(dk.cpu().numpy(), dk_ref, rtol, atol * scale * 10, "dk")


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("case", CASES)
def test_conv_forward_backward(ext, reference_modules, case, dtype):
    nlat, nlon, radius, types, _, window = case
    c = make_case(nlat, nlon, radius, types, 1, dtype=dtype, window=window)
    a0 = types.get(0, 0)
    w = sum(4 * a for n, a in types.items() if n)
    e = c.source.shape[0]
    v, g = seeded((c.n_nodes, c.width), 13, dtype, 2)
    rc, = seeded((e, a0), 14, dtype)
    cc, = seeded((e, w), 15, dtype)
    t = torch.from_numpy
    ref = reference_modules["gm_fused_attention_cpu"]
    args = (t(rc), t(cc), t(c.transport), t(c.angular), t(c.rho), t(c.weights), t(c.desc), t(c.row_ptr), t(c.source), a0, w)
    out_ref = ref.conv_forward(t(v), *args).numpy()
    dv_ref, drc_ref, dcc_ref = (x.numpy() for x in ref.conv_backward(t(g), t(v), *args))
    dev = [cuda(x) for x in (rc, cc, c.transport, c.angular, c.rho, c.weights, c.desc, c.row_ptr, c.source)]
    out = ext.conv_forward(cuda(v), *dev, a0, w)
    rtol, atol = tolerances(dtype)
    assert_close(out.cpu().numpy(), out_ref, rtol, atol * magnitude(out_ref), "conv out")
    dv, drc, dcc = ext.conv_backward(cuda(g), cuda(v), *dev, a0, w)
    assert_close(dv.cpu().numpy(), dv_ref, rtol, atol * magnitude(dv_ref), "dv")
    assert_close(drc.cpu().numpy(), drc_ref, rtol, atol * magnitude(drc_ref), "drc")
    assert_close(dcc.cpu().numpy(), dcc_ref, rtol, atol * magnitude(dcc_ref), "dcc")


def test_softmax_large_neighbourhood_spills_to_global(ext):
    """A row whose logits exceed the shared-memory budget keeps them in alpha."""
    n, deg, heads, d = 3, 30000, 2, 4
    rng = np.random.default_rng(0)
    q = rng.standard_normal((n, d)).astype(np.float32)
    k = rng.standard_normal((n, d)).astype(np.float32)
    source = np.concatenate([rng.integers(0, n, deg), [1], [0, 2]]).astype(np.int64)
    row_ptr = np.array([0, deg, deg + 1, deg + 3], np.int64)
    e = source.shape[0]
    transport = np.tile(np.array([[[1.0, 0.0], [0.6, 0.8]]], np.float32), (e, 1, 1))
    bias = rng.standard_normal(e).astype(np.float32)
    inside = (rng.random(e) > 0.2).astype(np.uint8)
    inside[[0, deg, deg + 1]] = 1
    desc = np.array([[1, 1, 0, 0, 2]], np.int64)
    want = O.softmax_forward(q, k, transport, bias, inside, desc, row_ptr, source, heads, 0.5)
    got = ext.softmax_forward(cuda(q), cuda(k), cuda(transport), cuda(bias), cuda(inside), cuda(desc), cuda(row_ptr), cuda(source),
                              heads, 0.5, deg)
    assert_close(got.cpu().numpy(), want, 2e-5, 1e-7, "alpha (spilled logits)")


def test_float32_masked_edge_never_sets_the_shift(ext):
    """The reference's float32 boundary case (tests/nn/test_fused_attention.py:376-404)."""
    desc = np.array([[0, 1, 0, 0, 1]], np.int64)
    q = np.array([[1.0], [1.0]], np.float32)
    k = np.array([[1.0], [1e4]], np.float32)
    row_ptr = np.array([0, 2, 3], np.int64)
    source = np.array([0, 1, 1], np.int64)
    transport = np.tile(np.array([[[1.0, 0.0]]], np.float32), (3, 1, 1))
    bias = np.array([0.0, np.log(np.finfo(np.float32).tiny), 0.0], np.float32)
    inside = np.array([1, 0, 1], np.uint8)
    alpha = ext.softmax_forward(cuda(q), cuda(k), cuda(transport), cuda(bias), cuda(inside), cuda(desc), cuda(row_ptr), cuda(source),
                                1, 1.0, 2)
    assert alpha.cpu().numpy().reshape(-1).tolist() == [1.0, 0.0, 1.0]


def test_empty_problems_and_isolated_nodes(ext):
    dev = torch.device("cuda")
    desc = torch.tensor([[0, 2, 0, 0, 1]], device=dev)
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=dev)
    # no nodes at all
    alpha = ext.softmax_forward(z(0, 2), z(0, 2), z(0, 1, 2), z(0), z(0, dt=torch.uint8), desc, z(1, dt=torch.int64), z(0, dt=torch.int64), 1, 1.0, 1)
    assert alpha.shape == (0, 1)
    # nodes without any edge: conv output is zero, softmax backward gives zero dq
    out = ext.conv_forward(torch.ones(3, 2, device=dev), z(0), z(0), z(0, 1, 2), z(0, 1, 2), z(0), z(0), desc, z(4, dt=torch.int64),
                           z(0, dt=torch.int64), 2, 0)
    assert torch.equal(out, z(3, 2))
    dq, dk = ext.softmax_backward(z(0, 1), torch.ones(3, 2, device=dev), torch.ones(3, 2, device=dev), z(0, 1, 2), z(0),
                                  z(0, dt=torch.uint8), desc, z(4, dt=torch.int64), z(0, dt=torch.int64), z(0, 1), 1, 1.0, 1)
    assert torch.equal(dq, z(3, 2)) and torch.equal(dk, z(3, 2))


def test_contract_errors_match_the_reference_wording(ext):
    dev = torch.device("cuda")
    q = torch.zeros(2, 2, device=dev)
    with pytest.raises(RuntimeError, match="contiguous"):
        ext.softmax_forward(q.t(), q, torch.zeros(1, 1, 2, device=dev), torch.zeros(1, device=dev),
                            torch.zeros(1, dtype=torch.uint8, device=dev), torch.tensor([[0, 2, 0, 0, 1]], device=dev),
                            torch.tensor([0, 1, 1], device=dev), torch.tensor([0], device=dev), 1, 1.0, 1)
    with pytest.raises(RuntimeError, match="at most 8 heads"):
        ext.softmax_forward(q, q, torch.zeros(1, 1, 2, device=dev), torch.zeros(1, device=dev),
                            torch.zeros(1, dtype=torch.uint8, device=dev), torch.tensor([[0, 2, 0, 0, 1]], device=dev),
                            torch.tensor([0, 1, 1], device=dev), torch.tensor([0], device=dev), 9, 1.0, 1)


def test_autograd_functions_run_end_to_end(ext):
    """Softmax.apply / Depthwise.apply with the reference's argument orders."""
    from gm_attention_b200.nn import fused_attention as fa

    c = make_case(8, 16, 2 * math.pi / 8, {0: 3, 1: 2, 2: 1}, 2, dtype=np.float64)
    q, k = (cuda(x).requires_grad_(True) for x in seeded((c.n_nodes, c.width), 21, np.float64, 2))
    tables = [cuda(x) for x in (c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source)]
    alpha = fa.Softmax.apply(q, k, *tables, c.heads, c.scale, c.max_degree)
    weight = cuda(seeded(tuple(alpha.shape), 22, np.float64)[0])
    (alpha * weight).sum().backward()
    dq_ref, dk_ref = O.softmax_backward(weight.cpu().numpy(), q.detach().cpu().numpy(), k.detach().cpu().numpy(), c.transport, c.desc,
                                        c.row_ptr, c.source, alpha.detach().cpu().numpy(), c.heads, c.scale)
    assert_close(q.grad.cpu().numpy(), dq_ref, 1e-10, 1e-11, "dq through autograd")
    assert_close(k.grad.cpu().numpy(), dk_ref, 1e-10, 1e-11, "dk through autograd")


def test_chunked_scores_equal_the_whole_edge_set(ext):
    """Exact chunking over contiguous target ranges (reference ``nn/attention.py:344-402``): every chunk holds whole
    neighbourhoods, its constants are views of the parent's, and the softmax stays a partition of unity inside it --
    the op over the chunks, concatenated, equals the op over the whole edge set bit for bit."""
    from gm_attention_b200.fields import FieldType
    from gm_attention_b200.geometry import compute_edge_geometry, midpoint_lattice
    from gm_attention_b200.nn import fused_attention as fa

    dev = torch.device("cuda", 0)
    lattice = midpoint_lattice(12, 24, dev)
    cutoff = 2 * math.pi / 12
    edges = compute_edge_geometry(lattice, lattice.frames, cutoff, max_frequency=2, dtype=torch.float32)
    heads, attn = 2, FieldType({0: 4, 1: 4, 2: 4})
    owner = type("Layer", (), {})()
    p = fa._plan(owner, attn, attn.scaled(heads), heads)
    desc = fa.descriptors(owner, p, dev)
    q, k = (cuda(x) for x in seeded((lattice.n_nodes, p.width), 21, np.float32, 2))
    scale = 1.0 / math.sqrt(attn.dimension)
    whole = fa.geometry(edges, cutoff, "quartic", torch.float32)
    alpha = ext.softmax_forward(q, k, whole.transport, whole.bias, whole.inside, desc, whole.row_ptr, whole.source, heads, scale, whole.max_degree)
    pieces = []
    for first in range(0, lattice.n_nodes, 37):
        last = min(lattice.n_nodes, first + 37)
        chunk, e_first, e_last = edges.target_range(first, last)
        fa.register_chunk(chunk, edges, e_first, e_last)
        g = fa.geometry(chunk, cutoff, "quartic", torch.float32)
        assert g.base is whole and g.transport.data_ptr() == whole.transport[e_first:e_last].data_ptr()
        part = ext.softmax_forward(q, k, g.transport, g.bias, g.inside, desc, g.row_ptr, g.source, heads, scale, max(g.max_degree, 1))
        sums = torch.zeros(lattice.n_nodes, heads, device=dev).index_add_(0, chunk.target_index, part)
        assert torch.allclose(sums[first:last], torch.ones_like(sums[first:last]), atol=1e-5)
        pieces.append(part)
    assert torch.equal(torch.cat(pieces), alpha)
