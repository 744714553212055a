"""Factored steerable kernel (forward, aggregate, backward, aggregated backward)
and pair-term kernels against the reference's own compiled CPU drivers, through
the extension shim and the C ABI.  float64 to 1e-10; float32 rtol 1e-4 / atol
1e-5 scaled by magnitude (the reference's own test tolerances,
tests/nn/test_fused_factored.py:126-158, 272-334)."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from tests.helpers import assert_close, cuda, make_case, seeded

pytestmark = pytest.mark.gpu


def blocks_for(type_in: dict[int, int], type_out: dict[int, int]):
    """Readout order of the reference kernel: real (0, 0) first, then for every (n, m) pair linear, then antilinear."""
    blocks, powers = [], {}
    if 0 in type_in and 0 in type_out:
        blocks.append((0, 0, "real"))
    for n in sorted(type_in):
        for m in sorted(type_out):
            if n == 0 and m == 0:
                continue
            blocks.append((n, m, "linear"))
            powers[(n, m, "linear")] = abs(m - n)
            if n >= 1 and m >= 1:
                blocks.append((n, m, "antilinear"))
                powers[(n, m, "antilinear")] = m + n
    return blocks, powers


FACTORED_CASES = [
    ({0: 2, 1: 2}, {0: 2, 1: 3}, 5),
    ({0: 8, 1: 8, 2: 8}, {0: 4, 1: 4, 2: 4}, 17),  # value kernel of the 32 x 64 configuration: 13 blocks, wc 48, wr 4
    ({1: 3}, {0: 2, 2: 2}, 4),                       # no real block
    ({0: 32, 1: 32, 2: 32, 3: 32}, {0: 8, 1: 8, 2: 8, 3: 8}, 17),  # the 128 x 256 layer (32 x (m <= 3) -> 8 x (m <= 3)): packed width 392 > the reference's 320
]


def factored_problem(type_in, type_out, k, dtype, seed):
    from gm_attention_b200.fields import FieldType
    from gm_attention_b200.nn import fused_factored as ff

    c = make_case(8, 16, 2 * math.pi / 8, {0: 1}, 1, dtype=dtype, max_frequency=6)
    blocks, powers = blocks_for(type_in, type_out)
    p = ff.plan_blocks(blocks, FieldType(type_out), powers)
    e, n = c.source.shape[0], c.n_nodes
    h, = seeded((e, k - 1), seed, dtype)
    zc, = seeded((n, k, p.wc, 2), seed + 1, dtype)
    zr, = seeded((n, k, p.wr), seed + 2, dtype)
    desc = np.array([b.row() for b in p.blocks], np.int32).reshape(-1, 8)
    return c, p, h, zc, zr, desc


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("case", FACTORED_CASES)
def test_factored_against_reference_driver(reference_modules, case, dtype):
    from gm_attention_b200.nn import fused_factored as ff

    type_in, type_out, k = case
    c, p, h, zc, zr, desc = factored_problem(type_in, type_out, k, dtype, 61)
    too_wide_for_reference = 2 * p.wc + p.wr > 320
    ext = ff.extension(True)
    t = torch.from_numpy
    order, group_ptr, group_source = ff.source_groups(t(c.source))
    dev = [cuda(x) for x in (h, zc, zr, c.angular, c.transport, c.rho, desc, c.source)]
    groups = [x.cuda() for x in (order, group_ptr, group_source)]
    rows = ext.forward(*dev, *groups, p.d_out, p.max_bm)
    weights, = seeded((c.source.shape[0],), 64, dtype)
    out = ext.aggregate(rows, cuda(weights), cuda(c.row_ptr))
    g_rows, = seeded((c.source.shape[0], p.d_out), 65, dtype)
    g_nodes, = seeded((c.n_nodes, p.d_out), 66, dtype)
    dh, dzc, dzr = ext.backward(cuda(g_rows), *dev, *groups)
    agg = ext.backward_aggregated(cuda(g_nodes), cuda(c.target), cuda(weights), rows, *dev, *groups)
    rtol, atol = (1e-10, 1e-11) if dtype == np.float64 else (1e-4, 1e-5)
    if too_wide_for_reference:
        # the reference refuses this width; check the linear-algebra identities instead:
        # aggregate = weighted segment sum of the rows, and <g, rows> = <dh, h> + <dZ, Z> (the map is bilinear in (h~, Z))
        rows_np = rows.cpu().numpy().astype(np.float64)
        want = np.add.reduceat(rows_np * weights[:, None], c.row_ptr[:-1], axis=0)
        assert_close(out.cpu().numpy(), want, 10 * rtol, 10 * atol * max(1.0, np.abs(want).max()), "aggregate")
        lhs = float((g_rows.astype(np.float64) * rows_np).sum())
        zsum = float((dzc.cpu().numpy().astype(np.float64) * zc).sum() + (dzr.cpu().numpy().astype(np.float64) * zr).sum())
        assert abs(zsum - lhs) <= 1e-3 * abs(lhs) + 1e-6  # rows are linear in Z
        # ... and the numpy restatement of the reference arithmetic, which has no width limit
        from oracle import ops_np

        mag = lambda x: max(1.0, float(np.abs(x).max())) if x.size else 1.0
        rows_np2 = ops_np.factored_forward(h, zc, zr, c.angular, c.transport, c.rho, desc, c.source, p.d_out)
        assert_close(rows.cpu().numpy(), rows_np2, 10 * rtol, 10 * atol * mag(rows_np2), "rows vs restatement")
        for name, got, ref_np in zip(("dh", "dzc", "dzr"), (dh, dzc, dzr),
                                     ops_np.factored_backward(g_rows, h, zc, zr, c.angular, c.transport, c.rho, desc, c.source)):
            assert_close(got.cpu().numpy(), ref_np, 10 * rtol, 100 * atol * mag(ref_np), name + " vs restatement")
        return
    ref = reference_modules["gm_factored_cpu"]
    cpu = [t(x) for x in (h, zc, zr, c.angular, c.transport, c.rho, desc, c.source)]
    rows_ref = ref.forward(*cpu, order, group_ptr, group_source, p.d_out, p.max_bm)
    mag = lambda x: max(1.0, float(np.abs(x).max())) if x.size else 1.0
    assert_close(rows.cpu().numpy(), rows_ref.numpy(), rtol, atol * mag(rows_ref.numpy()), "rows")
    out_ref = ref.aggregate(rows_ref, t(weights), t(c.row_ptr))
    assert_close(out.cpu().numpy(), out_ref.numpy(), rtol, 10 * atol * mag(out_ref.numpy()), "aggregate")
    for name, got, want in zip(("dh", "dzc", "dzr"), (dh, dzc, dzr), ref.backward(t(g_rows), *cpu, order, group_ptr, group_source)):
        assert_close(got.cpu().numpy(), want.numpy(), rtol, 10 * atol * mag(want.numpy()), name)
    agg_ref = ref.backward_aggregated(t(g_nodes), t(c.target), t(weights), rows_ref, *cpu, order, group_ptr, group_source)
    for name, got, want in zip(("dh", "dzc", "dzr", "dweights"), agg, agg_ref):
        assert_close(got.cpu().numpy(), want.numpy(), rtol, 100 * atol * mag(want.numpy()), "aggregated " + name)


def test_source_groups_known_answer():
    """The grouping of the reference's tests/nn/test_fused_factored.py:105-123."""
    from gm_attention_b200.nn import fused_factored as ff

    order, ptr, sources = ff.source_groups(torch.tensor([2, 1, 2, 0, 1, 2]))
    assert order.tolist() == [3, 1, 4, 0, 2, 5] and ptr.tolist() == [0, 1, 3, 6] and sources.tolist() == [0, 1, 2]


def test_factored_autograd_functions():
    from gm_attention_b200.nn import fused_factored as ff

    c, p, h, zc, zr, desc = factored_problem({0: 2, 1: 2}, {0: 2, 1: 3}, 5, np.float64, 71)
    order, group_ptr, group_source = (x.cuda() for x in ff.source_groups(torch.from_numpy(c.source)))
    H, ZC, ZR = (cuda(x).requires_grad_(True) for x in (h, zc, zr))
    W = cuda(seeded((c.source.shape[0],), 72, np.float64)[0]).requires_grad_(True)
    tables = [cuda(x) for x in (c.angular, c.transport, c.rho, desc, c.source)]
    out = ff.FactoredAggregate.apply(H, ZC, ZR, W, *tables, cuda(c.target), cuda(c.row_ptr), order, group_ptr, group_source, p.d_out, p.max_bm)
    rows = ff.Factored.apply(H, ZC, ZR, *tables, order, group_ptr, group_source, p.d_out, p.max_bm)
    want = torch.segment_reduce(rows * W[:, None], "sum", offsets=cuda(c.row_ptr))
    assert torch.allclose(out, want, rtol=1e-10, atol=1e-11)
    g = cuda(seeded(tuple(out.shape), 73, np.float64)[0])
    grads_a = torch.autograd.grad((out * g).sum(), (H, ZC, ZR, W), retain_graph=True)
    grads_b = torch.autograd.grad((want * g).sum(), (H, ZC, ZR, W))
    for a, b in zip(grads_a, grads_b):
        assert torch.allclose(a, b, rtol=1e-9, atol=1e-10)


PAIR_CASES = [
    (3, 2, 5, 2 | 8),          # real block: U_REAL | OUT_REAL
    (4, 8, 16, 1 | 2),         # 0 -> m: MATRIX_COMPLEX | U_REAL
    (8, 4, 16, 1 | 4 | 8),     # n -> 0: MATRIX_COMPLEX | CONJ_U | OUT_REAL
    (16, 16, 16, 1),           # linear
    (2, 3, 7, 1 | 4),          # antilinear
]


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("case", PAIR_CASES)
def test_pairs_against_reference_driver(reference_modules, case, dtype):
    from gm_attention_b200.nn import fused_pairs as fp

    a, b, trunk, flags = case
    ref = reference_modules["gm_fused_pairs_cpu"]
    ext = fp.extension()
    e = 301
    width = (2 if flags & 1 else 1) * a * b
    cdt = torch.complex64 if dtype == np.float32 else torch.complex128
    rnd = lambda shape, seed: torch.from_numpy(seeded(shape, seed, dtype)[0])
    cx = lambda shape, seed: torch.view_as_complex(rnd((*shape, 2), seed))
    hidden, weight, bias = rnd((e, trunk), 81), rnd((width, trunk), 82), rnd((width,), 83)
    u = rnd((e, a), 84) if flags & 2 else cx((e, a), 84)
    pre = torch.polar(torch.ones(e, dtype=torch.from_numpy(np.zeros(1, dtype)).dtype), rnd((e,), 85))
    post = torch.polar(torch.ones(e, dtype=pre.real.dtype), rnd((e,), 86))
    scale = rnd((e,), 87).abs()
    out0 = rnd((e, b), 88) if flags & 8 else cx((e, b), 88)
    grad_out = rnd((e, b), 89) if flags & 8 else cx((e, b), 89)
    assert pre.dtype == cdt
    out_ref = out0.clone()
    ref.forward(hidden, weight, bias, u, pre, post, scale, out_ref, a, b, flags)
    out = out0.clone().cuda()
    dev = [x.cuda() for x in (hidden, weight, bias, u, pre, post, scale)]
    ext.forward(*dev, out, a, b, flags)
    rtol, atol = (1e-10, 1e-11) if dtype == np.float64 else (1e-4, 1e-5)
    as_np = lambda x: torch.view_as_real(x).cpu().numpy() if x.is_complex() else x.cpu().numpy()
    mag = lambda x: max(1.0, float(np.abs(x).max()))
    assert_close(as_np(out), as_np(out_ref), rtol, atol * mag(as_np(out_ref)), "out")
    gu_ref, gh_ref, gk_ref = torch.ones_like(u), torch.ones_like(hidden), torch.zeros(width, e, dtype=hidden.dtype)
    ref.backward(hidden, weight, bias, u, pre, post, scale, grad_out, gu_ref, gh_ref, gk_ref, a, b, flags)
    gu, gh, gk = torch.ones_like(u).cuda(), torch.ones_like(hidden).cuda(), torch.zeros(width, e, dtype=hidden.dtype).cuda()
    ext.backward(*dev, grad_out.cuda(), gu, gh, gk, a, b, flags)
    for name, got, want in (("grad_u", gu, gu_ref), ("grad_hidden", gh, gh_ref), ("grad_k", gk, gk_ref)):
        assert_close(as_np(got), as_np(want), rtol, 10 * atol * mag(as_np(want)), name)


def test_pairs_plan_order():
    """Term order of the reference planner (tests/nn/test_fused_pairs.py:136-147): m outer, n inner; linear before antilinear."""
    from types import SimpleNamespace

    from gm_attention_b200.fields import FieldType
    from gm_attention_b200.nn import fused_pairs as fp

    tin, tout = FieldType({0: 2, 1: 3}), FieldType({0: 1, 1: 2})
    ranges, powers = {}, {}
    offset = 0
    for n, m in [(0, 1), (1, 0), (1, 1)]:
        width = 2 * tout.multiplicity(m) * tin.multiplicity(n)
        ranges[(n, m, "linear")], powers[(n, m, "linear")] = slice(offset, offset + width), abs(m - n)
        offset += width
        if n and m:
            ranges[(n, m, "antilinear")], powers[(n, m, "antilinear")] = slice(offset, offset + width), m + n
            offset += width
    kernel = SimpleNamespace(field_type_in=tin, field_type_out=tout, _pair_ranges=ranges, _pair_powers=powers)
    terms = fp.plan(kernel)
    assert [(t.n, t.m, t.role) for t in terms] == [(0, 0, "real"), (1, 0, "linear"), (0, 1, "linear"), (1, 1, "linear"), (1, 1, "antilinear")]
    assert [t.flags for t in terms] == [2 | 8, 1 | 4 | 8, 1 | 2, 1, 1 | 4]
    assert [(t.pre_order, t.post_order) for t in terms] == [(None, None), (1, None), (None, 1), (0, None), (2, None)]


# ----------------------------------------------------------------------------- the pair-term driver (_FusedPairs, forward_general)

DRIVER_CASES = [
    ({0: 2, 1: 2, 2: 1}, {0: 1, 1: 2, 2: 2}, True),
    ({0: 2, 1: 2, 2: 1}, {0: 1, 1: 2, 2: 2}, False),
    ({0: 3}, {0: 2}, True),
    ({1: 2, 2: 1}, {1: 1, 2: 2}, True),
    ({0: 2, 1: 1}, {1: 2}, True),
    ({1: 2}, {0: 2}, True),
    ({1: 16}, {1: 16}, True),
    ({0: 5, 1: 7}, {0: 6, 2: 5}, True),  # block sides outside the reference's CPU size list
]


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("field_in, field_out, bias", DRIVER_CASES)
def test_pairs_driver_matches_the_pair_loop(field_in, field_out, bias, dtype):
    """``forward_general`` (one launch per term, blocked readout gradient) against the plain-PyTorch pair loop on the
    same device: values and every gradient (input field, trunk, both heads), the logic of the reference's
    ``tests/nn/test_fused_pairs.py:73-93``.  float64 1e-11 / 1e-10; float32 1e-5 relative to the tensor's magnitude."""
    from gm_attention_b200.fields import FeatureField
    from gm_attention_b200.geometry import compute_edge_geometry, midpoint_lattice
    from gm_attention_b200.nn import fused_pairs as fp

    from tests.helpers import StandInKernel

    dev = torch.device("cuda", 0)
    lattice = midpoint_lattice(6, 12, dev)
    cutoff = 1.4 * math.pi / 6
    edges = compute_edge_geometry(lattice, lattice.frames, cutoff, max_frequency=4, dtype=dtype)
    kernel = StandInKernel(field_in, field_out, cutoff, trunk=16, bias=bias, dtype=dtype).to(dev)
    flat0 = torch.randn(lattice.n_nodes, kernel.field_type_in.dimension, generator=torch.Generator().manual_seed(5), dtype=dtype).to(dev)

    def run(fused: bool):
        flat = flat0.clone().requires_grad_(True)
        x = FeatureField.from_flat(kernel.field_type_in, flat)
        out = fp.forward_general(kernel, x, edges).coefficients if fused else kernel.pair_loop(x, edges)
        loss = sum((out[m] * torch.linspace(0.1, 1.0, out[m].numel(), dtype=dtype, device=dev).reshape(out[m].shape)).sum() for m in out)
        return {m: v.detach() for m, v in out.items()}, [g.detach() for g in torch.autograd.grad(loss, [flat, *kernel.parameters()])]

    y_plain, g_plain = run(False)
    y_fused, g_fused = run(True)
    tol_y, tol_g = (1e-11, 1e-10) if dtype == torch.float64 else (1e-5, 1e-5)
    for m in y_plain:
        scale = max(1.0, float(y_plain[m].abs().max()))
        assert float((y_fused[m] - y_plain[m]).abs().max()) <= tol_y * scale, m
    for a, b in zip(g_fused, g_plain):
        assert float((a - b).abs().max()) <= tol_g * max(1.0, float(b.abs().max()))
