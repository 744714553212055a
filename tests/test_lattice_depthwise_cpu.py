"""CPU pins of the depthwise path: the radial network and the C oracle against fixtures produced by the reference's own
Python (``tests/golden/make_golden.py: depthwise_case`` -- a depthwise ``SO2Convolution`` through the eager path), and
the folded 2 x 2 matrices against the message formula of ``nn/depthwise.py:176-191``."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import geometry_np as G
from oracle import oracle as O

from tests.helpers import descriptor_rows, window_values

from gm_attention_b200.fields import FieldType

GOLDEN = Path(__file__).resolve().parent / "golden"
CASES = ["plain", "normalized"]


def load_network(z, dtype=torch.float64, device="cpu"):
    from gm_attention_b200.nn.lattice_depthwise import RadialCoefficients

    net = RadialCoefficients(z["rc"].shape[1], z["cc"].shape[1], float(z["radius"]), n_radial_basis=4, radial_hidden_features=(16,),
                             dtype=dtype, device=device)
    state = {k.replace("__", "."): torch.from_numpy(z[k]).to(dtype) for k in z.files if "__" in k and not k.startswith("grad__")}
    net.load_state_dict(state, strict=False)
    return net


@pytest.mark.parametrize("name", CASES)
def test_radial_network_matches_the_reference(name):
    z = np.load(GOLDEN / f"depthwise_{name}.npz")
    rc, cc = load_network(z)(torch.from_numpy(z["distances"]))
    np.testing.assert_allclose(rc.detach().numpy(), z["rc"], rtol=1e-12, atol=1e-13)
    np.testing.assert_allclose(cc.detach().numpy(), z["cc"], rtol=1e-12, atol=1e-13)


@pytest.mark.parametrize("name", CASES)
def test_oracle_depthwise_matches_the_reference_eager_path(name):
    """The C restatement of the depthwise op (forward and backward) on the reference's own coefficients equals the
    reference's eager gather / kernel / weighted segment sum and autograd's field gradient."""
    z = np.load(GOLDEN / f"depthwise_{name}.npz")
    nlat, nlon, radius = int(z["nlat"]), int(z["nlon"]), float(z["radius"])
    e = G.lattice_edges(G.midpoint_lattice(nlat, nlon), radius, 4, np.float64)
    np.testing.assert_allclose(e.distances, z["distances"], rtol=0, atol=1e-12)
    head = FieldType({int(n): int(a) for n, a in z["types"]})
    desc = descriptor_rows(head, 1)
    weights = window_values(e.distances, radius, "hard") * e.tangent_quadrature_weights
    if int(z["normalize"]):
        mass = np.maximum(np.add.reduceat(weights, e.row_ptr[:-1]), 1e-12)
        weights = weights / np.repeat(mass, np.diff(e.row_ptr))
    stack = lambda c: np.ascontiguousarray(np.stack([c.real, c.imag], -1))
    a0, w = z["rc"].shape[1], z["cc"].shape[1]
    args = (z["rc"][None], z["cc"][None], stack(e.transport_phases), stack(e.angular_phases), e.distances / radius, weights, desc, e.row_ptr,
            e.source_index, a0, w)
    out = O.conv_forward(z["v"], *args)
    dv, _, _ = O.conv_backward(z["dout"], z["v"], *args)
    np.testing.assert_allclose(out, z["out"], rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(dv, z["dv"], rtol=1e-11, atol=1e-12)


def test_fold_is_the_reference_message():
    from gm_attention_b200.nn.lattice_depthwise import ConvTables, fold

    head = FieldType({0: 4, 1: 3, 2: 2})
    rows = tuple(tuple(int(x) for x in r) for r in descriptor_rows(head, 1))
    gen = torch.Generator().manual_seed(0)
    n = 50
    unit = lambda: torch.polar(torch.ones(n, 2, dtype=torch.float32), torch.rand(n, 2, generator=gen) * 6.28)
    tau, omega = unit(), unit() * torch.rand(n, 2, generator=gen)
    weights = torch.rand(n, generator=gen) + 0.1
    t = ConvTables(None, rows, 4, 20, 4 + 4 * 5, None, None, torch.rand(n, generator=gen), weights, tau, omega)
    rc, cc = torch.randn(n, 4, generator=gen), torch.randn(n, 20, generator=gen)
    table = fold(rc, cc, t)
    assert table.shape == (n, 24)
    torch.testing.assert_close(table[:, :4], rc * weights[:, None])
    z = torch.randn(n, 5, dtype=torch.complex64, generator=gen)
    column, copy = 0, 0
    for index, (freq, copies) in enumerate(((1, 3), (2, 2))):
        block = cc[:, column:column + 4 * copies].reshape(n, 2, copies, 2)
        a, b = torch.view_as_complex(block[:, 0].contiguous()), torch.view_as_complex(block[:, 1].contiguous())
        zt = tau[:, index:index + 1] * z[:, copy:copy + copies]
        want = weights[:, None] * (a * zt + omega[:, index:index + 1] * b * zt.conj())  # nn/depthwise.py:188
        m = table[:, 4 + 4 * copy:4 + 4 * (copy + copies)].reshape(n, copies, 2, 2)
        zz = z[:, copy:copy + copies]
        got = torch.complex(m[..., 0, 0] * zz.real + m[..., 0, 1] * zz.imag, m[..., 1, 0] * zz.real + m[..., 1, 1] * zz.imag)
        torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)
        column += 4 * copies
        copy += copies


def _apply_on_the_host(x, table, cnt, lo, off, items, nlat, nlon, halo, transpose):
    """What ``gm_lattice_conv_apply`` computes, as numpy loops over (target row, window, offset)."""
    y = np.zeros_like(x)
    grid = x.reshape(nlat, nlon, -1)
    out = y.reshape(nlat, nlon, -1)
    span = 2 * halo + 1
    for i in range(nlat):
        for c in range(span):
            j = i + c - halo
            n = int(cnt[i, c])
            if not (0 <= j < nlat) or n == 0:
                continue
            for d in range(n):
                entry = table[int(off[i, c]) + d]
                source = np.roll(grid[j], -(int(lo[i, c]) + d), axis=0)  # source[l] = x[j, l + lo + d]
                for kind, col, fcol in items:
                    if kind == 1:
                        out[i, :, col] += entry[fcol] * source[:, col]
                        out[i, :, col + 1] += entry[fcol + 1] * source[:, col + 1]
                    else:
                        m = entry[fcol:fcol + 4].reshape(2, 2)
                        m = m.T if transpose else m
                        out[i, :, col] += m[0, 0] * source[:, col] + m[0, 1] * source[:, col + 1]
                        out[i, :, col + 1] += m[1, 0] * source[:, col] + m[1, 1] * source[:, col + 1]
    return y


@pytest.mark.parametrize("normalize", [False, True])
def test_tables_and_fold_reproduce_the_depthwise_op_on_the_host(normalize):
    """The host side of the lattice convolution -- windows, entry origins, transposed entry order, items, fold -- without a
    GPU: the table applied along the windows by plain numpy loops equals the reference's depthwise op (C oracle) on the
    same coefficients expanded to every edge, forward and for the field gradient (transposed windows, transposed matrices)."""
    import math
    from types import SimpleNamespace

    from tests.helpers import make_case, seeded

    from gm_attention_b200.nn.lattice_depthwise import conv_tables, fold

    head = {0: 4, 1: 3, 2: 2}
    c = make_case(8, 16, 2.5 * math.pi / 8, head, 1, dtype=np.float64)
    weights = c.weights
    if normalize:
        mass = np.add.reduceat(c.weights, c.row_ptr[:-1])
        weights = c.weights / np.repeat(np.maximum(mass, 1e-12), np.diff(c.row_ptr))
    t = torch.from_numpy
    geometry = SimpleNamespace(transport=t(c.transport.astype(np.float32)), angular=t(c.angular.astype(np.float32)), rho=t(c.rho.astype(np.float32)),
                               bias=t(c.bias.astype(np.float32)), inside=t(c.inside), row_ptr=t(c.row_ptr), source=t(c.source))
    tables = conv_tables(geometry, t((c.rho * c.radius).astype(np.float32)), t(weights.astype(np.float32)), descriptor_rows(c.head_type, 1), c.nlat, c.nlon)
    lat = tables.lattice
    assert tables.n_entries * c.nlon == c.source.shape[0] and tables.table_width == 4 + 4 * 5
    a0, w = 4, 20
    rc_t, = seeded((tables.n_entries, a0), 51, np.float32)
    cc_t, = seeded((tables.n_entries, w), 52, np.float32)
    table = fold(t(rc_t), t(cc_t), tables).numpy().astype(np.float64)
    v, g = seeded((c.n_nodes, c.width), 53, np.float64, 2)
    # the same coefficients on every edge of an entry
    span = 2 * lat.halo + 1
    cnt, lo, off = (x.numpy() for x in (lat.win_cnt, lat.win_lo, lat.win_off))
    ri, li, rj, lj = c.target // c.nlon, c.target % c.nlon, c.source // c.nlon, c.source % c.nlon
    win = (ri, rj - ri + lat.halo)
    entry = off[win] + (lj - li - lo[win]) % c.nlon
    args = (rc_t[entry].astype(np.float64)[None], cc_t[entry].astype(np.float64)[None], c.transport, c.angular, c.rho, weights, c.desc, c.row_ptr,
            c.source, a0, w)
    want = O.conv_forward(v, *args)
    want_dv, _, _ = O.conv_backward(g, v, *args)
    items = tables.items.numpy().tolist()
    got = _apply_on_the_host(v, table, cnt, lo, off, items, c.nlat, c.nlon, lat.halo, False)
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5 * np.abs(want).max())
    t_table = table[lat.t_entry.numpy()]
    got_dv = _apply_on_the_host(g, t_table, lat.t_win_cnt.numpy(), lat.t_win_lo.numpy(), lat.t_win_off.numpy(), items, c.nlat, c.nlon, lat.halo, True)
    np.testing.assert_allclose(got_dv, want_dv, rtol=1e-5, atol=1e-5 * np.abs(want_dv).max())
