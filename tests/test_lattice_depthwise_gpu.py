"""The lattice depthwise convolution (coefficient table per (row pair, offset) instead of a per-edge stream) against the
reference's depthwise op (``nn/fused/attention.h:174-232, 265-287``, restated in ``oracle/gm_oracle.c`` and pinned to the
reference's compiled driver) fed with the SAME coefficients expanded to every edge.

* whole problem on small lattices, float32 and bf16 storage, batches 1 / 3 / 4 (every samples-per-CTA variant), plain and
  normalised aggregation weights: output, field gradient, and the coefficient gradient summed over the edges of an entry;
* 256 x 512, radius 4 pi / 256, batch 4, 64 x (m = 0, 1, 2) (a_0 = 64, W = 512, 22 999 040 edges per sample): sampled
  targets and sources (complete rows, exact), the coefficient gradient of one complete lattice row, and -- on the whole
  problem -- the adjoint identities  <g, y> = <table, dtable> = <dv, v>  that hold because y is bilinear in (table, v).

Tolerances: float32 1e-5 relative with an absolute part of 1e-5 of the tensor's largest magnitude for sums of hundreds
to thousands of terms; bf16 storage 2e-2 of the largest magnitude against the oracle in float32 on the rounded inputs.
"""

from __future__ import annotations

import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from oracle import geometry_np as G
from oracle import oracle as O
from oracle import sampled as S

from tests.helpers import assert_close, cuda, descriptor_rows, make_case, rel_err, seeded

pytestmark = pytest.mark.gpu


def magnitude(a) -> float:
    return max(float(np.abs(a).max()), 1.0)


def entry_of(tables, target: np.ndarray, source: np.ndarray) -> np.ndarray:
    """Table entry of every edge (target <- source), from the windows alone."""
    lat = tables.lattice
    span = 2 * lat.halo + 1
    cnt, lo, off = (x.cpu().numpy().reshape(-1) for x in (lat.win_cnt, lat.win_lo, lat.win_off))
    ri, li, rj, lj = target // lat.nlon, target % lat.nlon, source // lat.nlon, source % lat.nlon
    w = ri * span + (rj - ri + lat.halo)
    d = (lj - li - lo[w]) % lat.nlon
    assert (d < cnt[w]).all()
    return off[w] + d


def package_tables(c, head_type, normalize: bool):
    from gm_attention_b200.nn.lattice_depthwise import conv_tables

    weights = c.weights
    if normalize:
        mass = np.add.reduceat(c.weights, c.row_ptr[:-1])
        weights = (c.weights / np.repeat(np.maximum(mass, 1e-12), np.diff(c.row_ptr))).astype(c.weights.dtype)
    geometry = SimpleNamespace(transport=cuda(c.transport.astype(np.float32)), angular=cuda(c.angular.astype(np.float32)),
                               rho=cuda(c.rho.astype(np.float32)), bias=cuda(c.bias.astype(np.float32)), inside=cuda(c.inside),
                               row_ptr=cuda(c.row_ptr), source=cuda(c.source))
    rows = descriptor_rows(c.head_type, 1)
    return conv_tables(geometry, cuda((c.rho * c.radius).astype(np.float32)), cuda(weights.astype(np.float32)), rows, c.nlat, c.nlon), weights


@pytest.mark.parametrize("batch,storage,normalize", [(1, "f32", False), (3, "f32", True), (4, "f32", False), (3, "bf16", False), (4, "bf16", True)])
def test_whole_problem(batch, storage, normalize):
    from gm_attention_b200.nn.lattice_depthwise import lattice_depthwise

    head = {0: 4, 1: 3, 2: 2}
    c = make_case(16, 32, 3 * math.pi / 16, head, 1, dtype=np.float32)
    a0, w = 4, 4 * 3 + 4 * 2
    tables, weights = package_tables(c, head, normalize)
    n_entries = tables.n_entries
    rc_t, = seeded((n_entries, a0), 31, np.float32)
    cc_t, = seeded((n_entries, w), 32, np.float32)
    fields = seeded((batch * c.n_nodes, c.width), 33, np.float32, 2)
    bf16 = storage == "bf16"
    if bf16:
        dev = [torch.from_numpy(x).bfloat16().cuda() for x in fields]
        fields = [x.float().cpu().numpy() for x in dev]
    else:
        dev = [cuda(x) for x in fields]
    v, g = fields
    entry = entry_of(tables, c.target, c.source)
    rc, cc = rc_t[entry], cc_t[entry]
    args = (rc[None], cc[None], c.transport, c.angular, c.rho, weights, c.desc, c.row_ptr, c.source, a0, w)
    want_out, want_dv = np.zeros_like(v), np.zeros_like(v)
    want_drc, want_dcc = np.zeros_like(rc_t), np.zeros_like(cc_t)
    for b in range(batch):
        rows = slice(b * c.n_nodes, (b + 1) * c.n_nodes)
        want_out[rows] = O.conv_forward(v[rows], *args)
        dv, drc, dcc = O.conv_backward(g[rows], v[rows], *args)
        want_dv[rows] = dv
        np.add.at(want_drc, entry, drc.reshape(-1, a0))
        np.add.at(want_dcc, entry, dcc.reshape(-1, w))
    V = dev[0].requires_grad_(True)
    RC, CC = cuda(rc_t).requires_grad_(True), cuda(cc_t).requires_grad_(True)
    out = lattice_depthwise(V, RC, CC, tables)
    out.backward(dev[1])
    got = {"out": out.detach(), "dv": V.grad, "drc": RC.grad, "dcc": CC.grad}
    want = {"out": want_out, "dv": want_dv, "drc": want_drc, "dcc": want_dcc}
    for name in want:
        a = got[name].float().cpu().numpy()
        if bf16:
            assert rel_err(a, want[name]) < 2e-2, name
        else:
            assert_close(a, want[name], 1e-5, 1e-5 * magnitude(want[name]), name)


def test_only_true_neighbours_are_touched():
    """One Inf in the field reaches exactly the targets that see that node, as in the reference's edge loop."""
    from gm_attention_b200.nn.lattice_depthwise import fold, _apply

    head = {0: 4, 1: 3, 2: 2}
    c = make_case(16, 32, 3 * math.pi / 16, head, 1, dtype=np.float32)
    tables, _ = package_tables(c, head, False)
    rc_t, = seeded((tables.n_entries, 4), 41, np.float32)
    cc_t, = seeded((tables.n_entries, 20), 42, np.float32)
    v, = seeded((c.n_nodes, c.width), 43, np.float32)
    node = 5 * c.nlon + 31
    v[node, 5] = np.inf  # the imaginary part of the first m = 1 copy
    out = _apply(cuda(v), fold(cuda(rc_t), cuda(cc_t), tables), tables, False).cpu().numpy()
    seen_by = np.unique(c.target[c.source == node])
    bad = np.flatnonzero(~np.isfinite(out).all(1))
    assert np.array_equal(bad, seen_by)
    assert np.isfinite(out[:, :4]).all() and np.isfinite(out[:, 10:]).all()  # other channels stay finite everywhere


# ----------------------------------------------------------------------------- 256 x 512, radius 4 pi / 256, batch 4

NLAT, NLON, BATCH, COPIES = 256, 512, 4, 64
HEAD = {0: COPIES, 1: COPIES, 2: COPIES}
RADIUS = 4 * math.pi / NLAT


@pytest.fixture(scope="module")
def big():
    from gm_attention_b200.fields import FieldType
    from gm_attention_b200.geometry import compute_edge_geometry, midpoint_lattice
    from gm_attention_b200.nn import fused_attention as fa
    from gm_attention_b200.nn.lattice_depthwise import conv_tables

    dev = torch.device("cuda", 0)
    lattice = midpoint_lattice(NLAT, NLON, dev)
    edges = compute_edge_geometry(lattice, lattice.frames, RADIUS, max_frequency=4, dtype=torch.float32)
    assert edges.n_edges == 22_999_040
    geo = fa.geometry(edges, RADIUS, "hard", torch.float32)
    rows = descriptor_rows(FieldType(HEAD), 1)
    tables = conv_tables(geo, edges.distances.float(), geo.weights, rows, NLAT, NLON)
    assert tables.n_entries == 22_999_040 // NLON
    gen = torch.Generator(device="cuda").manual_seed(5)
    a0, w = COPIES, 8 * COPIES
    rc_t = torch.randn(tables.n_entries, a0, generator=gen, device=dev) / 4
    cc_t = torch.randn(tables.n_entries, w, generator=gen, device=dev) / 4
    return tables, rows, rc_t, cc_t


@pytest.mark.parametrize("storage", ["f32", "bf16"])
def test_sampled_targets_256x512(big, storage):
    from gm_attention_b200.nn.lattice_depthwise import lattice_depthwise

    tables, rows, rc_t, cc_t = big
    n1, D = NLAT * NLON, 5 * COPIES
    a0, w = COPIES, 8 * COPIES
    dtype = torch.bfloat16 if storage == "bf16" else torch.float32
    gen = torch.Generator(device="cuda").manual_seed(6)
    V, Gd = (torch.randn(BATCH * n1, D, generator=gen, device="cuda").to(dtype) for _ in range(2))
    V.requires_grad_(True)
    RC, CC = rc_t.clone().requires_grad_(True), cc_t.clone().requires_grad_(True)
    out = lattice_depthwise(V, RC, CC, tables)
    out.backward(Gd)
    # adjoint identities on the whole problem (float64 sums of the kernels' own results)
    from gm_attention_b200.nn.lattice_depthwise import fold, _table_gradient

    table = fold(rc_t, cc_t, tables)
    dtable = _table_gradient(Gd, V.detach(), tables)
    lhs = float((Gd.double() * out.detach().double()).sum())
    assert abs(float((table.double() * dtable.double()).sum()) - lhs) < (2e-2 if storage == "bf16" else 1e-4) * abs(lhs)
    assert abs(float((V.grad.double() * V.detach().double()).sum()) - lhs) < (2e-2 if storage == "bf16" else 1e-4) * abs(lhs)
    # sampled targets / sources of the LAST sample against the oracle
    lat = G.midpoint_lattice(NLAT, NLON)
    t_rows = [0, 1, 4, 9, NLAT // 2, NLAT - 1]
    targets = np.array([r * NLON + col for r in t_rows for col in (0, NLON - 1, NLON // 2 + 1)], np.int64)
    sources = np.array([9 * NLON, (NLAT // 2) * NLON + NLON - 1, 40 * NLON + 7], np.int64)
    sample = S.sample_problem(lat, RADIUS, targets, sources, 4, np.float32)
    b = BATCH - 1
    pick = lambda x, nodes: x[torch.from_numpy(b * n1 + nodes).cuda()].float().cpu().numpy()
    tgt = np.repeat(sample.nodes, np.diff(sample.row_ptr))
    entry = entry_of(tables, tgt, sample.nodes[sample.source_index])
    rc, cc = rc_t[torch.from_numpy(entry).cuda()].cpu().numpy(), cc_t[torch.from_numpy(entry).cuda()].cpu().numpy()
    want = S.run_conv(sample, pick(V.detach(), sample.nodes), pick(Gd, sample.nodes), rc, cc, rows, RADIUS, a0, w)
    got = {"out": pick(out.detach(), sample.targets), "dv": pick(V.grad, sample.sources)}
    for name in got:
        if storage == "bf16":
            assert rel_err(got[name], want[name]) < 2e-2, name
        else:
            assert_close(got[name], want[name], 1e-5, 1e-5 * magnitude(want[name]), name)
    # the coefficient gradient of every entry of ONE complete lattice row (row 9: 421 neighbours per node): all 512
    # targets of the row, all samples, per-edge gradients of the oracle summed per entry
    row = 9
    row_targets = row * NLON + np.arange(NLON, dtype=np.int64)
    whole = S.sample_problem(lat, RADIUS, row_targets, np.zeros(0, np.int64), 4, np.float32)
    tgt = np.repeat(whole.nodes, np.diff(whole.row_ptr))
    entry = entry_of(tables, tgt, whole.nodes[whole.source_index])
    index = torch.from_numpy(entry).cuda()
    rc, cc = rc_t[index].cpu().numpy(), cc_t[index].cpu().numpy()
    first, count = int(entry.min()), int(entry.max()) - int(entry.min()) + 1
    want_rc, want_cc = np.zeros((count, a0), np.float64), np.zeros((count, w), np.float64)
    for s in range(BATCH):
        rows_of = lambda x: x[torch.from_numpy(s * n1 + whole.nodes).cuda()].float().cpu().numpy()
        r = S.run_conv(whole, rows_of(V.detach()), rows_of(Gd), rc, cc, rows, RADIUS, a0, w)
        np.add.at(want_rc, entry - first, r["drc"])
        np.add.at(want_cc, entry - first, r["dcc"])
    got_rc, got_cc = RC.grad[first:first + count].cpu().numpy(), CC.grad[first:first + count].cpu().numpy()
    covered = np.unique(entry - first)
    for name, a, ref in (("drc", got_rc, want_rc), ("dcc", got_cc, want_cc)):
        if storage == "bf16":
            assert rel_err(a[covered], ref[covered]) < 2e-2, name
        else:
            assert_close(a[covered], ref[covered].astype(np.float32), 1e-4, 1e-5 * magnitude(ref), name)


# ----------------------------------------------------------------------------- the reference's own convolution layer

@pytest.mark.parametrize("name", ["plain", "normalized"])
def test_reference_convolution_layer(name):
    """A depthwise ``SO2Convolution`` with its radial network, as the reference's Python evaluates it through its eager
    path (fixtures of ``tests/golden/make_golden.py: depthwise_case``, float64), against the package's chain in float32:
    geometry on the device, radial network on the table entries, fold, apply; gradients of the field and of every
    parameter of the network."""
    from pathlib import Path

    from gm_attention_b200.fields import FieldType
    from gm_attention_b200.geometry import compute_edge_geometry, midpoint_lattice
    from gm_attention_b200.nn import fused_attention as fa
    from gm_attention_b200.nn.lattice_depthwise import conv_tables, lattice_depthwise
    from tests.test_lattice_depthwise_cpu import load_network

    z = np.load(Path(__file__).resolve().parent / "golden" / f"depthwise_{name}.npz")
    nlat, nlon, radius = int(z["nlat"]), int(z["nlon"]), float(z["radius"])
    head = FieldType({int(n): int(a) for n, a in z["types"]})
    dev = torch.device("cuda", 0)
    lattice = midpoint_lattice(nlat, nlon, dev)
    edges = compute_edge_geometry(lattice, lattice.frames, radius, max_frequency=4, dtype=torch.float32)
    geo = fa.geometry(edges, radius, "hard", torch.float32)
    weights = geo.aggregation_weights(bool(int(z["normalize"])), 1e-12)
    tables = conv_tables(geo, edges.distances.float(), weights, descriptor_rows(head, 1), nlat, nlon)
    net = load_network(z, torch.float32, dev)
    v = cuda(z["v"].astype(np.float32)).requires_grad_(True)
    out = lattice_depthwise(v, *net(tables.distances), tables)
    out.backward(cuda(z["dout"].astype(np.float32)))
    assert_close(out.detach().cpu().numpy(), z["out"].astype(np.float32), 2e-5, 2e-5 * magnitude(z["out"]), "out")
    assert_close(v.grad.cpu().numpy(), z["dv"].astype(np.float32), 2e-5, 2e-5 * magnitude(z["dv"]), "dv")
    for key, parameter in net.named_parameters():
        want = z["grad__" + key.replace(".", "__")].astype(np.float32)
        assert_close(parameter.grad.cpu().numpy(), want, 1e-4, 1e-4 * magnitude(want), key)
