"""The equiangular-lattice fast path of the fused layer against the oracle and
against the general CSR kernels: forward and the deterministic two-pass
backward, float32 (1e-5 relative / 1e-6 absolute, absolute part scaled by the
tensor's magnitude) and bf16 storage (2e-2 relative to the magnitude)."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from oracle import oracle as O

from tests.helpers import assert_close, cuda, make_case, rel_err, seeded

pytestmark = pytest.mark.gpu

CASES = [
    # nlat, nlon, radius, head type, heads, window, batch
    (16, 32, 2 * math.pi / 16, {0: 4, 1: 4, 2: 4}, 2, "hard", 2),         # 2 heads of 4 x (m = 0, 1, 2)
    (12, 24, 3 * math.pi / 12, {0: 16, 1: 16, 2: 16}, 4, "hard", 1),      # headline layout; polar windows are whole rows
    (8, 16, 2.5 * math.pi / 8, {0: 2, 1: 2}, 4, "quartic", 2),             # pairs outside the quartic window's support
    (10, 20, 2 * math.pi / 10, {0: 8, 1: 8, 2: 8, 3: 8}, 4, "hard", 1),   # 4 heads of 8 x (m = 0..3)
    (8, 256, 1.2 * math.pi / 8, {0: 4, 1: 4, 2: 4}, 2, "hard", 1),        # wide windows: several staged chunks per row
    (8, 16, 2 * math.pi / 8, {1: 6, 2: 6}, 1, "hard", 2),                 # no scalar block, runs of 2 with idle slots
    (8, 16, 2 * math.pi / 8, {0: 3, 2: 5}, 2, "hard", 1),                 # odd multiplicities: unaligned runs
]


def tables_for(c):
    from gm_attention_b200.attention import AttentionTables, build_lattice_tables

    rows = tuple(tuple(int(x) for x in row) for row in c.desc)
    general = AttentionTables(cuda(c.transport), cuda(c.bias), cuda(c.inside), cuda(c.row_ptr), cuda(c.source), rows, c.heads, c.scale)
    return general, build_lattice_tables(general, c.nlat, c.nlon, rows, c.heads, c.scale)


@pytest.mark.parametrize("case", CASES)
def test_lattice_matches_oracle_float32(case):
    from gm_attention_b200.attention import lattice_attention_backward, lattice_attention_forward

    batch = case[6]
    c = make_case(*case[:5], dtype=np.float32, window=case[5])
    q, k, v, g = seeded((batch * c.n_nodes, c.width), 51, np.float32, 4)
    want = O.attention_forward(q, k, v, c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, batch)
    grads = O.attention_backward(g, q, k, v, c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, batch)
    _, lat = tables_for(c)
    assert lat.n_edges == c.source.shape[0]
    Q, K, V, G = cuda(q), cuda(k), cuda(v), cuda(g)
    out, lse = lattice_attention_forward(Q, K, V, lat)
    assert_close(out.cpu().numpy(), want, 1e-5, 1e-6 * max(1.0, np.abs(want).max()), "out")
    got = lattice_attention_backward(G, Q, K, V, out, lse, lat)
    for name, a, b in zip(("dq", "dk", "dv"), got, grads):
        assert_close(a.cpu().numpy(), b, 1e-5, 1e-5 * max(1.0, np.abs(b).max()), name)


@pytest.mark.parametrize("case", CASES[:4])
def test_lattice_bf16_storage(case):
    from gm_attention_b200.attention import lattice_attention_backward, lattice_attention_forward

    batch = case[6]
    c = make_case(*case[:5], dtype=np.float32, window=case[5])
    rounded = [torch.from_numpy(x).bfloat16() for x in seeded((batch * c.n_nodes, c.width), 52, np.float32, 4)]
    q, k, v, g = (x.float().numpy() for x in rounded)
    want = O.attention_forward(q, k, v, c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, batch)
    grads = O.attention_backward(g, q, k, v, c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, batch)
    _, lat = tables_for(c)
    Q, K, V, G = (x.cuda() for x in rounded)
    out, lse = lattice_attention_forward(Q, K, V, lat)
    assert rel_err(out.float().cpu().numpy(), want) < 2e-2
    got = lattice_attention_backward(G, Q, K, V, out, lse, lat)
    for name, a, b in zip(("dq", "dk", "dv"), got, grads):
        assert rel_err(a.float().cpu().numpy(), b) < 2e-2, name


def test_lattice_agrees_with_the_general_kernels_and_is_deterministic():
    from gm_attention_b200.attention import (attention_backward, attention_forward, lattice_attention_backward,
                                             lattice_attention_forward)

    c = make_case(16, 32, 3 * math.pi / 16, {0: 16, 1: 16, 2: 16}, 4, dtype=np.float32)
    general, lat = tables_for(c)
    Q, K, V, G = (cuda(x) for x in seeded((2 * c.n_nodes, c.width), 53, np.float32, 4))
    out_a, lse_a = attention_forward(Q, K, V, general)
    out_b, lse_b = lattice_attention_forward(Q, K, V, lat)
    assert_close(out_b.cpu().numpy(), out_a.cpu().numpy(), 1e-5, 2e-6, "out")
    assert_close(lse_b.cpu().numpy(), lse_a.cpu().numpy(), 1e-5, 1e-5, "lse")
    first = lattice_attention_backward(G, Q, K, V, out_b, lse_b, lat)
    again = lattice_attention_backward(G, Q, K, V, out_b, lse_b, lat)
    for a, b in zip(first, again):
        assert torch.equal(a, b)  # no atomics: bit-identical reruns
    for name, a, b in zip(("dq", "dk", "dv"), first, attention_backward(G, Q, K, V, out_a, lse_a, general)):
        assert_close(a.cpu().numpy(), b.cpu().numpy(), 1e-5, 1e-5 * max(1.0, float(b.abs().max())), name)


def test_lattice_through_autograd_and_unsupported_layout():
    from gm_attention_b200.attention import GaugeAttention, build_lattice_tables, lattice_layout_supported

    c = make_case(8, 16, 2 * math.pi / 8, {0: 4, 1: 4, 2: 4}, 2, dtype=np.float32)
    _, lat = tables_for(c)
    q, k, v = (cuda(x).requires_grad_(True) for x in seeded((c.n_nodes, c.width), 54, np.float32, 3))
    g, = seeded((c.n_nodes, c.width), 55, np.float32)
    out = GaugeAttention.apply(q, k, v, lat)
    (out * cuda(g)).sum().backward()
    grads = O.attention_backward(g, q.detach().cpu().numpy(), k.detach().cpu().numpy(), v.detach().cpu().numpy(), c.transport, c.bias,
                                 c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, 1)
    for name, a, b in zip(("dq", "dk", "dv"), (q.grad, k.grad, v.grad), grads):
        assert_close(a.cpu().numpy(), b, 1e-5, 1e-5 * max(1.0, np.abs(b).max()), name)
    odd = make_case(6, 12, 2 * math.pi / 6, {1: 3, 3: 2}, 1, dtype=np.float32)
    rows = tuple(tuple(int(x) for x in row) for row in odd.desc)
    assert not lattice_layout_supported(rows)
    assert lattice_layout_supported(lat.desc_rows)


#: headline head layout on a lattice wide enough for the TMA staging path: tiles that wrap the longitude seam and
#: tiles that do not, windows from a few positions (one staged chunk) to whole rows (several chunks)
TMA_CASE = (6, 256, 1.2 * math.pi / 6, {0: 16, 1: 16, 2: 16}, 2, "hard", 2)
TC_CASES = [CASES[0], CASES[1], CASES[2], CASES[3], CASES[4], (8, 16, 2 * math.pi / 8, {1: 6, 2: 6}, 1, "hard", 2), TMA_CASE]


@pytest.fixture(params=["one-head", "four-heads"])
def kernel_family(request, monkeypatch):
    """The two tensor-core kernel families: one head per CTA (default) and all four heads of a tile per CTA (opt-in;
    layouts it does not serve fall through to the first)."""
    from gm_attention_b200 import attention

    monkeypatch.setattr(attention, "FOUR_HEADS", "1" if request.param == "four-heads" else "0")
    return request.param


FOUR_HEAD_CASES = [
    (12, 48, 3 * math.pi / 12, {0: 16, 1: 16, 2: 16}, 4, "hard", 2),      # headline layout: whole-row polar windows, tiles across the seam
    (6, 256, 1.2 * math.pi / 6, {0: 16, 1: 16, 2: 16}, 4, "hard", 2),     # wide windows: several chunks per row pair, tensor copies and seam chunks
    (10, 64, 2 * math.pi / 10, {0: 16, 1: 16}, 4, "quartic", 1),          # one complex frequency, masked pairs inside the windows
    (8, 40, 2 * math.pi / 8, {0: 16, 1: 16, 2: 16, 3: 16}, 4, "hard", 1), # three complex frequencies (20-word entries), the smallest row length served
]


@pytest.mark.parametrize("case", FOUR_HEAD_CASES)
def test_four_head_kernels_match_the_oracle_and_the_one_head_kernels(case, monkeypatch):
    """The persistent four-heads-per-CTA kernels (128-byte rows, producer / consumer warps): forward and both backward
    passes against the oracle (2e-2 of each tensor's magnitude) and against the one-head kernels on the same inputs;
    bit-identical reruns; no wait on a barrier ran out."""
    import ctypes

    from gm_attention_b200 import _lib, attention
    from gm_attention_b200.attention import four_head_layout_supported, lattice_attention_backward, lattice_attention_forward

    batch = case[6]
    c = make_case(*case[:5], dtype=np.float32, window=case[5])
    rounded = [torch.from_numpy(x).bfloat16() for x in seeded((batch * c.n_nodes, c.width), 62, np.float32, 4)]
    q, k, v, g = (x.float().numpy() for x in rounded)
    want = O.attention_forward(q, k, v, c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, batch)
    grads = O.attention_backward(g, q, k, v, c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, batch)
    _, lat = tables_for(c)
    assert four_head_layout_supported(lat, c.width)
    Q, K, V, G = (x.cuda() for x in rounded)
    results = {}
    # the other family: the one-head tensor-core kernels, or the FMA lattice kernels where those have no instantiation
    # (16 copies of three complex frequencies)
    other_tc = attention.tensor_core_layout_supported(lat.desc_rows)
    for family in ("1", "0"):
        monkeypatch.setattr(attention, "FOUR_HEADS", family)
        tc = True if family == "1" else other_tc
        out, lse = lattice_attention_forward(Q, K, V, lat, tensor_cores=tc)
        results[family] = (out, lse, *lattice_attention_backward(G, Q, K, V, out, lse, lat, tensor_cores=tc))
    monkeypatch.setattr(attention, "FOUR_HEADS", "1")
    out, lse = lattice_attention_forward(Q, K, V, lat, tensor_cores=True)
    again = (out, lse, *lattice_attention_backward(G, Q, K, V, out, lse, lat, tensor_cores=True))
    for a, b in zip(results["1"], again):
        assert torch.equal(a, b)
    for name, a, b in zip(("out", "dq", "dk", "dv"), (results["1"][0], *results["1"][2:]), (want, *grads)):
        assert rel_err(a.float().cpu().numpy(), b) < 2e-2, name
    for name, a, b in zip(("out", "lse", "dq", "dk", "dv"), results["1"], results["0"]):
        assert rel_err(a.float().cpu().numpy(), b.float().cpu().numpy()) < 2e-2, name
    expired = ctypes.c_int(-1)
    _lib.call("gm_lattice_attention_tc4_wait_expired", ctypes.byref(expired))
    assert expired.value == 0


@pytest.mark.parametrize("case", TC_CASES)
def test_tensor_core_forward_bf16(case):
    """mma.sync Gram / value tiles against the oracle (2e-2 of the output's magnitude) and against the FMA
    lattice kernel on the same bf16 inputs (they differ only by the bf16 rounding of the attention weights)."""
    from gm_attention_b200.attention import lattice_attention_forward, tensor_core_layout_supported

    batch = case[6]
    c = make_case(*case[:5], dtype=np.float32, window=case[5])
    rounded = [torch.from_numpy(x).bfloat16() for x in seeded((batch * c.n_nodes, c.width), 57, np.float32, 3)]
    q, k, v = (x.float().numpy() for x in rounded)
    want = O.attention_forward(q, k, v, c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, batch)
    _, lat = tables_for(c)
    assert tensor_core_layout_supported(lat.desc_rows)
    Q, K, V = (x.cuda() for x in rounded)
    out_tc, lse_tc = lattice_attention_forward(Q, K, V, lat, tensor_cores=True)
    out_fma, lse_fma = lattice_attention_forward(Q, K, V, lat, tensor_cores=False)
    assert rel_err(out_tc.float().cpu().numpy(), want) < 2e-2
    assert rel_err(out_tc.float().cpu().numpy(), out_fma.float().cpu().numpy()) < 2e-2
    assert_close(lse_tc.cpu().numpy(), lse_fma.cpu().numpy(), 1e-4, 1e-4, "lse")


@pytest.mark.parametrize("case", TC_CASES)
def test_tensor_core_backward_bf16(case):
    """Both backward passes on tensor cores against the oracle (fp32 on the bf16-rounded inputs, 2e-2 of each
    gradient's magnitude); reruns are bit-identical (no atomics)."""
    from gm_attention_b200.attention import lattice_attention_backward, lattice_attention_forward

    batch = case[6]
    c = make_case(*case[:5], dtype=np.float32, window=case[5])
    rounded = [torch.from_numpy(x).bfloat16() for x in seeded((batch * c.n_nodes, c.width), 58, np.float32, 4)]
    q, k, v, g = (x.float().numpy() for x in rounded)
    grads = O.attention_backward(g, q, k, v, c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, batch)
    _, lat = tables_for(c)
    Q, K, V, G = (x.cuda() for x in rounded)
    out, lse = lattice_attention_forward(Q, K, V, lat, tensor_cores=True)
    got = lattice_attention_backward(G, Q, K, V, out, lse, lat, tensor_cores=True)
    again = lattice_attention_backward(G, Q, K, V, out, lse, lat, tensor_cores=True)
    for name, a, b, a2 in zip(("dq", "dk", "dv"), got, grads, again):
        assert rel_err(a.float().cpu().numpy(), b) < 2e-2, name
        assert torch.equal(a, a2), name


def test_tma_staging_equals_per_thread_staging(monkeypatch):
    """The two staging paths of the tensor-core kernels (TMA tensor copies; per-thread cp.async) feed the same
    arithmetic: results are bit-identical, and no wait on a copy barrier ever ran out."""
    import ctypes

    from gm_attention_b200 import _lib
    from gm_attention_b200.attention import lattice_attention_backward, lattice_attention_forward

    batch = TMA_CASE[6]
    c = make_case(*TMA_CASE[:5], dtype=np.float32, window=TMA_CASE[5])
    _, lat = tables_for(c)
    Q, K, V, G = (torch.from_numpy(x).bfloat16().cuda() for x in seeded((batch * c.n_nodes, c.width), 60, np.float32, 4))
    results = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("GM_LATTICE_TMA", mode)
        out, lse = lattice_attention_forward(Q, K, V, lat, tensor_cores=True)
        results[mode] = (out, lse, *lattice_attention_backward(G, Q, K, V, out, lse, lat, tensor_cores=True))
    for a, b in zip(results["1"], results["0"]):
        assert torch.equal(a, b)
    assert torch.isfinite(results["1"][0].float()).all()
    expired = ctypes.c_int(-1)
    _lib.call("gm_lattice_attention_tc_wait_expired", ctypes.byref(expired))
    assert expired.value == 0


def test_host_pipeline_equals_the_device_path():
    """Host-resident fields, sample chunks pipelined over three streams: same numbers as one device-resident call."""
    from gm_attention_b200.attention import HostPipeline, lattice_attention_backward, lattice_attention_forward

    batch = 5
    c = make_case(8, 16, 2 * math.pi / 8, {0: 4, 1: 4, 2: 4}, 2, dtype=np.float32)
    _, lat = tables_for(c)
    host = [torch.from_numpy(x).pin_memory() for x in seeded((batch * c.n_nodes, c.width), 59, np.float32, 4)]
    outs = [torch.empty_like(host[0]).pin_memory() for _ in range(4)]
    pipe = HostPipeline(lat, batch, c.width, torch.float32, torch.device("cuda", 0), chunk=1)
    for _ in range(2):  # the second run reuses the staging buffers
        pipe.run(*host, *outs)
        torch.cuda.synchronize()
    for x in outs:
        x.zero_()
    for _ in range(3):  # enqueue-only calls overlap one another; join before reading
        pipe.run(*host, *outs, wait=False)
    pipe.join()
    torch.cuda.synchronize()
    Q, K, V, G = (x.cuda() for x in host)
    out, lse = lattice_attention_forward(Q, K, V, lat)
    want = (out, *lattice_attention_backward(G, Q, K, V, out, lse, lat))
    for got, ref in zip(outs, want):
        assert torch.equal(got, ref.cpu())


def test_layer_split_around_a_halo_exchange_equals_one_call():
    """The row subsets used to overlap the halo exchange (interior / boundary target rows; halo / owned source rows)
    reproduce the unsplit forward and backward of a rank's band bit for bit (one GPU, no exchange: the band of rank 1
    of 3 with its halo rows filled from the full fields)."""
    import dataclasses

    from gm_attention_b200.attention import AttentionTables, build_lattice_tables, lattice_attention_backward, lattice_attention_forward
    from gm_attention_b200.fields import FieldType
    from gm_attention_b200.geometry import midpoint_lattice
    from gm_attention_b200.nn import fused_attention as fa
    from gm_attention_b200.parallel import BandPlan, band_geometry, overlap_tables

    dev = torch.device("cuda", 0)
    nlat, nlon, heads, batch = 24, 64, 2, 2
    radius = 2.5 * math.pi / nlat
    attn = FieldType({0: 16, 1: 16, 2: 16})
    full = attn.scaled(heads)
    lattice = midpoint_lattice(nlat, nlon, dev)
    plan = BandPlan(nlat, nlon, lattice.band(radius), (0, 7, 16, 24))
    rank = 1
    elo, ehi = plan.extended(rank)
    edges = band_geometry(lattice, plan, rank, radius, max_frequency=2, dtype=torch.float32)
    geo = fa.geometry(edges, radius, "hard", torch.float32)
    p = fa._plan(type("Layer", (), {})(), attn, full, heads)
    gen = AttentionTables(geo.transport, geo.bias, geo.inside, geo.row_ptr, geo.source, p.rows, heads, 1 / math.sqrt(attn.dimension))
    t = build_lattice_tables(gen, ehi - elo, nlon, p.rows, heads, gen.scale)
    split = overlap_tables(t, plan, rank)
    assert split.interior.row_order.numel() > 0 and split.boundary.row_order.numel() > 0
    assert split.interior.row_order.numel() + split.boundary.row_order.numel() == t.row_order.numel()
    assert split.halo_sources.t_row_order.numel() + split.owned_sources.t_row_order.numel() == t.t_row_order.numel()
    n = batch * (ehi - elo) * nlon
    Q, K, V, G = (torch.from_numpy(x).bfloat16().to(dev) for x in seeded((n, full.dimension), 61, np.float32, 4))
    out, lse = lattice_attention_forward(Q, K, V, t)
    want = (out, lse, *lattice_attention_backward(G, Q, K, V, out, lse, t))
    out2, lse2 = lattice_attention_forward(Q, K, V, split.interior)
    lattice_attention_forward(Q, K, V, split.boundary, out=out2, lse=lse2)
    ws = (torch.zeros_like(Q), torch.zeros_like(Q), torch.zeros_like(Q), torch.empty((n, heads), dtype=torch.float32, device=dev))
    lattice_attention_backward(G, Q, K, V, out2, lse2, split.full, passes=3, workspace=ws)
    lattice_attention_backward(G, Q, K, V, out2, lse2, split.halo_sources, passes=4, workspace=ws)
    lattice_attention_backward(G, Q, K, V, out2, lse2, split.owned_sources, passes=4, workspace=ws)
    for a, b in zip(want, (out2, lse2, *ws[:3])):
        assert torch.equal(a, b)
