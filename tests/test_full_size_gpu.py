"""Parity at the sizes the benchmark configurations name, not at scaled-down lattices.

* 32 x 64, radius 2 pi / 32, batch 2, 2 heads of 4 x (m = 0, 1, 2), float32 (136 192 edges): WHOLE problem
  against the reference's compiled CPU driver (scores + softmax op) and the C oracle (fused layer), on the
  general CSR kernels, the FMA lattice kernels and -- bf16 storage -- the tensor-core lattice kernels.
* 128 x 256, radius 3 pi / 128, batch 4, 4 heads of 8 x (m = 0..3) (D = 224) and 256 x 512, radius 3 pi / 256,
  batch 8, 4 heads of 16 x (m = 0, 1, 2) (D = 320): the whole layer is minutes of CPU oracle work, so the
  oracle runs on SAMPLED targets and sources (``oracle/sampled.py``: rows next to the pole with whole-row
  windows, rows 3, 6 and 8, the equator, both columns at the longitude seam; complete rows, exact) of one
  sample of the batch, float32 and bf16 storage.  The GPU side is the package's own chain at full size:
  geometry built on the device, per-edge constants, compact lattice tables, kernels over the whole batch.

Tolerances: float32 1e-5 relative / 1e-6 absolute for outputs; gradients sum hundreds to thousands of
terms of both signs, so their absolute part is 1e-5 of the tensor's largest magnitude.  bf16 storage:
2e-2 of the tensor's largest magnitude, against the oracle in float32 on the bf16-rounded inputs.
"""

from __future__ import annotations

import math
from functools import lru_cache

import numpy as np
import pytest
import torch

from oracle import geometry_np as G
from oracle import oracle as O
from oracle import sampled as S

from tests.helpers import assert_close, cuda, descriptor_rows, make_case, rel_err, seeded

pytestmark = pytest.mark.gpu

SMALL = (32, 64, 2 * math.pi / 32, {0: 4, 1: 4, 2: 4}, 2)  # whole problem, batch 2
SAMPLED = {
    "128x256": dict(nlat=128, nlon=256, radius_rows=3, head_type={0: 8, 1: 8, 2: 8, 3: 8}, heads=4, batch=4),
    "256x512": dict(nlat=256, nlon=512, radius_rows=3, head_type={0: 16, 1: 16, 2: 16}, heads=4, batch=8),
}


def magnitude(a) -> float:
    return max(float(np.abs(a).max()), 1.0)


# ----------------------------------------------------------------------------- 32 x 64: the whole problem

def test_scores_softmax_op_32x64(reference_modules):
    from gm_attention_b200.nn import fused_attention as fa

    ext = fa.extension(True)
    c = make_case(*SMALL, dtype=np.float32)
    assert c.source.shape[0] == 68096 and c.max_degree == 129
    batch = 2  # the reference's batch is the tiled disjoint-union graph: run the op per sample, as its drivers would on a tiled table
    t = torch.from_numpy
    ref = reference_modules["gm_fused_attention_cpu"]
    tables_h = (t(c.transport), t(c.bias), t(c.inside), t(c.desc), t(c.row_ptr), t(c.source))
    tables_d = [cuda(x) for x in (c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source)]
    for b in range(batch):
        q, k = seeded((c.n_nodes, c.width), 70 + b, np.float32, 2)
        da, = seeded((c.source.shape[0], c.heads), 80 + b, np.float32)
        alpha_ref = ref.softmax_forward(t(q), t(k), *tables_h, c.heads, c.scale, c.max_degree)
        dq_ref, dk_ref = ref.softmax_backward(t(da), t(q), t(k), *tables_h, alpha_ref, c.heads, c.scale, c.max_degree)
        alpha = ext.softmax_forward(cuda(q), cuda(k), *tables_d, c.heads, c.scale, c.max_degree)
        assert_close(alpha.cpu().numpy(), alpha_ref.numpy(), 1e-5, 1e-6, "alpha")
        dq, dk = ext.softmax_backward(cuda(da), cuda(q), cuda(k), *tables_d, alpha_ref.cuda(), c.heads, c.scale, c.max_degree)
        assert_close(dq.cpu().numpy(), dq_ref.numpy(), 1e-5, 1e-5 * magnitude(dq_ref.numpy()), "dq")
        assert_close(dk.cpu().numpy(), dk_ref.numpy(), 1e-5, 1e-5 * magnitude(dk_ref.numpy()), "dk")


@pytest.mark.parametrize("path", ["csr", "lattice_fma", "lattice_tc_bf16"])
def test_fused_layer_32x64(path):
    from gm_attention_b200.attention import (AttentionTables, attention_backward, attention_forward, build_lattice_tables,
                                             lattice_attention_backward, lattice_attention_forward)

    batch = 2
    c = make_case(*SMALL, dtype=np.float32)
    fields = seeded((batch * c.n_nodes, c.width), 71, np.float32, 4)
    bf16 = path == "lattice_tc_bf16"
    if bf16:
        rounded = [torch.from_numpy(x).bfloat16() for x in fields]
        fields = [x.float().numpy() for x in rounded]
        dev = [x.cuda() for x in rounded]
    else:
        dev = [cuda(x) for x in fields]
    q, k, v, g = fields
    want = O.attention_forward(q, k, v, c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, batch)
    grads = O.attention_backward(g, q, k, v, c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, c.heads, c.scale, batch)
    rows = tuple(tuple(int(x) for x in row) for row in c.desc)
    general = AttentionTables(cuda(c.transport), cuda(c.bias), cuda(c.inside), cuda(c.row_ptr), cuda(c.source), rows, c.heads, c.scale)
    Q, K, V, Gd = dev
    if path == "csr":
        out, lse = attention_forward(Q, K, V, general)
        got = attention_backward(Gd, Q, K, V, out, lse, general)
    else:
        lat = build_lattice_tables(general, c.nlat, c.nlon, rows, c.heads, c.scale)
        out, lse = lattice_attention_forward(Q, K, V, lat, tensor_cores=bf16)
        got = lattice_attention_backward(Gd, Q, K, V, out, lse, lat, tensor_cores=bf16)
    if bf16:
        assert rel_err(out.float().cpu().numpy(), want) < 2e-2
        for name, a, b in zip(("dq", "dk", "dv"), got, grads):
            assert rel_err(a.float().cpu().numpy(), b) < 2e-2, name
    else:
        assert_close(out.cpu().numpy(), want, 1e-5, 1e-6 * magnitude(want), "out")
        for name, a, b in zip(("dq", "dk", "dv"), got, grads):
            assert_close(a.cpu().numpy(), b, 1e-5, 1e-5 * magnitude(b), name)


# ----------------------------------------------------------------------------- 128 x 256 and 256 x 512: sampled targets

@lru_cache(maxsize=2)
def device_problem(name: str):
    """The package's own chain at full size: device geometry -> per-edge constants -> general and lattice tables."""
    from gm_attention_b200.attention import AttentionTables, build_lattice_tables
    from gm_attention_b200.fields import FieldType
    from gm_attention_b200.geometry import compute_edge_geometry, midpoint_lattice
    from gm_attention_b200.nn import fused_attention as fa

    cfg = SAMPLED[name]
    dev = torch.device("cuda", 0)
    radius = cfg["radius_rows"] * math.pi / cfg["nlat"]
    attn = FieldType(cfg["head_type"])
    lattice = midpoint_lattice(cfg["nlat"], cfg["nlon"], dev)
    edges = compute_edge_geometry(lattice, lattice.frames, radius, max_frequency=max(cfg["head_type"]), dtype=torch.float32)
    geo = fa.geometry(edges, radius, "hard", torch.float32)
    plan = fa._plan(type("Layer", (), {})(), attn, attn.scaled(cfg["heads"]), cfg["heads"])
    general = AttentionTables(geo.transport, geo.bias, geo.inside, geo.row_ptr, geo.source, plan.rows, cfg["heads"], 1.0 / math.sqrt(attn.dimension))
    lat = build_lattice_tables(general, cfg["nlat"], cfg["nlon"], plan.rows, cfg["heads"], general.scale)
    return general, lat, plan.width


@lru_cache(maxsize=2)
def oracle_sample(name: str) -> S.Sample:
    cfg = SAMPLED[name]
    targets, sources = S.default_sample_nodes(cfg["nlat"], cfg["nlon"])
    return S.sample_problem(G.midpoint_lattice(cfg["nlat"], cfg["nlon"]), cfg["radius_rows"] * math.pi / cfg["nlat"], targets, sources,
                            max(cfg["head_type"]), np.float32)


def sampled_check(name: str, dtype: torch.dtype, path: str) -> dict[str, float]:
    from gm_attention_b200.attention import (attention_backward, attention_forward, lattice_attention_backward,
                                             lattice_attention_forward)
    from gm_attention_b200.fields import FieldType

    cfg = SAMPLED[name]
    general, lat, width = device_problem(name)
    n1, batch = cfg["nlat"] * cfg["nlon"], cfg["batch"]
    gen = torch.Generator(device="cuda").manual_seed(90)
    Q, K, V, Gd = (torch.randn(batch * n1, width, generator=gen, device="cuda", dtype=torch.float32).to(dtype) for _ in range(4))
    if path == "csr":
        out, lse = attention_forward(Q, K, V, general)
        dq, dk, dv = attention_backward(Gd, Q, K, V, out, lse, general)
    else:
        out, lse = lattice_attention_forward(Q, K, V, lat)
        dq, dk, dv = lattice_attention_backward(Gd, Q, K, V, out, lse, lat)
    sample = oracle_sample(name)
    b = batch - 1  # the last sample: the batch stride is exercised
    rows = lambda x, nodes: x[torch.from_numpy(b * n1 + nodes).cuda()].float().cpu().numpy()
    want = S.run(sample, lambda nodes: tuple(rows(x, nodes) for x in (Q, K, V, Gd)), descriptor_rows(FieldType(cfg["head_type"]), cfg["heads"]),
                 cfg["heads"], general.scale)
    got = {"out": rows(out, sample.targets), "dq": rows(dq, sample.targets), "dk": rows(dk, sample.sources), "dv": rows(dv, sample.sources)}
    worst = {}
    for name_, w in want.items():
        if dtype == torch.bfloat16:
            worst[name_] = rel_err(got[name_], w)
            assert worst[name_] < 2e-2, (name_, worst[name_])
        else:
            assert_close(got[name_], w, 1e-5, (1e-6 if name_ == "out" else 1e-5) * magnitude(w), name_)
    return worst


@pytest.mark.parametrize("name", list(SAMPLED))
def test_sampled_targets_float32_lattice(name):
    sampled_check(name, torch.float32, "lattice")


@pytest.mark.parametrize("name", list(SAMPLED))
def test_sampled_targets_bf16_tensor_cores(name):
    sampled_check(name, torch.bfloat16, "lattice")


def test_sampled_targets_bf16_four_head_kernels_256x512(monkeypatch):
    """The opt-in four-heads-per-CTA kernels at the headline size."""
    from gm_attention_b200 import attention

    monkeypatch.setattr(attention, "FOUR_HEADS", "1")
    sampled_check("256x512", torch.bfloat16, "lattice")


def test_sampled_targets_float32_general_kernels_128x256():
    sampled_check("128x256", torch.float32, "csr")
