"""Latitude-band sharding on real GPUs (NCCL, one process per GPU): the sharded fused layer with halo exchange
against the unsharded layer on one GPU.  Needs at least two GPUs; skipped otherwise."""

from __future__ import annotations

import math
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank: int, world: int, port: int, out_dir: str, kind: str) -> None:
    """One rank.  A failure is written to ``fail<rank>`` and the process leaves at once, WITHOUT the collective tear-down:
    the other ranks may be inside a collective waiting for this one, and the parent ends them."""
    import traceback

    try:
        _rank_body(rank, world, port, out_dir, kind)
    except BaseException:  # noqa: BLE001
        with open(os.path.join(out_dir, f"fail{rank}"), "w") as f:
            f.write(traceback.format_exc())
        os._exit(1)


def _rank_body(rank: int, world: int, port: int, out_dir: str, kind: str) -> None:
    import torch.distributed as dist

    from gm_attention_b200.attention import AttentionTables, build_lattice_tables, lattice_attention_backward, lattice_attention_forward
    from gm_attention_b200.fields import FieldType
    from gm_attention_b200.geometry import compute_edge_geometry, midpoint_lattice
    from gm_attention_b200.nn import fused_attention as fa
    from gm_attention_b200.parallel import BandPlan, HaloExchanger, NativeHaloExchanger, PeerHaloExchanger, band_geometry, row_degrees

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    nlat, nlon, batch, heads = 24, 48, 2, 4
    radius = 3 * math.pi / nlat
    attn = FieldType({0: 16, 1: 16, 2: 16})
    full = attn.scaled(heads)
    D = full.dimension
    owner = type("Layer", (), {})()
    rows = fa._plan(owner, attn, full, heads).rows
    scale = 1.0 / math.sqrt(attn.dimension)
    lattice = midpoint_lattice(nlat, nlon, device)
    plan = BandPlan.balanced(nlat, nlon, lattice.band(radius), row_degrees(lattice, radius), world)
    lo, hi = plan.owned(rank)
    elo, ehi = plan.extended(rank)

    def tables_of(edges, n_rows):
        g = fa.geometry(edges, radius, "hard", torch.float32)
        general = AttentionTables(g.transport, g.bias, g.inside, g.row_ptr, g.source, rows, heads, scale)
        return build_lattice_tables(general, n_rows, nlon, rows, heads, scale)

    local = tables_of(band_geometry(lattice, plan, rank, radius, max_frequency=2), ehi - elo)
    gen = torch.Generator().manual_seed(7)
    fields = [torch.randn(batch, nlat, nlon, D, generator=gen).to(device) for _ in range(4)]  # same on every rank
    q, k, v, g = (f[:, elo:ehi].contiguous() for f in fields)
    k[:, : lo - elo] = float("nan"); k[:, hi - elo:] = float("nan")  # halos must come from the owners
    v[:, : lo - elo] = float("nan"); v[:, hi - elo:] = float("nan")
    # the library's own copy kernels into the neighbour's mapped buffer, its NCCL groups, or torch.distributed point-to-point
    halo = {"peer-memory": lambda: PeerHaloExchanger(plan, rank, device), "library-nccl": lambda: NativeHaloExchanger(plan, rank, device),
            "torch-distributed": lambda: HaloExchanger(plan, rank)}[kind]()
    try:
        halo.fill_halos(k, v)
    except RuntimeError as exc:
        if kind == "peer-memory" and "not available on this machine" in str(exc):  # every rank raises together
            open(os.path.join(out_dir, f"skip{rank}"), "w").close()
            dist.destroy_process_group()
            return
        raise
    flat = lambda t: t.reshape(-1, D)
    out, lse = lattice_attention_forward(flat(q), flat(k), flat(v), local, tensor_cores=False)
    dq, dk, dv = lattice_attention_backward(flat(g), flat(q), flat(k), flat(v), out, lse, local, tensor_cores=False)
    shape = (batch, ehi - elo, nlon, D)
    dk, dv = dk.view(shape), dv.view(shape)
    halo.reduce_halos(dk, dv)
    # unsharded on this GPU
    whole = tables_of(compute_edge_geometry(lattice, lattice.frames, radius, max_frequency=2, dtype=torch.float32), nlat)
    Q, K, V, G = (flat(f.contiguous()) for f in fields)
    want_out, want_lse = lattice_attention_forward(Q, K, V, whole, tensor_cores=False)
    want = [want_out, *lattice_attention_backward(G, Q, K, V, want_out, want_lse, whole, tensor_cores=False)]
    own = slice(lo - elo, hi - elo)
    for name, got, ref in zip(("out", "dq", "dk", "dv"), (out.view(shape), dq.view(shape), dk, dv), want):
        ref = ref.view(batch, nlat, nlon, D)[:, lo:hi]
        err = float((got[:, own] - ref).abs().max() / ref.abs().max().clamp_min(1.0))
        assert err < 1e-5, f"rank {rank} {name}: {err}"
    # bf16 node fields on the tensor-core kernels: the layer run AROUND the exchange (interior rows while the halos
    # travel, own source rows while the halo sums travel) equals the plain exchange-compute-exchange order bit for
    # bit, and both agree with the unsharded layer to bf16 accuracy
    from gm_attention_b200.parallel import overlap_tables

    qb, kb, vb, gb = (f[:, elo:ehi].contiguous().bfloat16() for f in fields)
    if kind == "peer-memory":  # its buffers are sized for one field shape and dtype: a second exchanger for the bf16 fields
        halo32, halo = halo, PeerHaloExchanger(plan, rank, device)
    halo.fill_halos(kb, vb)
    o1, l1 = lattice_attention_forward(flat(qb), flat(kb), flat(vb), local)
    g1 = lattice_attention_backward(flat(gb), flat(qb), flat(kb), flat(vb), o1, l1, local)
    halo.reduce_halos(g1[1].view(shape), g1[2].view(shape))
    split = overlap_tables(local, plan, rank)
    kb2, vb2 = kb.clone(), vb.clone()
    kb2[:, : lo - elo] = 0; kb2[:, hi - elo:] = 0
    vb2[:, : lo - elo] = 0; vb2[:, hi - elo:] = 0
    pending = halo.start_fill(kb2, vb2)
    o2, l2 = lattice_attention_forward(flat(qb), flat(kb2), flat(vb2), split.interior)
    halo.finish_fill(pending)
    lattice_attention_forward(flat(qb), flat(kb2), flat(vb2), split.boundary, out=o2, lse=l2)
    ws = (torch.zeros_like(flat(qb)), torch.zeros_like(flat(qb)), torch.zeros_like(flat(qb)),
          torch.empty((flat(qb).shape[0], heads), dtype=torch.float32, device=device))
    lattice_attention_backward(flat(gb), flat(qb), flat(kb2), flat(vb2), o2, l2, split.full, passes=3, workspace=ws)
    lattice_attention_backward(flat(gb), flat(qb), flat(kb2), flat(vb2), o2, l2, split.halo_sources, passes=4, workspace=ws)
    pending = halo.start_reduce(ws[1].view(shape), ws[2].view(shape))
    lattice_attention_backward(flat(gb), flat(qb), flat(kb2), flat(vb2), o2, l2, split.owned_sources, passes=4, workspace=ws)
    halo.finish_reduce(pending)
    for name, x, y in zip(("out", "dq", "dk", "dv"), (o1, *g1), (o2, *ws[:3])):
        assert torch.equal(x.view(shape)[:, own], y.view(shape)[:, own]), f"rank {rank} overlapped {name}"
    for name, got, ref in zip(("out", "dq", "dk", "dv"), (o2, *ws[:3]), want):
        ref = ref.view(batch, nlat, nlon, D)[:, lo:hi]
        err = float((got.view(shape)[:, own].float() - ref).abs().max() / ref.abs().max().clamp_min(1.0))
        assert err < 2e-2, f"rank {rank} bf16 {name}: {err}"
    if kind == "peer-memory":
        assert halo.error() == 0 and halo32.error() == 0
    open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    for exchanger in (halo, locals().get("halo32")):
        if exchanger is not None and hasattr(exchanger, "close"):
            exchanger.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("kind", ["peer-memory", "library-nccl", "torch-distributed"])
def test_sharded_layer_on_gpus(tmp_path, kind):
    import torch.multiprocessing as mp

    import time

    world = min(torch.cuda.device_count(), 4)
    context = mp.spawn(_rank, args=(world, _free_port(), str(tmp_path), kind), nprocs=world, join=False)
    deadline = time.monotonic() + 180  # a rank that failed leaves the others inside a collective: end them, do not wait
    try:
        while not context.join(timeout=2):
            failed = [f for f in os.listdir(tmp_path) if f.startswith("fail")]
            if failed or time.monotonic() > deadline:
                break
    except Exception:  # noqa: BLE001  (a rank's exit code: the fail file below says why)
        pass
    for process in context.processes:
        if process.is_alive():
            process.terminate()
    for process in context.processes:
        process.join(10)
    failures = {f: open(os.path.join(tmp_path, f)).read() for f in sorted(os.listdir(tmp_path)) if f.startswith("fail")}
    assert not failures, "\n".join(f"{name}:\n{text}" for name, text in failures.items())
    made = sorted(os.listdir(tmp_path))
    if made == [f"skip{r}" for r in range(world)]:
        pytest.skip("these GPUs cannot map each other's memory")
    assert made == [f"ok{r}" for r in range(world)]


def test_peer_protocol_on_one_gpu():
    """The send / landing kernels of the peer-memory exchange with the "neighbour's" block being this process's own: every
    kernel finds its flag already raised by the kernel before it on the stream, so nothing ever waits on a concurrent
    kernel.  Three steps of copy and of add, bf16 and float32; the flags must carry the step, or the landing would run
    out of patience and report it."""
    import ctypes

    from gm_attention_b200 import _lib

    device = torch.device("cuda", 0)
    batch, rows, nlon, width, r0, r1 = 3, 10, 8, 40, 2, 5
    for dtype in (torch.bfloat16, torch.float32):
        elem = torch.empty((), dtype=dtype).element_size()
        row_bytes = nlon * width * elem
        slab, sample = (r1 - r0) * row_bytes, rows * row_bytes
        buffer_bytes = 2 * batch * slab
        block, handle = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
        _lib.call("gm_peer_alloc", buffer_bytes + 4 * 128, ctypes.byref(block), ctypes.addressof(handle))
        words = [block.value + buffer_bytes + 128 * i for i in range(4)]  # data flag, acknowledgement, send ticket, land ticket
        try:
            gen = torch.Generator(device="cuda").manual_seed(3)
            for step in (1, 2, 3):
                src = [torch.randn(batch, rows, nlon, width, generator=gen, device=device).to(dtype) for _ in range(2)]
                dst = [torch.randn(batch, rows, nlon, width, generator=gen, device=device).to(dtype) for _ in range(2)]
                before = [d.clone() for d in dst]
                pointers = lambda fields: (ctypes.c_void_p * 2)(*[f.data_ptr() + r0 * row_bytes for f in fields])
                stream = torch.cuda.current_stream(device).cuda_stream
                add = step == 2
                _lib.call("gm_peer_send", pointers(src), 2, batch, slab, sample, block.value, words[1], words[2], words[0], step, stream)
                _lib.call("gm_peer_land", pointers(dst), 2, batch, slab, sample, block.value, int(add), _lib.dtype_code(dtype), words[0], words[3],
                          words[1], step, stream)
                torch.cuda.synchronize()
                code = ctypes.c_int(-1)
                _lib.call("gm_peer_error", ctypes.byref(code))
                assert code.value == 0
                for s_, d_, b_ in zip(src, dst, before):
                    want = b_.clone()
                    want[:, r0:r1] = (b_[:, r0:r1].float() + s_[:, r0:r1].float()).to(dtype) if add else s_[:, r0:r1]
                    assert torch.equal(d_, want)
        finally:
            torch.cuda.synchronize()
            _lib.call("gm_peer_free", block)


def test_peer_protocol_two_neighbours_in_one_launch():
    """The two-neighbour form of the send / landing kernels, again with this process's own block standing in for both
    neighbours' (every flag is already raised when its kernel starts): two lanes with different row ranges in one launch."""
    import ctypes

    from gm_attention_b200 import _lib

    device = torch.device("cuda", 0)
    batch, rows, nlon, width = 2, 12, 8, 24
    ranges = [(0, 3), (8, 10)]
    dtype = torch.bfloat16
    row_bytes = nlon * width * 2
    sample = rows * row_bytes
    slabs = [(b - a) * row_bytes for a, b in ranges]
    offsets = [0, 2 * batch * slabs[0]]
    buffers_end = offsets[1] + 2 * batch * slabs[1]
    block, handle = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
    _lib.call("gm_peer_alloc", buffers_end + 8 * 128, ctypes.byref(block), ctypes.addressof(handle))
    word = lambda lane, i: block.value + buffers_end + 128 * (4 * lane + i)  # per lane: data flag, acknowledgement, send / land ticket
    array = lambda kind, values: (kind * len(values))(*values)
    try:
        gen = torch.Generator(device="cuda").manual_seed(4)
        for step in (1, 2):
            src = [torch.randn(batch, rows, nlon, width, generator=gen, device=device).to(dtype) for _ in range(2)]
            dst = [torch.randn(batch, rows, nlon, width, generator=gen, device=device).to(dtype) for _ in range(2)]
            before = [d.clone() for d in dst]
            bases = lambda fields: array(ctypes.c_void_p, [f.data_ptr() + a * row_bytes for a, _ in ranges for f in fields])
            stream = torch.cuda.current_stream(device).cuda_stream
            common = (2, batch, array(ctypes.c_int64, slabs), sample, array(ctypes.c_void_p, [block.value + o for o in offsets]))
            steps = array(ctypes.c_uint32, [step, step])
            _lib.call("gm_peer_send_many", 2, bases(src), *common, array(ctypes.c_void_p, [word(l, 1) for l in range(2)]),
                      array(ctypes.c_void_p, [word(l, 2) for l in range(2)]), array(ctypes.c_void_p, [word(l, 0) for l in range(2)]), steps, stream)
            add = step == 2
            _lib.call("gm_peer_land_many", 2, bases(dst), *common, int(add), _lib.dtype_code(dtype), array(ctypes.c_void_p, [word(l, 0) for l in range(2)]),
                      array(ctypes.c_void_p, [word(l, 3) for l in range(2)]), array(ctypes.c_void_p, [word(l, 1) for l in range(2)]), steps, stream)
            torch.cuda.synchronize()
            code = ctypes.c_int(-1)
            _lib.call("gm_peer_error", ctypes.byref(code))
            assert code.value == 0
            for s_, d_, b_ in zip(src, dst, before):
                want = b_.clone()
                for a, b in ranges:
                    want[:, a:b] = (b_[:, a:b].float() + s_[:, a:b].float()).to(dtype) if add else s_[:, a:b]
                assert torch.equal(d_, want)
    finally:
        torch.cuda.synchronize()
        _lib.call("gm_peer_free", block)
