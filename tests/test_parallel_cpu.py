"""Latitude-band sharding on CPU ranks (gloo, world size 2 and 3): the band
plan, the forward halo exchange, the backward halo reduction, and the whole
sharded layer (oracle kernels standing in for the GPU ones) against the
unsharded oracle."""

from __future__ import annotations

import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gm_attention_b200.parallel import BandPlan, HaloExchanger, balanced_cuts


def test_balanced_cuts_minimise_the_bottleneck():
    cost = [1537, 1459, 1263, 681, 505, 407, 337, 293] + [29] * 240 + [293, 337, 407, 505, 681, 1263, 1459, 1537]
    for parts in (2, 4, 8):
        cuts = balanced_cuts(cost, parts)
        assert cuts[0] == 0 and cuts[-1] == len(cost) and all(b > a for a, b in zip(cuts, cuts[1:]))
        loads = [sum(cost[a:b]) for a, b in zip(cuts, cuts[1:])]
        assert max(loads) <= 1.06 * sum(cost) / parts + max(cost) * (parts == 8)
    with pytest.raises(ValueError):
        balanced_cuts([1, 2], 3)


def test_band_plan_overlaps():
    plan = BandPlan(16, 8, 3, (0, 2, 8, 16))  # a 2-row polar band: rank 2's halo reaches past rank 1
    assert plan.owned(0) == (0, 2) and plan.extended(0) == (0, 5)
    assert plan.needs(0, 1) == (2, 5) and plan.needs(0, 2) is None
    assert plan.needs(1, 0) == (0, 2) and plan.needs(1, 2) == (8, 11)
    assert plan.needs(2, 1) == (5, 8) and plan.needs(2, 0) is None
    wide = BandPlan(16, 8, 3, (0, 1, 2, 16))
    assert wide.needs(2, 0) == (0, 1) and wide.needs(0, 2) == (2, 4)  # halo spans ranks +-1 and +-2


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, cuts: tuple[int, ...], result_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as O
        from tests.helpers import make_case, seeded

        nlat, nlon, heads, batch = 12, 8, 2, 2
        c = make_case(nlat, nlon, 2.4 * math.pi / nlat, {0: 2, 1: 2}, heads, dtype=np.float64)
        D = c.width
        halo = int(np.abs(c.target // nlon - c.source // nlon).max())
        plan = BandPlan(nlat, nlon, halo, cuts)
        lo, hi = plan.owned(rank)
        elo, ehi = plan.extended(rank)
        ex = HaloExchanger(plan, rank)
        q, k, v, g = (x.reshape(batch, nlat, nlon, D) for x in seeded((batch * c.n_nodes, D), 5, np.float64, 4))

        # 1. forward exchange: halo rows arrive bit-exact from their owners
        local = lambda x: torch.from_numpy(np.ascontiguousarray(x[:, elo:ehi])).clone()
        K, V = local(k), local(v)
        K[:, : lo - elo] = float("nan"); K[:, hi - elo:] = float("nan")
        V[:, : lo - elo] = float("nan"); V[:, hi - elo:] = float("nan")
        ex.fill_halos(K, V)
        assert torch.equal(K, local(k)) and torch.equal(V, local(v))

        # 2. the sharded layer: local edges = edges whose target this rank owns, node indices relative to the extended rows
        mine = (c.target // nlon >= lo) & (c.target // nlon < hi)
        rows_ext = ehi - elo
        tgt, src = c.target[mine] - elo * nlon, c.source[mine] - elo * nlon
        assert src.min() >= 0 and src.max() < rows_ext * nlon  # the halo covers every source
        row_ptr = np.zeros(rows_ext * nlon + 1, np.int64)
        np.cumsum(np.bincount(tgt, minlength=rows_ext * nlon), out=row_ptr[1:])
        flat = lambda t: np.ascontiguousarray(t.numpy().reshape(batch * rows_ext * nlon, D))
        Q, G = local(q), local(g)
        args = (c.transport[mine], c.bias[mine], c.inside[mine], c.desc, row_ptr, src, heads, c.scale, batch)
        out = O.attention_forward(flat(Q), flat(K), flat(V), *args).reshape(batch, rows_ext, nlon, D)
        dq, dk, dv = (torch.from_numpy(x.reshape(batch, rows_ext, nlon, D)) for x in O.attention_backward(flat(G), flat(Q), flat(K), flat(V), *args))
        ex.reduce_halos(dk, dv)

        # 3. against the unsharded oracle on the whole sphere
        full = (c.transport, c.bias, c.inside, c.desc, c.row_ptr, c.source, heads, c.scale, batch)
        want = O.attention_forward(q.reshape(-1, D), k.reshape(-1, D), v.reshape(-1, D), *full).reshape(batch, nlat, nlon, D)
        wq, wk, wv = (x.reshape(batch, nlat, nlon, D) for x in O.attention_backward(g.reshape(-1, D), q.reshape(-1, D), k.reshape(-1, D),
                                                                                   v.reshape(-1, D), *full))
        own = slice(lo - elo, hi - elo)
        np.testing.assert_allclose(out[:, own], want[:, lo:hi], rtol=1e-12, atol=1e-13)
        np.testing.assert_allclose(dq.numpy()[:, own], wq[:, lo:hi], rtol=1e-11, atol=1e-12)
        np.testing.assert_allclose(dk.numpy()[:, own], wk[:, lo:hi], rtol=1e-11, atol=1e-12)
        np.testing.assert_allclose(dv.numpy()[:, own], wv[:, lo:hi], rtol=1e-11, atol=1e-12)
        assert float(dk[:, : lo - elo].abs().sum() + dk[:, hi - elo:].abs().sum()) == 0.0  # halo rows handed back and cleared
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cuts", [(0, 6, 12), (0, 2, 12), (0, 1, 3, 12)])
def test_sharded_layer_equals_unsharded(tmp_path, cuts):
    world = len(cuts) - 1
    mp.spawn(_worker, args=(world, _free_port(), cuts, str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == [f"ok{r}" for r in range(world)]


def _silent_peer(rank: int, world: int, port: int, result_dir: str) -> None:
    """Rank 1 never posts its side of the exchange: rank 0's wait runs out and reports it (no hang)."""
    import time

    from gm_attention_b200.parallel import HaloTimeout

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        plan = BandPlan(8, 4, 1, (0, 4, 8))
        field = torch.zeros(1, plan.extended(rank)[1] - plan.extended(rank)[0], 4, 3)
        if rank == 0:
            ex = HaloExchanger(plan, rank, timeout=1.5)
            start = time.monotonic()
            try:
                ex.fill_halos(field)
            except HaloTimeout as exc:
                assert "did not complete" in str(exc) and time.monotonic() - start < 30
                open(os.path.join(result_dir, "timed_out"), "w").close()
        else:
            time.sleep(4.0)  # posts nothing; stays alive until rank 0 has given up
        open(os.path.join(result_dir, f"done{rank}"), "w").close()
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001  (the aborted exchange may have left the group unusable)
            pass


def test_a_peer_that_never_posts_times_out(tmp_path):
    mp.spawn(_silent_peer, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["done0", "done1", "timed_out"]
