"""Expert-parallel dispatch/combine bookkeeping on CPU: world size 2 over gloo, with a stand-in
expert function (no GPU, no oracle): expert e maps x to x * (e + 1)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from moe4all_b200.ep import ExpertParallel

E, K, NE = 8, 3, 16


def fake_route(x):
    # deterministic, rank-dependent, distinct experts per row
    R = x.shape[0]
    base = (x[:, 0].abs() * 1000).to(torch.int64)
    ids = torch.stack([(base + 3 * s) % E for s in range(K)], 1).to(torch.int32)
    wts = torch.softmax(x[:, 1:1 + K], 1)
    return ids, wts


def make_band_fn(rank, e_local):
    lo = rank * e_local

    def fn(x_rows, ids, wts):
        ids = ids.to(torch.int64)
        mine = ((ids >= lo) & (ids < lo + e_local)).to(torch.float32)
        coef = ((ids.to(torch.float32) + 1) * wts * mine).sum(1, keepdim=True)
        return x_rows * coef
    return fn


def finish(moe, x):
    return moe


def expected(x):
    ids, wts = fake_route(x)
    return (x[:, None, :] * (ids.to(torch.float32) + 1)[..., None] * wts[..., None]).sum(1)


def worker(rank, world, port, rows_per_rank, fail_rank, ret, static=False):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(100 + rank)
        x = torch.randn(rows_per_rank[rank], NE)
        ep = ExpertParallel(E, K, fake_route, make_band_fn(rank, E // world), finish)
        if fail_rank == rank:
            # a rank whose expert function returns the wrong number of rows must raise, not hang
            ep.band_fn = lambda xr, i, w: xr[:-1] if xr.shape[0] else xr.new_zeros(1, xr.shape[1])
        try:
            out = ep.forward(x, rows_equal=static)
            ok = torch.allclose(out, expected(x), rtol=1e-5, atol=1e-6)
            ret[rank] = "ok" if ok else "mismatch"
        except RuntimeError as e:
            ret[rank] = "raised: " + str(e)[:60]
    finally:
        dist.destroy_process_group()


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run(world, rows_per_rank, fail_rank=-1, static=False):
    ret = mp.Manager().dict()
    mp.spawn(worker, args=(world, free_port(), rows_per_rank, fail_rank, ret, static), nprocs=world, join=True)
    return dict(ret)


def test_ep_world2_matches_direct_sum():
    assert run(2, [37, 5]) == {0: "ok", 1: "ok"}


def test_ep_world2_fixed_shape_exchange():
    # equal rows on every rank: every row goes to every rank, foreign pairs carry negative ids
    assert run(2, [19, 19], static=True) == {0: "ok", 1: "ok"}


def test_ep_world2_with_an_empty_rank():
    # a rank with no tokens still serves its experts
    assert run(2, [0, 23]) == {0: "ok", 1: "ok"}


def test_ep_world1_identity():
    # world 1 is the identity lowering (crates/infr-vulkan/src/adapter.rs:27494-27701)
    torch.manual_seed(3)
    x = torch.randn(11, NE)
    ep = ExpertParallel(E, K, fake_route, make_band_fn(0, E), finish)
    assert torch.allclose(ep.forward(x), expected(x), rtol=1e-5, atol=1e-6)


def test_expert_count_must_divide(monkeypatch):
    # crates/infr-vulkan/src/ep.rs:171-176: n_expert % world == 0 or the split is refused
    monkeypatch.setattr(dist, "is_initialized", lambda: True)
    monkeypatch.setattr(dist, "get_world_size", lambda group=None: 2)
    monkeypatch.setattr(dist, "get_rank", lambda group=None: 0)
    with pytest.raises(ValueError):
        ExpertParallel(7, 2, fake_route, make_band_fn(0, 3), finish)


def test_bad_expert_fn_raises_on_the_host():
    r = run(2, [9, 9], fail_rank=1)
    assert r[1].startswith("raised"), r
