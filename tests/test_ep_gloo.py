"""Expert-parallel dispatch/combine bookkeeping on CPU: world size 2 over gloo, with a stand-in
expert function (no GPU, no oracle): y = x * (global expert id + 1)."""
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


def make_expert_fn(rank, e_local):
    def fn(xg, seg_off):
        y = torch.empty_like(xg)
        for e in range(e_local):
            a, b = int(seg_off[e]), int(seg_off[e + 1])
            y[a:b] = xg[a:b] * float(rank * e_local + e + 1)
        return y
    return fn


def combine(y_sorted, pos_of_pair, wts, x):
    R = x.shape[0]
    y = y_sorted[pos_of_pair.long()].reshape(R, K, x.shape[1])
    return (y * wts[..., None]).sum(1)


def expected(x):
    ids, wts = fake_route(x)
    return (x[:, None, :] * (ids.to(torch.float32) + 1)[..., None] * wts[..., None]).sum(1)


def worker(rank, world, port, rows_per_rank, fail_rank, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(100 + rank)
        x = torch.randn(rows_per_rank[rank], NE)
        ep = ExpertParallel(E, K, fake_route, make_expert_fn(rank, E // world), combine)
        if fail_rank == rank:
            # a rank whose expert function returns the wrong number of rows must raise, not hang
            ep.expert_fn = lambda xg, seg: xg[:-1] if xg.shape[0] else xg
        try:
            out = ep.forward(x)
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


def run(world, rows_per_rank, fail_rank=-1):
    ret = mp.Manager().dict()
    mp.spawn(worker, args=(world, free_port(), rows_per_rank, fail_rank, ret), nprocs=world, join=True)
    return dict(ret)


def test_ep_world2_matches_direct_sum():
    assert run(2, [37, 5]) == {0: "ok", 1: "ok"}


def test_ep_world2_with_an_empty_rank():
    # a rank with no tokens still serves its experts
    assert run(2, [0, 23]) == {0: "ok", 1: "ok"}


def test_ep_world1_identity():
    # world 1 is the identity lowering (crates/infr-vulkan/src/adapter.rs:27494-27701)
    torch.manual_seed(3)
    x = torch.randn(11, NE)
    ep = ExpertParallel(E, K, fake_route, make_expert_fn(0, E), combine)
    assert torch.allclose(ep.forward(x), expected(x), rtol=1e-5, atol=1e-6)


def test_expert_count_must_divide(monkeypatch):
    # crates/infr-vulkan/src/ep.rs:171-176: n_expert % world == 0 or the split is refused
    monkeypatch.setattr(dist, "is_initialized", lambda: True)
    monkeypatch.setattr(dist, "get_world_size", lambda group=None: 2)
    monkeypatch.setattr(dist, "get_rank", lambda group=None: 0)
    with pytest.raises(ValueError):
        ExpertParallel(7, 2, fake_route, make_expert_fn(0, 3), combine)


def test_bad_expert_fn_raises_on_the_host():
    r = run(2, [9, 9], fail_rank=1)
    assert r[1].startswith("raised"), r
