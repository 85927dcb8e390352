"""GPU: expert-parallel layer (all-to-all dispatch/combine over NCCL) against the single-device
result - the reference's own EP check is world-1 vs world-N identity
(crates/infr-vulkan/src/adapter.rs:27494-27701).  Runs at world size 2 when the box has two GPUs,
else at world size 1 (identity lowering)."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

NE, E, K, NFF, ROWS = 512, 16, 4, 256, 48


def worker(rank, world, port, ret):
    import torch.distributed as dist
    from moe4all_b200 import CudaBackend, MoeFfn
    from moe4all_b200.devgen import DeviceLayer
    from moe4all_b200.ep import CudaExpertParallelLayer

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dev = f"cuda:{rank}"
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(dev))
    try:
        be = CudaBackend(rank)
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            el = E // world
            banded = DeviceLayer(be, 7, NE, E, NFF, sh_ff=NFF, device=dev, router_std=0.05, band=(rank * el, el))
            full = DeviceLayer(be, 7, NE, E, NFF, sh_ff=NFF, device=dev, router_std=0.05)
            gen = torch.Generator(device=dev)
            gen.manual_seed(5)
            x_all = torch.randn(world * ROWS, NE, generator=gen, device=dev)  # same on every rank
            x = x_all[rank * ROWS:(rank + 1) * ROWS].contiguous()
            layer = CudaExpertParallelLayer(be, banded, E, K, NFF, NE)
            out = layer.forward(x)
            out_static = layer.forward(x, rows_equal=True)  # fixed-shape exchange (world > 1), same sums
            # single-device result for the same rows
            dst = torch.empty_like(x)
            b = full.b
            be.moe_ffn(MoeFfn(x=be.wrap_tensor(x), router=b["router"], gate_exps=b["gate"], up_exps=b["up"], down_exps=b["down"],
                              dst=be.wrap_tensor(dst), rows=ROWS, ne=NE, n_expert=E, n_used=K, n_ff_exp=NFF, sh_gate=b["sh_gate"],
                              sh_up=b["sh_up"], sh_down=b["sh_down"], sh_gate_inp=b["sh_gate_inp"], sh_ff=NFF, path=2))
            be.sync()
            torch.cuda.synchronize()
            ref = dst.cpu().numpy()
            got = out.cpu().numpy()
            rel = float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-3))
            rel = max(rel, float(np.abs(out_static.cpu().numpy() - ref).max() / max(np.abs(ref).max(), 1e-3)))
            ret[rank] = (rel, float(np.abs(ref).max()))
    finally:
        if world > 1:
            dist.destroy_process_group()


def test_ep_matches_single_device():
    import torch.multiprocessing as mp

    world = 2 if torch.cuda.device_count() >= 2 else 1
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    if world == 1:
        ret = {}
        worker(0, 1, port, ret)
    else:
        ret = mp.Manager().dict()
        mp.spawn(worker, args=(world, port, ret), nprocs=world, join=True)
        ret = dict(ret)
    assert len(ret) == world
    for rank, (rel, mag) in ret.items():
        assert mag > 0
        assert rel < 1e-4, f"rank {rank}: expert-parallel result differs from single device by {rel:.2e}"
