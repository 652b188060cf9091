"""World-size-2 gloo test of the data-parallel host logic (no GPU): batch-divisor / noise-share
bookkeeping and the bucketed SUM/mean gradient reducer."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, overlap, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flashdp4review_b200.distributed import DPGradReducer, init_data_parallel
        from flashdp4review_b200.layers._common import dp_scalars
        from flashdp4review_b200.layers.utils import DPParameter

        assert init_data_parallel() == (rank, world)
        div, noise = dp_scalars(local_batch=8, noise_multiplier=2.0, param_id=7, step=3)
        assert div == 8 * world
        assert abs(noise.std - 2.0 / (8 * world) ** 0.5) < 1e-12
        assert (noise.rank, noise.world, noise.param_id, noise.step) == (rank, world, 7, 3)

        torch.manual_seed(0)
        model = nn.Sequential(nn.Linear(6, 5), nn.Linear(5, 3))
        model[0].weight = DPParameter(model[0].weight.data)       # DP tensor: SUM
        model[0].bias = DPParameter(model[0].bias.data)
        red = DPGradReducer(model, bucket_bytes=64, overlap=overlap)
        assert len(red.buckets) >= 2
        for step in range(2):
            model.zero_grad()
            x = torch.full((4, 6), float(rank + 1 + step))
            model(x).sum().backward()
            local = [p.grad.clone() for p in model.parameters()]
            red.finish()
            gathered = [[torch.zeros_like(g) for _ in range(world)] for g in local]
            for g, lst in zip(local, gathered):
                dist.all_gather(lst, g)
            for p, lst in zip(model.parameters(), gathered):
                want = sum(lst) if getattr(p, "requires_dp", False) else sum(lst) / world
                assert torch.allclose(p.grad, want, rtol=1e-6, atol=1e-6)
        red.remove()
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("overlap", [True, False])
def test_reducer_and_dp_bookkeeping_world2(overlap):
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, overlap, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=120)
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        assert dict(results) == {0: "ok", 1: "ok"}


def test_set_data_parallel_validation():
    from flashdp4review_b200 import runtime
    with pytest.raises(ValueError):
        runtime.set_data_parallel(2, 2)
    with pytest.raises(ValueError):
        runtime.set_data_parallel(0, 0)
    runtime.set_data_parallel(0, 1)
