"""World-size-2 gloo test of the data-parallel host logic (no GPU): batch-divisor / noise-share
bookkeeping and the bucketed SUM/mean gradient reducer."""
import copy
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


def _worker(rank, world, port, overlap, as_view, results):
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
        model = nn.Sequential(nn.Linear(6, 5), nn.Linear(5, 3))      # odd sizes: bucket slices need padding
        model[0].weight = DPParameter(model[0].weight.data)       # DP tensor: SUM
        model[0].bias = DPParameter(model[0].bias.data)
        twin = copy.deepcopy(model)          # same weights, no reducer: yields the local gradients
        red = DPGradReducer(model, bucket_bytes=64, overlap=overlap, grad_as_bucket_view=as_view)
        assert len(red.buckets) >= 2
        for step in range(3):
            if step == 2:
                model.zero_grad(set_to_none=True)     # detaches bucket views; the reducer re-attaches
            else:
                red.zero_grad()
            x = torch.full((4, 6), float(rank + 1 + step))
            model(x).sum().backward()
            twin.zero_grad()
            twin(x).sum().backward()
            local = [p.grad.clone() for p in twin.parameters()]
            red.finish()
            gathered = [[torch.zeros_like(g) for _ in range(world)] for g in local]
            for g, lst in zip(local, gathered):
                dist.all_gather(lst, g)
            for p, lst in zip(model.parameters(), gathered):
                want = sum(lst) if getattr(p, "requires_dp", False) else sum(lst) / world
                assert torch.allclose(p.grad, want, rtol=1e-6, atol=1e-6)
            if as_view:
                assert all(p.grad.data_ptr() == red._views[id(p)].data_ptr() for p in model.parameters())
                assert all(p.grad.data_ptr() % 64 == 0 for p in model.parameters())

        # gradient accumulation: two micro-steps, one collective after the second
        from flashdp4review_b200 import runtime
        red.zero_grad()
        twin.zero_grad()
        for micro in range(2):
            with runtime.accumulate(micro, 2):
                div, noise = dp_scalars(local_batch=8, noise_multiplier=2.0, param_id=7, step=4 + micro)
                assert div == 8 * world * 2
                assert noise.std == (0.0 if micro == 0 else 2.0 / (8 * world * 2) ** 0.5)
                red.set_sync(micro == 1)
                x = torch.full((4, 6), float(rank + 3 + micro))
                model(x).sum().backward()
                twin(x).sum().backward()
                if micro == 0:
                    red.finish()                      # no collective: nothing may change
        local = [p.grad.clone() for p in twin.parameters()]
        red.finish()
        gathered = [[torch.zeros_like(g) for _ in range(world)] for g in local]
        for g, lst in zip(local, gathered):
            dist.all_gather(lst, g)
        for p, lst in zip(model.parameters(), gathered):
            want = sum(lst) if getattr(p, "requires_dp", False) else sum(lst) / world
            assert torch.allclose(p.grad, want, rtol=1e-6, atol=1e-6)
        assert runtime.accumulation() == (0, 1)
        red.remove()
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("overlap,as_view", [(True, False), (False, False), (True, True), (False, True)])
def test_reducer_and_dp_bookkeeping_world2(overlap, as_view):
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, overlap, as_view, results)) for r in range(world)]
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


def test_accumulation_validation():
    from flashdp4review_b200 import runtime
    with pytest.raises(ValueError):
        runtime.set_accumulation(2, 2)
    with pytest.raises(ValueError):
        runtime.set_accumulation(0, 0)
    with runtime.accumulate(1, 4):
        assert runtime.accumulation() == (1, 4)
    assert runtime.accumulation() == (0, 1)
