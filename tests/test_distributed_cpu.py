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

        from flashdp4review_b200 import runtime as _rt
        _rt.manual_seed(1000 + rank)                  # ranks start with different keys ...
        assert init_data_parallel() == (rank, world)
        seeds = [None] * world
        dist.all_gather_object(seeds, _rt.get_seed())
        assert seeds == [1000] * world                # ... and continue with rank 0's
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


def _leaver(rank, world, port, results):
    """Rank 1 leaves between steps (none of its collectives in flight); rank 0 learns of it through a
    finite process-group timeout on its next collective, not by hanging."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from flashdp4review_b200.distributed import DPGradReducer, init_data_parallel
    init_data_parallel()
    torch.manual_seed(0)
    model = nn.Linear(6, 5)
    red = DPGradReducer(model, overlap=False)
    model(torch.ones(4, 6)).sum().backward()
    red.finish()                                   # step 0: both ranks present
    results[(rank, "step0")] = "ok"
    if rank == 1:
        os._exit(0)                                # gone before step 1, without a goodbye
    red.zero_grad()
    model(torch.ones(4, 6)).sum().backward()
    t0 = time.time()
    try:
        red.finish()
        results[(rank, "step1")] = "no error"
    except Exception as e:                         # gloo: connection closed by peer, or the timeout
        results[(rank, "step1")] = f"{type(e).__name__} after {time.time() - t0:.1f}s"
    os._exit(0)


def test_rank_that_leaves_between_steps_ends_the_next_collective_with_an_error():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_leaver, args=(r, world, port, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=90)
        assert all(not p.is_alive() for p in procs)
        res = dict(results)
    assert res[(0, "step0")] == "ok" and res[(1, "step0")] == "ok"
    assert (0, "step1") in res and res[(0, "step1")] != "no error", res


def test_noise_state_round_trip_never_repeats_a_step():
    """The Philox step word of a layer's k-th backward is base + k; a resumed run restores the seed and
    continues above the highest step the saved run drew with."""
    from flashdp4review_b200 import runtime
    saved_seed, saved = runtime.get_seed(), runtime.noise_state()
    try:
        runtime.manual_seed(5)
        runtime.set_noise_state({"seed": 5, "step": 0})
        first = [runtime.noise_step(k) for k in (1, 2, 3)]
        state = runtime.noise_state()
        assert state == {"seed": 5, "step": max(first)}
        runtime.manual_seed(99)                               # a new process would start like this
        runtime.set_noise_state(state)
        assert runtime.get_seed() == 5
        resumed = [runtime.noise_step(k) for k in (1, 2, 3)]  # fresh layers count from 1 again
        assert min(resumed) > max(first)
        assert runtime.noise_state()["step"] == max(resumed)
    finally:
        runtime.manual_seed(saved_seed)
        runtime.set_noise_state(saved)


def test_default_seed_is_not_a_constant():
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = f"import sys; sys.path.insert(0, {root!r}); from flashdp4review_b200 import runtime; print(runtime.get_seed())"
    a, b = (subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300).stdout.strip()
            for _ in range(2))
    assert a and b and a != b and int(a) != 0


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
