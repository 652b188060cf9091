"""Process-wide DP run state: noise seed, parameter ids, data-parallel layout.

The reference keeps no such state (it draws from torch's global generator and knows one GPU).
Here the noise is a pure function of (seed, param_id, step, element index), and a
data-parallel job is described once so every layer scales by the global batch and draws only
its share of the noise before the all-reduce of the clipped sums.
"""
import contextlib
import itertools
import os

_ids = itertools.count(1)


class _Run:
    seed = 0
    world = 1
    rank = 0
    input_grad_impl = "library"   # "library": cuBLAS via torch (as the reference); "native": fdp_linear_dgrad
    micro_index = 0               # gradient accumulation: which micro-step of `micro_steps` runs now
    micro_steps = 1


_run = _Run()


def manual_seed(seed: int):
    """Fix the Philox key of every DP layer's noise (reproducible runs)."""
    _run.seed = int(seed)


def get_seed() -> int:
    return _run.seed


def set_data_parallel(rank: int, world: int):
    """Declare that the batch each DP layer sees is one of `world` equal shards.

    Layers then divide by world*B_local and use std = noise_multiplier/sqrt(world*B_local); rank r
    draws only its 1/world share of the noise elements, so the SUM all-reduce of the gradients
    (see flashdp4review_b200.distributed) yields the gradient and exactly one noise draw of the
    concatenated batch.
    """
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad data-parallel layout rank={rank} world={world}")
    _run.rank, _run.world = int(rank), int(world)
    if world > 1:
        # The persistent GEMM grids otherwise take every SM (a CTA holds an SM's whole shared memory) and
        # the NCCL kernels of the gradient all-reduce cannot start beside them.  Leaving a dozen SMs free
        # measured +5 % on 8 GPUs.  The library reads this once, at its first tensor-core launch.
        os.environ.setdefault("FDP_TC_RESERVE_SMS", "12")


def data_parallel():
    return _run.rank, _run.world


def set_accumulation(micro_index: int, micro_steps: int):
    """Declare that the next backward pass is micro-step `micro_index` of `micro_steps` whose
    gradients autograd adds up before one optimizer step.

    The reference divides by the micro-batch and draws fresh noise in every backward
    (flashdp/layers/linear.py:72-80), so accumulating k micro-steps yields k times the mean and k
    noise draws.  With this setting every micro-step divides by the whole logical batch
    (micro_steps * world * B_local) and only the last one adds noise, with
    std = noise_multiplier / sqrt(whole batch): the accumulated gradient equals one step on the
    concatenated batch.
    """
    if micro_steps < 1 or not (0 <= micro_index < micro_steps):
        raise ValueError(f"bad accumulation state micro_index={micro_index} micro_steps={micro_steps}")
    _run.micro_index, _run.micro_steps = int(micro_index), int(micro_steps)


def accumulation():
    return _run.micro_index, _run.micro_steps


@contextlib.contextmanager
def accumulate(micro_index: int, micro_steps: int):
    """`with accumulate(i, k): loss_i.backward()` -- set_accumulation for the block, then back to
    single-step behaviour."""
    set_accumulation(micro_index, micro_steps)
    try:
        yield
    finally:
        set_accumulation(0, 1)


def set_input_grad_impl(name: str):
    """Which GEMMs the DP layers use beside the DP kernels: "library" = cuBLAS through torch, as the
    reference does (flashdp/layers/linear.py:43, :62-67); "native" = this package's own tcgen05 GEMMs
    for the input gradient (any dtype) and, for bf16/fp16, the forward product with the bias added in
    the epilogue."""
    if name not in ("library", "native"):
        raise ValueError("input_grad_impl must be 'library' or 'native'")
    _run.input_grad_impl = name


def input_grad_impl():
    return _run.input_grad_impl


def next_param_id() -> int:
    """A fresh id per DP parameter tensor, in construction order."""
    return next(_ids)
