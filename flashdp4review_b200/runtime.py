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
    # Philox key of the noise.  Drawn from the OS by default: a fixed default would make the noise of
    # every run a publicly computable function of (construction order, step).  manual_seed() fixes it.
    seed = int.from_bytes(os.urandom(8), "little")
    step_base = 0                 # added to every layer's own backward counter (see noise_state)
    step_high = 0                 # largest step value any layer has drawn noise with so far
    world = 1
    rank = 0
    # SMs the persistent GEMM grids leave free while DPGradReducer has an all-reduce in flight.  0 by
    # default: in a training step the collective kernels find room between the step's many ordinary
    # kernels (GPT-2-medium on two GPUs: 95.1 ms per step without a reservation, 97.1 ms with 12 SMs)
    reserve_sms = int(os.environ.get("FDP_DP_RESERVE_SMS", "0"))
    fp32_mode = "tensor"          # "tensor": three bf16 tensor-core products where the shape allows; "exact": fp32 FMA kernels
    input_grad_impl = "auto"      # forward / input-gradient products of the DP layers: see set_input_grad_impl
    micro_index = 0               # gradient accumulation: which micro-step of `micro_steps` runs now
    micro_steps = 1
    device_step = False           # the noise step is read from a device counter (use_device_noise_step)
    device_counters = None        # device index -> one-element int32 tensor


_run = _Run()


def manual_seed(seed: int):
    """Fix the Philox key of every DP layer's noise (reproducible runs)."""
    _run.seed = int(seed)


def get_seed() -> int:
    return _run.seed


def use_device_noise_step(on: bool = True):
    """Read the noise step on the GPU.  By default each DP layer counts its own backward passes on the
    host and passes the count to its kernels, which is all an eagerly executed loop needs.  A training
    step captured in a CUDA graph replays the same kernel arguments, hence the same noise, every time.
    With this switch on, every layer passes a fixed step plus a pointer to a per-device counter that
    the kernels add when they run; `advance_noise_step()` -- one tiny kernel, to be called once per
    training step, inside the captured region -- increments it, so every replay draws fresh noise."""
    _run.device_step = bool(on)


def device_noise_counter(device=None):
    """The current (or given) CUDA device's noise-step counter, a one-element int32 tensor, or None
    when `use_device_noise_step` is off."""
    if not _run.device_step:
        return None
    import torch
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if _run.device_counters is None:
        _run.device_counters = {}
    t = _run.device_counters.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _run.device_counters[idx] = t
    return t


def advance_noise_step(n: int = 1):
    """counter += n on the current device's stream (see use_device_noise_step); a no-op when off."""
    t = device_noise_counter()
    if t is not None:
        t.add_(int(n))


def noise_step(local_count: int) -> int:
    """Philox step word of a layer's `local_count`-th backward: the run's base plus the layer's own
    counter, so that after `set_noise_state` no (parameter, step) pair of the earlier run recurs.
    With the device counter on, the host part is the constant base + 1 and the counter does the counting."""
    if _run.device_step:
        return (_run.step_base + 1) & 0xFFFFFFFF
    step = (_run.step_base + int(local_count)) & 0xFFFFFFFF
    if step > _run.step_high:
        _run.step_high = step
    return step


def noise_state() -> dict:
    """What a checkpoint must keep beside the model and optimizer state for the DP noise: the seed
    and the highest step drawn so far.  Without it a resumed run would count its layers' steps from
    zero again and, under the same seed, repeat the noise tensors of steps 1..N exactly -- noise an
    observer of both runs could cancel."""
    high = _run.step_high
    for t in (_run.device_counters or {}).values():      # reads the counters back: a synchronisation
        high = max(high, (_run.step_base + 1 + int(t.item())) & 0xFFFFFFFF)
    return {"seed": _run.seed, "step": high}


def set_noise_state(state: dict):
    """Resume: same seed, and every layer's step counter continues above the saved high-water mark."""
    _run.seed = int(state["seed"])
    _run.step_base = int(state["step"])
    _run.step_high = max(_run.step_high, _run.step_base)


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


def reserve_sms() -> int:
    """SMs to leave free for the collective kernels while an all-reduce overlaps GEMMs."""
    return _run.reserve_sms if _run.world > 1 else 0


@contextlib.contextmanager
def sm_reservation(n=12):
    """`with sm_reservation():` -- the library's persistent GEMM grids launched inside the block leave
    `n` SMs free, so that a collective kernel launched beside them can run.  A persistent CTA holds a
    whole SM's shared memory; without the reservation an all-reduce enqueued beside a long GEMM cannot
    start before that GEMM has ended.  Worth it where GEMMs of this library run back to back beside the
    collective (one DP layer's backward: 1.83-1.85 ms per step with 12 SMs reserved around the
    input-gradient GEMM, 1.88 ms without, on two GPUs); outside such a block the grids take every SM."""
    from . import _lib
    n = int(n)
    lib = _lib.load()
    prev = lib.fdp_set_sm_reserve(n)
    try:
        yield
    finally:
        lib.fdp_set_sm_reserve(prev)


def check_device_status(device=-1):
    """Raise RuntimeError if a kernel of the library reported, since the last check, that one of its
    bounded waits ran out (its outputs are then undefined).  A host read, no synchronisation: it sees
    what the GPU has reported so far, so call it once per step before the optimizer uses the gradients
    (DPGradReducer.finish does).  The flag stays up, and every library call on that device fails,
    until clear_device_status()."""
    from . import _lib
    _lib.check(_lib.load().fdp_async_status(int(device)), "device status")


def clear_device_status(device=-1):
    from . import _lib
    _lib.load().fdp_clear_async_status(int(device))


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


def set_fp32_mode(name: str):
    """How fp32 layers compute their DP weight gradients.  "tensor" (default): shapes with 64-aligned
    features and sequence length (at least 128 each) run on the tensor cores as three bf16 products
    (x = hi + lo; hi*hi + hi*lo + lo*hi) whose fp32 accumulators are drained into registers every few K
    stages -- within 1e-5 of float64 like the fp32-FMA kernels (measured 4e-6 on the gradient, 4e-7 on the
    norms at 4096x4096) and about six times faster; other shapes use the FMA kernels.  "exact": always
    the fp32-FMA kernels, the reference's own arithmetic."""
    if name not in ("exact", "tensor"):
        raise ValueError("fp32_mode must be 'exact' or 'tensor'")
    _run.fp32_mode = name


def fp32_mode():
    return _run.fp32_mode


def set_input_grad_impl(name: str):
    """Which GEMMs the DP layers use beside the DP kernels, i.e. for the forward product and the input
    gradient.  "library": cuBLAS through torch, as the reference does (flashdp/layers/linear.py:43,
    :62-67).  "auto" (default): this package's own tcgen05 GEMMs (bias added in the epilogue) wherever one
    of them takes the shape -- for fp32 layers that is three bf16 products within 1e-5, about five times
    cuBLAS's fp32 GEMM -- and cuBLAS elsewhere.  "native": the package's kernels for every 16-bit shape,
    the generic ones included."""
    if name not in ("library", "native", "auto"):
        raise ValueError("input_grad_impl must be 'library', 'native' or 'auto'")
    _run.input_grad_impl = name


def input_grad_impl():
    return _run.input_grad_impl


def next_param_id() -> int:
    """A fresh id per DP parameter tensor, in construction order."""
    return next(_ids)
