"""Shared pieces of the DP layer backward passes."""
from .. import runtime
from ..core.ops import NoiseSpec, noise_std
from ..distributed import direct_reducer


class DPLayerMixin:
    """Hyper-parameters and noise bookkeeping common to the DP layers."""

    def _init_dp(self, C, clamp_value, noise_multiplier, n_tensors=2):
        self.dp = True
        self.C = C
        self.clamp_value = clamp_value
        self.noise_multiplier = noise_multiplier
        self._dp_param_ids = [runtime.next_param_id() for _ in range(n_tensors)]
        self._dp_step = 0

    def _next_step(self):
        self._dp_step += 1
        return runtime.noise_step(self._dp_step)


def reshape_to_3d(input, grad_output):
    """(B,T,.) views of the saved input and the upstream gradient: 2-D gets T=1, >3-D folds the
    middle axes into T (flashdp/layers/linear.py:51-58)."""
    if input.dim() == 2:
        return input.unsqueeze(1), grad_output.unsqueeze(1)
    if input.dim() > 3:
        B = input.shape[0]
        return input.reshape(B, -1, input.shape[-1]), grad_output.reshape(B, -1, grad_output.shape[-1])
    return input, grad_output


def dp_scalars(local_batch, noise_multiplier, param_id, step, param_id2=0):
    """(batch_divisor, NoiseSpec) for one backward call under the current run layout."""
    rank, world = runtime.data_parallel()
    micro_index, micro_steps = runtime.accumulation()
    global_batch = local_batch * world * micro_steps
    # under gradient accumulation only the last micro-step carries the (single) noise draw
    std = noise_std(noise_multiplier, global_batch) if micro_index == micro_steps - 1 else 0.0
    return global_batch, NoiseSpec(std=std, seed=runtime.get_seed(),
                                   param_id=param_id, param_id2=param_id2, step=step, rank=rank, world=world,
                                   step_device=runtime.device_noise_counter() if std != 0.0 else None)


def direct_grad_target(param):
    """The bucket slice a DP weight gradient may be written into directly, or None.

    A DPGradReducer built with grad_as_bucket_view=True offers the slice once per accumulation
    cycle (the first gradient of the cycle overwrites it: no zero fill, no accumulate pass by
    autograd); later gradients of the same cycle go the ordinary way and are added by autograd.
    """
    reducer = direct_reducer(param)
    return reducer.claim_direct(param) if reducer is not None else None


def direct_grad_done(param):
    """Tell the reducer that the gradient written into the claimed slice is complete (queued on
    the current stream), as autograd's post-accumulate hook would have."""
    direct_reducer(param).direct_written(param)


def autocast_dtype(*tensors):
    """The CUDA autocast dtype if autocast is on and the tensors live on a GPU, else None.

    Under autocast the DP layers behave like their plain twins (nn.Linear, Conv1D): operands are
    cast to the autocast dtype in forward, the output comes out in it, and the cast input is what
    backward sees -- so the upstream gradient is 16-bit and the tensor-core kernels run.  (In the
    reference the Conv1D forward adds an fp32 bias to the bf16 product, the output and hence the
    whole backward become fp32 -- flashdp/layers/transformers_conv1d.py:40-43.)
    """
    import torch
    if torch.is_autocast_enabled("cuda") and all(t is None or t.is_cuda for t in tensors):
        return torch.get_autocast_dtype("cuda")
    return None
