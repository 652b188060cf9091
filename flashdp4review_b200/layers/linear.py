"""DPLinear: nn.Linear whose backward yields per-sample-clipped, noised parameter gradients.

Same constructor and attributes as the reference's DPLinear (flashdp/layers/linear.py:11-32).
Backward = `_DPLinearFunc.backward` (flashdp/layers/linear.py:49-104): grad_input, then one
library call for the weight gradient (norms -> clip factors -> clipped sum / B -> noise) and one
for the bias gradient.  Unlike the reference, 2-D and >3-D inputs get a grad_input of the
input's own shape, and grad_output is left unmodified.
"""
import torch
import torch.nn as nn
from torch.autograd.function import Function

from .. import runtime
from ..core import ops
from ..core.ops import RuntimeAutoTuner
from .utils import DPParameter as Parameter
from ._common import (DPLayerMixin, reshape_to_3d, dp_scalars, autocast_dtype, direct_grad_target,
                      direct_grad_done)


class _DPLinearFunc(Function):
    @staticmethod
    def forward(ctx, input, weight, bias, layer):
        dt = autocast_dtype(input, weight)
        x = input if dt is None else input.to(dt)
        w = weight if dt is None else weight.to(dt)
        ctx.save_for_backward(x, weight, bias, w if dt is not None else None)
        ctx.layer = layer
        ctx.input_dtype = input.dtype
        if x.is_cuda and ops.native_product_ok(
                x.dtype, x.numel() // x.shape[-1], w.shape[1], w.shape[0]):
            return ops.linear_forward(x, w, bias, "out_in")     # library GEMM, bias added in its epilogue
        output = x @ w.t()
        if bias is not None:
            output += bias if dt is None else bias.to(dt)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        input, weight, bias, w_cast = ctx.saved_tensors
        layer = ctx.layer
        x3, g3 = reshape_to_3d(input, grad_output)
        w_for_dx = weight if w_cast is None else w_cast
        B = x3.shape[0]
        step = layer._next_step()
        grad_input = grad_weight = grad_bias = None

        if ctx.needs_input_grad[0]:
            if ops.native_product_ok(
                    g3.dtype, g3.numel() // g3.shape[-1], w_for_dx.shape[0], w_for_dx.shape[1]):
                grad_input = ops.linear_input_grad(g3, w_for_dx, "out_in", out_dtype=ctx.input_dtype)
            else:
                grad_input = g3 @ w_for_dx.to(g3.dtype)
            grad_input = grad_input.reshape(input.shape)

        if ctx.needs_input_grad[1]:
            div, noise = dp_scalars(B, layer.noise_multiplier, layer._dp_param_ids[0], step)
            target = direct_grad_target(weight)      # a gradient-bucket slice, or None
            grad_weight = ops.dp_linear_weight_grad(
                x3, g3, layer.C, layer.clamp_value, batch_divisor=div, noise=noise,
                layout="out_in", out_dtype=weight.dtype, norm_algo=layer.norm_algo, out=target)
            if grad_weight.shape != weight.shape:
                raise RuntimeError(f"grad_weight shape {grad_weight.shape} is not equal to weight shape {weight.shape}")
            if target is not None:
                direct_grad_done(weight)
                grad_weight = None                    # already where the optimizer and the all-reduce read it

        if bias is not None and ctx.needs_input_grad[2]:
            div, noise = dp_scalars(B, layer.noise_multiplier, layer._dp_param_ids[1], step)
            grad_bias = ops.dp_bias_grad(g3, layer.C, layer.clamp_value, batch_divisor=div,
                                         noise=noise, out_dtype=bias.dtype)
            if grad_bias.shape != bias.shape:
                raise RuntimeError(f"grad_bias shape {grad_bias.shape} is not equal to bias shape {bias.shape}")

        return grad_input, grad_weight, grad_bias, None


class DPLinear(nn.Linear, DPLayerMixin):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None,
                 dtype=None, C: float = 1.0, clamp_value: float = 1.0, noise_multiplier: float = 1.0,
                 auto_tune: bool = True, norm_algo: str = "auto"):
        # `bias=None` means no bias, anything else (True, False, a tensor) means bias:
        # the reference's rule (flashdp/layers/linear.py:14), kept for drop-in behaviour
        use_bias = bias is not None
        super().__init__(in_features, out_features, use_bias, device=device, dtype=dtype)
        self._init_dp(C, clamp_value, noise_multiplier)
        self.runtime_tuner = RuntimeAutoTuner(enable=auto_tune)
        self.norm_algo = norm_algo
        self.weight = Parameter(self.weight.data)
        if use_bias:
            self.bias = Parameter(self.bias.data)

    def forward(self, input):
        return _DPLinearFunc.apply(input, self.weight, self.bias, self)
