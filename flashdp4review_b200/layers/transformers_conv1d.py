"""DPConv1D: the GPT-2 style `transformers.pytorch_utils.Conv1D` (weight [nx, nf]) with DP backward.

Constructor as flashdp/layers/transformers_conv1d.py:12-24.  The weight gradient comes out in the
weight's own [nx, nf] orientation (that of flashdp/core/transformers_conv1d_clip.py:22-28), so
rectangular layers such as GPT-2's c_attn work; the reference's backward raises on nf != nx
because it produces [nf, nx] (flashdp/layers/transformers_conv1d.py:79-81, :94-95).

`compat_inplace_bias_scale=True` reproduces the reference's order of operations, where the bias
gradient is taken first and scales grad_output in place, so grad_input and the weight gradient
see c_bias[b] * grad_output (flashdp/layers/transformers_conv1d.py:59-81).  Off by default.
"""
import torch
import torch.nn as nn
from torch.autograd.function import Function

try:
    from transformers.pytorch_utils import Conv1D
except Exception:  # transformers absent: a minimal stand-in with the same parameters
    class Conv1D(nn.Module):
        def __init__(self, nf, nx):
            super().__init__()
            self.nf, self.nx = nf, nx
            self.weight = nn.Parameter(torch.empty(nx, nf))
            self.bias = nn.Parameter(torch.zeros(nf))
            nn.init.normal_(self.weight, std=0.02)

        def forward(self, x):
            return torch.addmm(self.bias, x.view(-1, x.size(-1)), self.weight).view(x.size()[:-1] + (self.nf,))

from .. import runtime
from ..core import ops
from ..core.ops import RuntimeAutoTuner
from .utils import DPParameter as Parameter
from ._common import (DPLayerMixin, reshape_to_3d, dp_scalars, autocast_dtype, direct_grad_target,
                      direct_grad_done)


class _DPConv1DFunc(Function):
    @staticmethod
    def forward(ctx, bias, input, weight, layer):
        dt = autocast_dtype(input, weight)
        x = input if dt is None else input.to(dt)
        w = weight if dt is None else weight.to(dt)
        ctx.save_for_backward(bias, x, weight, w if dt is not None else None)
        ctx.layer = layer
        ctx.input_dtype = input.dtype
        if x.is_cuda and ops.native_product_ok(
                x.dtype, x.numel() // x.shape[-1], w.shape[0], w.shape[1]):
            return ops.linear_forward(x, w, bias, "in_out")     # library GEMM, bias added in its epilogue
        return x @ w + (bias if dt is None else bias.to(dt))

    @staticmethod
    def backward(ctx, grad_output):
        bias, input, weight, w_cast = ctx.saved_tensors
        layer = ctx.layer
        w_for_dx = weight if w_cast is None else w_cast
        x3, g3 = reshape_to_3d(input, grad_output)
        B = x3.shape[0]
        step = layer._next_step()
        grad_input = grad_weight = grad_bias = None

        if ctx.needs_input_grad[0] or layer.compat_inplace_bias_scale:
            div, noise = dp_scalars(B, layer.noise_multiplier, layer._dp_param_ids[1], step)
            grad_bias, _, factors = ops.dp_bias_grad(g3, layer.C, layer.clamp_value, batch_divisor=div,
                                                     noise=noise, out_dtype=bias.dtype, return_norms=True)
            if layer.compat_inplace_bias_scale:
                g3 = g3 * factors.to(g3.dtype).view(B, 1, 1)
            if grad_bias.shape != bias.shape:
                raise RuntimeError(f"grad_bias shape {grad_bias.shape} is not equal to bias shape {bias.shape}")
            if not ctx.needs_input_grad[0]:
                grad_bias = None

        if ctx.needs_input_grad[1]:
            if ops.native_product_ok(
                    g3.dtype, g3.numel() // g3.shape[-1], w_for_dx.shape[1], w_for_dx.shape[0]):
                grad_input = ops.linear_input_grad(g3, w_for_dx, "in_out", out_dtype=ctx.input_dtype)
            else:
                grad_input = g3 @ w_for_dx.to(g3.dtype).t()
            grad_input = grad_input.reshape(input.shape)

        if ctx.needs_input_grad[2]:
            div, noise = dp_scalars(B, layer.noise_multiplier, layer._dp_param_ids[0], step)
            target = direct_grad_target(weight)      # a gradient-bucket slice, or None
            grad_weight = ops.dp_linear_weight_grad(
                x3, g3, layer.C, layer.clamp_value, batch_divisor=div, noise=noise,
                layout="in_out", out_dtype=weight.dtype, norm_algo=layer.norm_algo, out=target)
            if grad_weight.shape != weight.shape:
                raise RuntimeError(f"grad_weight shape {grad_weight.shape} is not equal to weight shape {weight.shape}")
            if target is not None:
                direct_grad_done(weight)
                grad_weight = None                    # already where the optimizer and the all-reduce read it

        return grad_bias, grad_input, grad_weight, None


class DPConv1D(Conv1D, DPLayerMixin):
    def __init__(self, nf, nx, C: float = 1.0, clamp_value: float = 1.0, noise_multiplier: float = 1.0,
                 auto_tune: bool = True, norm_algo: str = "auto", compat_inplace_bias_scale: bool = False):
        super().__init__(nf, nx)
        self._init_dp(C, clamp_value, noise_multiplier)
        self.nf = nf
        self.runtime_tuner = RuntimeAutoTuner(enable=auto_tune)
        self.norm_algo = norm_algo
        self.compat_inplace_bias_scale = compat_inplace_bias_scale
        self.weight = Parameter(self.weight.data)
        self.bias = Parameter(self.bias.data)

    def forward(self, x):
        size_out = x.size()[:-1] + (self.nf,)
        return _DPConv1DFunc.apply(self.bias, x, self.weight, self).view(size_out)
