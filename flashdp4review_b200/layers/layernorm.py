"""DPLayerNorm: LayerNorm over the last dimension with per-sample-clipped, noised dgamma/dbeta.

Constructor as flashdp/layers/layernorm.py:25-66.  Forward and dx are the standard LayerNorm of
the reference's fused kernels (flashdp/core/layernorm_clip.py:11-60, :95-103).  The affine
gradients follow the reference's per-sample path (`layernorm_dw_clip` / `layernorm_db_clip`,
flashdp/core/layernorm_clip.py:163-198, called from flashdp/layers/layernorm.py:128-165) for both
`use_fused` settings: the reference's fused kernel saturates a shared buffer element-wise under a
spin lock, adds no noise and depends on block order (flashdp/core/layernorm_clip.py:109-131), so
it cannot be reproduced or relied on; and the per-sample path's second noise draw, which the
reference adds to grad_weight (flashdp/layers/layernorm.py:150), goes to grad_bias here.

`compat_fused_saturation=True` (with use_fused) reproduces the reference's fused arithmetic instead --
element-wise saturation of 64..256 row-group buffers, no division by the batch, no noise
(flashdp/layers/layernorm.py:170-204) -- with the rows of a buffer taken in increasing order.  It is
there for comparisons with the reference's default; it is not differentially private.
"""
import numbers

import torch
import torch.nn as nn
from torch.autograd.function import Function

from ..core import ops
from .utils import DPParameter as Parameter
from ._common import DPLayerMixin, dp_scalars


class _DPLayerNormFunc(Function):
    @staticmethod
    def forward(ctx, input, weight, bias, layer):
        y, buf, _ = ops.layernorm_fwd_fused(input, weight, bias, layer.eps)
        ctx.save_for_backward(input, weight, buf["mean"], buf["rstd"])
        ctx.layer = layer
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, grad_output):
        input, weight, mean, rstd = ctx.saved_tensors
        layer = ctx.layer
        if layer.compat_fused_saturation:
            clip_args = torch.tensor([layer.C, layer.clamp_value])
            dx, dw_, db_, args = ops.layernorm_bwd_clip_fused(grad_output, input, weight, None, clip_args,
                                                             {"mean": mean, "rstd": rstd})
            dw, db = ops.layernorm_dwdb_fused(weight, None, dw_, db_, args)
            return (dx if ctx.needs_input_grad[0] else None, dw if ctx.needs_input_grad[1] else None,
                    db if ctx.has_bias and ctx.needs_input_grad[2] else None, None)
        B = input.shape[0] if input.dim() > 1 else 1
        step = layer._next_step()
        div, noise = dp_scalars(B, layer.noise_multiplier, layer._dp_param_ids[0], step,
                                param_id2=layer._dp_param_ids[1])
        need_db = ctx.has_bias and ctx.needs_input_grad[2]
        dx, dw, db = ops.dp_layernorm_backward(
            grad_output, input, weight, mean, rstd, layer.C, layer.clamp_value, batch_divisor=div,
            noise=noise, need_dx=ctx.needs_input_grad[0], need_dbeta=need_db)
        if dx is not None and dx.shape != input.shape:
            raise RuntimeError(f"grad_input shape {dx.shape} is not equal to input shape {input.shape}")
        if not ctx.needs_input_grad[1]:
            dw = None
        return dx, dw, db, None


class DPLayerNorm(nn.LayerNorm, DPLayerMixin):
    def __init__(self, normalized_shape, eps: float = 1e-5, elementwise_affine: bool = True,
                 bias: bool = True, device=None, dtype=None, use_fused: bool = True, C: float = 1.0,
                 clamp_value: float = 1.0, noise_multiplier: float = 1.0,
                 compat_fused_saturation: bool = False) -> None:
        if isinstance(normalized_shape, numbers.Integral):
            normalized_shape = (normalized_shape,)
        use_bias = bias is not None   # the reference's rule (flashdp/layers/layernorm.py:42)
        if use_fused and not use_bias:
            raise NotImplementedError("In fused mode, bias must be enabled. Set use_fused=False to use the default implementation.")
        super().__init__(normalized_shape, eps, elementwise_affine, use_bias, device=device, dtype=dtype)
        self.use_fused = use_fused
        self.compat_fused_saturation = bool(compat_fused_saturation) and use_fused
        self._init_dp(C, clamp_value, noise_multiplier)
        if self.elementwise_affine:
            self.weight = Parameter(self.weight.data)
            if use_bias:
                self.bias = Parameter(self.bias.data)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if len(self.normalized_shape) != 1:
            raise NotImplementedError("Currently layernorm only support normalized_dim=-1.")
        if self.normalized_shape[0] != input.shape[-1]:
            raise NotImplementedError("Currently layernorm only support normalized_dim=-1.")
        if not self.elementwise_affine:
            return torch.nn.functional.layer_norm(input, self.normalized_shape, None, None, self.eps)
        bias = self.bias if self.bias is not None else torch.zeros_like(self.weight)
        return _DPLayerNormFunc.apply(input, self.weight, bias, self)
