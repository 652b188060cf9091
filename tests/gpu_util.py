"""Helpers of the GPU parity tests: tolerances and oracle comparison."""
import numpy as np
import torch

from oracle import dp_oracle as O
from conftest import rel_err, norm_err

# Parity tolerances of the path: per-sample norms max_b |n^ - n|/n and gradients
# max|g^ - g| / max|g|, against the oracle evaluated in float64 on the SAME (rounded) inputs.
TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2, torch.float16: 1e-2}


def dev():
    return torch.device("cuda:0")


def rand_case(B, T, n_in, n_out, g_scale, seed, dtype):
    X, G, W = O.make_linear_inputs(B, T, n_in, n_out, g_scale, seed, dtype=dtype)
    return X, G, W


def check_wgrad(X, G, C, clamp, dtype, layout="out_in", norm_algo="auto", out_dtype=None, tol=None, fp32_tensor=None):
    from flashdp4review_b200.core import ops
    tol = tol or TOL[dtype]
    dW, norms, factors = ops.dp_linear_weight_grad(
        X.to(dev()), G.to(dev()), C, clamp, layout=layout, norm_algo=norm_algo,
        out_dtype=out_dtype, return_norms=True, fp32_tensor=fp32_tensor)
    torch.cuda.synchronize()
    want, wn = O.linear_weight_grad(G, X, C, clamp, layout=layout)
    got = dW.float().cpu().numpy()
    assert got.shape == want.shape
    if wn.max() > 0:
        assert norm_err(norms.cpu().numpy(), wn) < tol, (norms.cpu().numpy(), wn)
    f = O.clip_factor(wn, C, clamp)
    assert np.allclose(factors.cpu().numpy(), f, rtol=max(tol, 1e-5) * 2, atol=0)
    out_tol = tol if (out_dtype or dtype) == torch.float32 or dtype != torch.float32 else 1e-2
    assert rel_err(got, want) < out_tol, rel_err(got, want)
    return dW, norms
