"""Shape fuzzing of the weight-gradient entry point with hypothesis: arbitrary small shapes straddle
the boundary between the generic kernels and the tensor-core kernels (row pitch multiple of 16 bytes,
at least 128 features, T >= 64) and the boundaries of the 128x256x64 tiles."""
import pytest
import torch
from hypothesis import given, settings, strategies as st, HealthCheck

from oracle import dp_oracle as O
from gpu_util import check_wgrad

pytestmark = pytest.mark.gpu

dims = st.sampled_from([8, 24, 64, 120, 128, 136, 192, 256, 264, 320, 384, 520])


@settings(max_examples=30, deadline=None, suppress_health_check=list(HealthCheck), derandomize=True)
@given(B=st.integers(1, 5), T=st.sampled_from([1, 7, 33, 64, 96, 128, 130, 192, 256, 320]), n_in=dims, n_out=dims,
       dtype=st.sampled_from([torch.float32, torch.bfloat16, torch.float16]),
       layout=st.sampled_from(["out_in", "in_out"]), C=st.sampled_from([1e-3, 0.05, 1.0, 1e6]),
       clamp=st.sampled_from([0.25, 1.0]))
def test_wgrad_fuzz(B, T, n_in, n_out, dtype, layout, C, clamp):
    X, G, _ = O.make_linear_inputs(B, T, n_in, n_out, 2e-2, seed=B * 1000 + T + n_in + n_out, dtype=dtype)
    if B > 1:
        G[0] *= 25.0
    check_wgrad(X, G, C, clamp, dtype, layout=layout)


@settings(max_examples=20, deadline=None, suppress_health_check=list(HealthCheck), derandomize=True)
@given(B=st.integers(1, 5), T=st.sampled_from([64, 128, 192, 256, 320, 512]), n_in=st.sampled_from([64, 128, 192, 256, 320, 576]),
       n_out=st.sampled_from([128, 192, 256, 384, 640]), layout=st.sampled_from(["out_in", "in_out"]),
       algo=st.sampled_from(["auto", "gram", "direct"]), C=st.sampled_from([1e-3, 0.05, 1e6]))
def test_fp32_tensor_mode_fuzz(B, T, n_in, n_out, layout, algo, C):
    """fp32 inputs with `fp32_tensor=True`: shapes on both sides of what the three-product tensor-core
    path takes (64-aligned features of at least 128, T a multiple of 64 and at least 128); the others
    fall back to the fp32-FMA kernels.  The fp32 tolerance 1e-5 either way."""
    from flashdp4review_b200.core import ops
    from conftest import rel_err, norm_err
    from gpu_util import dev
    X, G, _ = O.make_linear_inputs(B, T, n_in, n_out, 2e-2, seed=B + T + n_in + n_out)
    if B > 1:
        G[0] *= 25.0
    dW, norms, _ = ops.dp_linear_weight_grad(X.to(dev()), G.to(dev()), C, 1.0, layout=layout, norm_algo=algo,
                                             return_norms=True, fp32_tensor=True)
    want, wn = O.linear_weight_grad(G, X, C, 1.0, layout=layout)
    assert norm_err(norms.cpu().numpy(), wn) < 1e-5 and rel_err(dW.cpu().numpy(), want) < 1e-5
