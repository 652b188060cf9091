"""GPU parity of the LayerNorm forward / backward / per-sample affine gradients."""
import numpy as np
import pytest
import torch

from oracle import dp_oracle as O
from conftest import rel_err, norm_err
from gpu_util import TOL, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from flashdp4review_b200.core import ops
    return ops


def _case(B, T, d, dtype, seed):
    gen = torch.Generator().manual_seed(seed)
    X = (torch.randn(B, T, d, generator=gen) * 1.5 + 0.3).to(dtype)
    DY = (torch.randn(B, T, d, generator=gen) * 0.2).to(dtype)
    DY[0] *= 30
    gamma = torch.randn(d, generator=gen) * 0.1 + 1.0
    beta = torch.randn(d, generator=gen) * 0.1
    return X, DY, gamma, beta


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(4, 9, 40), (2, 33, 1024), (3, 70, 768), (1, 5, 7), (2, 16, 2048),
                                   (2, 8, 4096), (2, 3, 8192), (3, 64, 100), (2, 40, 1030)])
def test_layernorm_fwd_bwd(shape, dtype, ops):
    B, T, d = shape
    X, DY, gamma, beta = _case(B, T, d, dtype, seed=B * 1000 + d)
    tol = TOL[dtype]
    y, buf, _ = ops.layernorm_fwd_fused(X.to(dev()), gamma.to(dev()), beta.to(dev()), 1e-5)
    wy, wmean, wrstd = O.layernorm_fwd(X, gamma, beta, 1e-5)
    assert rel_err(y.float().cpu().numpy(), wy) < tol
    assert rel_err(buf["mean"].cpu().numpy().reshape(B, T), wmean) < 1e-5
    assert norm_err(buf["rstd"].cpu().numpy().reshape(B, T), wrstd) < 2e-5
    dx, dg, db, ng, nb = ops.dp_layernorm_backward(DY.to(dev()), X.to(dev()), gamma.to(dev()),
                                                   buf["mean"], buf["rstd"], 0.9, 1.0, return_norms=True)
    xhat = (X.double().numpy() - wmean[..., None]) * wrstd[..., None]
    wdg, wdb, wng, wnb = O.layernorm_affine_grads(DY, xhat, 0.9, 1.0)
    assert norm_err(ng.cpu().numpy(), wng) < max(tol, 2e-5)
    assert norm_err(nb.cpu().numpy(), wnb) < max(tol, 2e-5)
    assert rel_err(dg.cpu().numpy(), wdg) < max(tol, 2e-5)
    assert rel_err(db.cpu().numpy(), wdb) < max(tol, 2e-5)
    wdx = O.layernorm_bwd_dx(DY, X, gamma, wmean, wrstd)
    assert rel_err(dx.float().cpu().numpy(), wdx) < max(tol, 5e-5)


def test_layernorm_against_reference_fixture(golden, ops):
    g = golden("layers.npz")
    X, DY = torch.from_numpy(g["ln_X"]), torch.from_numpy(g["ln_DY"])
    gamma, beta = torch.from_numpy(g["ln_gamma"]), torch.from_numpy(g["ln_beta"])
    y, buf, _ = ops.layernorm_fwd_fused(X.to(dev()), gamma.to(dev()), beta.to(dev()), 1e-5)
    assert rel_err(y.cpu().numpy(), g["ln_y"]) < 1e-5
    dx, dg, db = ops.dp_layernorm_backward(DY.to(dev()), X.to(dev()), gamma.to(dev()), buf["mean"],
                                           buf["rstd"], float(g["ln_C"]), 1.0)
    assert rel_err(dg.cpu().numpy(), g["ln_dgamma"]) < 2e-5
    assert rel_err(db.cpu().numpy(), g["ln_dbeta_fn"]) < 2e-5
    assert rel_err(dx.cpu().numpy(), g["ln_dx"]) < 5e-5
    # the drop-in functions take the already normalised activation
    xhat = (X - X.mean(-1, keepdim=True)) / torch.sqrt(X.var(-1, keepdim=True, unbiased=False) + 1e-5)
    dgw = ops.layernorm_dw_clip(xhat.to(dev()), DY.to(dev()), gamma.to(dev()).reshape(1, 1, -1),
                                torch.Tensor([float(g["ln_C"])]), torch.Tensor([1.0]))
    dgb = ops.layernorm_db_clip(DY.to(dev()), beta.to(dev()).reshape(1, 1, -1),
                                torch.Tensor([float(g["ln_C"])]), torch.Tensor([1.0]))
    assert dgw.shape == (1, 1, X.shape[-1])
    assert rel_err(dgw.cpu().numpy().reshape(-1), g["ln_dgamma_fn"]) < 2e-5
    assert rel_err(dgb.cpu().numpy().reshape(-1), g["ln_dbeta_fn"]) < 2e-5


def test_layernorm_noise_and_determinism(ops):
    B, T, d = 4, 16, 1024
    X, DY, gamma, beta = _case(B, T, d, torch.bfloat16, 3)
    y, buf, _ = ops.layernorm_fwd_fused(X.to(dev()), gamma.to(dev()), beta.to(dev()), 1e-5)
    ns = ops.NoiseSpec(std=0.5, seed=77, param_id=5, param_id2=6, step=2)
    r0 = ops.dp_layernorm_backward(DY.to(dev()), X.to(dev()), gamma.to(dev()), buf["mean"], buf["rstd"], 1.0, 1.0)
    r1 = ops.dp_layernorm_backward(DY.to(dev()), X.to(dev()), gamma.to(dev()), buf["mean"], buf["rstd"], 1.0, 1.0, noise=ns)
    r2 = ops.dp_layernorm_backward(DY.to(dev()), X.to(dev()), gamma.to(dev()), buf["mean"], buf["rstd"], 1.0, 1.0, noise=ns)
    for a, b in zip(r1, r2):
        assert torch.equal(a, b)                          # bit-reproducible
    assert np.abs((r1[1] - r0[1]).cpu().numpy() - O.gaussian_noise(d, 0.5, 77, 5, 2)).max() < 1e-5
    assert np.abs((r1[2] - r0[2]).cpu().numpy() - O.gaussian_noise(d, 0.5, 77, 6, 2)).max() < 1e-5
    assert torch.equal(r0[0], r1[0])                      # dx carries no noise


def test_layernorm_shape_limit(ops):
    from flashdp4review_b200 import _lib
    lib = _lib.load()
    assert lib.fdp_layernorm_bwd_workspace_bytes(0, 4, 8) == 0
    x = torch.zeros(2, 2, 8200, device=dev())
    m = torch.zeros(4, device=dev())
    with pytest.raises(RuntimeError):
        ops.dp_layernorm_backward(x, x, torch.ones(8200, device=dev()), m, m, 1.0, 1.0)


@pytest.mark.parametrize("shape,dtype", [((4, 300, 256), torch.float32), ((2, 1024, 1024), torch.bfloat16),
                                         ((3, 50, 72), torch.float32), ((1, 40, 2048), torch.float16)])
def test_fused_saturation_compat_mode(shape, dtype, ops):
    """`compat_fused_saturation`: the reference's fused dgamma / dbeta arithmetic with a fixed row order
    (flashdp/core/layernorm_clip.py:109-131) against its CPU restatement; bit-equal reruns; dx is the
    ordinary LayerNorm input gradient."""
    import flashdp4review_b200 as fdp
    B, T, d = shape
    gen = torch.Generator().manual_seed(sum(shape))
    X = (torch.randn(B, T, d, generator=gen) * 1.5 + 0.3).to(dtype)
    DY = (torch.randn(B, T, d, generator=gen) * 0.2).to(dtype)
    C = 0.05                                         # |buffer| passes C within a few rows: the saturation acts
    ln = fdp.DPLayerNorm(d, C=C, clamp_value=1.0, compat_fused_saturation=True).to(dev())
    x = X.to(dev()).requires_grad_(True)
    ln(x).backward(DY.to(dev()))
    g1, b1 = ln.weight.grad.clone(), ln.bias.grad.clone()
    _, wmean, wrstd = O.layernorm_fwd(X, np.ones(d), np.zeros(d), 1e-5)
    xhat = (X.double().numpy() - wmean[..., None]) * wrstd[..., None]
    wg, wb, _, _ = O.layernorm_fused_saturation(DY, xhat, C, 1.0)
    tol = 1e-4 if dtype == torch.float32 else 2e-2   # xhat from the kernel's own fp32 statistics; saturating recurrences amplify
    assert rel_err(g1.cpu().numpy(), wg) < tol and rel_err(b1.cpu().numpy(), wb) < tol
    assert rel_err(x.grad.float().cpu().numpy(), O.layernorm_bwd_dx(DY, X, np.ones(d), wmean, wrstd)) < (1e-5 if dtype == torch.float32 else 1e-2)
    ln.weight.grad = None
    ln.bias.grad = None
    x2 = X.to(dev()).requires_grad_(True)
    ln(x2).backward(DY.to(dev()))
    assert torch.equal(ln.weight.grad, g1) and torch.equal(ln.bias.grad, b1)
    # not the per-sample clipping of the default mode
    ref = fdp.DPLayerNorm(d, C=C, clamp_value=1.0, noise_multiplier=0.0).to(dev())
    x3 = X.to(dev()).requires_grad_(True)
    ref(x3).backward(DY.to(dev()))
    assert rel_err(ref.weight.grad.cpu().numpy(), g1.cpu().numpy()) > 1e-2
