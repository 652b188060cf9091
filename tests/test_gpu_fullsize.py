"""The benchmark description's full-size shapes.  First against an independent float64 evaluation of
the reference's per-sample algorithm on the same GPU (torch float64 matmuls: every per-sample norm
and the whole clipped mean, tensor-wide); then through properties that need no second evaluation: agreement of the two norm algorithms, a float64 spot check of two samples'
norms, a float64 check of one 64x64 block of the clipped sum, invariance of the all-clipped
gradient to a rescaling of the upstream gradient, linearity when nothing is clipped, and bit-equal
reruns.  LayerNorm at full size is cheap enough for a direct oracle comparison."""
import numpy as np
import pytest
import torch

from oracle import dp_oracle as O
from conftest import rel_err, norm_err
from gpu_util import dev

pytestmark = pytest.mark.gpu

# (name, B, T, n_in, n_out, g_scale, layout): config 2 (Linear 4096x4096), config 3 (GPT-2 c_attn as
# Conv1D), one Llama-2-7B-shaped MLP projection at seq 2048
CASES = [("linear_4096x4096_b32_t1024", 32, 1024, 4096, 4096, 1e-3, "out_in"),
         ("conv1d_1024x3072_b16_t1024", 16, 1024, 1024, 3072, 1e-3, "in_out"),
         ("llama_up_proj_4096x11008_b4_t2048", 4, 2048, 4096, 11008, 1e-3, "out_in")]


def _fp64_reference(G, X, C, clamp, layout):
    """`_weight_grad_block_clip` (flashdp/core/linear_clip.py:94-104) followed by `.div_(B)`
    (flashdp/layers/linear.py:72-73), one sample at a time in float64 on the device."""
    B = G.shape[0]
    acc = torch.zeros(G.shape[-1], X.shape[-1], dtype=torch.float64, device=G.device)
    norms = torch.empty(B, dtype=torch.float64, device=G.device)
    for b in range(B):
        g = G[b].double().t() @ X[b].double()
        norms[b] = torch.linalg.norm(g)
        acc += g * torch.clamp(C / (norms[b] + 1e-10), max=clamp)
    acc /= B
    return (acc if layout == "out_in" else acc.t().contiguous()), norms


@pytest.mark.parametrize("sigma", [0.0, 1.0])
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_full_size_whole_tensor_against_float64(case, sigma):
    """All B norms and every element of dW at the full sizes, bf16 tolerance 1e-2 (observed: norms
    ~1e-3 from the bf16 products' fp32 accumulation, dW ~2e-3).  With the noise on, the host
    restatement of the noise stream is subtracted first."""
    from flashdp4review_b200.core import ops
    _, B, T, n_in, n_out, gs, layout = case
    gen = torch.Generator(device="cuda").manual_seed(0)
    X = torch.randn(B, T, n_in, device=dev(), generator=gen).to(torch.bfloat16)
    G = (torch.randn(B, T, n_out, device=dev(), generator=gen) * gs).to(torch.bfloat16)
    G[1] *= 3.0
    G[B - 1] *= 1e-4                                # one sample below the clipping threshold
    C = 1.0
    std = sigma / float(np.sqrt(B))
    noise = ops.NoiseSpec(std, 7, 3, 0, 11) if sigma > 0 else None
    dW, norms, factors = ops.dp_linear_weight_grad(X, G, C, 1.0, layout=layout, out_dtype=torch.float32,
                                                   return_norms=True, noise=noise)
    want, wn = _fp64_reference(G, X, C, 1.0, layout)
    err_n = float(((norms.double() - wn).abs() / wn).max())
    assert err_n < 1e-2, err_n
    assert float(factors[B - 1]) == 1.0 and float(factors[1]) < 1.0
    got = dW.double()
    if sigma > 0:
        z = O.gaussian_noise(dW.numel(), std, 7, 3, 11).reshape(dW.shape)
        got = got - torch.from_numpy(z).to(got.device)
        # the device draws in fp32, the host restatement in float64 (they agree to 3e-6), and the sum
        # gradient + noise is rounded at the noise's magnitude
        slack = 4e-6
    else:
        slack = 0.0
    err = float((got - want).abs().max() / want.abs().max())
    assert err < 1e-2 + slack / float(want.abs().max()), err


@pytest.mark.parametrize("shape", [(8, 1024, 4096, 4096, "out_in"), (4, 128, 768, 768, "out_in"),
                                   (3, 320, 1024, 576, "in_out"), (2, 2048, 1024, 3072, "in_out")],
                         ids=lambda s: "x".join(map(str, s)))
def test_fp32_inputs_on_the_tensor_cores(shape):
    """fp32 G and X with 64-aligned shapes run as three bf16 products (hi*hi + hi*lo + lo*hi) on the
    tensor cores, their accumulators drained into registers every few K stages.  Norms and clipped mean
    against float64 at the fp32 tolerance 1e-5, as the default (`fp32_tensor=None`) and on request; the
    fp32-FMA kernels (`fp32_tensor=False`) on the same inputs hold it too."""
    from flashdp4review_b200.core import ops
    B, T, n_in, n_out, layout = shape
    gen = torch.Generator(device="cuda").manual_seed(3)
    X = torch.randn(B, T, n_in, device=dev(), generator=gen)
    G = torch.randn(B, T, n_out, device=dev(), generator=gen) * 1e-2
    G[0] *= 30.0
    G[B - 1] *= 1e-5
    C = 1.0
    want, wn = _fp64_reference(G, X, C, 1.0, layout)
    for algo, mode in (("auto", None), ("gram", True), ("direct", True)):
        dW, norms, factors = ops.dp_linear_weight_grad(X, G, C, 1.0, layout=layout, norm_algo=algo, return_norms=True,
                                                       fp32_tensor=mode)
        assert dW.dtype == torch.float32
        err_n = float(((norms.double() - wn).abs() / wn).max())
        err = float((dW.double() - want).abs().max() / want.abs().max())
        assert err_n < 1e-5 and err < 1e-5, (algo, err_n, err)
    if B * T * n_in * n_out <= 2 ** 32:                       # the fp32-FMA kernels: same tolerance
        dW, norms, _ = ops.dp_linear_weight_grad(X, G, C, 1.0, layout=layout, return_norms=True, fp32_tensor=False)
        assert float(((norms.double() - wn).abs() / wn).max()) < 1e-5
        assert float((dW.double() - want).abs().max() / want.abs().max()) < 1e-5
    again = ops.dp_linear_weight_grad(X, G, C, 1.0, layout=layout, fp32_tensor=True)
    assert torch.equal(again, ops.dp_linear_weight_grad(X, G, C, 1.0, layout=layout, fp32_tensor=True))
    # noise on top: the host stream, subtracted, leaves the same gradient
    noisy = ops.dp_linear_weight_grad(X, G, C, 1.0, layout=layout, noise=ops.NoiseSpec(0.01, 5, 2, 0, 9), fp32_tensor=True)
    z = O.gaussian_noise(noisy.numel(), 0.01, 5, 2, 9).reshape(noisy.shape)
    assert float((noisy.double() - torch.from_numpy(z).to(noisy.device) - want).abs().max() / want.abs().max()) < 1e-4


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_full_size_properties(case):
    from flashdp4review_b200.core import ops
    _, B, T, n_in, n_out, gs, layout = case
    gen = torch.Generator(device="cuda").manual_seed(0)
    X = torch.randn(B, T, n_in, device=dev(), generator=gen).to(torch.bfloat16)
    G = (torch.randn(B, T, n_out, device=dev(), generator=gen) * gs).to(torch.bfloat16)
    G[1] *= 3.0
    C = 1.0
    run = lambda g, c=C, algo="auto": ops.dp_linear_weight_grad(X, g, c, 1.0, layout=layout, norm_algo=algo,
                                                                out_dtype=torch.float32, return_norms=True)
    dW, norms, factors = run(G)
    dW2, norms2, _ = run(G)
    assert torch.equal(dW, dW2) and torch.equal(norms, norms2)            # bit-reproducible
    # the two norm algorithms are independent computations of the same numbers
    _, norms_d, _ = run(G, algo="direct")
    _, norms_g, _ = run(G, algo="gram")
    assert norm_err(norms_d.cpu().numpy(), norms_g.cpu().numpy()) < 2e-3
    # float64 spot check of two samples' norms through the Gram identity
    for b in (0, 1):
        Gb, Xb = G[b].double().cpu().numpy(), X[b].double().cpu().numpy()
        want = np.sqrt(np.sum((Gb @ Gb.T) * (Xb @ Xb.T)))
        assert abs(float(norms[b]) / want - 1) < 1e-2
    assert torch.all(factors < 1.0)                                       # every sample is clipped at C = 1
    f = factors.double().cpu().numpy()
    assert np.allclose(f, O.clip_factor(norms.double().cpu().numpy(), C, 1.0), rtol=1e-5)
    # one 64x64 block of the clipped sum in float64, from the kernel's own factors
    r0, c0 = 64 * 3, 64 * 5
    Gs = G[:, :, r0:r0 + 64].double().cpu().numpy() if layout == "out_in" else G[:, :, c0:c0 + 64].double().cpu().numpy()
    Xs = X[:, :, c0:c0 + 64].double().cpu().numpy() if layout == "out_in" else X[:, :, r0:r0 + 64].double().cpu().numpy()
    if layout == "out_in":
        want = sum(f[b] * Gs[b].T @ Xs[b] for b in range(B)) / B
    else:
        want = sum(f[b] * Xs[b].T @ Gs[b] for b in range(B)) / B
    got = dW[r0:r0 + 64, c0:c0 + 64].double().cpu().numpy()
    assert np.abs(got - want).max() / float(dW.abs().max()) < 2e-3
    # all samples clipped: c_b scales as 1/|G_b|, so doubling G must not change the result
    dW_scaled, _, _ = run(G * 2)
    assert rel_err(dW_scaled.cpu().numpy(), dW.cpu().numpy()) < 1e-2
    # nothing clipped (huge C): the result is linear in G
    a, _, fa = run(G, c=1e9)
    b2, _, _ = run(G * 2, c=1e9)
    assert torch.all(fa == 1.0)
    assert rel_err(b2.cpu().numpy(), 2 * a.cpu().numpy()) < 1e-2
    # sum over samples of clipped norms bounds the result: ||B*dW|| <= sum_b c_b*||g_b|| <= B*C
    assert float(dW.double().norm()) * B <= B * C * (1 + 1e-3)


def test_full_size_bias_and_input_grad():
    from flashdp4review_b200.core import ops
    B, T, n_in, n_out = 16, 1024, 1024, 3072
    gen = torch.Generator(device="cuda").manual_seed(1)
    G = (torch.randn(B, T, n_out, device=dev(), generator=gen) * 1e-3).to(torch.bfloat16)
    W = (torch.randn(n_in, n_out, device=dev(), generator=gen) * 0.02).to(torch.bfloat16)
    db, norms, _ = ops.dp_bias_grad(G, 1.0, 1.0, return_norms=True, out_dtype=torch.float32)
    want, wn, _ = O.linear_bias_grad(G.float().cpu(), 1.0, 1.0)
    assert norm_err(norms.cpu().numpy(), wn) < 1e-2 and rel_err(db.cpu().numpy(), want) < 1e-2
    dX = ops.linear_input_grad(G, W, "in_out", out_dtype=torch.float32)
    rows = torch.arange(0, B * T, 997, device=dev())
    want = G.reshape(-1, n_out)[rows].double() @ W.double().t()
    assert rel_err(dX.reshape(-1, n_in)[rows].cpu().numpy(), want.cpu().numpy()) < 1e-2


def test_full_size_layernorm_against_oracle():
    from flashdp4review_b200.core import ops
    B, T, d = 16, 1024, 1024
    gen = torch.Generator().manual_seed(2)
    X = (torch.randn(B, T, d, generator=gen) * 1.3 + 0.2).to(torch.bfloat16)
    DY = (torch.randn(B, T, d, generator=gen) * 1e-3).to(torch.bfloat16)
    gamma, beta = torch.ones(d), torch.zeros(d)
    y, buf, _ = ops.layernorm_fwd_fused(X.to(dev()), gamma.to(dev()), beta.to(dev()), 1e-5)
    wy, wmean, wrstd = O.layernorm_fwd(X, gamma, beta, 1e-5)
    assert rel_err(y.float().cpu().numpy(), wy) < 1e-2
    dx, dg, db, ng, nb = ops.dp_layernorm_backward(DY.to(dev()), X.to(dev()), gamma.to(dev()), buf["mean"],
                                                   buf["rstd"], 1.0, 1.0, return_norms=True)
    xhat = (X.double().numpy() - wmean[..., None]) * wrstd[..., None]
    wdg, wdb, wng, wnb = O.layernorm_affine_grads(DY, xhat, 1.0, 1.0)
    assert norm_err(ng.cpu().numpy(), wng) < 1e-2 and norm_err(nb.cpu().numpy(), wnb) < 1e-2
    assert rel_err(dg.cpu().numpy(), wdg) < 1e-2 and rel_err(db.cpu().numpy(), wdb) < 1e-2
    assert rel_err(dx.float().cpu().numpy(), O.layernorm_bwd_dx(DY, X, gamma, wmean, wrstd)) < 1e-2
