"""DPLinear / DPConv1D / DPLayerNorm against the fixtures made by the reference's own autograd
Functions (noise_multiplier = 0), plus the behaviours that differ from the reference by design."""
import pytest
import torch
import torch.nn as nn

from oracle import dp_oracle as O
from conftest import rel_err
from gpu_util import dev

pytestmark = pytest.mark.gpu


def test_dplinear_matches_reference_function(golden):
    from flashdp4review_b200 import DPLinear
    g = golden("layers.npz")
    B, T, n_in, n_out = (int(v) for v in g["lin_meta"])
    lin = DPLinear(n_in, n_out, bias=True, C=float(g["lin_C"]), clamp_value=1.0, noise_multiplier=0.0).to(dev())
    with torch.no_grad():
        lin.weight.copy_(torch.from_numpy(g["lin_W"]))
        lin.bias.copy_(torch.from_numpy(g["lin_b"]))
    x = torch.from_numpy(g["lin_X"]).to(dev()).requires_grad_(True)
    y = lin(x)
    Gd = torch.from_numpy(g["lin_G"]).to(dev())
    keep = Gd.clone()
    y.backward(Gd)
    assert rel_err(y.detach().cpu().numpy(), g["lin_y"]) < 1e-5
    assert rel_err(x.grad.cpu().numpy(), g["lin_dx"]) < 1e-5
    assert rel_err(lin.weight.grad.cpu().numpy(), g["lin_dW"]) < 1e-5
    assert rel_err(lin.bias.grad.cpu().numpy(), g["lin_db"]) < 1e-5
    assert torch.equal(Gd, keep)          # upstream gradient not modified
    assert lin.dp and lin.weight.requires_dp and type(lin.weight).__name__ == "DPParameter"


@pytest.mark.parametrize("impl", ["library", "native", "auto"])
def test_dplinear_2d_and_4d_inputs(impl):
    import flashdp4review_b200 as fdp
    fdp.set_input_grad_impl(impl)
    try:
        lin = fdp.DPLinear(16, 24, C=0.5, noise_multiplier=0.0).to(dev())
        for shape in [(6, 16), (3, 2, 5, 16)]:
            lin.zero_grad()
            x = torch.randn(*shape, device=dev(), requires_grad=True)
            y = lin(x)
            gy = torch.randn_like(y) * 0.1
            y.backward(gy)
            assert x.grad.shape == x.shape      # the reference returns a reshaped grad and autograd rejects it
            B = shape[0]
            want, _ = O.linear_weight_grad(gy.reshape(B, -1, 24).cpu(), x.detach().reshape(B, -1, 16).cpu(), 0.5, 1.0)
            assert rel_err(lin.weight.grad.cpu().numpy(), want) < 1e-5
            assert rel_err(x.grad.cpu().numpy(), (gy.double().cpu() @ lin.weight.double().cpu()).detach().numpy()) < 1e-5
    finally:
        fdp.set_input_grad_impl("auto")


def test_dpconv1d_rectangular_and_compat(golden):
    from flashdp4review_b200 import DPConv1D
    g = golden("layers.npz")
    B, T, n_in, n_out = (int(v) for v in g["lin_meta"])
    C = float(g["lin_C"])
    X, G, W = g["lin_X"], g["lin_G"], g["lin_W"]
    # compat mode reproduces the reference's bias-first in-place scaling (dx and dW see c_bias*G)
    conv = DPConv1D(n_out, n_in, C=C, noise_multiplier=0.0, compat_inplace_bias_scale=True).to(dev())
    with torch.no_grad():
        conv.weight.copy_(torch.from_numpy(W.T.copy()))
    x = torch.from_numpy(X).to(dev()).requires_grad_(True)
    y = conv(x)
    y.backward(torch.from_numpy(G).to(dev()))
    assert rel_err(y.detach().cpu().numpy(), g["conv_y"]) < 1e-5
    assert rel_err(conv.bias.grad.cpu().numpy(), g["conv_db"]) < 1e-5
    assert rel_err(x.grad.cpu().numpy(), g["conv_dx"]) < 1e-5
    # the reference returns [nf,nx]; ours is the weight's own [nx,nf] orientation
    assert rel_err(conv.weight.grad.cpu().numpy(), g["conv_dW_ref_orientation"].T) < 1e-5
    # default mode: plain per-sample clipping, rectangular weights work (the reference raises)
    conv = DPConv1D(40, 24, C=0.6, noise_multiplier=0.0).to(dev())
    x = torch.randn(3, 11, 24, device=dev(), requires_grad=True)
    y = conv(x)
    gy = torch.randn_like(y) * 0.05
    y.backward(gy)
    want, _ = O.linear_weight_grad(gy.cpu(), x.detach().cpu(), 0.6, 1.0, layout="in_out")
    assert conv.weight.grad.shape == (24, 40)
    assert rel_err(conv.weight.grad.cpu().numpy(), want) < 1e-5
    wdb, _, _ = O.linear_bias_grad(gy.cpu(), 0.6, 1.0)
    assert rel_err(conv.bias.grad.cpu().numpy(), wdb) < 1e-5
    assert rel_err(x.grad.cpu().numpy(), (gy.double().cpu() @ conv.weight.double().cpu().t()).detach().numpy()) < 1e-5


def test_dplayernorm_matches_reference_module(golden):
    from flashdp4review_b200 import DPLayerNorm
    g = golden("layers.npz")
    B, T, d = (int(v) for v in g["ln_meta"])
    for fused in (True, False):
        ln = DPLayerNorm(d, eps=1e-5, use_fused=fused, C=float(g["ln_C"]), noise_multiplier=0.0).to(dev())
        with torch.no_grad():
            ln.weight.copy_(torch.from_numpy(g["ln_gamma"]))
            ln.bias.copy_(torch.from_numpy(g["ln_beta"]))
        x = torch.from_numpy(g["ln_X"]).to(dev()).requires_grad_(True)
        y = ln(x)
        y.backward(torch.from_numpy(g["ln_DY"]).to(dev()))
        assert rel_err(y.detach().cpu().numpy(), g["ln_y"]) < 1e-5
        assert rel_err(x.grad.cpu().numpy(), g["ln_dx"]) < 5e-5
        assert rel_err(ln.weight.grad.cpu().numpy(), g["ln_dgamma"]) < 2e-5
        assert rel_err(ln.bias.grad.cpu().numpy(), g["ln_dbeta"]) < 2e-5
    with pytest.raises(NotImplementedError):
        DPLayerNorm(d, bias=None, use_fused=True)


def test_layer_noise_is_seeded_and_per_step():
    import flashdp4review_b200 as fdp
    fdp.manual_seed(123)
    lin = fdp.DPLinear(64, 64, C=1.0, noise_multiplier=2.0).to(dev())
    x = torch.randn(16, 4, 64, device=dev())
    gy = torch.randn(16, 4, 64, device=dev()) * 0.01
    grads = []
    for _ in range(2):
        lin.zero_grad()
        lin(x).backward(gy)
        grads.append(lin.weight.grad.clone())
    assert not torch.equal(grads[0], grads[1])            # a fresh draw every step
    clean, _ = O.linear_weight_grad(gy.cpu(), x.cpu(), 1.0, 1.0)
    resid = grads[0].cpu().numpy() - clean
    assert abs(resid.std() / (2.0 / 4.0) - 1) < 0.05        # std = noise_multiplier / sqrt(B)
    # same seed, same parameter id, same step -> same bits
    lin._dp_step = 0
    lin.zero_grad()
    lin(x).backward(gy)
    assert torch.equal(lin.weight.grad, grads[0])


def test_autocast_bf16_gives_fp32_param_grads():
    import flashdp4review_b200 as fdp
    lin = fdp.DPLinear(128, 64, C=1.0, noise_multiplier=0.0).to(dev())
    x = torch.randn(4, 64, 128, device=dev())
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = lin(x)
    assert y.dtype == torch.bfloat16
    gy = (torch.randn(4, 64, 64, device=dev()) * 0.01).to(torch.bfloat16)
    y.backward(gy)
    assert lin.weight.grad.dtype == torch.float32
    want, _ = O.linear_weight_grad(gy.cpu(), x.to(torch.bfloat16).cpu(), 1.0, 1.0)
    assert rel_err(lin.weight.grad.cpu().numpy(), want) < 1e-2


def test_native_gemms_bf16_layer_matches_oracle():
    """With set_input_grad_impl("native") forward, input gradient and DP gradients all come from the library."""
    import flashdp4review_b200 as fdp
    from flashdp4review_b200 import _lib
    fdp.set_input_grad_impl("native")
    try:
        X, G, W = O.make_linear_inputs(4, 128, 256, 384, 1e-2, seed=33, dtype=torch.bfloat16)
        for kind in ("linear", "conv1d"):
            if kind == "linear":
                layer = fdp.DPLinear(256, 384, C=0.1, noise_multiplier=0.0).to(dev()).to(torch.bfloat16)
                with torch.no_grad():
                    layer.weight.copy_(W)
                    layer.bias.copy_(torch.linspace(-1, 1, 384))
            else:
                layer = fdp.DPConv1D(384, 256, C=0.1, noise_multiplier=0.0).to(dev()).to(torch.bfloat16)
                with torch.no_grad():
                    layer.weight.copy_(W.t())
                    layer.bias.copy_(torch.linspace(-1, 1, 384))
            x = X.to(dev()).requires_grad_(True)
            n0 = _lib.load().fdp_launch_count()
            y = layer(x)
            y.backward(G.to(dev()))
            assert _lib.load().fdp_launch_count() - n0 >= 8          # forward, dX, wgrad and bias kernels ran
            bias = layer.bias.detach().double().cpu().numpy()
            assert rel_err(y.detach().float().cpu().numpy(), X.double().numpy() @ W.double().numpy().T + bias) < 1e-2
            assert rel_err(x.grad.float().cpu().numpy(), G.double().numpy() @ W.double().numpy()) < 1e-2
            want, _ = O.linear_weight_grad(G, X, 0.1, 1.0, layout="out_in" if kind == "linear" else "in_out")
            assert rel_err(layer.weight.grad.float().cpu().numpy(), want) < 1e-2
    finally:
        fdp.set_input_grad_impl("auto")


def test_wrapped_model_trains_one_step():
    import flashdp4review_b200 as fdp
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(32, 64), nn.LayerNorm(64), nn.GELU(), nn.Linear(64, 8)).to(dev())
    fdp.wrap_with_flashdp_layers(model, target_modules=[nn.Linear, nn.LayerNorm], skip_layers=["3"],
                                 C=1.0, noise_multiplier=0.5, feedback=False)
    assert type(model[0]).__name__ == "DPLinear" and type(model[1]).__name__ == "DPLayerNorm"
    assert type(model[3]) is nn.Linear
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    x = torch.randn(8, 10, 32, device=dev())
    loss = model(x).square().mean()
    loss.backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())
    opt.step()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
def test_batch_sharding_equals_single_rank(dtype, tol):
    """Data-parallel semantics without a collective: two 'ranks' each run the DP backward on half of
    the batch (divisor and noise std of the global batch, each drawing its share of the noise); the
    SUM of their gradients must equal the single-rank gradient of the whole batch -- the clipped
    part to tolerance, the noise part exactly (same Philox stream, disjoint element groups)."""
    from flashdp4review_b200.core import ops
    B, T, n_in, n_out, world = 8, 128, 256, 384, 2
    X, G, _ = O.make_linear_inputs(B, T, n_in, n_out, 1e-2, seed=17, dtype=dtype)
    G[2] *= 20.0
    Xd, Gd = X.to(dev()), G.to(dev())
    std = ops.noise_std(1.5, B)
    for std_ in (0.0, std):
        full_ns = ops.NoiseSpec(std=std_, seed=5, param_id=3, step=9)
        want = ops.dp_linear_weight_grad(Xd, Gd, 0.05, 1.0, noise=full_ns, out_dtype=torch.float32)
        want_b = ops.dp_bias_grad(Gd, 0.05, 1.0, noise=full_ns, out_dtype=torch.float32)
        acc = torch.zeros_like(want)
        acc_b = torch.zeros_like(want_b)
        half = B // world
        for r in range(world):
            ns = ops.NoiseSpec(std=std_, seed=5, param_id=3, step=9, rank=r, world=world)
            sl = slice(r * half, (r + 1) * half)
            acc += ops.dp_linear_weight_grad(Xd[sl], Gd[sl], 0.05, 1.0, batch_divisor=B, noise=ns,
                                             out_dtype=torch.float32)
            acc_b += ops.dp_bias_grad(Gd[sl], 0.05, 1.0, batch_divisor=B, noise=ns, out_dtype=torch.float32)
        assert rel_err(acc.cpu().numpy(), want.cpu().numpy()) < tol
        assert rel_err(acc_b.cpu().numpy(), want_b.cpu().numpy()) < tol
    # noise alone: the shards' draws add up to the single-rank draw bit for bit
    Z = torch.zeros_like(Gd)
    one = ops.dp_linear_weight_grad(Xd, Z, 1.0, 1.0, noise=ops.NoiseSpec(std, 5, 3, 0, 9), out_dtype=torch.float32)
    two = sum(ops.dp_linear_weight_grad(Xd[:4], Z[:4], 1.0, 1.0, batch_divisor=B, out_dtype=torch.float32,
                                        noise=ops.NoiseSpec(std, 5, 3, 0, 9, r, 2)) for r in range(2))
    assert torch.equal(one, two)


def test_gradient_accumulation_equals_one_step_on_the_whole_batch():
    """Two micro-steps of 4 samples under runtime.accumulate add up to the gradient of one step on
    all 8 samples (divisor 8, per-sample clipping unchanged), and only the last micro-step draws
    noise, with the std of the whole batch."""
    import flashdp4review_b200 as fdp
    from flashdp4review_b200 import runtime
    B, T, n_in, n_out = 8, 32, 64, 48
    X, G, W = O.make_linear_inputs(B, T, n_in, n_out, 5e-2, seed=23)
    G[1] *= 30.0

    def grads(sigma, micro_steps):
        fdp.manual_seed(3)
        torch.manual_seed(0)              # same initial bias in every run
        lin = fdp.DPLinear(n_in, n_out, C=0.4, noise_multiplier=sigma).to(dev())
        ln = fdp.DPLayerNorm(n_out, C=0.4, noise_multiplier=sigma).to(dev())
        with torch.no_grad():
            lin.weight.copy_(W)
        per = B // micro_steps
        for i in range(micro_steps):
            with runtime.accumulate(i, micro_steps):
                sl = slice(i * per, (i + 1) * per)
                ln(lin(X[sl].to(dev()))).backward(G[sl].to(dev()))
        return [p.grad.clone() for p in (lin.weight, lin.bias, ln.weight, ln.bias)]

    whole, split = grads(0.0, 1), grads(0.0, 2)
    for a, b in zip(whole, split):
        assert rel_err(b.cpu().numpy(), a.cpu().numpy()) < 1e-5
    noisy = grads(2.0, 2)
    resid = (noisy[0] - split[0]).flatten()
    want = 2.0 / B ** 0.5
    assert abs(float(resid.std()) / want - 1.0) < 0.05 and abs(float(resid.mean())) < 4 * want / resid.numel() ** 0.5
    assert runtime.accumulation() == (0, 1)


def test_weight_gradients_written_straight_into_the_bucket():
    """With DPGradReducer(grad_as_bucket_view=True) the DP layers write dW into the bucket slice
    (no autograd accumulate pass): same values as the ordinary route, p.grad is the slice, a second
    backward of the same cycle is added by autograd, zero_grad() starts a new cycle."""
    import flashdp4review_b200 as fdp
    from flashdp4review_b200.distributed import DPGradReducer
    torch.manual_seed(0)

    def make():
        torch.manual_seed(1)
        return nn.Sequential(fdp.DPLinear(32, 50, C=0.3, noise_multiplier=0.0),    # 50: slices need padding
                             fdp.DPConv1D(40, 50, C=0.3, noise_multiplier=0.0),
                             fdp.DPLayerNorm(40, C=0.3, noise_multiplier=0.0)).to(dev())

    x = torch.randn(4, 6, 32, device=dev())
    g = torch.randn(4, 6, 40, device=dev()) * 0.1
    plain = make()
    plain(x).backward(g)
    model = make()
    red = DPGradReducer(model, bucket_bytes=1 << 12, grad_as_bucket_view=True)
    model(x).backward(g)
    red.finish()
    for p, q in zip(model.parameters(), plain.parameters()):
        assert p.grad.data_ptr() == red._views[id(p)].data_ptr()
        assert torch.equal(p.grad, q.grad)
    model(x).backward(g)                      # no zero_grad: accumulates like torch does
    for p, q in zip(model.parameters(), plain.parameters()):
        assert rel_err(p.grad.cpu().numpy(), 2 * q.grad.cpu().numpy()) < 1e-6
    red.zero_grad()
    model(x).backward(g)
    for p, q in zip(model.parameters(), plain.parameters()):
        assert torch.equal(p.grad, q.grad)
    model.zero_grad(set_to_none=True)         # the optimizer's default: slices are claimed anew
    model(x).backward(g)
    red.finish()
    for p, q in zip(model.parameters(), plain.parameters()):
        assert torch.equal(p.grad, q.grad)
    red.remove()
