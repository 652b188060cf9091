"""The library's calls inside a captured CUDA graph: every entry point only enqueues work on the
caller's stream (kernels, one memset), so a training step's DP calls can be captured once and replayed.
The noise step is a launch parameter, so a replay draws the same noise as the capture did -- the test
compares a replay on new inputs with eager calls that use the same step."""
import pytest
import torch

from oracle import dp_oracle as O
from gpu_util import dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_replay_of_captured_calls_equals_eager_calls(dtype):
    from flashdp4review_b200.core import ops
    B, T, n_in, n_out = 4, 256, 512, 384
    Xa, Ga, W = O.make_linear_inputs(B, T, n_in, n_out, 1e-3, seed=11, dtype=dtype)
    Xb, Gb, _ = O.make_linear_inputs(B, T, n_in, n_out, 1e-3, seed=12, dtype=dtype)
    Xa, Ga, Xb, Gb, W = (t.to(dev()) for t in (Xa, Ga, Xb, Gb, W))
    gamma = torch.linspace(0.5, 1.5, n_in, device=dev())
    beta = torch.zeros(n_in, device=dev())
    ns = ops.NoiseSpec(0.3, 21, 5, 6, 4)

    def calls(X, G):
        dW = ops.dp_linear_weight_grad(X, G, 1e-2, 1.0, noise=ns, out_dtype=torch.float32)
        db = ops.dp_bias_grad(G, 1e-2, 1.0, noise=ns)
        dX = ops.linear_input_grad(G, W, "out_in")
        _, buf, _ = ops.layernorm_fwd_fused(X, gamma, beta, 1e-5)
        dx, dg, dbeta = ops.dp_layernorm_backward(X, X, gamma, buf["mean"], buf["rstd"], 1e-2, 1.0, noise=ns)
        return [dW, db, dX, dx, dg, dbeta]

    want = [t.clone() for t in calls(Xb, Gb)]
    X, G = Xa.clone(), Ga.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):            # warm-up outside the capture: workspace, kernel attributes
        calls(X, G)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = calls(X, G)
    X.copy_(Xb)
    G.copy_(Gb)
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    for got, w in zip(outs, want):
        assert torch.equal(got, w)


def test_device_step_counter_gives_fresh_noise_on_every_replay():
    """`NoiseSpec.step_device` / `fdp_dp_params.step_device`: the kernels add a device counter to the step
    word when they run.  Zero gradients, so the outputs are the noise itself: replay k of a graph that also
    increments the counter equals the host stream of step 10 + k, on the tensor-core path (epilogue noise
    and split-K fix-up), the generic path and the bias gradient."""
    import numpy as np
    from flashdp4review_b200.core import ops
    counter = torch.zeros(1, dtype=torch.int32, device=dev())
    ns = ops.NoiseSpec(0.5, 77, 3, 0, 10, step_device=counter)
    Xt = torch.zeros(2, 256, 512, device=dev(), dtype=torch.bfloat16)
    Gt = torch.zeros(2, 256, 384, device=dev(), dtype=torch.bfloat16)
    Xs = torch.zeros(3, 50, 72, device=dev())
    Gs = torch.zeros(3, 50, 40, device=dev())

    def calls():
        a = ops.dp_linear_weight_grad(Xt, Gt, 1.0, 1.0, noise=ns, out_dtype=torch.float32)
        b = ops.dp_linear_weight_grad(Xs, Gs, 1.0, 1.0, noise=ns)
        c = ops.dp_bias_grad(Gt, 1.0, 1.0, noise=ns, out_dtype=torch.float32)
        return a, b, c

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        calls()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = calls()
        counter.add_(1)
    counter.zero_()
    for k in range(3):
        graph.replay()
        torch.cuda.synchronize()
        for got in outs:
            want = O.gaussian_noise(got.numel(), 0.5, 77, 3, 10 + k).reshape(got.shape)
            assert np.abs(got.cpu().numpy() - want).max() < 3e-6, k
    assert int(counter.item()) == 3


def test_layers_with_the_device_step_counter():
    """`use_device_noise_step()`: the layers pass the counter; `advance_noise_step()` moves every layer's
    noise to the next step, and `noise_state()` reports the step reached."""
    import numpy as np
    import flashdp4review_b200 as fdp
    from flashdp4review_b200 import runtime
    fdp.manual_seed(5)
    fdp.use_device_noise_step(True)
    try:
        lin = fdp.DPLinear(512, 384, bias=False, C=1.0, noise_multiplier=1.0).to(dev()).to(torch.bfloat16)
        pid = lin._dp_param_ids[0]
        base = runtime.noise_step(0)
        x = torch.zeros(4, 256, 512, device=dev(), dtype=torch.bfloat16)
        start = int(runtime.device_noise_counter().item())
        seen = []
        for k in range(2):
            lin.weight.grad = None
            lin(x).sum().backward()
            got = lin.weight.grad.float().cpu().numpy()
            want = O.gaussian_noise(got.size, 1.0 / np.sqrt(4), 5, pid, base + start + k).reshape(got.shape)
            assert np.abs(got - want).max() < 1e-2      # the gradient is stored in bf16
            seen.append(got)
            fdp.advance_noise_step()
        assert np.abs(seen[0] - seen[1]).max() > 0.1
        assert fdp.noise_state()["step"] >= base + start + 2
    finally:
        fdp.use_device_noise_step(False)
