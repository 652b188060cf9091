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
