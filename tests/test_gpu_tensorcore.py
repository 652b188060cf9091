"""The tcgen05 / TMEM / TMA kernels (bf16 and fp16, 16-byte-aligned row pitches) against the oracle:
both norm algorithms, the clipped-sum GEMM in both orientations, partial tiles, the input gradient."""
import numpy as np
import pytest
import torch

from oracle import dp_oracle as O
from conftest import rel_err, norm_err
from gpu_util import dev, check_wgrad

pytestmark = pytest.mark.gpu

# (B, T, n_in, n_out): full tiles, partial tiles in M / N / K, T not a multiple of the tile
SHAPES = [(2, 128, 256, 128), (3, 64, 136, 200), (2, 256, 512, 384), (1, 192, 768, 1024),
          (4, 320, 264, 520), (2, 1024, 256, 256), (2, 512, 256, 128), (1, 768, 128, 256), (5, 448, 384, 640)]


@pytest.mark.parametrize("algo", ["direct", "gram", "auto"])
@pytest.mark.parametrize("shape", SHAPES)
def test_wgrad_tensorcore(shape, algo):
    B, T, n_in, n_out = shape
    X, G, _ = O.make_linear_inputs(B, T, n_in, n_out, 1e-3, seed=sum(shape), dtype=torch.bfloat16)
    G[0] *= 40.0                      # one sample clipped harder than the others
    check_wgrad(X, G, 1e-2, 1.0, torch.bfloat16, norm_algo=algo)


@pytest.mark.parametrize("shape", [(2, 128, 256, 128), (3, 64, 136, 200)])
def test_wgrad_tensorcore_conv1d_layout_fp16_fp32out(shape):
    B, T, n_in, n_out = shape
    X, G, _ = O.make_linear_inputs(B, T, n_in, n_out, 1e-2, seed=7, dtype=torch.float16)
    check_wgrad(X, G, 0.05, 1.0, torch.float16, layout="in_out")
    check_wgrad(X, G, 0.05, 1.0, torch.float16, layout="out_in", out_dtype=torch.float32, tol=2e-3)


def test_gram_T_not_multiple_of_tile():
    # T = 200: the direct algorithm is not eligible (a K stage would cross samples); Gram masks rows
    X, G, _ = O.make_linear_inputs(3, 200, 256, 128, 1e-3, seed=21, dtype=torch.bfloat16)
    check_wgrad(X, G, 1e-2, 1.0, torch.bfloat16, norm_algo="auto")


def test_norm_algorithms_agree_and_are_deterministic():
    from flashdp4review_b200.core import ops
    X, G, _ = O.make_linear_inputs(4, 256, 512, 256, 1e-3, seed=3, dtype=torch.bfloat16)
    Xd, Gd = X.to(dev()), G.to(dev())
    res = {}
    for algo in ("direct", "gram"):
        a = ops.dp_linear_weight_grad(Xd, Gd, 1e-2, 1.0, norm_algo=algo, return_norms=True)
        b = ops.dp_linear_weight_grad(Xd, Gd, 1e-2, 1.0, norm_algo=algo, return_norms=True)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])      # bit-reproducible
        res[algo] = a
    assert norm_err(res["direct"][1].cpu().numpy(), res["gram"][1].cpu().numpy()) < 1e-4


def test_tensorcore_noise_matches_host_stream():
    from flashdp4review_b200.core import ops
    X = torch.zeros(2, 128, 256, device=dev(), dtype=torch.bfloat16)
    G = torch.zeros(2, 128, 384, device=dev(), dtype=torch.bfloat16)
    ns = ops.NoiseSpec(std=0.75, seed=99, param_id=4, step=6)
    for layout, shape in (("out_in", (384, 256)), ("in_out", (256, 384))):
        a = ops.dp_linear_weight_grad(X, G, 1.0, 1.0, noise=ns, layout=layout, out_dtype=torch.float32)
        want = O.gaussian_noise(384 * 256, 0.75, 99, 4, 6).reshape(shape)
        assert np.abs(a.cpu().numpy() - want).max() < 3e-6
    # partition over ranks
    acc = sum(ops.dp_linear_weight_grad(X, G, 1.0, 1.0, layout="out_in", out_dtype=torch.float32,
                                        noise=ops.NoiseSpec(0.75, 99, 4, 0, 6, r, 2)) for r in range(2))
    assert np.abs(acc.cpu().numpy() - O.gaussian_noise(384 * 256, 0.75, 99, 4, 6).reshape(384, 256)).max() < 3e-6


@pytest.mark.parametrize("layout", ["out_in", "in_out"])
@pytest.mark.parametrize("shape", [(256, 256, 128), (200, 136, 328), (1024, 512, 768)])
def test_input_grad_tensorcore(shape, layout):
    from flashdp4review_b200.core import ops
    rows, n_in, n_out = shape
    gen = torch.Generator().manual_seed(rows)
    G = (torch.randn(2, rows // 2, n_out, generator=gen) * 0.1).to(torch.bfloat16)
    W = (torch.randn(n_out, n_in, generator=gen) * 0.05).to(torch.bfloat16)
    Wd = W if layout == "out_in" else W.t().contiguous()
    dX = ops.linear_input_grad(G.to(dev()), Wd.to(dev()), layout)
    want = G.double().numpy() @ W.double().numpy()
    assert rel_err(dX.float().cpu().numpy(), want) < 1e-2


def test_no_bounded_wait_ran_out():
    """After a tensor-core call the status word at the head of the workspace is still zero."""
    from flashdp4review_b200 import _lib
    lib = _lib.load()
    B, T, n_in, n_out = 2, 128, 256, 256
    X = torch.randn(B, T, n_in, device=dev(), dtype=torch.bfloat16)
    G = torch.randn(B, T, n_out, device=dev(), dtype=torch.bfloat16)
    dW = torch.empty(n_out, n_in, device=dev(), dtype=torch.bfloat16)
    ws = torch.empty(lib.fdp_linear_wgrad_workspace_bytes(B, T, n_in, n_out, _lib.FDP_BF16, 0),
                     dtype=torch.uint8, device=dev())
    p = _lib.DPParams(1.0, 1.0, 0.0, 0, 0, 0, 0, 0, 0, 1)
    import ctypes
    st = lib.fdp_linear_wgrad(G.data_ptr(), X.data_ptr(), dW.data_ptr(), None, None, B, T, n_in, n_out,
                              _lib.FDP_BF16, _lib.FDP_BF16, 0, 0, ctypes.byref(p), ws.data_ptr(), ws.numel(),
                              torch.cuda.current_stream().cuda_stream)
    assert st == 0
    assert lib.fdp_device_status(ws.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0


_VARIANT_CHILD = r"""
import sys, torch, numpy as np
sys.path.insert(0, %r)
from oracle import dp_oracle as O
from flashdp4review_b200.core import ops
dev = torch.device("cuda:0")
worst = 0.0
for shape in [(2, 256, 512, 384), (3, 320, 264, 520), (2, 1024, 256, 256)]:
    B, T, n_in, n_out = shape
    X, G, W = O.make_linear_inputs(B, T, n_in, n_out, 1e-3, seed=sum(shape), dtype=torch.bfloat16)
    G[0] *= 40.0
    for layout in ("out_in", "in_out"):
        dW, norms, _ = ops.dp_linear_weight_grad(X.to(dev), G.to(dev), 1e-2, 1.0, layout=layout, return_norms=True)
        want, wn = O.linear_weight_grad(G, X, 1e-2, 1.0, layout=layout)
        worst = max(worst, float(np.abs(dW.float().cpu().numpy() - want).max() / np.abs(want).max()),
                    float((np.abs(norms.cpu().numpy() - wn) / wn).max()))
    dX = ops.linear_input_grad(G.to(dev), W.to(dev), "out_in")
    wdx = G.double().numpy() @ W.double().numpy()
    worst = max(worst, float(np.abs(dX.float().cpu().numpy() - wdx).max() / np.abs(wdx).max()))
torch.cuda.synchronize()
print("WORST", worst)
"""


@pytest.mark.parametrize("env", [{"FDP_TC_CTAS": "1"}, {"FDP_WGRAD_PRESCALE": "1"},
                                 {"FDP_TC_CTAS": "1", "FDP_WGRAD_PRESCALE": "1"}, {"FDP_TC_RESERVE_SMS": "16"},
                                 {"FDP_PDL": "0"}])
def test_kernel_variants_selected_by_environment(env):
    """Single-CTA tiles, the pre-scale path and a reduced grid are chosen once per process, so each
    is exercised in a child process and checked against the oracle at the bf16 tolerance."""
    import os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", _VARIANT_CHILD % root], env={**os.environ, **env},
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    worst = float(r.stdout.strip().split("WORST")[-1])
    assert worst < 1e-2, worst


_DIGEST_CHILD = r"""
import sys, hashlib, torch
sys.path.insert(0, %r)
from oracle import dp_oracle as O
from flashdp4review_b200.core import ops
dev = torch.device("cuda:0")
h = hashlib.sha256()
ns = ops.NoiseSpec(0.5, 7, 3, 4, 9)
for shape in [(4, 256, 512, 384), (8, 1024, 1024, 768), (3, 320, 264, 520), (300, 1, 136, 264), (3, 50, 72, 40)]:
    B, T, n_in, n_out = shape
    X, G, W = O.make_linear_inputs(B, T, n_in, n_out, 1e-3, seed=sum(shape), dtype=torch.bfloat16)
    X, G = X.to(dev), G.to(dev)
    for _ in range(3):      # back to back: the chains of consecutive calls overlap if anything can
        dW, norms, _ = ops.dp_linear_weight_grad(X, G, 1e-2, 1.0, noise=ns, return_norms=True, out_dtype=torch.float32)
        db = ops.dp_bias_grad(G, 1e-2, 1.0, noise=ns)
        h.update(dW.cpu().numpy().tobytes()); h.update(norms.cpu().numpy().tobytes()); h.update(db.float().cpu().numpy().tobytes())
    gamma = torch.linspace(0.5, 1.5, n_in, device=dev); beta = torch.zeros(n_in, device=dev)
    y, buf, _ = ops.layernorm_fwd_fused(X, gamma, beta, 1e-5)
    for _ in range(3):
        dx, dg, dbeta = ops.dp_layernorm_backward(X, X, gamma, buf["mean"], buf["rstd"], 1e-2, 1.0, noise=ns)
        for t in (dx, dg, dbeta):
            h.update(t.float().cpu().numpy().tobytes())
torch.cuda.synchronize()
print("DIGEST", h.hexdigest())
"""


def test_dependent_launches_do_not_change_a_bit():
    """The second and later kernels of a call are programmatic dependent launches unless FDP_PDL=0.
    Weight gradient (tensor-core, short-sequence and generic paths), bias gradient and LayerNorm
    backward, three calls in a row each, noise on: the outputs hash the same either way."""
    import os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    digests = []
    for env in ({"FDP_PDL": "1"}, {"FDP_PDL": "0"}):
        r = subprocess.run([sys.executable, "-c", _DIGEST_CHILD % root], env={**os.environ, **env},
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        digests.append(r.stdout.strip().split("DIGEST")[-1].strip())
    assert digests[0] == digests[1] and len(digests[0]) == 64


# short sequences (T < 64): norms through the small Gram kernel, clipped sum as one GEMM over B*T rows
SHORT = [(512, 1, 256, 384), (300, 1, 136, 264), (64, 7, 256, 128), (16, 32, 384, 256), (9, 63, 128, 520),
         (4096, 1, 128, 128)]


@pytest.mark.parametrize("layout", ["out_in", "in_out"])
@pytest.mark.parametrize("shape", SHORT)
def test_wgrad_short_sequences_bf16(shape, layout):
    B, T, n_in, n_out = shape
    X, G, _ = O.make_linear_inputs(B, T, n_in, n_out, 1e-2, seed=sum(shape), dtype=torch.bfloat16)
    G[0] *= 40.0
    G[B // 2] *= 1e-2
    check_wgrad(X, G, 0.05, 1.0, torch.bfloat16, layout=layout)


@pytest.mark.parametrize("shape", [(512, 1, 64, 48), (40, 5, 72, 136), (6, 33, 264, 96), (3, 63, 40, 24)])
def test_wgrad_short_sequences_fp32_and_direct_hint(shape):
    B, T, n_in, n_out = shape
    X, G, _ = O.make_linear_inputs(B, T, n_in, n_out, 1e-2, seed=sum(shape))
    G[0] *= 40.0
    _, n_gram = check_wgrad(X, G, 0.05, 1.0, torch.float32)
    _, n_direct = check_wgrad(X, G, 0.05, 1.0, torch.float32, norm_algo="direct")
    assert norm_err(n_gram.cpu().numpy(), n_direct.cpu().numpy()) < 1e-5


def test_dplinear_2d_large_batch_bf16():
    """2-D inputs (T = 1) with a batch large enough for the tensor-core clipped sum."""
    import flashdp4review_b200 as fdp
    B, n_in, n_out = 1024, 256, 128
    X, G, W = O.make_linear_inputs(B, 1, n_in, n_out, 1e-1, seed=77, dtype=torch.bfloat16)
    lin = fdp.DPLinear(n_in, n_out, C=0.3, noise_multiplier=0.0, dtype=torch.bfloat16).to(dev())
    with torch.no_grad():
        lin.weight.copy_(W)
    x = X[:, 0].to(dev()).requires_grad_(True)
    lin(x).backward(G[:, 0].to(dev()))
    want, _ = O.linear_weight_grad(G, X, 0.3, 1.0)
    want_b = O.linear_bias_grad(G, 0.3, 1.0)[0]
    assert rel_err(lin.weight.grad.float().cpu().numpy(), want) < 1e-2
    assert rel_err(lin.bias.grad.float().cpu().numpy(), want_b) < 1e-2
    assert x.grad.shape == x.shape


@pytest.mark.parametrize("w_layout", ["out_in", "in_out"])
@pytest.mark.parametrize("shape", [(2048, 1024, 768), (512, 256, 520), (4096, 4096, 1024), (130, 128, 136)],
                         ids=lambda s: "x".join(map(str, s)))
def test_fp32_forward_and_input_gradient_on_the_tensor_cores(shape, w_layout):
    """fp32 `linear_forward` / `linear_input_grad` as three bf16 tensor-core products with chained
    accumulation (the package default for fp32 where K is a multiple of 64): within the fp32 tolerance
    1e-5 of float64, bias included, output widths that are not multiples of the tile included; the
    flag off gives the fp32-FMA kernels, also within 1e-5."""
    from flashdp4review_b200.core import ops
    rows, n_in, n_out = shape
    gen = torch.Generator(device="cuda").manual_seed(rows + n_in + n_out)
    X = torch.randn(rows, n_in, device=dev(), generator=gen)
    G = torch.randn(rows, n_out, device=dev(), generator=gen) * 1e-2
    W = torch.randn(n_out, n_in, device=dev(), generator=gen) * 0.02
    bias = torch.randn(n_out, device=dev(), generator=gen)
    Wl = W if w_layout == "out_in" else W.t().contiguous()
    want_y = X.double() @ W.double().t() + bias.double()
    want_dx = G.double() @ W.double()
    from flashdp4review_b200 import runtime
    before = runtime.input_grad_impl()
    try:
        for impl, want in (("auto", n_in % 64 == 0 and rows >= 128), ("library", False)):
            runtime.set_input_grad_impl(impl)
            assert ops.native_product_ok(torch.float32, rows, n_in, n_out) == want
    finally:
        runtime.set_input_grad_impl(before)
    for mode in (None, True, False):
        y = ops.linear_forward(X, Wl, bias, w_layout, fp32_tensor=mode)
        dx = ops.linear_input_grad(G, Wl, w_layout, fp32_tensor=mode)
        assert y.dtype == torch.float32 and dx.dtype == torch.float32
        ey = float((y.double() - want_y).abs().max() / want_y.abs().max())
        ex = float((dx.double() - want_dx).abs().max() / want_dx.abs().max())
        assert ey < 1e-5 and ex < 1e-5, (mode, ey, ex)


def test_first_cuda_call_of_a_thread_may_be_a_library_call():
    """A host thread that has made no CUDA call yet has no context bound (an autograd worker thread
    running a DP layer's backward as its first node is such a thread).  The tensor-map encoder is a
    driver entry point and does not bind one on demand, so every entry point binds the device's
    primary context itself: a tensor-core GEMM called first thing in a new thread works."""
    import threading
    from flashdp4review_b200.core import ops
    X, G, W = O.make_linear_inputs(4, 256, 512, 384, 1e-3, seed=2, dtype=torch.bfloat16)
    g, w = G.to(dev()), W.to(dev())
    want = (G.double().reshape(-1, 384) @ W.double()).numpy()
    torch.cuda.synchronize()
    box = {}

    def work():
        try:
            box["dx"] = ops.linear_input_grad(g, w, "out_in")
        except Exception as e:      # surfaces in the main thread below
            box["err"] = e
    t = threading.Thread(target=work)
    t.start()
    t.join()
    assert "err" not in box, box.get("err")
    torch.cuda.synchronize()
    got = box["dx"].float().cpu().numpy().reshape(-1, 512)
    assert np.abs(got - want).max() / np.abs(want).max() < 1e-2
