"""GPU parity of the Linear / Conv1D weight, bias and input gradients against the oracle and the
fixtures made by the reference.  Every call goes through the C ABI (ctypes -> libfdp_b200.so)."""
import ctypes
import math

import numpy as np
import pytest
import torch

from oracle import dp_oracle as O
from conftest import rel_err, norm_err
from gpu_util import TOL, dev, check_wgrad

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from flashdp4review_b200.core import ops
    return ops


def test_library_loaded_and_device_ok():
    from flashdp4review_b200 import _lib
    lib = _lib.load()
    assert lib.fdp_abi_version() == _lib.ABI_VERSION
    assert lib.fdp_check_device(0) == 0


def test_cfg1_against_reference_fixture(golden, ops):
    g = golden("linear_cfg1.npz")
    B, T, n_in, n_out = (int(v) for v in g["meta"])
    X, G, W = O.make_linear_inputs(B, T, n_in, n_out, float(g["g_scale"]), int(g["seed"]))
    dW, norms = check_wgrad(X, G, 1.0, 1.0, torch.float32)
    assert norm_err(norms.cpu().numpy(), g["wnorms"]) < 1e-5
    got = dW.cpu().numpy()
    assert np.abs(got[::16, ::16] - g["dW_sub"]).max() / float(g["dW_absmax"]) < 1e-5
    db, bn, _ = ops.dp_bias_grad(G.to(dev()), 1.0, 1.0, return_norms=True)
    assert norm_err(bn.cpu().numpy(), g["bnorms"]) < 1e-5
    assert rel_err(db.cpu().numpy(), g["db"]) < 1e-5


def test_small_reference_fixtures(golden, ops):
    g = golden("linear_small.npz")
    for i in range(int(g["n_cases"])):
        C, clamp = (float(v) for v in g[f"c{i}_hp"])
        X, G = torch.from_numpy(g[f"c{i}_X"]), torch.from_numpy(g[f"c{i}_G"])
        dW, norms = check_wgrad(X, G, C, clamp, torch.float32)
        assert rel_err(dW.cpu().numpy(), g[f"c{i}_dW"]) < 1e-5, i
        assert norm_err(norms.cpu().numpy(), g[f"c{i}_wnorms"]) < 1e-5, i
        db = ops.dp_bias_grad(G.to(dev()), C, clamp)
        assert rel_err(db.cpu().numpy(), g[f"c{i}_db"]) < 1e-5, i


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 1, 8, 8), (2, 7, 24, 8), (3, 64, 136, 64), (3, 130, 64, 136),
                                   (2, 33, 72, 40), (1, 200, 100, 36), (5, 16, 768, 24)])
def test_ragged_shapes(shape, dtype):
    B, T, n_in, n_out = shape
    X, G, _ = O.make_linear_inputs(B, T, n_in, n_out, 2e-2, seed=sum(shape), dtype=dtype)
    check_wgrad(X, G, 0.5, 1.0, dtype)
    check_wgrad(X, G, 0.5, 1.0, dtype, layout="in_out")


def test_mixed_all_none_clipped():
    X, G, _ = O.make_linear_inputs(4, 32, 64, 48, 1e-2, seed=3)
    G[0] *= 50
    G[3] *= 0.01
    for C, clamp in [(1.0, 1.0), (1e-6, 1.0), (1e6, 1.0), (1.0, 0.25), (3.0, 7.0)]:
        check_wgrad(X, G, C, clamp, torch.float32)


def test_zero_gradient(ops):
    X, G, _ = O.make_linear_inputs(2, 8, 16, 16, 1.0, seed=1)
    G.zero_()
    dW, norms, factors = ops.dp_linear_weight_grad(X.to(dev()), G.to(dev()), 1.0, 0.75, return_norms=True)
    assert float(dW.abs().max()) == 0.0 and float(norms.abs().max()) == 0.0
    assert torch.all(factors == 0.75)          # norm 0 -> C/1e-10 saturates at clamp_value
    db = ops.dp_bias_grad(G.to(dev()), 1.0, 0.75)
    assert float(db.abs().max()) == 0.0


def test_fp32_output_from_bf16_inputs():
    X, G, _ = O.make_linear_inputs(3, 40, 72, 56, 1e-2, seed=5, dtype=torch.bfloat16)
    check_wgrad(X, G, 1.0, 1.0, torch.bfloat16, out_dtype=torch.float32, tol=2e-3)


def test_batch_divisor_and_drop_in_functions(ops):
    X, G, _ = O.make_linear_inputs(3, 12, 24, 16, 5e-2, seed=8)
    s = ops.linear_weight_flashdp(X.to(dev()), G.to(dev()), 0.7, 1.0, None)      # clipped SUM
    want, _ = O.linear_weight_grad(G, X, 0.7, 1.0, batch_divisor=1)
    assert rel_err(s.cpu().numpy(), want) < 1e-5
    s2 = ops.bmtm_clip(G.to(dev()), X.to(dev()), clip_args=torch.tensor([0.7, 1.0]))
    assert torch.equal(s, s2)
    c = ops.conv1d_weight_flashdp(X.to(dev()), G.to(dev()), 0.7, 1.0)
    assert rel_err(c.cpu().numpy(), want.T) < 1e-5
    d6 = ops.dp_linear_weight_grad(X.to(dev()), G.to(dev()), 0.7, 1.0, batch_divisor=6)
    assert rel_err(d6.cpu().numpy(), want / 6) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 5, 8), (3, 64, 136), (4, 130, 768), (2, 1, 3), (3, 77, 1000)])
def test_bias_grad(shape, dtype, ops):
    B, T, n_out = shape
    gen = torch.Generator().manual_seed(B * 100 + T)
    G = (torch.randn(B, T, n_out, generator=gen) * 0.05).to(dtype)
    G[0] *= 20
    db, norms, factors = ops.dp_bias_grad(G.to(dev()), 0.8, 1.0, return_norms=True)
    want, wn, wf = O.linear_bias_grad(G, 0.8, 1.0)
    tol = TOL[dtype]
    assert norm_err(norms.cpu().numpy(), wn) < tol
    assert rel_err(db.float().cpu().numpy(), want) < tol
    # the input is not modified (the reference scales it in place)
    assert torch.equal(G, G.clone())


def test_bias_input_left_untouched(ops):
    G = torch.randn(3, 9, 40, device=dev()) * 3
    keep = G.clone()
    ops.linear_bias_grad_clip(G, 1.0, 1.0)
    assert torch.equal(G, keep)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout", ["out_in", "in_out"])
def test_input_grad(layout, dtype, ops):
    X, G, W = O.make_linear_inputs(3, 37, 72, 40, 1e-1, seed=12, dtype=dtype)
    Wd = W if layout == "out_in" else W.t().contiguous()
    dX = ops.linear_input_grad(G.to(dev()), Wd.to(dev()), layout)
    want = G.double().numpy() @ W.double().numpy()
    assert dX.shape == X.shape
    assert rel_err(dX.float().cpu().numpy(), want) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layout", ["out_in", "in_out"])
@pytest.mark.parametrize("shape", [(3, 37, 72, 40), (2, 128, 256, 384), (1, 200, 136, 328)])
def test_forward_gemm(shape, layout, dtype, ops):
    B, T, n_in, n_out = shape
    X, _, W = O.make_linear_inputs(B, T, n_in, n_out, 1e-1, seed=21, dtype=dtype)
    bias = (torch.linspace(-0.5, 0.5, n_out)).to(dtype)
    Wd = W if layout == "out_in" else W.t().contiguous()
    for b in (None, bias):
        Y = ops.linear_forward(X.to(dev()), Wd.to(dev()), None if b is None else b.to(dev()), layout)
        want = X.double().numpy() @ W.double().numpy().T + (0 if b is None else b.double().numpy())
        assert Y.shape == (B, T, n_out)
        assert rel_err(Y.float().cpu().numpy(), want) < TOL[dtype]


# ---- noise ---------------------------------------------------------------------------------------
def _noise_only(ops, n_out, n_in, std, seed, pid, step, rank=0, world=1, layout="out_in", dtype=torch.float32):
    X = torch.zeros(2, 4, n_in, device=dev(), dtype=dtype)
    G = torch.zeros(2, 4, n_out, device=dev(), dtype=dtype)
    ns = ops.NoiseSpec(std=std, seed=seed, param_id=pid, step=step, rank=rank, world=world)
    return ops.dp_linear_weight_grad(X, G, 1.0, 1.0, noise=ns, layout=layout, out_dtype=torch.float32)


def test_noise_matches_host_philox_and_is_deterministic(ops):
    a = _noise_only(ops, 40, 24, 0.5, seed=2 ** 40 + 17, pid=3, step=11)
    b = _noise_only(ops, 40, 24, 0.5, seed=2 ** 40 + 17, pid=3, step=11)
    assert torch.equal(a, b)
    want = O.gaussian_noise(40 * 24, 0.5, 2 ** 40 + 17, 3, 11).reshape(40, 24)
    assert np.abs(a.cpu().numpy() - want).max() < 2e-6
    for kw in (dict(seed=2 ** 40 + 18, pid=3, step=11), dict(seed=2 ** 40 + 17, pid=4, step=11),
               dict(seed=2 ** 40 + 17, pid=3, step=12)):
        assert not torch.equal(a, _noise_only(ops, 40, 24, 0.5, **kw))
    # Conv1D orientation: same stream indexed by the output's own flat index
    c = _noise_only(ops, 40, 24, 0.5, seed=2 ** 40 + 17, pid=3, step=11, layout="in_out")
    assert np.abs(c.cpu().numpy().reshape(-1) - want.reshape(-1)).max() < 2e-6


def test_noise_statistics(ops):
    from scipy import stats
    z = _noise_only(ops, 1024, 1024, 0.25, seed=9, pid=1, step=1).cpu().numpy().reshape(-1)
    n = z.size
    assert abs(z.mean()) < 4 * 0.25 / math.sqrt(n)
    assert abs(z.std() / 0.25 - 1) < 0.01
    assert stats.kstest(z[:200000] / 0.25, "norm").pvalue > 1e-3


def test_noise_partition_over_ranks_sums_to_single_rank_noise(ops):
    full = _noise_only(ops, 24, 40, 1.0, seed=5, pid=2, step=3)
    acc = torch.zeros_like(full)
    for r in range(4):
        part = _noise_only(ops, 24, 40, 1.0, seed=5, pid=2, step=3, rank=r, world=4)
        assert int((part != 0).sum()) <= full.numel() // 4 + 4
        acc += part
    assert torch.equal(acc, full)


def test_bias_noise(ops):
    G = torch.zeros(2, 3, 4096, device=dev())
    ns = ops.NoiseSpec(std=0.5, seed=1, param_id=9, step=2)
    db = ops.dp_bias_grad(G, 1.0, 1.0, noise=ns)
    assert np.abs(db.cpu().numpy() - O.gaussian_noise(4096, 0.5, 1, 9, 2)).max() < 2e-6


# ---- ABI error behaviour ---------------------------------------------------------------------------
def test_abi_status_codes():
    from flashdp4review_b200 import _lib
    lib = _lib.load()
    p = _lib.DPParams(1.0, 1.0, 0.0, 0, 0, 0, 0, 0, 0, 1)
    t = torch.zeros(2 * 4 * 8, device=dev())
    ws = torch.empty(1 << 20, dtype=torch.uint8, device=dev())
    args = dict(B=2, T=4, n_in=8, n_out=8)

    def call(G=t.data_ptr(), X=t.data_ptr(), dW=t.data_ptr(), dt=_lib.FDP_F32, layout=0, algo=0, B=2,
             wsp=ws.data_ptr(), wsn=ws.numel(), pp=p):
        return lib.fdp_linear_wgrad(G, X, dW, None, None, B, 4, 8, 8, dt, _lib.FDP_F32, layout, algo,
                                    ctypes.byref(pp) if pp is not None else None, wsp, wsn, None)
    assert call() == _lib.FDP_OK
    assert call(G=None) == _lib.FDP_ERR_ARG
    assert call(B=0) == _lib.FDP_ERR_ARG
    assert call(layout=5) == _lib.FDP_ERR_ARG
    assert call(dt=7) == _lib.FDP_ERR_DTYPE
    assert call(G=t.data_ptr() + 4) == _lib.FDP_OK            # generic kernels: single-element accesses
    big = torch.zeros(2 * 64 * 256 + 8, device=dev(), dtype=torch.bfloat16)
    tc = lambda off: lib.fdp_linear_wgrad(big.data_ptr() + off, big.data_ptr(), big.data_ptr(), None, None, 2, 64, 128,
                                          256, _lib.FDP_BF16, _lib.FDP_BF16, 0, 0, ctypes.byref(p), ws.data_ptr(),
                                          ws.numel(), None)
    assert ws.numel() < lib.fdp_linear_wgrad_workspace_bytes(2, 64, 128, 256, _lib.FDP_BF16, 0)
    assert tc(0) == _lib.FDP_ERR_WORKSPACE                   # tensor-core shape: needs its parking area
    ws_tc = torch.empty(lib.fdp_linear_wgrad_workspace_bytes(2, 64, 128, 256, _lib.FDP_BF16, 0), dtype=torch.uint8, device=dev())
    tc2 = lambda off: lib.fdp_linear_wgrad(big.data_ptr() + off, big.data_ptr(), big.data_ptr(), None, None, 2, 64, 128,
                                           256, _lib.FDP_BF16, _lib.FDP_BF16, 0, 0, ctypes.byref(p), ws_tc.data_ptr(),
                                           ws_tc.numel(), None)
    assert tc2(4) == _lib.FDP_ERR_ALIGN                      # TMA operands must sit on 16-byte boundaries
    assert call(wsp=None) == _lib.FDP_ERR_WORKSPACE
    assert call(wsn=8) == _lib.FDP_ERR_WORKSPACE
    assert call(pp=None) == _lib.FDP_ERR_ARG
    torch.cuda.synchronize()
    with pytest.raises(KeyError):
        from flashdp4review_b200.core import ops
        ops.dp_linear_weight_grad(torch.zeros(1, 1, 8, device=dev(), dtype=torch.int8),
                                  torch.zeros(1, 1, 8, device=dev(), dtype=torch.int8), 1.0, 1.0)
    with pytest.raises(RuntimeError):
        from flashdp4review_b200.core import ops
        ops.dp_linear_weight_grad(torch.zeros(1, 1, 8), torch.zeros(1, 1, 8), 1.0, 1.0)   # CPU tensors


def test_views_with_a_storage_offset(ops):
    """A contiguous view that starts off a 16-byte boundary (x[1:] of a 3-column fp32 tensor; a bf16
    tensor-core shape shifted by one row of 8 bytes): the generic kernels read it in place, the
    tensor-core path gets an aligned copy from the operator layer."""
    gen = torch.Generator().manual_seed(4)
    Xf = torch.randn(5, 6, 3, generator=gen)
    Gf = torch.randn(5, 6, 5, generator=gen) * 0.1
    got = ops.dp_linear_weight_grad(Xf.to(dev())[1:], Gf.to(dev())[1:], 0.5, 1.0)
    want, _ = O.linear_weight_grad(Gf[1:], Xf[1:], 0.5, 1.0)
    assert rel_err(got.cpu().numpy(), want) < 1e-5
    Xb = torch.randn(3 * 64 * 132 + 4, generator=gen).to(torch.bfloat16)
    Gb = (torch.randn(3 * 64 * 136 + 4, generator=gen) * 0.01).to(torch.bfloat16)
    xv = Xb.to(dev())[4:].view(3, 64, 132)[:, :, :128].contiguous()
    gv = Gb.to(dev())[4:].view(3, 64, 136)
    assert gv.data_ptr() % 16 == 8
    got = ops.dp_linear_weight_grad(xv, gv, 0.05, 1.0, out_dtype=torch.float32)
    want, _ = O.linear_weight_grad(gv.cpu(), xv.cpu(), 0.05, 1.0)
    assert rel_err(got.cpu().numpy(), want) < 1e-2


@pytest.mark.parametrize("shape", [(3, 256, 768, 768), (2, 200, 520, 264), (2, 512, 256, 192), (1, 130, 1024, 512)])
def test_fp32_exact_norm_algorithms_agree(shape):
    """fp32 inputs on the exact (fp32 FMA) kernels: the product form and the Gram form of the per-sample
    norm, and the automatic choice between them, all hold the fp32 tolerance; partial blocks (T not a
    multiple of 128, features not multiples of 128) included."""
    B, T, n_in, n_out = shape
    X, G, _ = O.make_linear_inputs(B, T, n_in, n_out, 1e-2, seed=sum(shape))
    G[0] *= 40.0
    norms = {}
    for algo in ("auto", "direct", "gram"):
        _, n = check_wgrad(X, G, 0.05, 1.0, torch.float32, norm_algo=algo, fp32_tensor=False)
        norms[algo] = n.cpu().numpy()
    assert norm_err(norms["direct"], norms["gram"]) < 1e-5


def test_two_dimensional_inputs_with_more_than_65535_rows(ops):
    """A 2-D layer input is `rows` samples of one row each (flashdp/layers/linear.py:51-53); the batch is
    not a grid dimension of any kernel, so it may exceed 65535."""
    B = 70001
    gen = torch.Generator().manual_seed(8)
    X = torch.randn(B, 1, 40, generator=gen)
    G = torch.randn(B, 1, 24, generator=gen) * 0.05
    G[::7] *= 30
    dW, norms, _ = ops.dp_linear_weight_grad(X.to(dev()), G.to(dev()), 0.5, 1.0, return_norms=True)
    want, wn = O.linear_weight_grad(G, X, 0.5, 1.0)
    # the clipped sum runs over 70001 signed terms per element in fp32: its rounding alone reaches 1e-5
    assert norm_err(norms.cpu().numpy(), wn) < 1e-5 and rel_err(dW.cpu().numpy(), want) < 3e-5
    dWd, nd, _ = ops.dp_linear_weight_grad(X.to(dev()), G.to(dev()), 0.5, 1.0, return_norms=True, norm_algo="direct")
    assert norm_err(nd.cpu().numpy(), wn) < 1e-5 and rel_err(dWd.cpu().numpy(), want) < 3e-5
    db, nb, _ = ops.dp_bias_grad(G.to(dev()), 0.5, 1.0, return_norms=True)
    wdb, wnb, _ = O.linear_bias_grad(G, 0.5, 1.0)
    assert norm_err(nb.cpu().numpy(), wnb) < 1e-5 and rel_err(db.cpu().numpy(), wdb) < 1e-5
    # LayerNorm with as many samples
    d = 32
    xl = torch.randn(B, d, generator=gen)
    dy = torch.randn(B, d, generator=gen) * 0.1
    y, buf, _ = ops.layernorm_fwd_fused(xl.to(dev()), torch.ones(d, device=dev()), torch.zeros(d, device=dev()), 1e-5)
    _, dg, dbt = ops.dp_layernorm_backward(dy.to(dev()), xl.to(dev()), torch.ones(d, device=dev()), buf["mean"], buf["rstd"],
                                           0.2, 1.0)
    _, wmean, wrstd = O.layernorm_fwd(xl, np.ones(d), np.zeros(d), 1e-5)
    xhat = (xl.double().numpy() - wmean[..., None]) * wrstd[..., None]
    wdg, wdbt, _, _ = O.layernorm_affine_grads(dy.reshape(B, 1, d), xhat.reshape(B, 1, d), 0.2, 1.0)
    assert rel_err(dg.cpu().numpy(), wdg) < 2e-5 and rel_err(dbt.cpu().numpy(), wdbt) < 2e-5


def test_core_exports_match_the_reference_and_mm_fused(ops):
    """Every name flashdp.core exports (flashdp/core/__init__.py:1-11) exists here; mm_fused is the plain
    product with fp32 accumulation and output (flashdp/core/linear_clip.py:64-91)."""
    from flashdp4review_b200 import core
    for name in ("mm_clip", "bmm_clip", "bmtm_clip", "mm_fused", "linear_weight_flashdp", "linear_bias_grad_clip",
                 "layernorm_dw_clip", "layernorm_db_clip", "layernorm_fwd_fused", "layernorm_bwd_clip_fused",
                 "layernorm_dwdb_fused"):
        assert callable(getattr(core, name)), name
    gen = torch.Generator().manual_seed(2)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        A = torch.randn(3, 50, 136, generator=gen).to(dtype)
        Bm = (torch.randn(136, 264, generator=gen) * 0.1).to(dtype)
        out = core.mm_fused(A.to(dev()), Bm.to(dev()))
        assert out.dtype == torch.float32 and out.shape == (3, 50, 264)
        assert rel_err(out.cpu().numpy(), A.double().numpy() @ Bm.double().numpy()) < tol
    with pytest.raises(ValueError):
        core.mm_fused(torch.zeros(4, 5, device=dev()), torch.zeros(6, 3, device=dev()))


def test_bounded_wait_that_runs_out_is_reported_and_sticky():
    """A one-warp kernel waits about a millisecond on a barrier nobody arrives on.  It must return
    normally, leave its code in the workspace word and in the device's host-visible word, make every
    later compute call fail with FDP_ERR_TIMEOUT (RuntimeError in Python) until the flag is cleared,
    and leave the device fully usable."""
    from flashdp4review_b200 import _lib, runtime
    from flashdp4review_b200.core import ops
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.zeros(256, dtype=torch.uint8, device=dev())
    assert lib.fdp_async_status(-1) == _lib.FDP_OK
    try:
        assert lib.fdp_selftest_wait_timeout(2_000_000, ws.data_ptr(), ws.numel(), stream) == _lib.FDP_OK
        assert lib.fdp_device_status(ws.data_ptr(), stream) == _lib.FDP_ERR_TIMEOUT
        assert int(ws[:4].view(torch.int32).item()) == 9
        assert lib.fdp_async_status(-1) == _lib.FDP_ERR_TIMEOUT
        with pytest.raises(RuntimeError, match="bounded device-side wait"):
            runtime.check_device_status()
        X = torch.zeros(2, 4, 8, device=dev())
        with pytest.raises(RuntimeError, match="bounded device-side wait"):
            ops.dp_linear_weight_grad(X, X, 1.0, 1.0)
        with pytest.raises(RuntimeError, match="bounded device-side wait"):
            ops.dp_bias_grad(X, 1.0, 1.0)
    finally:
        runtime.clear_device_status()
    assert lib.fdp_async_status(-1) == _lib.FDP_OK
    X, G, _ = O.make_linear_inputs(2, 64, 128, 128, 1e-2, seed=3, dtype=torch.bfloat16)
    got = ops.dp_linear_weight_grad(X.to(dev()), G.to(dev()), 0.05, 1.0, out_dtype=torch.float32)
    want, _ = O.linear_weight_grad(G, X, 0.05, 1.0)
    assert rel_err(got.cpu().numpy(), want) < 1e-2


def test_bmm_clip_and_per_token_mm_clip(ops):
    """The two operators flashdp.core exports beside bmtm_clip (flashdp/core/__init__.py:1-3):
    bmm_clip sums clip(A_b B_b) over the batch, mm_clip clips every rank-one term a_k b_k^T."""
    import numpy as np
    gen = torch.Generator().manual_seed(12)
    A = torch.randn(3, 20, 14, generator=gen) * 0.3
    Bm = torch.randn(3, 14, 24, generator=gen)
    A[1] *= 10.0
    clip = torch.tensor([0.9, 1.0])
    got = ops.bmm_clip(A.to(dev()), Bm.to(dev()), clip_args=clip).cpu().numpy()
    want = np.zeros((20, 24))
    for b in range(3):
        P = A[b].double().numpy() @ Bm[b].double().numpy()
        want += O.clip_factor(np.linalg.norm(P), 0.9, 1.0) * P
    assert rel_err(got, want) < 1e-5

    m1 = torch.randn(40, 50, generator=gen) * 0.2
    m2 = torch.randn(50, 32, generator=gen)
    m1[:, 7] *= 30.0
    got = ops.mm_clip(m1.to(dev()), m2.to(dev()), clip_args=clip).cpu().numpy()
    a, b = m1.double().numpy(), m2.double().numpy()
    f = O.clip_factor(np.linalg.norm(a, axis=0) * np.linalg.norm(b, axis=1), 0.9, 1.0)
    assert rel_err(got, (a * f[None, :]) @ b) < 1e-5
