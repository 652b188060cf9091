"""The Gaussian noise of the clipped-sum GEMM's per-sample epilogue (sequences of 256 rows or more,
a multiple of 64): the path the default benchmark workload takes.  There the noise of a whole tile is
added into the epilogue registers between sample segments, and a tile whose K range is split gets
it from the warp that sums the parked parts.  Checked here: the stream equals the host restatement
of Philox4x32-10 + Box-Muller element for element, its statistics on top of a non-zero gradient,
the partition over ranks, bit-equal reruns, and the same with single-CTA tiles (child process).

The reference draws torch.normal(0, noise_multiplier / sqrt(B)) from the global generator
(flashdp/layers/linear.py:74-80); only the distribution is a parity target, the stream is this
library's own.
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import dp_oracle as O
from gpu_util import dev

pytestmark = pytest.mark.gpu

STD, SEED, PID, STEP = 0.75, 99, 4, 6


def _spec(rank=0, world=1, std=STD):
    from flashdp4review_b200.core import ops
    return ops.NoiseSpec(std, SEED, PID, 0, STEP, rank, world)


def _want(shape, std=STD):
    return O.gaussian_noise(shape[0] * shape[1], std, SEED, PID, STEP).reshape(shape)


# (B, T, n_in, n_out): whole tiles only / K-split few-tile shapes whose cuts fall inside samples /
# partial tiles in both dimensions
ZERO_SHAPES = [(2, 256, 512, 384), (5, 512, 1024, 1024), (2, 1024, 256, 256), (3, 320, 264, 520), (1, 256, 2048, 1024)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("layout", ["out_in", "in_out"])
@pytest.mark.parametrize("shape", ZERO_SHAPES)
def test_zero_gradient_yields_the_host_noise_stream(shape, layout, dtype):
    from flashdp4review_b200.core import ops
    B, T, n_in, n_out = shape
    X = torch.zeros(B, T, n_in, device=dev(), dtype=dtype)
    G = torch.zeros(B, T, n_out, device=dev(), dtype=dtype)
    oshape = (n_out, n_in) if layout == "out_in" else (n_in, n_out)
    want = _want(oshape)
    got = ops.dp_linear_weight_grad(X, G, 1.0, 1.0, noise=_spec(), layout=layout, out_dtype=torch.float32,
                                    batch_divisor=3 * B)     # a divisor that is no power of two
    assert np.abs(got.cpu().numpy() - want).max() < 3e-6
    # 16-bit output: the same stream, rounded once
    got16 = ops.dp_linear_weight_grad(X, G, 1.0, 1.0, noise=_spec(), layout=layout, out_dtype=dtype)
    want16 = torch.from_numpy(want).to(torch.float32).to(dtype).float().numpy()
    tol = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    assert np.abs(got16.float().cpu().numpy() - want16).max() <= tol * np.abs(want).max()
    # the ranks' shares add up to the single-rank draw, each element drawn by exactly one rank
    for world in (2, 4):
        parts = [ops.dp_linear_weight_grad(X, G, 1.0, 1.0, noise=_spec(r, world), layout=layout,
                                           out_dtype=torch.float32) for r in range(world)]
        nonzero = sum((p != 0).to(torch.int32) for p in parts)
        assert int(nonzero.max()) <= 1
        assert np.abs(sum(parts).cpu().numpy() - want).max() < 3e-6


def test_split_k_tail_tiles_get_their_noise_once():
    """4096 x 4096 with K = 4 x 1024: 256 pair tiles on 74 CTA pairs leave a tail wave whose tiles are
    cut along K; their noise is added by the warp that sums the parts."""
    from flashdp4review_b200.core import ops
    B, T, n = 4, 1024, 4096
    X = torch.zeros(B, T, n, device=dev(), dtype=torch.bfloat16)
    G = torch.zeros(B, T, n, device=dev(), dtype=torch.bfloat16)
    got = ops.dp_linear_weight_grad(X, G, 1.0, 1.0, noise=_spec(), out_dtype=torch.float32)
    assert np.abs(got.cpu().numpy() - _want((n, n))).max() < 3e-6


@pytest.mark.parametrize("shape", [(2, 256, 1024, 1024), (5, 512, 1024, 1024)])
def test_noise_statistics_on_top_of_a_gradient(shape):
    """dW(sigma) - dW(0) over 2^20 elements: mean, variance and Kolmogorov-Smirnov against N(0, std^2),
    and bit-equal reruns with the noise on."""
    from scipy import stats
    from flashdp4review_b200.core import ops
    B, T, n_in, n_out = shape
    X, G, _ = O.make_linear_inputs(B, T, n_in, n_out, 1e-3, seed=5, dtype=torch.bfloat16)
    Xd, Gd = X.to(dev()), G.to(dev())
    std = 0.5 / np.sqrt(B)
    run = lambda s: ops.dp_linear_weight_grad(Xd, Gd, 1.0, 1.0, noise=_spec(std=s), out_dtype=torch.float32)
    clean, noisy, again = run(0.0), run(std), run(std)
    assert torch.equal(noisy, again)
    z = (noisy - clean).double().cpu().numpy().ravel() / std
    n = z.size
    assert n >= 1 << 20
    assert abs(z.mean()) < 4.0 / np.sqrt(n)
    assert abs(z.var() - 1.0) < 0.01
    assert stats.kstest(z[:: 4], "norm").pvalue > 1e-3
    # the draw does not depend on the gradient it is added to
    want = _want((n_out, n_in), std=1.0).ravel()
    assert np.abs(z - want).max() < 1e-3      # rounding of (dW + noise) - dW in fp32


_CHILD = r"""
import sys, numpy as np, torch
sys.path.insert(0, %r)
sys.path.insert(0, %r)
from oracle import dp_oracle as O
from flashdp4review_b200.core import ops
dev = torch.device("cuda:0")
worst = 0.0
for (B, T, n_in, n_out) in [(2, 256, 512, 384), (5, 512, 1024, 1024), (3, 320, 264, 520)]:
    X = torch.zeros(B, T, n_in, device=dev, dtype=torch.bfloat16)
    G = torch.zeros(B, T, n_out, device=dev, dtype=torch.bfloat16)
    for layout, shape in (("out_in", (n_out, n_in)), ("in_out", (n_in, n_out))):
        want = O.gaussian_noise(n_in * n_out, 0.75, 99, 4, 6).reshape(shape)
        got = ops.dp_linear_weight_grad(X, G, 1.0, 1.0, noise=ops.NoiseSpec(0.75, 99, 4, 0, 6), layout=layout,
                                        out_dtype=torch.float32)
        worst = max(worst, float(np.abs(got.cpu().numpy() - want).max()))
        acc = sum(ops.dp_linear_weight_grad(X, G, 1.0, 1.0, noise=ops.NoiseSpec(0.75, 99, 4, 0, 6, r, 2), layout=layout,
                                            out_dtype=torch.float32) for r in range(2))
        worst = max(worst, float(np.abs(acc.cpu().numpy() - want).max()))
torch.cuda.synchronize()
print("WORST", worst)
"""


@pytest.mark.parametrize("env", [{"FDP_TC_CTAS": "1"}, {"FDP_TC_RESERVE_SMS": "20"}, {"FDP_PDL": "0"}])
def test_noise_stream_with_single_cta_tiles_and_a_reduced_grid(env):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", _CHILD % (root, os.path.join(root, "tests"))],
                       env={**os.environ, **env}, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert float(r.stdout.strip().split("WORST")[-1]) < 3e-6
