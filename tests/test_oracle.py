"""The CPU oracle against the fixtures produced by the reference's own pure-PyTorch path."""
import math

import numpy as np

from oracle import dp_oracle as O
from conftest import rel_err, norm_err

FP32_TOL = 1e-5  # the fp32 parity tolerance of the path (norms and clipped gradients)


def test_cfg1_against_reference(golden):
    g = golden("linear_cfg1.npz")
    B, T, n_in, n_out = (int(v) for v in g["meta"])
    X, G, W = O.make_linear_inputs(B, T, n_in, n_out, float(g["g_scale"]), int(g["seed"]))
    # the generator recipe reproduces the very tensors the fixture was made from
    assert np.array_equal(X[0, 0, :8].numpy(), g["x_probe"])
    assert np.array_equal(G[0, 0, :8].numpy(), g["g_probe"])
    dW, norms = O.linear_weight_grad(G, X, float(g["C"]), float(g["clamp"]))
    assert norm_err(norms, g["wnorms"]) < FP32_TOL
    assert np.abs(dW[::16, ::16] - g["dW_sub"]).max() / float(g["dW_absmax"]) < FP32_TOL
    assert abs(dW.sum() - float(g["dW_sum"])) < 1e-4 * math.sqrt(float(g["dW_sumsq"]))
    assert abs((dW ** 2).sum() / float(g["dW_sumsq"]) - 1) < 1e-5
    db, bnorms, _ = O.linear_bias_grad(G, float(g["C"]), float(g["clamp"]))
    assert norm_err(bnorms, g["bnorms"]) < FP32_TOL
    assert rel_err(db, g["db"]) < FP32_TOL
    # Gram identity used by the tensor-core norm kernel
    assert norm_err(O.per_sample_wgrad_norms_gram(G, X), norms) < 1e-9


def test_small_cases_against_reference(golden):
    g = golden("linear_small.npz")
    for i in range(int(g["n_cases"])):
        C, clamp = (float(v) for v in g[f"c{i}_hp"])
        X, G = g[f"c{i}_X"], g[f"c{i}_G"]
        dW, norms = O.linear_weight_grad(G, X, C, clamp)
        assert norm_err(norms, g[f"c{i}_wnorms"]) < FP32_TOL, i
        assert rel_err(dW, g[f"c{i}_dW"]) < FP32_TOL, i
        db, bnorms, _ = O.linear_bias_grad(G, C, clamp)
        assert norm_err(bnorms, g[f"c{i}_bnorms"]) < FP32_TOL, i
        assert rel_err(db, g[f"c{i}_db"]) < FP32_TOL, i
        dWt, _ = O.linear_weight_grad(G, X, C, clamp, layout="in_out")
        assert np.array_equal(dWt, dW.T)
    assert float(g["zero_dW_absmax"]) == 0.0
    dW0, n0 = O.linear_weight_grad(np.zeros((2, 4, 8)), np.ones((2, 4, 8)), 1.0, 1.0)
    assert np.all(dW0 == 0) and np.all(n0 == 0)


def test_mixed_clip_case_is_mixed(golden):
    g = golden("linear_small.npz")
    C, clamp = (float(v) for v in g["c2_hp"])
    f = O.clip_factor(g["c2_wnorms"], C, clamp)
    assert (f < clamp).any() and (f == clamp).any()


def test_layer_linear_against_reference(golden):
    g = golden("layers.npz")
    C = float(g["lin_C"])
    X, G, W = g["lin_X"], g["lin_G"], g["lin_W"]
    dW, _ = O.linear_weight_grad(G, X, C, 1.0)
    db, _, _ = O.linear_bias_grad(G, C, 1.0)
    assert rel_err(dW, g["lin_dW"]) < FP32_TOL
    assert rel_err(db, g["lin_db"]) < FP32_TOL
    assert rel_err(G.astype(np.float64) @ W, g["lin_dx"]) < FP32_TOL


def test_conv1d_reference_quirk_is_bias_first(golden):
    """The reference's Conv1D backward scales grad_output by the bias clip factors in place
    before dx and dW are computed (flashdp/layers/transformers_conv1d.py:59-81)."""
    g = golden("layers.npz")
    C = float(g["lin_C"])
    X, G, W = g["lin_X"], g["lin_G"], g["lin_W"]
    db, _, c = O.linear_bias_grad(G, C, 1.0)
    assert rel_err(db, g["conv_db"]) < FP32_TOL
    Gs = G * c[:, None, None]
    assert rel_err(Gs @ W.astype(np.float64), g["conv_dx"]) < FP32_TOL
    dW, _ = O.linear_weight_grad(Gs, X, C, 1.0)          # [out,in], the reference's (wrong) orientation
    assert rel_err(dW, g["conv_dW_ref_orientation"]) < FP32_TOL


def test_layernorm_against_reference(golden):
    g = golden("layers.npz")
    C = float(g["ln_C"])
    X, DY, gamma, beta = g["ln_X"], g["ln_DY"], g["ln_gamma"], g["ln_beta"]
    y, mean, rstd = O.layernorm_fwd(X, gamma, beta, 1e-5)
    assert rel_err(y, g["ln_y"]) < FP32_TOL
    xhat = (X - mean[..., None]) * rstd[..., None]
    dgamma, dbeta, _, _ = O.layernorm_affine_grads(DY, xhat, C, 1.0)
    assert rel_err(dgamma, g["ln_dgamma_fn"]) < FP32_TOL
    assert rel_err(dbeta, g["ln_dbeta_fn"]) < FP32_TOL
    assert rel_err(dgamma, g["ln_dgamma"]) < FP32_TOL      # through the module, sigma = 0
    assert rel_err(dbeta, g["ln_dbeta"]) < FP32_TOL
    assert rel_err(O.layernorm_bwd_dx(DY, X, gamma, mean, rstd), g["ln_dx"]) < 5e-5


def test_torch_port_matches_float64():
    X, G, W = O.make_linear_inputs(3, 20, 24, 16, 5e-2, 9)
    acc = O.torch_port_weight_grad_block_clip(G, X, 0.8, 1.0) / 3
    dW, _ = O.linear_weight_grad(G, X, 0.8, 1.0)
    assert rel_err(acc.numpy(), dW) < FP32_TOL
    gi, gw, gb = O.torch_port_linear_backward(G, X, W, 0.8, 1.0, 0.0, True)
    db, _, _ = O.linear_bias_grad(G, 0.8, 1.0)
    assert rel_err(gw.numpy(), dW) < FP32_TOL and rel_err(gb.numpy(), db) < FP32_TOL


def test_philox_known_answers():
    # Random123 known-answer vectors for philox4x32-10
    kat = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
           ((0xffffffff,) * 4, (0xffffffff,) * 2, (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
           ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
            (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]
    for ctr, key, want in kat:
        got = O.philox4x32_10(np.array([ctr], dtype=np.uint32), np.array(key, dtype=np.uint32))[0]
        assert tuple(int(v) for v in got) == want


def test_noise_stream_statistics(golden):
    n = 1 << 20
    z = O.gaussian_noise(n, 0.5, seed=7, param_id=3, step=11)
    assert abs(z.mean()) < 4 * 0.5 / math.sqrt(n)
    assert abs(z.std() / 0.5 - 1) < 0.01
    from scipy import stats
    assert stats.kstest(z[:200000] / 0.5, "norm").pvalue > 1e-3
    assert not np.array_equal(z[:64], O.gaussian_noise(64, 0.5, 7, 4, 11))
    assert np.array_equal(z[:64], O.gaussian_noise(64, 0.5, 7, 3, 11))
    g = golden("noise_stats.npz")   # the reference's own noise: std = noise_multiplier/sqrt(B)
    assert abs(float(g["resid_std"]) / float(g["expected_std"]) - 1) < 0.03


def test_fused_saturation_restatement_against_a_row_by_row_loop():
    """The vectorised restatement of the reference's fused LayerNorm accumulation
    (flashdp/core/layernorm_clip.py:104-131 with a fixed row order) against the same recurrence written
    row by row, as the Triton program of one row would apply it."""
    import numpy as np
    from oracle import dp_oracle as O
    rng = np.random.default_rng(0)
    rows, d, C, clamp = 600, 8, 0.05, 1.0
    dy = rng.normal(size=(rows, d)).astype(np.float32) * 0.2
    xh = rng.normal(size=(rows, d)).astype(np.float32)
    G = O.layernorm_saturate_groups(rows, d)
    assert G == 256
    bw = np.zeros((G, d), np.float32)
    bb = np.zeros((G, d), np.float32)
    seen = np.zeros(G, bool)
    f = lambda b: np.minimum(np.float32(C) / (np.abs(b) + np.float32(1e-10)), np.float32(clamp))
    for r in range(rows):
        g = r % G
        pw, pb = dy[r] * xh[r], dy[r]
        if seen[g]:
            pw = pw + bw[g] * f(bw[g])
            pb = pb + bb[g] * f(bb[g])
        bw[g], bb[g], seen[g] = pw, pb, True
    dg, db, dw_, db_ = O.layernorm_fused_saturation(dy, xh, C, clamp)
    assert np.allclose(dw_, bw, rtol=1e-6, atol=1e-8) and np.allclose(db_, bb, rtol=1e-6, atol=1e-8)
    assert np.allclose(dg, bw.sum(0), rtol=1e-5, atol=1e-5) and np.allclose(db, bb.sum(0), rtol=1e-5, atol=1e-5)   # fp32 sums of 256 signed terms, two orders
    assert O.layernorm_saturate_groups(40, 2048) == 40 and O.layernorm_saturate_groups(10 ** 6, 8192) == 96
