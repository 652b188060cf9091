"""Generate the golden fixtures by running the REFERENCE's own pure-PyTorch per-sample path.

Run where a checkout of the reference is available:

    python tests/golden/make_golden.py /path/to/FlashDP4Review

The script imports `flashdp` from that path, drives `_weight_grad_block_clip`,
`linear_bias_grad_clip`, `layernorm_dw_clip`, `layernorm_db_clip` and the three autograd
Functions on CPU (the layers' runtime tuner is replaced by a stub that always returns the
pure-PyTorch function, since the stock tuner times the Triton path first and cannot run without
a GPU -- flashdp/core/utils.py:24-37), and writes small `.npz` files beside itself.  Nothing in
the test-suite reads the reference at run time; it reads these files.
"""
import math
import os
import sys

sys.dont_write_bytecode = True
HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FLASHDP_REFERENCE", "")
if not REF or not os.path.isdir(os.path.join(REF, "flashdp")):
    sys.exit("usage: make_golden.py <path to the reference checkout>")
sys.path.insert(0, REF)
sys.path.insert(0, REPO)

import numpy as np
import torch

from flashdp.core.linear_clip import _weight_grad_block_clip, linear_bias_grad_clip
from flashdp.core.layernorm_clip import layernorm_dw_clip, layernorm_db_clip
from flashdp.layers.linear import DPLinear
from flashdp.layers.layernorm import DPLayerNorm
from flashdp.layers.transformers_conv1d import DPConv1D
from oracle.dp_oracle import make_linear_inputs


class StubTuner:
    """Always picks the second candidate: the pure-PyTorch per-sample function."""
    def choose_function(self, funcs, *a, **k):
        return funcs[1]

    def final_tune(self):
        pass


def np32(t):
    return t.detach().float().numpy().copy()


def linear_case(B, T, n_in, n_out, g_scale, C, clamp, seed):
    X, G, W = make_linear_inputs(B, T, n_in, n_out, g_scale, seed)
    clip_args = torch.tensor([C, clamp])
    acc = _weight_grad_block_clip(G, X, clip_args=clip_args)
    # per-sample norms exactly as the reference computes them (einsum + torch.norm)
    norms = torch.stack([torch.norm(torch.einsum("k...m,k...n->kmn", G[b:b + 1], X[b:b + 1]),
                                    p=2, dim=(-1, -2)).reshape(()) for b in range(B)])
    Gc = G.clone()
    db = linear_bias_grad_clip(Gc, C, clamp)      # mutates Gc in place
    bnorms = torch.norm(G.reshape(B, -1), p=2, dim=-1)
    return X, G, W, acc / B, norms, db, bnorms


def main():
    torch.manual_seed(1234)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    out = {}

    # ---- config 1 of the benchmark description: fp32 B=4 T=128 768->768, bias, C=1 ----------
    X, G, W, dW, norms, db, bnorms = linear_case(4, 128, 768, 768, 1e-2, 1.0, 1.0, 0)
    np.savez_compressed(
        os.path.join(HERE, "linear_cfg1.npz"),
        meta=np.array([4, 128, 768, 768]), g_scale=1e-2, C=1.0, clamp=1.0, seed=0,
        dW_sub=np32(dW)[::16, ::16], dW_sum=float(dW.double().sum()),
        dW_sumsq=float((dW.double() ** 2).sum()), dW_absmax=float(dW.abs().max()),
        wnorms=np32(norms), db=np32(db), bnorms=np32(bnorms),
        x_probe=np32(X)[0, 0, :8], g_probe=np32(G)[0, 0, :8])
    print("cfg1 weight norms", norms.tolist(), "bias norms", bnorms.tolist())

    # ---- small cases kept in full (inputs included) ---------------------------------------
    small = {}
    cases = [  # B, T, in, out, g_scale, C, clamp, seed
        (1, 1, 8, 8, 1.0, 1.0, 1.0, 1),
        (2, 7, 24, 8, 1e-1, 1.0, 1.0, 2),
        (3, 64, 136, 64, 1e-2, 0.5, 1.0, 3),      # mixed: some samples clipped, some not
        (3, 130, 64, 136, 1e-3, 1.0, 1.0, 4),     # none clipped (factor saturates at clamp)
        (2, 33, 72, 40, 1e-2, 1.0, 0.25, 5),      # clamp_value < 1
        (5, 16, 32, 48, 3e-2, 2.0, 1.0, 6),
    ]
    for i, (B, T, n_in, n_out, gs, C, clamp, seed) in enumerate(cases):
        X, G, W, dW, norms, db, bnorms = linear_case(B, T, n_in, n_out, gs, C, clamp, seed)
        if i == 2:  # rescale two samples so that the clip is genuinely mixed
            G[0] *= 30.0
            G[2] *= 0.03
            clip_args = torch.tensor([C, clamp])
            dW = _weight_grad_block_clip(G, X, clip_args=clip_args) / B
            norms = torch.stack([torch.norm(G[b].t() @ X[b]) for b in range(B)])
            db = linear_bias_grad_clip(G.clone(), C, clamp)
            bnorms = torch.norm(G.reshape(B, -1), p=2, dim=-1)
        small[f"c{i}_meta"] = np.array([B, T, n_in, n_out])
        small[f"c{i}_hp"] = np.array([C, clamp])
        for k, v in dict(X=X, G=G, dW=dW, wnorms=norms, db=db, bnorms=bnorms).items():
            small[f"c{i}_{k}"] = np32(v)
    # zero upstream gradient: norm 0 -> factor = clamp_value, gradient stays 0
    X, G, W = make_linear_inputs(2, 4, 8, 8, 1.0, 7)
    G.zero_()
    dW0 = _weight_grad_block_clip(G, X, clip_args=torch.tensor([1.0, 1.0])) / 2
    small["zero_dW_absmax"] = float(dW0.abs().max())
    small["n_cases"] = len(cases)
    np.savez_compressed(os.path.join(HERE, "linear_small.npz"), **small)

    # ---- layer level: the reference autograd Functions at noise_multiplier = 0 -------------
    lay = {}
    B, T, n_in, n_out = 3, 10, 16, 16
    X, G, W = make_linear_inputs(B, T, n_in, n_out, 5e-2, 11)
    lin = DPLinear(n_in, n_out, bias=True, C=0.7, clamp_value=1.0, noise_multiplier=0.0)
    lin.runtime_tuner = StubTuner()
    with torch.no_grad():
        lin.weight.copy_(W)
        lin.bias.copy_(torch.linspace(-0.1, 0.1, n_out))
    x = X.clone().requires_grad_(True)
    y = lin(x)
    y.backward(G.clone())
    lay.update(lin_meta=np.array([B, T, n_in, n_out]), lin_C=0.7, lin_X=np32(X), lin_G=np32(G),
               lin_W=np32(W), lin_b=np32(lin.bias), lin_y=np32(y), lin_dx=np32(x.grad),
               lin_dW=np32(lin.weight.grad), lin_db=np32(lin.bias.grad))

    # Conv1D (square, the only shape the reference's backward accepts): bias is computed
    # first and scales grad_output in place, so dx and dW see the bias-scaled gradient.
    conv = DPConv1D(n_out, n_in, C=0.7, clamp_value=1.0, noise_multiplier=0.0)
    conv.runtime_tuner = StubTuner()
    with torch.no_grad():
        conv.weight.copy_(W.t())
    x = X.clone().requires_grad_(True)
    y = conv(x)
    y.backward(G.clone())
    lay.update(conv_y=np32(y), conv_dx=np32(x.grad), conv_dW_ref_orientation=np32(conv.weight.grad),
               conv_db=np32(conv.bias.grad))

    # LayerNorm, unfused path = true per-sample clipping (flashdp/layers/layernorm.py:108-167)
    B, T, d = 4, 9, 40
    gen = torch.Generator().manual_seed(21)
    X = torch.randn(B, T, d, generator=gen) * 1.5 + 0.3
    DY = torch.randn(B, T, d, generator=gen) * 0.2
    gamma = torch.randn(d, generator=gen) * 0.1 + 1.0
    beta = torch.randn(d, generator=gen) * 0.1
    ln = DPLayerNorm(d, eps=1e-5, use_fused=False, C=0.9, clamp_value=1.0, noise_multiplier=0.0)
    with torch.no_grad():
        ln.weight.copy_(gamma)
        ln.bias.copy_(beta)
    x = X.clone().requires_grad_(True)
    y = ln(x)
    y.backward(DY.clone())
    mean = X.mean(-1, keepdim=True)
    xhat = (X - mean) / torch.sqrt(X.var(-1, keepdim=True, unbiased=False) + 1e-5)
    dgw = layernorm_dw_clip(xhat, DY, gamma.reshape(1, 1, d), torch.Tensor([0.9]), torch.Tensor([1.0]))
    dgb = layernorm_db_clip(DY, beta.reshape(1, 1, d), torch.Tensor([0.9]), torch.Tensor([1.0]))
    lay.update(ln_meta=np.array([B, T, d]), ln_C=0.9, ln_X=np32(X), ln_DY=np32(DY),
               ln_gamma=np32(gamma), ln_beta=np32(beta), ln_y=np32(y), ln_dx=np32(x.grad),
               ln_dgamma=np32(ln.weight.grad).reshape(-1), ln_dbeta_fn=np32(dgb).reshape(-1),
               ln_dgamma_fn=np32(dgw).reshape(-1), ln_dbeta=np32(ln.bias.grad).reshape(-1))
    np.savez_compressed(os.path.join(HERE, "layers.npz"), **lay)

    # ---- noise statistics of the reference at sigma = 1 (distribution is the parity target) --
    torch.manual_seed(0)
    B, T, n_in, n_out = 16, 4, 64, 64
    X, G, W = make_linear_inputs(B, T, n_in, n_out, 1e-2, 31)
    lin = DPLinear(n_in, n_out, bias=True, C=1.0, clamp_value=1.0, noise_multiplier=2.0)
    lin.runtime_tuner = StubTuner()
    x = X.clone().requires_grad_(True)
    lin(x).backward(G.clone())
    clean = _weight_grad_block_clip(G, X, clip_args=torch.tensor([1.0, 1.0])) / B
    resid = lin.weight.grad - clean
    np.savez_compressed(os.path.join(HERE, "noise_stats.npz"), B=B, noise_multiplier=2.0,
                        resid_std=float(resid.std()), resid_mean=float(resid.mean()),
                        expected_std=2.0 / math.sqrt(B), n=resid.numel())
    print("reference noise std", float(resid.std()), "expected", 2.0 / math.sqrt(B))


if __name__ == "__main__":
    main()
