"""Whole models through the wrap API on the GPU: a two-block Llama-2-7B-shaped decoder at full layer
sizes (d 4096, SwiGLU 11008, seq 2048, micro-batch 4, bf16), every Linear but lm_head wrapped, each DP
layer's weight gradient compared with a float64 evaluation of the reference's per-sample algorithm
(`_weight_grad_block_clip`, flashdp/core/linear_clip.py:94-104, then `.div_(B)`,
flashdp/layers/linear.py:72-73) on the inputs and upstream gradients that layer actually saw."""
import pytest
import torch

from gpu_util import dev

pytestmark = pytest.mark.gpu


def _fp64_clipped_mean(G, X, C, clamp):
    B = G.shape[0]
    acc = torch.zeros(G.shape[-1], X.shape[-1], dtype=torch.float64, device=G.device)
    norms = []
    for b in range(B):
        g = G[b].double().t() @ X[b].double()
        n = torch.linalg.norm(g)
        norms.append(float(n))
        acc += g * torch.clamp(C / (n + 1e-10), max=clamp)
    return acc / B, norms


def test_llama_shaped_two_blocks_layer_by_layer():
    import bench
    import flashdp4review_b200 as fdp
    from flashdp4review_b200.layers.linear import DPLinear
    torch.manual_seed(0)
    C = 1e-3                       # small enough that most samples are clipped in most layers
    model = bench.build_llama(layers=2, dtype=torch.bfloat16, device=dev())
    fdp.wrap_with_flashdp_layers(model, target_modules=[torch.nn.Linear], skip_layers=["lm_head"], C=C,
                                 noise_multiplier=0.0, feedback=False)
    layers = {n: m for n, m in model.named_modules() if isinstance(m, DPLinear)}
    assert len(layers) == 14 and not isinstance(model.lm_head, DPLinear)
    seen = {}
    hooks = []
    for name, m in layers.items():
        hooks.append(m.register_forward_hook(lambda mod, inp, out, name=name: seen.setdefault(name, {}).update(x=inp[0].detach())))
        hooks.append(m.register_full_backward_hook(lambda mod, gi, go, name=name: seen[name].update(g=go[0].detach())))
    gen = torch.Generator().manual_seed(42)
    tok = torch.randint(0, 32000, (4, 2049), generator=gen).to(dev())
    logits = model(tok[:, :-1])
    loss = torch.nn.functional.cross_entropy(logits.float().view(-1, 32000), tok[:, 1:].reshape(-1))
    loss.backward()
    torch.cuda.synchronize()
    for h in hooks:
        h.remove()
    worst = 0.0
    clipped = 0
    for name, m in layers.items():
        X, G = seen[name]["x"], seen[name]["g"]
        assert X.shape[:2] == (4, 2048) and G.shape[:2] == (4, 2048)
        want, norms = _fp64_clipped_mean(G, X, C, 1.0)
        clipped += sum(n > C for n in norms)
        got = m.weight.grad.double()
        assert got.shape == want.shape
        # the gradient is stored in the weight's dtype (bf16): one rounding on top of the bf16 tolerance
        err = float((got - want).abs().max() / want.abs().max())
        worst = max(worst, err)
        assert err < 1e-2 + 2.0 ** -8, (name, err)
    assert clipped > 0
    assert model.lm_head.weight.grad is not None
