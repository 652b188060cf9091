"""CPU oracle for the DP-SGD backward hot path (TEST INFRASTRUCTURE, not product code).

This module restates, in float64 numpy, the arithmetic of the reference's pure-PyTorch
per-sample path.  Only the tests, the smoke check and the `cpu_baseline` / `--impl reference`
legs of the benchmark may import it; the product package never does.

Parity pin: the reference ships no tests and no golden vectors for this path, so the oracle
is pinned against outputs of the reference's own Python run on CPU (the fixtures under
``tests/golden/`` and the script beside them that imports the reference to make them).

Per parameter tensor, with ``f(n) = min(clamp_value, C / (n + 1e-10))``
(flashdp/core/clip_fn.py:6-8):

* Linear weight ``[out,in]``:  ``dW = (1/B) * sum_b f(||G_b^T X_b||_F) * G_b^T X_b``
  (flashdp/core/linear_clip.py:94-104, flashdp/layers/linear.py:72-73)
* Conv1D weight ``[in,out]``: the transpose of the above
  (flashdp/core/transformers_conv1d_clip.py:22-28)
* bias ``[out]``: ``db = (1/(B*T)) * sum_b f(||G_b||_F) * sum_t G_b[t,:]``
  (flashdp/core/linear_clip.py:116-123) -- the norm is over the whole T x out block
* LayerNorm: ``dgamma = (1/B) sum_b f(||sum_t dy_b*xhat_b||_2) * sum_t dy_b*xhat_b`` and
  ``dbeta`` alike with ``sum_t dy_b`` (flashdp/core/layernorm_clip.py:163-198)
* noise: ``+ N(0, (noise_multiplier/sqrt(B))^2)`` per element (flashdp/layers/linear.py:74-80)
"""
from __future__ import annotations

import math

import numpy as np

EPS_NORM = 1e-10  # flashdp/core/clip_fn.py:8


def _f64(a) -> np.ndarray:
    if hasattr(a, "detach"):  # torch tensor
        a = a.detach().to("cpu").double().numpy()
    return np.asarray(a, dtype=np.float64)


# --------------------------------------------------------------------------------------
# clip factor -- flashdp/core/clip_fn.py:6-8
# --------------------------------------------------------------------------------------
def clip_factor(norm, C: float, clamp_value: float) -> np.ndarray:
    """``clamp(C / (norm + 1e-10), max=clamp_value)``."""
    norm = _f64(norm)
    return np.minimum(C / (norm + EPS_NORM), clamp_value)


# --------------------------------------------------------------------------------------
# Linear / Conv1D weight gradient -- flashdp/core/linear_clip.py:94-104
# --------------------------------------------------------------------------------------
def per_sample_wgrad_norms(G, X) -> np.ndarray:
    """Frobenius norm of each sample's ``G_b^T X_b`` (linear_clip.py:99-100)."""
    G, X = _f64(G), _f64(X)
    out = np.empty(G.shape[0])
    for b in range(G.shape[0]):
        out[b] = np.linalg.norm(G[b].T @ X[b])
    return out


def per_sample_wgrad_norms_gram(G, X) -> np.ndarray:
    """Same norms through ``||G^T X||_F^2 = sum_{t,s} (G G^T)_{ts} (X X^T)_{ts}``."""
    G, X = _f64(G), _f64(X)
    out = np.empty(G.shape[0])
    for b in range(G.shape[0]):
        out[b] = math.sqrt(max(float(np.sum((G[b] @ G[b].T) * (X[b] @ X[b].T))), 0.0))
    return out


def linear_weight_grad(G, X, C: float, clamp_value: float, batch_divisor: int | None = None,
                       layout: str = "out_in"):
    """Clipped mean weight gradient and the per-sample norms.

    Follows `_weight_grad_block_clip` (flashdp/core/linear_clip.py:94-104) with BK=1 and the
    ``.div_(B)`` of flashdp/layers/linear.py:72-73.  ``layout='in_out'`` gives the Conv1D
    orientation of flashdp/core/transformers_conv1d_clip.py:22-28.
    Returns ``(dW, norms)``.
    """
    G, X = _f64(G), _f64(X)
    B = G.shape[0]
    div = B if batch_divisor is None else batch_divisor
    acc = np.zeros((G.shape[-1], X.shape[-1]))
    norms = np.empty(B)
    for b in range(B):
        g = G[b].T @ X[b]                       # einsum 'k...m,k...n->kmn', one sample
        norms[b] = np.linalg.norm(g)            # torch.norm(p=2, dim=(-1,-2))
        acc += clip_factor(norms[b], C, clamp_value) * g
    acc /= div
    return (acc if layout == "out_in" else acc.T.copy()), norms


# --------------------------------------------------------------------------------------
# bias gradient -- flashdp/core/linear_clip.py:116-123
# --------------------------------------------------------------------------------------
def linear_bias_grad(G, C: float, clamp_value: float, batch_divisor: int | None = None):
    """``mean over the B*T rows of (c_b * G)``; the norm of sample b is over its T*out block.

    Returns ``(db, norms, factors)``.  The reference scales ``grad_output`` in place
    (linear_clip.py:121); this restatement leaves its input untouched.
    """
    G = _f64(G)
    B, T = G.shape[0], G.shape[1]
    div = B if batch_divisor is None else batch_divisor
    norms = np.linalg.norm(G.reshape(B, -1), axis=1)
    c = clip_factor(norms, C, clamp_value)
    db = (c[:, None] * G.sum(axis=1)).sum(axis=0) / (div * T)
    return db, norms, c


# --------------------------------------------------------------------------------------
# LayerNorm -- forward flashdp/core/layernorm_clip.py:11-60, per-sample clip :163-198
# --------------------------------------------------------------------------------------
def layernorm_fwd(x, gamma, beta, eps: float):
    """Row-wise mean / biased variance / rstd / affine output (layernorm_clip.py:31-59)."""
    x, gamma, beta = _f64(x), _f64(gamma), _f64(beta)
    mean = x.mean(axis=-1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    rstd = 1.0 / np.sqrt(var + eps)
    y = (x - mean) * rstd * gamma + beta
    return y, mean[..., 0], rstd[..., 0]


def layernorm_bwd_dx(dy, x, gamma, mean, rstd):
    """Input gradient of LayerNorm (flashdp/core/layernorm_clip.py:95-103)."""
    dy, x, gamma = _f64(dy), _f64(x), _f64(gamma)
    mean, rstd = _f64(mean)[..., None], _f64(rstd)[..., None]
    xhat = (x - mean) * rstd
    wdy = gamma * dy
    c1 = (xhat * wdy).mean(axis=-1, keepdims=True)
    c2 = wdy.mean(axis=-1, keepdims=True)
    return (wdy - (xhat * c1 + c2)) * rstd


def layernorm_affine_grads(dy, xhat, C: float, clamp_value: float,
                           batch_divisor: int | None = None):
    """Per-sample clipped dgamma / dbeta for ``(B, T, d)`` tensors.

    `layernorm_dw_clip` (layernorm_clip.py:163-180) and `layernorm_db_clip` (:183-198): sum over
    the non-batch, non-feature axes, L2 norm over d, clip, mean over B.
    Returns ``(dgamma, dbeta, norms_gamma, norms_beta)``.
    """
    dy, xhat = _f64(dy), _f64(xhat)
    B, d = dy.shape[0], dy.shape[-1]
    div = B if batch_divisor is None else batch_divisor
    dyr, xr = dy.reshape(B, -1, d), xhat.reshape(B, -1, d)
    gw = (dyr * xr).sum(axis=1)
    gb = dyr.sum(axis=1)
    nw, nb = np.linalg.norm(gw, axis=1), np.linalg.norm(gb, axis=1)
    dgamma = (clip_factor(nw, C, clamp_value)[:, None] * gw).sum(axis=0) / div
    dbeta = (clip_factor(nb, C, clamp_value)[:, None] * gb).sum(axis=0) / div
    return dgamma, dbeta, nw, nb


def layernorm_saturate_groups(rows: int, d: int) -> int:
    """GROUP_SIZE_M of flashdp/core/layernorm_clip.py:261-264, capped by the row count (:309)."""
    g = 64
    if d <= 8192:
        g = 96
    if d <= 4096:
        g = 128
    if d <= 1024:
        g = 256
    return min(g, rows)


def layernorm_fused_saturation(dy, xhat, C: float, clamp_value: float, round_to=None):
    """The reference's FUSED dgamma / dbeta (flashdp/core/layernorm_clip.py:104-131, :134-160) with the
    rows of each of the G buffers added in increasing row order (the reference's order is whatever its
    spin lock yields): row r goes to buffer r % G; the first row of a buffer is stored, every later one
    is added to the buffer after the buffer was scaled element-wise by min(clamp, C / (|buf| + 1e-10)).
    Arithmetic in float32 like the reference's accumulation dtype; `round_to` (a torch dtype) rounds
    the per-row partials as the reference's `.to(w.dtype)` does.  Returns (dgamma, dbeta, dw_, db_)."""
    import torch
    dy = torch.as_tensor(_f64(dy)).float()
    xh = torch.as_tensor(_f64(xhat)).float()
    d = dy.shape[-1]
    dy, xh = dy.reshape(-1, d), xh.reshape(-1, d)
    rows = dy.shape[0]
    G = layernorm_saturate_groups(rows, d)
    bw = torch.zeros(G, d)
    bb = torch.zeros(G, d)
    f = lambda b: torch.clamp(C / (b.abs() + EPS_NORM), max=clamp_value)
    for k, r0 in enumerate(range(0, rows, G)):
        pw, pb = dy[r0:r0 + G] * xh[r0:r0 + G], dy[r0:r0 + G].clone()
        if round_to is not None:
            pw, pb = pw.to(round_to).float(), pb.to(round_to).float()
        n = pw.shape[0]
        if k == 0:
            bw[:n], bb[:n] = pw, pb
        else:
            bw[:n] = pw + bw[:n] * f(bw[:n])
            bb[:n] = pb + bb[:n] * f(bb[:n])
    return bw.sum(0).numpy(), bb.sum(0).numpy(), bw.numpy(), bb.numpy()


# --------------------------------------------------------------------------------------
# Gaussian noise: counter-based restatement of what the CUDA epilogues draw.
# The reference draws torch.normal(std=noise_multiplier/sqrt(B)) from the global generator
# (flashdp/layers/linear.py:74-80); only the distribution is a parity target.
# --------------------------------------------------------------------------------------
_PHILOX_M0, _PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32_10(ctr: np.ndarray, key: np.ndarray) -> np.ndarray:
    """Philox4x32-10 (Salmon et al., SC'11).  ``ctr``: (n,4) uint32, ``key``: (2,) uint32."""
    c = ctr.astype(np.uint64).copy()
    k0, k1 = np.uint64(key[0]), np.uint64(key[1])
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(_PHILOX_M0) * c[:, 0]
        p1 = np.uint64(_PHILOX_M1) * c[:, 2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        n0 = (hi1 ^ c[:, 1] ^ k0) & mask
        n2 = (hi0 ^ c[:, 3] ^ k1) & mask
        c = np.stack([n0, lo1, n2, lo0], axis=1)
        k0 = (k0 + np.uint64(_PHILOX_W0)) & mask
        k1 = (k1 + np.uint64(_PHILOX_W1)) & mask
    return c.astype(np.uint32)


def gaussian_noise(n: int, std: float, seed: int, param_id: int, step: int) -> np.ndarray:
    """The standard-normal stream of the CUDA epilogues, scaled by ``std``.

    Element ``i`` uses Philox counter ``(i>>2 low, i>>2 high, param_id, step)`` under key
    ``(seed low, seed high)``; lanes 0/1 are the cos/sin Box-Muller pair of words (0,1) and
    lanes 2/3 that of words (2,3); a word ``w`` maps to the uniform ``((w >> 9) + 0.5) * 2^-23``
    (exactly representable in fp32, so host and device agree on it bit for bit).
    """
    groups = (n + 3) // 4
    idx = np.arange(groups, dtype=np.uint64)
    ctr = np.stack([idx & np.uint64(0xFFFFFFFF), idx >> np.uint64(32),
                    np.full(groups, param_id, np.uint64), np.full(groups, step, np.uint64)], axis=1)
    key = np.array([seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF], dtype=np.uint64)
    r = (philox4x32_10(ctr, key) >> np.uint32(9)).astype(np.float64)
    u = (r + 0.5) * (2.0 ** -23)
    z = np.empty((groups, 4))
    for p in range(2):
        rad = np.sqrt(-2.0 * np.log(u[:, 2 * p]))
        ang = 2.0 * math.pi * u[:, 2 * p + 1]
        z[:, 2 * p] = rad * np.cos(ang)
        z[:, 2 * p + 1] = rad * np.sin(ang)
    return std * z.reshape(-1)[:n]


# --------------------------------------------------------------------------------------
# The same path as a sequence of torch CPU ops, op for op as the reference issues them.
# Used for the timed CPU baseline and to cross-check the float64 restatement in fp32.
# --------------------------------------------------------------------------------------
def torch_port_weight_grad_block_clip(grad_output, input, C: float, clamp_value: float):
    """Op-for-op port of `_weight_grad_block_clip` (flashdp/core/linear_clip.py:94-104), BK=1."""
    import torch
    M, K, N = grad_output.shape[-1], input.shape[0], input.shape[-1]
    acc = torch.zeros([M, N], dtype=input.dtype)
    for k in range(K):
        g = torch.einsum("k...m,k...n->kmn", grad_output[k:k + 1], input[k:k + 1])
        n = torch.norm(g, p=2, dim=(-1, -2), keepdim=True)
        f = torch.clamp(C / (n + EPS_NORM), max=clamp_value)
        g.mul_(f)
        acc += g.sum(0)
    return acc


def torch_port_linear_backward(grad_output, input, weight, C, clamp_value, noise_multiplier,
                               with_bias: bool):
    """Port of `_DPLinearFunc.backward` (flashdp/layers/linear.py:49-104) on CPU tensors."""
    import torch
    B = input.shape[0]
    grad_input = grad_output @ weight.to(grad_output.dtype)
    gw = torch_port_weight_grad_block_clip(grad_output, input.to(grad_output.dtype), C,
                                           clamp_value).div_(B)
    gw.add_(torch.normal(mean=0.0, std=noise_multiplier / math.sqrt(B), size=gw.shape,
                         dtype=gw.dtype) if noise_multiplier > 0 else torch.zeros_like(gw))
    gb = None
    if with_bias:
        flat = grad_output.clone().view(B, -1)
        n = torch.norm(flat, p=2, dim=-1, keepdim=True)
        flat.mul_(torch.clamp(C / (n + EPS_NORM), max=clamp_value))
        gb = flat.view(-1, grad_output.shape[-1]).mean(0)
        if noise_multiplier > 0:
            gb.add_(torch.normal(mean=0.0, std=noise_multiplier / math.sqrt(B), size=gb.shape,
                                 dtype=gb.dtype))
    return grad_input, gw, gb


# --------------------------------------------------------------------------------------
# Synthetic inputs shared by tests, golden fixtures and the benchmark
# --------------------------------------------------------------------------------------
def make_linear_inputs(B, T, n_in, n_out, g_scale, seed=0, dtype=None):
    """fp32 CPU tensors drawn in the fixed order X, G, W from one generator.

    X ~ N(0,1) (B,T,in); G ~ N(0,g_scale^2) (B,T,out); W ~ N(0,0.02^2) (out,in).
    ``dtype`` (e.g. torch.bfloat16) rounds the tensors after generation.
    """
    import torch
    gen = torch.Generator().manual_seed(seed)
    X = torch.randn(B, T, n_in, generator=gen)
    G = torch.randn(B, T, n_out, generator=gen) * g_scale
    W = torch.randn(n_out, n_in, generator=gen) * 0.02
    if dtype is not None:
        X, G, W = X.to(dtype), G.to(dtype), W.to(dtype)
    return X, G, W
