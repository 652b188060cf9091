"""Operator layer: the functions of the reference's `flashdp/core` package, backed by the
sm_100a CUDA library through its C ABI.

Same names and argument meaning as the reference (flashdp/core/__init__.py:1-11) so callers read
the same; the fused variants `dp_linear_weight_grad` / `dp_bias_grad` / `dp_layernorm_backward`
are what the layers call -- they fold the reference's `.div_(B)` and `torch.normal` noise
(flashdp/layers/linear.py:72-80) into the kernel epilogues.
Inputs are never modified (the reference's bias path scales grad_output in place,
flashdp/core/linear_clip.py:121).
"""
import math
from dataclasses import dataclass

import torch

from .. import _lib
from .._lib import DPParams

_DT = {torch.float32: _lib.FDP_F32, torch.bfloat16: _lib.FDP_BF16, torch.float16: _lib.FDP_F16}
NORM_ALGOS = {"auto": _lib.FDP_NORM_AUTO, "direct": _lib.FDP_NORM_DIRECT, "gram": _lib.FDP_NORM_GRAM}


def _dt(t):
    try:
        return _DT[t]
    except KeyError:
        # same exception class as the reference's dtype table lookup (flashdp/core/bmtm_clip_loop.py:139-142)
        raise KeyError(f"unsupported dtype {t}; supported: fp32, bf16, fp16") from None


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("flashdp4review_b200 kernels need CUDA tensors on a B200 (sm_100); "
                               "there is no CPU path")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(device):
    return torch.cuda.current_stream(device).cuda_stream


def _aligned(t):
    """`t` itself, or a copy when its storage offset leaves it off a 16-byte boundary (the
    tensor-core kernels move 16-byte vectors; .contiguous() keeps the offset of a contiguous view)."""
    return t if t.data_ptr() % 16 == 0 else t.clone(memory_format=torch.contiguous_format)


def _workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


@dataclass
class NoiseSpec:
    """Where the Gaussian noise of one call comes from.

    std = noise_multiplier / sqrt(global batch) (flashdp/layers/linear.py:76).  The stream is a
    function of (seed, param_id, step, element index) only, so it is reproducible and does not
    depend on how many ranks share the batch: rank r draws element groups g with g % world == r
    and the all-reduce of the clipped sums assembles the full noise tensor exactly once.
    """
    std: float = 0.0
    seed: int = 0
    param_id: int = 0
    param_id2: int = 0
    step: int = 0
    rank: int = 0
    world: int = 1
    step_device: object = None    # a one-element int32 CUDA tensor the kernels add to `step` when they run


def _params(C, clamp_value, batch_divisor, noise):
    noise = noise or NoiseSpec()
    return DPParams(float(C), float(clamp_value), float(noise.std), int(batch_divisor or 0),
                    int(noise.seed) & (2 ** 64 - 1), int(noise.param_id) & 0xFFFFFFFF,
                    int(noise.param_id2) & 0xFFFFFFFF, int(noise.step) & 0xFFFFFFFF,
                    int(noise.rank), int(noise.world),
                    noise.step_device.data_ptr() if noise.step_device is not None else None)


# ------------------------------------------------------------------------------------------------
# weight gradient
# ------------------------------------------------------------------------------------------------
def dp_linear_weight_grad(input, grad_output, C, clamp_value, *, batch_divisor=None, noise=None,
                          layout="out_in", out_dtype=None, norm_algo="auto", return_norms=False, out=None,
                          fp32_tensor=None):
    """Clipped, averaged, noised weight gradient of a Linear/Conv1D layer in one library call.

    input (B,T,in), grad_output (B,T,out).  Returns dW [out,in] (layout='out_in', nn.Linear) or
    [in,out] (layout='in_out', transformers Conv1D), and with return_norms the per-sample
    Frobenius norms and clip factors.  Computes
    (1/divisor) * sum_b min(clamp, C/(||G_b^T X_b||+1e-10)) * G_b^T X_b + N(0, noise.std^2).
    `out`: a contiguous tensor of the result's shape to write into (e.g. a slice of a gradient
    bucket) instead of a fresh allocation.
    `fp32_tensor` (default: runtime.fp32_mode() == "tensor", which is the package default): fp32 inputs
    with 64-aligned shapes run on the tensor cores as three bf16 products with short accumulation
    chains -- about six times faster than the fp32-FMA kernels and within the same 1e-5 of float64;
    False forces the FMA kernels.
    """
    lib = _lib.load()
    _require_cuda(input, grad_output)
    if input.dim() != 3 or grad_output.dim() != 3 or input.shape[:2] != grad_output.shape[:2]:
        raise RuntimeError(f"expected (B,T,in) and (B,T,out), got {tuple(input.shape)} and {tuple(grad_output.shape)}")
    G = _aligned(grad_output.contiguous())
    X = _aligned(input.to(G.dtype).contiguous())     # the reference casts input to the grad dtype (linear_clip.py:111)
    B, T, n_in = X.shape
    n_out = G.shape[-1]
    shape = (n_out, n_in) if layout == "out_in" else (n_in, n_out)
    if out is not None:
        if tuple(out.shape) != shape or not out.is_contiguous() or out.device != G.device:
            raise RuntimeError(f"out must be a contiguous {shape} tensor on {G.device}")
        dW, out_dtype = out, out.dtype
    else:
        out_dtype = out_dtype or G.dtype
        dW = torch.empty(shape, dtype=out_dtype, device=G.device)
    norms = torch.empty(B, dtype=torch.float32, device=G.device) if return_norms else None
    factors = torch.empty(B, dtype=torch.float32, device=G.device) if return_norms else None
    algo = NORM_ALGOS[norm_algo]
    if fp32_tensor is None:
        from .. import runtime
        fp32_tensor = runtime.fp32_mode() == "tensor"
    if fp32_tensor and G.dtype == torch.float32:
        algo |= _lib.FDP_FP32_TENSOR
    nbytes = lib.fdp_linear_wgrad_workspace_bytes(B, T, n_in, n_out, _dt(G.dtype), algo)
    ws = _workspace(nbytes, G.device)
    p = _params(C, clamp_value, batch_divisor, noise)
    with torch.cuda.device(G.device):
        st = lib.fdp_linear_wgrad(_ptr(G), _ptr(X), _ptr(dW), _ptr(norms), _ptr(factors), B, T, n_in,
                                  n_out, _dt(G.dtype), _dt(out_dtype),
                                  _lib.FDP_OUT_IN if layout == "out_in" else _lib.FDP_IN_OUT, algo,
                                  p, _ptr(ws), ws.numel(), _stream(G.device))
    _lib.check(st, "fdp_linear_wgrad")
    return (dW, norms, factors) if return_norms else dW


def linear_weight_flashdp(input, grad_output, C, clamp_value, runtime_tuner=None):
    """Drop-in for the reference function of the same name (flashdp/core/linear_clip.py:107-113):
    the clipped SUM over samples, [out,in], in grad_output's dtype.  `runtime_tuner` is accepted
    and ignored -- there is one implementation."""
    return dp_linear_weight_grad(input, grad_output, C, clamp_value, batch_divisor=1)


def conv1d_weight_flashdp(input, grad_output, C, clamp_value, runtime_tuner=None):
    """Conv1D orientation [in,out] (flashdp/core/transformers_conv1d_clip.py:22-28)."""
    return dp_linear_weight_grad(input, grad_output, C, clamp_value, batch_divisor=1, layout="in_out")


def bmtm_clip(tensor1, tensor2, clip_args=None):
    """`bmtm_clip(tensor1=(B,K,M), tensor2=(B,K,N), clip_args=[C, clamp])` -> sum_b clip(t1_b^T t2_b)
    (flashdp/core/bmtm_clip_loop.py:162-173)."""
    C, clamp = (float(v) for v in clip_args.tolist())
    return dp_linear_weight_grad(tensor2, tensor1, C, clamp, batch_divisor=1)


def bmm_clip(tensor1, tensor2, clip_args=None):
    """`bmm_clip(tensor1=(B,M,K), tensor2=(B,K,N), clip_args=[C, clamp])` -> sum_b clip(t1_b t2_b)
    (flashdp/core/bmm_clip_loop.py:150-162; exported by flashdp.core, called by no layer).  The
    library contracts over the shared leading axis of both operands, so tensor1 is laid out as
    (B,K,M) first -- one extra pass over tensor1."""
    return bmtm_clip(tensor1.transpose(1, 2).contiguous(), tensor2, clip_args)


def mm_clip(mat1, mat2, clip_args=None):
    """Per-token clipping: `mm_clip(mat1=(M,K), mat2=(K,N))` -> sum_k clip(a_k b_k^T), each outer
    product of column k of mat1 and row k of mat2 clipped by its own Frobenius norm
    ||a_k|| * ||b_k|| (flashdp/core/mm_clip_loop.py:127-139; called by no layer).  Every k is a
    sample with a single row, which the library handles as a short sequence."""
    return bmtm_clip(mat1.t().contiguous().unsqueeze(1), mat2.contiguous().unsqueeze(1), clip_args)


# ------------------------------------------------------------------------------------------------
# bias gradient
# ------------------------------------------------------------------------------------------------
def dp_bias_grad(grad_output, C, clamp_value, *, batch_divisor=None, noise=None, out_dtype=None,
                 return_norms=False):
    """(1/(divisor*T)) * sum_b c_b * sum_t G[b,t,:] + noise, with c_b from ||G_b||_F over T*out
    (flashdp/core/linear_clip.py:116-123)."""
    lib = _lib.load()
    _require_cuda(grad_output)
    if grad_output.dim() < 2:
        raise RuntimeError("grad_output must be at least (B, out)")
    G = grad_output.contiguous()
    B, n_out = G.shape[0], G.shape[-1]
    T = G.numel() // (B * n_out)
    out_dtype = out_dtype or G.dtype
    db = torch.empty(n_out, dtype=out_dtype, device=G.device)
    norms = torch.empty(B, dtype=torch.float32, device=G.device) if return_norms else None
    factors = torch.empty(B, dtype=torch.float32, device=G.device) if return_norms else None
    ws = _workspace(lib.fdp_bias_grad_workspace_bytes(B, T, n_out, _dt(G.dtype)), G.device)
    p = _params(C, clamp_value, batch_divisor, noise)
    with torch.cuda.device(G.device):
        st = lib.fdp_bias_grad(_ptr(G), _ptr(db), _ptr(norms), _ptr(factors), B, T, n_out,
                               _dt(G.dtype), _dt(out_dtype), p, _ptr(ws), ws.numel(), _stream(G.device))
    _lib.check(st, "fdp_bias_grad")
    return (db, norms, factors) if return_norms else db


def linear_bias_grad_clip(grad_output, C, clamp_value):
    """Drop-in for flashdp/core/linear_clip.py:116-123 (mean over the B*T rows of c_b*G)."""
    return dp_bias_grad(grad_output, C, clamp_value)


# ------------------------------------------------------------------------------------------------
# input gradient
# ------------------------------------------------------------------------------------------------
def native_product_ok(dtype, rows, K, N):
    """Whether a DP layer runs its forward / input-gradient product [rows, K] x [K, N] on this library's
    GEMMs, under runtime.input_grad_impl(): "library" never (cuBLAS through torch, as the reference);
    "auto" (default) where a tensor-core kernel of the library takes the shape -- bf16 / fp16 with
    8-aligned features, at least 128 rows and output columns and 64 contracted ones; fp32 in mode "tensor"
    with K a multiple of 64 and at least 128 of everything (three bf16 products); "native" also for every
    other 16-bit shape (generic kernels)."""
    from .. import runtime
    mode = runtime.input_grad_impl()
    if mode == "library":
        return False
    if dtype == torch.float32:
        return (runtime.fp32_mode() == "tensor" and rows >= 128 and K >= 128 and N >= 128
                and K % 64 == 0 and N % 8 == 0)
    if dtype not in (torch.bfloat16, torch.float16):
        return False
    return mode == "native" or (K % 8 == 0 and N % 8 == 0 and N >= 128 and K >= 64 and rows >= 128)


def _gemm_dtype_code(dtype, fp32_tensor):
    """dtype code of the forward / input-gradient entry points, with the fp32 tensor-core flag"""
    code = _dt(dtype)
    if dtype == torch.float32:
        if fp32_tensor is None:
            from .. import runtime
            fp32_tensor = runtime.fp32_mode() == "tensor"
        if fp32_tensor:
            code |= _lib.FDP_FP32_TENSOR
    return code


def linear_input_grad(grad_output, weight, w_layout="out_in", out_dtype=None, fp32_tensor=None):
    """grad_output @ weight (nn.Linear, weight [out,in]) or grad_output @ weight.t() (Conv1D,
    weight [in,out]) -- flashdp/layers/linear.py:62-67, transformers_conv1d.py:70-75.
    `out_dtype` (default: grad_output's) lets the kernel write the dtype autograd wants directly.
    `fp32_tensor` as in dp_linear_weight_grad: fp32 operands as three bf16 tensor-core products."""
    lib = _lib.load()
    _require_cuda(grad_output, weight)
    G = _aligned(grad_output.contiguous())
    W = _aligned(weight.to(G.dtype).contiguous())         # AMP: weight follows the grad dtype (linear.py:66)
    n_out = G.shape[-1]
    n_in = W.shape[1] if w_layout == "out_in" else W.shape[0]
    rows = G.numel() // n_out
    out_dtype = out_dtype or G.dtype
    dX = torch.empty(G.shape[:-1] + (n_in,), dtype=out_dtype, device=G.device)
    code = _gemm_dtype_code(G.dtype, fp32_tensor)
    ws = _workspace(lib.fdp_linear_dgrad_workspace_bytes(rows, n_in, n_out, code), G.device)
    with torch.cuda.device(G.device):
        st = lib.fdp_linear_dgrad(_ptr(G), _ptr(W), _ptr(dX), rows, n_in, n_out, code, _dt(out_dtype),
                                  _lib.FDP_OUT_IN if w_layout == "out_in" else _lib.FDP_IN_OUT,
                                  _ptr(ws), ws.numel(), _stream(G.device))
    _lib.check(st, "fdp_linear_dgrad")
    return dX


def linear_forward(input, weight, bias=None, w_layout="out_in", out_dtype=None, fp32_tensor=None):
    """input @ weight.t() + bias (nn.Linear, weight [out,in]) or input @ weight + bias (Conv1D, weight
    [in,out]) -- flashdp/layers/linear.py:41-46, transformers_conv1d.py:40-43."""
    lib = _lib.load()
    _require_cuda(input, weight, bias)
    X = _aligned(input.contiguous())
    W = _aligned(weight.to(X.dtype).contiguous())
    b = None if bias is None else _aligned(bias.to(X.dtype).contiguous())
    n_in = X.shape[-1]
    n_out = W.shape[0] if w_layout == "out_in" else W.shape[1]
    rows = X.numel() // n_in
    out_dtype = out_dtype or X.dtype
    Y = torch.empty(X.shape[:-1] + (n_out,), dtype=out_dtype, device=X.device)
    code = _gemm_dtype_code(X.dtype, fp32_tensor)
    ws = _workspace(lib.fdp_linear_dgrad_workspace_bytes(rows, n_out, n_in, code), X.device)
    with torch.cuda.device(X.device):
        st = lib.fdp_linear_fwd(_ptr(X), _ptr(W), _ptr(b), _ptr(Y), rows, n_in, n_out, code, _dt(out_dtype),
                                _lib.FDP_OUT_IN if w_layout == "out_in" else _lib.FDP_IN_OUT,
                                _ptr(ws), ws.numel(), _stream(X.device))
    _lib.check(st, "fdp_linear_fwd")
    return Y


def mm_fused(tensor1, tensor2):
    """Drop-in for flashdp/core/linear_clip.py:64-91 (exported by flashdp.core, called by no layer):
    tensor1 (..., K) @ tensor2 (K, ...) with fp32 accumulation, returned in the accumulation dtype
    (fp32), leading / trailing axes kept."""
    if tensor1.dtype not in _DT:
        raise KeyError("The type of input mat is not supported.")
    if tensor1.dim() < 2 or tensor2.dim() < 2:
        raise KeyError("The dimensions of input tensors must be at least 2.")
    if tensor1.shape[-1] != tensor2.shape[0]:
        raise ValueError("tensor1 last dimension must match tensor2 first dimension")
    a = tensor1.reshape(-1, tensor1.shape[-1])
    b = tensor2.reshape(tensor2.shape[0], -1)
    out = linear_forward(a, b, None, "in_out", out_dtype=torch.float32)
    return out.reshape(tensor1.shape[:-1] + tensor2.shape[1:])


# ------------------------------------------------------------------------------------------------
# LayerNorm
# ------------------------------------------------------------------------------------------------
def layernorm_fwd_fused(input, weight, bias, eps):
    """LayerNorm over the last dimension; returns (y, {'mean','rstd'}, args) like
    flashdp/core/layernorm_clip.py:201-239."""
    lib = _lib.load()
    _require_cuda(input, weight, bias)
    x = input.contiguous()
    d = x.shape[-1]
    rows = x.numel() // d
    if d * x.element_size() >= 65536:
        # same limit and exception as the reference (flashdp/core/layernorm_clip.py:220-221)
        raise RuntimeError("This layer norm doesn't support feature dim >= 64KB.")
    y = torch.empty_like(x)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    w = weight.contiguous()
    b = bias.to(w.dtype).contiguous()
    with torch.cuda.device(x.device):
        st = lib.fdp_layernorm_fwd(_ptr(x), _ptr(w), _ptr(b), _ptr(y), _ptr(mean), _ptr(rstd), rows, d,
                                   float(eps), _dt(x.dtype), _dt(w.dtype), _stream(x.device))
    _lib.check(st, "fdp_layernorm_fwd")
    return y, {"mean": mean, "rstd": rstd}, {"eps": eps}


def dp_layernorm_backward(grad_output, input, weight, mean, rstd, C, clamp_value, *,
                          batch_divisor=None, noise=None, need_dx=True, need_dbeta=True,
                          return_norms=False):
    """dx plus per-sample-clipped, averaged, noised dgamma / dbeta.

    dgamma = (1/divisor) sum_b f(||sum_t dy_b*xhat_b||_2) sum_t dy_b*xhat_b + noise, dbeta alike
    with sum_t dy_b (flashdp/core/layernorm_clip.py:163-198; noise flashdp/layers/layernorm.py:139-155,
    drawn once per tensor).  The sample axis is dim 0; every other leading axis is summed.
    """
    lib = _lib.load()
    _require_cuda(grad_output, input, weight)
    dy = grad_output.contiguous()
    x = input.contiguous()
    d = x.shape[-1]
    B = x.shape[0] if x.dim() > 1 else 1
    T = x.numel() // (B * d)
    w = weight.contiguous()
    dx = torch.empty_like(x) if need_dx else None
    dgamma = torch.empty(d, dtype=w.dtype, device=x.device)
    dbeta = torch.empty(d, dtype=w.dtype, device=x.device) if need_dbeta else None
    ng = torch.empty(B, dtype=torch.float32, device=x.device) if return_norms else None
    nb = torch.empty(B, dtype=torch.float32, device=x.device) if return_norms and need_dbeta else None
    ws = _workspace(lib.fdp_layernorm_bwd_workspace_bytes(B, T, d), x.device)
    p = _params(C, clamp_value, batch_divisor, noise)
    with torch.cuda.device(x.device):
        st = lib.fdp_layernorm_bwd(_ptr(dy), _ptr(x), _ptr(w), _ptr(mean), _ptr(rstd), _ptr(dx),
                                   _ptr(dgamma), _ptr(dbeta), _ptr(ng), _ptr(nb), B, T, d,
                                   _dt(x.dtype), _dt(w.dtype), p, _ptr(ws), ws.numel(), _stream(x.device))
    _lib.check(st, "fdp_layernorm_bwd")
    if return_norms:
        return dx, dgamma, dbeta, ng, nb
    return dx, dgamma, dbeta


def layernorm_bwd_clip_fused(grad_output, input, weight, bias, clip_args, buffer, args=None):
    """Compatibility drop-in for flashdp/core/layernorm_clip.py:241-286: returns (dx, dw_, db_, args)
    with dw_ / db_ the [G, d] buffers of the reference's element-wise saturating accumulation
    (buf <- partial + buf * min(clamp, C / (|buf| + 1e-10)), flashdp/core/layernorm_clip.py:109-131).
    The reference adds the rows of a buffer in the order its row programs win a spin lock; here they are
    added in increasing row order, so the result is reproducible.  This is NOT per-sample clipping and
    carries no noise: DP training uses dp_layernorm_backward."""
    lib = _lib.load()
    _require_cuda(grad_output, input, weight)
    C, clamp = (float(v) for v in clip_args.tolist())
    dy = grad_output.contiguous()
    x = input.contiguous()
    w = weight.contiguous()
    d = x.shape[-1]
    rows = x.numel() // d
    mean, rstd = buffer["mean"], buffer["rstd"]
    # dx: the standard LayerNorm input gradient (flashdp/core/layernorm_clip.py:95-103)
    dx, _, _ = dp_layernorm_backward(dy.reshape(1, rows, d), x.reshape(1, rows, d), w, mean, rstd, 1.0, 1.0,
                                     need_dx=True, need_dbeta=False)
    G = lib.fdp_layernorm_saturate_groups(rows, d)
    ws = torch.empty(2, G, d, dtype=torch.float32, device=x.device)
    dw = torch.empty(d, dtype=w.dtype, device=x.device)
    db = torch.empty(d, dtype=w.dtype, device=x.device)
    with torch.cuda.device(x.device):
        st = lib.fdp_layernorm_bwd_saturate(_ptr(dy), _ptr(x), _ptr(mean), _ptr(rstd), _ptr(dw), _ptr(db), rows, d,
                                            _dt(x.dtype), _dt(w.dtype), C, clamp, _ptr(ws), ws.numel() * 4,
                                            _stream(x.device))
    _lib.check(st, "fdp_layernorm_bwd_saturate")
    return dx.reshape(input.shape), ws[0], ws[1], {"GROUP_SIZE_M": G, "M": rows, "dw": dw, "db": db}


def layernorm_dwdb_fused(weight, bias, _dw, _db, args=None):
    """Compatibility drop-in for flashdp/core/layernorm_clip.py:289-315: the column sums of the G
    buffers (already formed by layernorm_bwd_clip_fused, which passes them on in `args`)."""
    if args is not None and "dw" in args:
        return args["dw"], args["db"]
    return _dw.sum(0).to(weight.dtype), _db.sum(0).to(weight.dtype)


def _ln_identity_stats(rows, device):
    return (torch.zeros(rows, dtype=torch.float32, device=device),
            torch.ones(rows, dtype=torch.float32, device=device))


def layernorm_dw_clip(input, grad_output, weight, C, clamp_value):
    """Drop-in for flashdp/core/layernorm_clip.py:163-180: `input` is the already normalised
    activation; returns the clipped mean of the per-sample sum(dy*xhat), shape (1,...,d)."""
    d = input.shape[-1]
    mean, rstd = _ln_identity_stats(input.numel() // d, input.device)
    ones = torch.ones(d, dtype=torch.float32, device=input.device)
    _, dg, _ = dp_layernorm_backward(grad_output, input, ones, mean, rstd, float(C), float(clamp_value),
                                     need_dx=False, need_dbeta=False)
    return dg.to(grad_output.dtype).reshape([1] * (input.dim() - 1) + [d])


def layernorm_db_clip(grad_output, bias, C, clamp_value):
    """Drop-in for flashdp/core/layernorm_clip.py:183-198."""
    d = grad_output.shape[-1]
    mean, rstd = _ln_identity_stats(grad_output.numel() // d, grad_output.device)
    ones = torch.ones(d, dtype=torch.float32, device=grad_output.device)
    _, _, db = dp_layernorm_backward(grad_output, grad_output, ones, mean, rstd, float(C),
                                     float(clamp_value), need_dx=False, need_dbeta=True)
    return db.to(grad_output.dtype).reshape([1] * (grad_output.dim() - 1) + [d])


class RuntimeAutoTuner:
    """Kept so that code written against the reference still constructs
    (flashdp/core/utils.py:15-47).  There is a single CUDA implementation per shape class, chosen
    from the shape, so nothing is timed at run time and nothing is tuned."""

    def __init__(self, enable=True, warmup_iterations=10, measure_iterations=100, log=False):
        self.enable = enable
        self.if_final_tune = False
        self.chosen_func = None
        self.warmup_iterations = warmup_iterations
        self.measure_iterations = measure_iterations
        self.log = log

    def choose_function(self, funcs_list, *args, **kwargs):
        self.chosen_func = funcs_list[0]
        return self.chosen_func

    def final_tune(self):
        self.if_final_tune = True


def noise_std(noise_multiplier, global_batch):
    """std of the per-element Gaussian: noise_multiplier / sqrt(B) (flashdp/layers/linear.py:76)."""
    return float(noise_multiplier) / math.sqrt(global_batch)
