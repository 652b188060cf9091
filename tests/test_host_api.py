"""CPU-side checks: the shared library loads and exports the whole C ABI, and the wrap API keeps
the reference's selection rules and errors (flashdp/api/wrap_model.py)."""
import os
import re

import pytest
import torch
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from flashdp4review_b200 import _lib
    lib = _lib.load()
    header = open(os.path.join(ROOT, "include", "fdp_b200.h")).read()
    declared = set(re.findall(r"\b(fdp_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/fdp_b200.h but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert lib.fdp_abi_version() == _lib.ABI_VERSION
    assert lib.fdp_status_string(0) == b"ok"
    assert b"workspace" in lib.fdp_status_string(_lib.FDP_ERR_WORKSPACE)
    # pure host-side queries work without a device
    assert lib.fdp_linear_wgrad_workspace_bytes(4, 128, 768, 768, _lib.FDP_F32, 0) > 0
    assert lib.fdp_linear_wgrad_workspace_bytes(0, 128, 768, 768, _lib.FDP_F32, 0) == 0
    assert lib.fdp_bias_grad_workspace_bytes(4, 128, 768, _lib.FDP_BF16) > 0
    assert lib.fdp_layernorm_bwd_workspace_bytes(16, 1024, 1024) > 0


def test_no_cpu_fallback():
    from flashdp4review_b200.core import ops
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.dp_linear_weight_grad(torch.zeros(1, 2, 8), torch.zeros(1, 2, 8), 1.0, 1.0)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.dp_bias_grad(torch.zeros(1, 2, 8), 1.0, 1.0)


def _model():
    return nn.Sequential(nn.Linear(8, 8), nn.LayerNorm(8),
                         nn.Sequential(nn.Linear(8, 4, bias=False), nn.ReLU()), nn.Linear(4, 2))


def test_wrap_argument_errors():
    from flashdp4review_b200 import wrap_with_flashdp_layers
    with pytest.raises(ValueError):
        wrap_with_flashdp_layers(_model())
    with pytest.raises(ValueError):
        wrap_with_flashdp_layers(_model(), target_modules=[])
    with pytest.raises(ValueError):
        wrap_with_flashdp_layers(_model(), target_layers=["0"])          # target_layers alone is rejected
    with pytest.raises(ValueError):
        wrap_with_flashdp_layers(_model(), target_modules=[nn.Conv2d])


def test_wrap_selection_rules():
    import flashdp4review_b200 as fdp
    m = fdp.wrap_with_flashdp_layers(_model(), target_modules=[nn.Linear, nn.LayerNorm], skip_layers=["3"],
                                     C=0.3, noise_multiplier=0.7, clamp_value=0.9, feedback=False)
    assert isinstance(m[0], fdp.DPLinear) and isinstance(m[1], fdp.DPLayerNorm)
    assert isinstance(m[2][0], fdp.DPLinear) and m[2][0].bias is None
    assert type(m[3]) is nn.Linear
    assert (m[0].C, m[0].noise_multiplier, m[0].clamp_value) == (0.3, 0.7, 0.9)
    # skipping a container does not skip its children (exact-name match only)
    m = fdp.wrap_with_flashdp_layers(_model(), target_modules=[nn.Linear], skip_layers=["2"], feedback=False)
    assert isinstance(m[2][0], fdp.DPLinear)
    # target_layers restricts the candidates
    m = fdp.wrap_with_flashdp_layers(_model(), target_modules=[nn.Linear], target_layers=["0"], feedback=False)
    assert isinstance(m[0], fdp.DPLinear) and type(m[3]) is nn.Linear


def test_wrap_keeps_weights_dtype_mode_and_ties():
    import flashdp4review_b200 as fdp

    class Tied(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(10, 8)
            self.body = nn.Linear(8, 8)
            self.lm_head = nn.Linear(8, 10, bias=False)
            self.lm_head.weight = self.emb.weight
    src = Tied().to(torch.bfloat16).eval()
    ref_w = src.body.weight.detach().clone()
    m = fdp.wrap_with_flashdp_layers(src, target_modules=[nn.Linear], skip_layers=["lm_head"], feedback=False)
    assert torch.equal(m.body.weight.detach(), ref_w)
    assert m.body.weight.dtype == torch.bfloat16 and not m.body.training
    assert m.lm_head.weight is m.emb.weight
    assert set(m.state_dict()) == set(Tied().state_dict())            # parameter names round-trip


def test_conv1d_twin_and_constructor_attributes():
    import flashdp4review_b200 as fdp
    from flashdp4review_b200.layers import Conv1D
    m = nn.Sequential(Conv1D(24, 8))
    fdp.wrap_with_flashdp_layers(m, target_modules=[Conv1D], feedback=False)
    assert isinstance(m[0], fdp.DPConv1D) and m[0].weight.shape == (8, 24) and m[0].nf == 24
    lin = fdp.DPLinear(4, 6, C=2.0, clamp_value=0.5, noise_multiplier=0.1, auto_tune=False)
    assert lin.dp and lin.runtime_tuner.enable is False and lin.weight.requires_dp
    ln = fdp.DPLayerNorm(6, use_fused=False, bias=None)
    assert ln.bias is None and ln.use_fused is False


def test_workspace_queries_are_pure_host_functions():
    """The *_workspace_bytes queries run without a GPU, reject nonsense with 0 and grow with the
    problem; every plan the launch would pick (tensor-core, short-sequence, generic) fits them."""
    from flashdp4review_b200 import _lib
    lib = _lib.load()
    q = lib.fdp_linear_wgrad_workspace_bytes
    assert q(0, 128, 256, 256, _lib.FDP_BF16, 0) == 0 and q(4, 128, 256, 256, 7, 0) == 0
    sizes = [q(B, T, 256, 384, dt, 0) for dt in (_lib.FDP_F32, _lib.FDP_BF16)
             for (B, T) in ((2, 7), (512, 1), (4, 128), (32, 1024))]
    assert all(s > 0 and s % 256 == 0 for s in sizes)
    assert q(64, 1024, 256, 384, _lib.FDP_BF16, 0) >= q(32, 1024, 256, 384, _lib.FDP_BF16, 0)
    b = lib.fdp_bias_grad_workspace_bytes
    assert b(0, 1, 1, _lib.FDP_F32) == 0
    assert 0 < b(4, 128, 768, _lib.FDP_F32) <= b(8, 128, 768, _lib.FDP_F32) <= b(8, 4096, 768, _lib.FDP_F32)
    ln = lib.fdp_layernorm_bwd_workspace_bytes
    assert ln(0, 1, 1) == 0
    assert 0 < ln(4, 9, 40) <= ln(16, 1024, 1024) <= ln(32, 1024, 4096)
    assert lib.fdp_linear_dgrad_workspace_bytes(4096, 256, 384, _lib.FDP_BF16) >= 0
    # fp32 on the tensor cores: the flag adds room for the bf16 halves of the operands where the shape
    # qualifies (64-aligned contracted dimension, at least 128 of everything) and nothing elsewhere
    t3 = _lib.FDP_F32 | _lib.FDP_FP32_TENSOR
    d = lib.fdp_linear_dgrad_workspace_bytes
    rows, n_in, n_out = 8192, 1024, 3072
    assert d(rows, n_in, n_out, _lib.FDP_F32) == 256
    assert d(rows, n_in, n_out, t3) >= 256 + 4 * (rows * n_out + n_out * n_in)
    assert d(rows, n_in, 1000, t3) == 256 and d(64, n_in, n_out, t3) == 256     # K % 64, too few rows
    w = lib.fdp_linear_wgrad_workspace_bytes
    plain, flagged = w(8, 1024, 4096, 4096, _lib.FDP_F32, 0), w(8, 1024, 4096, 4096, _lib.FDP_F32, _lib.FDP_FP32_TENSOR)
    assert flagged >= plain + 4 * 8 * 1024 * (4096 + 4096) - (1 << 20)
    assert w(8, 1000, 4096, 4096, _lib.FDP_F32, _lib.FDP_FP32_TENSOR) == w(8, 1000, 4096, 4096, _lib.FDP_F32, 0)
    assert w(8, 1024, 4096, 4096, _lib.FDP_BF16, _lib.FDP_FP32_TENSOR) == w(8, 1024, 4096, 4096, _lib.FDP_BF16, 0)


def test_gram_work_units_cover_the_block_triangle_once(tmp_path):
    """The Gram norm pass deals units of (t-block, two s-blocks); compiled for the host, the
    enumeration must cover every unordered block pair exactly once, with at most one single-block
    unit per sample, for every block count."""
    import shutil
    import subprocess
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no host C++ compiler")
    hdr = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                       "flashdp4review_b200", "csrc", "fdp_gram_units.h")
    src = tmp_path / "units.cpp"
    src.write_text('#include <cstdio>\n#include <set>\n#include <utility>\n#include "%s"\n' % hdr + r'''
int main() {
  for (int nb = 1; nb <= 160; ++nb) {
    std::set<std::pair<int, int>> seen;
    const int units = fdp::gram_units(nb);
    int singles = 0;
    for (int u = 0; u < units; ++u) {
      int i, j1, j2;
      fdp::gram_decode(nb, u, i, j1, j2);
      if (i < 0 || i >= nb || j1 < 0 || j1 >= nb || j2 >= nb) { std::printf("range nb=%d u=%d\n", nb, u); return 1; }
      if (j2 < 0) ++singles;
      const int js[2] = {j1, j2};
      for (int k = 0; k < 2; ++k) {
        if (js[k] < 0) continue;
        const std::pair<int, int> key(i < js[k] ? i : js[k], i < js[k] ? js[k] : i);
        if (!seen.insert(key).second) { std::printf("twice nb=%d (%d,%d)\n", nb, key.first, key.second); return 1; }
      }
    }
    if (static_cast<int>(seen.size()) != nb * (nb + 1) / 2) { std::printf("missing nb=%d\n", nb); return 1; }
    if (singles > 1 || units != (nb * (nb + 1) / 2 + 1) / 2) { std::printf("count nb=%d\n", nb); return 1; }
  }
  std::printf("ok\n");
  return 0;
}
''')
    exe = tmp_path / "units"
    subprocess.run([gxx, "-O1", "-std=c++17", "-o", str(exe), str(src)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip() == "ok", out.stdout


def test_forward_and_input_gradient_gemm_selection():
    """`set_input_grad_impl`: "library" never uses the package's GEMMs, "auto" (default) only where a
    tensor-core kernel takes the shape, "native" also the generic 16-bit kernels; fp32 only in fp32 mode
    "tensor" and with the contracted dimension a multiple of 64."""
    import torch
    from flashdp4review_b200 import runtime
    from flashdp4review_b200.core import ops
    before, before32 = runtime.input_grad_impl(), runtime.fp32_mode()
    try:
        assert before == "auto" and before32 == "tensor"
        bf, f32 = torch.bfloat16, torch.float32
        cases = {  # (dtype, rows, K, N): (library, auto, native)
            (bf, 8192, 1024, 3072): (False, True, True),
            (bf, 8192, 100, 3072): (False, False, True),      # K not a multiple of 8: generic kernel
            (bf, 64, 1024, 1024): (False, False, True),       # too few rows for a tile
            (f32, 8192, 1024, 3072): (False, True, True),
            (f32, 8192, 1000, 3072): (False, False, False),   # K not a multiple of 64: cuBLAS
            (f32, 96, 1024, 1024): (False, False, False),
            (torch.float64, 8192, 1024, 1024): (False, False, False),
        }
        for i, impl in enumerate(("library", "auto", "native")):
            runtime.set_input_grad_impl(impl)
            for (dt, rows, K, N), want in cases.items():
                assert ops.native_product_ok(dt, rows, K, N) == want[i], (impl, dt, rows, K, N)
        runtime.set_input_grad_impl("auto")
        runtime.set_fp32_mode("exact")
        assert not ops.native_product_ok(f32, 8192, 1024, 3072)
        with pytest.raises(ValueError):
            runtime.set_input_grad_impl("cublas")
    finally:
        runtime.set_input_grad_impl(before)
        runtime.set_fp32_mode(before32)
