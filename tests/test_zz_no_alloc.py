"""fdp_bias_grad_static -- the bias gradient for callers that cannot allocate device memory.

Some users of the C ABI have nowhere to get a workspace from: a host binding that owns no device
allocator, a process whose memory pool has already taken the whole GPU, or a step that must not
pay the device-wide synchronisation of cudaMalloc.  For them the library carries a fixed scratch
buffer (FDP_STATIC_SCRATCH_BYTES, 8 MiB) in its own image.  This test drives the entry point
through ctypes, twice in a row on different problems (the buffer is shared and keeps old
contents), and checks each result against fdp_bias_grad given an ordinary workspace and against
the CPU oracle, at the tolerances of the other parity tests; the amount of device memory in use
(as the driver reports it) must be the same before and after the calls.  It also checks that a
problem too large for the fixed buffer is refused with FDP_ERR_STATIC_LIMIT.  The file name sorts
last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import dp_oracle as O
from conftest import rel_err, norm_err
from gpu_util import TOL, dev

pytestmark = pytest.mark.gpu

_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def _params(lib_mod, std):
    return lib_mod.DPParams(0.8, 1.0, std, 0, 4242, 17, 0, 3, 0, 1)


def _with_workspace(lib_mod, lib, G, std):
    B, T, n_out = G.shape
    db = torch.empty(n_out, dtype=torch.float32, device=G.device)
    norms = torch.empty(B, dtype=torch.float32, device=G.device)
    factors = torch.empty(B, dtype=torch.float32, device=G.device)
    ws = torch.empty(lib.fdp_bias_grad_workspace_bytes(B, T, n_out, _DT[G.dtype]), dtype=torch.uint8, device=G.device)
    p = _params(lib_mod, std)
    st = lib.fdp_bias_grad(G.data_ptr(), db.data_ptr(), norms.data_ptr(), factors.data_ptr(), B, T, n_out,
                           _DT[G.dtype], 0, ctypes.byref(p), ws.data_ptr(), ws.numel(),
                           torch.cuda.current_stream().cuda_stream)
    assert st == 0
    return db, norms, factors


def _outputs(G):
    B, T, n_out = G.shape
    return (torch.empty(n_out, dtype=torch.float32, device=G.device),
            torch.empty(B, dtype=torch.float32, device=G.device),
            torch.empty(B, dtype=torch.float32, device=G.device))


def _static(lib_mod, lib, G, std, outputs=None):
    B, T, n_out = G.shape
    db, norms, factors = outputs if outputs is not None else _outputs(G)
    p = _params(lib_mod, std)
    st = lib.fdp_bias_grad_static(G.data_ptr(), db.data_ptr(), norms.data_ptr(), factors.data_ptr(), B, T,
                                  n_out, _DT[G.dtype], 0, ctypes.byref(p), torch.cuda.current_stream().cuda_stream)
    assert st == 0, lib.fdp_status_string(st)
    return db, norms, factors


def test_static_scratch_bias_grad_matches_workspace_variant_twice_in_a_row():
    from flashdp4review_b200 import _lib
    lib = _lib.load()
    gen = torch.Generator().manual_seed(5)
    big = (torch.randn(16, 256, 1024, generator=gen) * 0.05).to(torch.bfloat16).to(dev())
    small = (torch.randn(3, 70, 200, generator=gen) * 0.05).to(dev())
    small[0] *= 25
    _static(_lib, lib, small, 0.0)       # the first call on a device looks up the buffer's address
    torch.cuda.synchronize()
    for std in (0.0, 0.5):
        want = [_with_workspace(_lib, lib, g, std) for g in (big, small)]
        outs = [_outputs(big), _outputs(small)]      # the caller's outputs exist before the calls
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        # two calls back to back on the same stream: the second must not see the first one's partials
        got = [_static(_lib, lib, big, std, outs[0]), _static(_lib, lib, small, std, outs[1])]
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before             # the calls took nothing from the device
        for g, (db, n, f), (wdb, wn, wf) in zip((big, small), got, want):
            tol = TOL[g.dtype]
            assert norm_err(n.cpu().numpy(), wn.cpu().numpy()) < tol
            assert np.allclose(f.cpu().numpy(), wf.cpu().numpy(), rtol=tol, atol=0)
            assert rel_err(db.cpu().numpy(), wdb.cpu().numpy()) < tol
            # and against the oracle of the reference's bias path (flashdp/core/linear_clip.py:116-123)
            odb, on, of = O.linear_bias_grad(g.float().cpu(), 0.8, 1.0)
            assert norm_err(n.cpu().numpy(), on) < tol
            assert np.allclose(f.cpu().numpy(), of, rtol=2 * tol, atol=0)
            if std == 0.0:
                assert rel_err(db.cpu().numpy(), odb) < tol
            else:
                z = O.gaussian_noise(db.numel(), std, 4242, 17, 3)
                assert np.abs(db.cpu().numpy() - z - odb).max() < tol * np.abs(odb).max() + 3e-6


def test_static_scratch_limit_is_enforced():
    from flashdp4review_b200 import _lib
    lib = _lib.load()
    B, T, n_out = 256, 4096, 8192
    assert lib.fdp_bias_grad_workspace_bytes(B, T, n_out, 1) > _lib.FDP_STATIC_SCRATCH_BYTES
    dummy = torch.zeros(16, device=dev())
    p = _params(_lib, 0.0)
    st = lib.fdp_bias_grad_static(dummy.data_ptr(), dummy.data_ptr(), None, None, B, T, n_out, 1, 0,
                                  ctypes.byref(p), torch.cuda.current_stream().cuda_stream)
    assert st == _lib.FDP_ERR_STATIC_LIMIT
    assert b"FDP_STATIC_SCRATCH_BYTES" in lib.fdp_status_string(st)
    torch.cuda.synchronize()
