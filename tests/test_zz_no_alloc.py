"""The allocation-free key-split attention entry point, called through the C ABI.

`chitu_b200_attn_fwd_splitkv_static` exists for hosts that cannot give the library a scratch buffer
(a serving process whose own pool already owns all free device memory, or a plugin running in the
middle of another runtime's step where cudaMalloc is not an option): its partial results go to a
fixed 32 MiB array inside the library.  The test drives it twice in a row on the same GPU - the
array is shared and keeps the first call's contents - and compares each result with the ordinary
key-split entry point fed a caller-owned workspace, and with the single-pass kernel.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

# bf16 outputs of two schedules of the same arithmetic: same tolerance as the other attention tests
REL_MAX_ABS = 2e-2


def _call(lib, fn_name, q, k, v, n_splits, workspace=None):
    from chitudiffusion_b200 import _lib, ops

    B, Sq, H, D = q.shape
    out = torch.empty_like(q)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
    args = [
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), B, Sq, k.shape[1], H, D,
        _lib.i64_array(q.stride()), _lib.i64_array(k.stride()), _lib.i64_array(v.stride()),
        ctypes.c_float(D ** -0.5), _lib.DTYPE_BF16, n_splits,
    ]
    if workspace is not None:
        args += [workspace.data_ptr(), workspace.numel()]
    args += [ops.status_word(q.device).data_ptr(), int(torch.cuda.current_stream().cuda_stream)]
    rc = getattr(lib, fn_name)(*args)
    return rc, out, lse


def test_static_scratch_entry_point_matches_workspace_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from chitudiffusion_b200 import _lib, ops

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    gen = torch.Generator().manual_seed(2024)
    shapes = [(1, 300, 1500, 3, 4), (2, 130, 700, 2, 3)]  # second call: other shape, stale scratch underneath
    for B, Sq, Sk, H, n_splits in shapes:
        q = torch.randn(B, Sq, H, 128, generator=gen).to(torch.bfloat16).to(dev)
        k = torch.randn(B, Sk, H, 128, generator=gen).to(torch.bfloat16).to(dev)
        v = torch.randn(B, Sk, H, 128, generator=gen).to(torch.bfloat16).to(dev)
        need = int(lib.chitu_b200_attn_splitkv_workspace_bytes(B, Sq, H, 128, n_splits))
        ws = torch.zeros(need, dtype=torch.uint8, device=dev)  # the counters at its head must start at zero
        rc_ref, out_ref, lse_ref = _call(lib, "chitu_b200_attn_fwd_splitkv", q, k, v, n_splits, ws)
        assert rc_ref == 0, lib.chitu_b200_last_error()
        rc, out, lse = _call(lib, "chitu_b200_attn_fwd_splitkv_static", q, k, v, n_splits)
        assert rc == 0, lib.chitu_b200_last_error()
        torch.cuda.synchronize()
        ops.check_status(dev)
        scale = out_ref.float().abs().max().item()
        assert torch.isfinite(out.float()).all()
        assert (out.float() - out_ref.float()).abs().max().item() <= REL_MAX_ABS * scale
        assert (lse - lse_ref).abs().max().item() <= 1e-3
        single, _ = ops.attn_fwd(q, k, v, n_splits=1)
        assert (out.float() - single.float()).abs().max().item() <= REL_MAX_ABS * scale


def test_static_scratch_entry_point_rejects_oversized_requests():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from chitudiffusion_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    # 8 ranges x 40000 rows x 24 heads x 516 bytes is far beyond 32 MiB: refused before any launch
    q = torch.zeros(1, 8, 1, 128, dtype=torch.bfloat16, device=dev)
    st = _lib.i64_array((128 * 24 * 40000, 128 * 24, 128, 1))
    rc = lib.chitu_b200_attn_fwd_splitkv_static(
        q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), None, 1, 40000, 40000, 24, 128, st, st, st,
        ctypes.c_float(0.088), _lib.DTYPE_BF16, 8, None, None)
    assert rc == _lib.E_INVALID
    msg = lib.chitu_b200_last_error().decode()
    assert "scratch" in msg and "bytes" in msg
