"""GPU parity of the HBM-bound kernels (LSE combine, norm+rotary, layout copy) against the CPU oracle."""

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from chitudiffusion_b200 import ops as _ops

    return _ops


def test_lse_combine_golden(ops, golden):
    for name in ("lse_merge", "lse_merge_bf16"):
        c = golden[name]
        B, S, H, D = c["outs"][0].shape
        acc = torch.empty(B, S, H, D, device="cuda")
        lse = torch.empty(B, S, H, 1, device="cuda")
        for i, (bo, bl) in enumerate(zip(c["outs"], c["lses"])):
            ops.lse_combine(acc, lse, bo.cuda(), bl.cuda(), first=(i == 0))
        assert torch.allclose(acc.cpu(), c["out"], atol=2e-6, rtol=1e-5), name
        assert torch.allclose(lse.cpu(), c["lse"], atol=2e-6, rtol=1e-5), name


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_lse_combine_equals_full_attention(ops, dtype):
    torch.manual_seed(5)
    q = torch.randn(2, 70, 3, 128)
    k = torch.randn(2, 300, 3, 128)
    v = torch.randn(2, 300, 3, 128)
    full = oracle.sdpa_fp32(q, k, v)
    acc = torch.empty(2, 70, 3, 128, device="cuda")
    lse = torch.empty(2, 70, 3, device="cuda")
    final = torch.empty(2, 70, 3, 128, device="cuda", dtype=torch.bfloat16)
    bounds = [(0, 100), (100, 130), (130, 300)]
    for i, (a, b) in enumerate(bounds):
        o, l = oracle.sdpa_fp32(q, k[:, a:b], v[:, a:b], return_lse=True)
        ops.lse_combine(acc, lse, o.to(dtype).cuda(), l.cuda(), first=(i == 0), final_out=final if i == 2 else None)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(acc.cpu(), full, atol=tol)
    assert torch.allclose(final.float().cpu(), acc.cpu(), atol=1e-2)


def _wan_table(d, rows=1024):
    f = oracle.wan_rope_table(d, rows)
    return torch.stack([f.real, f.imag], dim=-1).to(torch.float32).contiguous()


@pytest.mark.parametrize("in_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 24, 2, 128, (2, 3, 4)), (2, 50, 12, 128, (3, 4, 4)), (1, 40, 40, 128, (2, 4, 5))])
def test_wan_norm_rope_matches_oracle(ops, in_dtype, shape):
    B, S, H, D, grid = shape
    torch.manual_seed(7)
    C = H * D
    x = (torch.randn(B, S, C) * 1.3).to(in_dtype)
    w = 1.0 + 0.1 * torch.randn(C)
    freqs = oracle.wan_rope_table(D)
    grids = torch.tensor([list(grid)] * B)
    ref = oracle.wan_rope_apply(oracle.wan_rms_norm(x, w, 1e-6).view(B, S, H, D), grids, freqs).to(torch.bfloat16)
    n_h = (D // 2) // 3
    n_t = D // 2 - 2 * n_h
    got = ops.qk_norm_rope(
        x.cuda(), H, w.cuda(), 1e-6, norm_mode=0, rope_mode=1, rope_table=_wan_table(D).cuda(), grid=grid,
        axis_split=(n_t, n_h),
    )
    diff = (got.float().cpu() - ref.float()).abs()
    # within one bf16 ulp everywhere, exact almost everywhere
    assert (diff <= ref.float().abs() * 2 ** -7 + 1e-6).all()
    assert (got.cpu() == ref).float().mean() > 0.995


def test_wan_norm_rope_cp_offset_and_send_layout(ops):
    """Rank-local positions plus output scattered as [U, B, s, H/U, D] (the Ulysses send layout)."""
    torch.manual_seed(8)
    B, s, H, D, cp, U = 1, 9, 4, 128, 3, 2
    grid = (2, 3, 4)
    freqs = oracle.wan_rope_table(D)
    n_h = (D // 2) // 3
    n_t = D // 2 - 2 * n_h
    for rank in range(cp):
        x = torch.randn(B, s, H * D)
        ref = oracle.wan_rope_apply_with_cp(x.view(B, s, H, D), torch.tensor([list(grid)]), freqs, cp, rank)
        ref = ref.to(torch.bfloat16)
        hc = H // U
        send = torch.zeros(U, B, s, hc, D, device="cuda", dtype=torch.bfloat16)
        ops.qk_norm_rope(
            x.cuda(), H, None, 1e-6, norm_mode=2, rope_mode=1, rope_table=_wan_table(D).cuda(), grid=grid,
            axis_split=(n_t, n_h), pos_offset=rank * s, out=send,
            out_strides=(s * hc * D, hc * D, B * s * hc * D, D), heads_per_group=hc,
        )
        want = ref.view(B, s, U, hc, D).permute(2, 0, 1, 3, 4)
        assert (send.cpu().float() - want.float()).abs().max() <= 2 ** -7 * want.float().abs().max()
        assert (send.cpu() == want).float().mean() > 0.995


def test_per_head_norm_axis_rope(ops):
    torch.manual_seed(9)
    B, S, H, D = 1, 70, 24, 128
    x = torch.randn(B, S, H * D).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(D)).to(torch.bfloat16)
    ids = torch.zeros(S, 3, dtype=torch.long)
    ids[6:, 1] = torch.arange(S - 6) // 8
    ids[6:, 2] = torch.arange(S - 6) % 8
    cos, sin = oracle.axis_rope_table(ids, (16, 56, 56))
    table = torch.stack([cos, sin], dim=-1).to(torch.float32).contiguous()
    ref = oracle.apply_rope_interleaved(oracle.per_head_rms_norm(x.view(B, S, H, D), w, 1e-6), cos, sin)
    got = ops.qk_norm_rope(x.cuda(), H, w.cuda(), 1e-6, norm_mode=1, rope_mode=2, rope_table=table.cuda(),
                           round_mid=False)
    assert (got.float().cpu() - ref).abs().max() <= 2 ** -7 * ref.abs().max() + 1e-3


def test_strided_copy_ulysses_layouts(ops):
    torch.manual_seed(10)
    B, s, U, hc, D = 2, 11, 4, 3, 128
    x = torch.randn(B, s, U * hc, D).to(torch.bfloat16).cuda()
    # pack heads: [B, s, U*hc, D] -> [U, B, s, hc, D]
    send = torch.empty(U, B, s, hc, D, dtype=torch.bfloat16, device="cuda")
    ops.strided_copy(x.view(B, s, U, hc * D).permute(2, 0, 1, 3).unsqueeze(3), send.view(U, B, s, 1, hc * D))
    want = x.view(B, s, U, hc, D).permute(2, 0, 1, 3, 4).contiguous()
    assert torch.equal(send, want)
    # unpack sequence: recv [U, B, s, hc, D] -> [B, U*s, hc, D]
    y = torch.empty(B, U, s, 1, hc * D, dtype=torch.bfloat16, device="cuda")
    ops.strided_copy(send.view(U, B, s, 1, hc * D).permute(1, 0, 2, 3, 4), y)
    ref = oracle.ulysses_scatter_heads([x.cpu()])  # U=1 trivial check of helper import
    assert torch.equal(y.view(B, U * s, hc, D), want.permute(1, 0, 2, 3, 4).reshape(B, U * s, hc, D))
    assert ref[0].shape == x.shape
