"""GPU checks of the DiT-block kernels and of the Wan block built on them.

Tolerances: the elementwise kernels compute in fp32 and round once to bf16, so they must sit within
one bf16 ulp of the fp32 torch form; the whole block (bf16 GEMMs, bf16 attention operands) is held to
max-abs <= 3e-2 * max|ref| and cosine >= 0.999 against the fp32 oracle and against the output of the
reference's own block (tests/golden/wan_block_golden.pt).
"""

import os

import pytest
import torch
import torch.nn.functional as F

import oracle

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "wan_block_golden.pt")


@pytest.fixture(scope="module")
def cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda", 0)


@pytest.mark.parametrize("B,L,C", [(1, 7, 128), (2, 33, 1536), (1, 50, 5120), (3, 5, 8192)])
def test_layernorm_modulate(cuda, B, L, C):
    from chitudiffusion_b200 import ops

    gen = torch.Generator().manual_seed(C + L)
    x = torch.randn(B, L, C, generator=gen) * 3 + 0.5
    mod = torch.randn(B, 6, C, generator=gen) * 0.3
    ref = F.layer_norm(x, (C,), None, None, 1e-6) * (1 + mod[:, 1:2]) + mod[:, 0:1]
    modc = mod.to(cuda)
    out = ops.layernorm_modulate(x.to(cuda), modc[:, 1], modc[:, 0], add_one=True)
    assert out.dtype == torch.bfloat16
    ulp = ref.abs().clamp_min(1e-3) * 2.0 ** -8
    assert ((out.float().cpu() - ref).abs() <= ulp).all()
    # affine form shared among batches
    wgt, bias = torch.randn(C, generator=gen), torch.randn(C, generator=gen)
    ref2 = F.layer_norm(x, (C,), wgt, bias, 1e-6)
    out2 = ops.layernorm_modulate(x.to(cuda), wgt.to(cuda), bias.to(cuda), out_dtype=torch.float16)
    assert out2.dtype == torch.float16
    assert ((out2.float().cpu() - ref2).abs() <= ref2.abs().clamp_min(1e-3) * 2.0 ** -10).all()


@pytest.mark.parametrize("B,L,C", [(1, 7, 128), (2, 33, 1536), (1, 50, 5120)])
def test_gate_residual(cuda, B, L, C):
    from chitudiffusion_b200 import ops

    gen = torch.Generator().manual_seed(C)
    x = torch.randn(B, L, C, generator=gen)
    y = torch.randn(B, L, C, generator=gen).to(torch.bfloat16)
    gate = torch.randn(B, 6, C, generator=gen)
    xc = x.to(cuda)
    ops.gate_residual(xc, y.to(cuda), gate.to(cuda)[:, 2])
    assert torch.allclose(xc.cpu(), x + y.float() * gate[:, 2:3], atol=1e-6, rtol=1e-6)
    xc = x.to(cuda)
    ops.gate_residual(xc, y.to(cuda))
    assert torch.allclose(xc.cpu(), x + y.float(), atol=1e-6, rtol=1e-6)


def _close(out, ref):
    out, ref = out.float().cpu(), ref.float()
    cos = F.cosine_similarity(out.flatten(), ref.flatten(), dim=0).item()
    return (out - ref).abs().max().item() / ref.abs().max().item(), cos


def test_wan_block_against_reference_golden(cuda):
    from chitudiffusion_b200 import B200AttnBackend
    from chitudiffusion_b200.dit import WanBlock

    g = torch.load(GOLDEN, weights_only=False)
    blk = WanBlock.from_reference_params({k: v.float() for k, v in g["params"].items()}, g["heads"], cuda)
    x = g["x"].float().to(cuda)
    out = blk(x, g["e"].float().to(cuda), g["grid"][0].tolist(), g["context"].to(cuda), B200AttnBackend("b200"))
    err, cos = _close(out, g["out"])
    assert err <= 3e-2 and cos >= 0.999, (err, cos)


def test_wan_block_against_oracle(cuda):
    from chitudiffusion_b200 import B200AttnBackend
    from chitudiffusion_b200.dit import WanBlock

    dim, heads, ffn, grid, T = 256, 2, 640, (3, 6, 8), 40
    L = grid[0] * grid[1] * grid[2]
    blk = WanBlock.random_init(dim, ffn, heads, cuda, seed=5, std=0.05)
    gen = torch.Generator().manual_seed(11)
    x = torch.randn(2, L, dim, generator=gen)
    e = 0.3 * torch.randn(2, 6, dim, generator=gen)
    ctx = torch.randn(2, T, dim, generator=gen).to(torch.bfloat16)
    w = {k: v.float().cpu() for k, v in blk.w.items()}
    C = dim
    params = {
        "self_attn.q.weight": w["qkv.weight"][:C], "self_attn.k.weight": w["qkv.weight"][C:2 * C],
        "self_attn.v.weight": w["qkv.weight"][2 * C:], "self_attn.q.bias": w["qkv.bias"][:C],
        "self_attn.k.bias": w["qkv.bias"][C:2 * C], "self_attn.v.bias": w["qkv.bias"][2 * C:],
        "self_attn.o.weight": w["o.weight"], "self_attn.o.bias": w["o.bias"],
        "self_attn.norm_q.weight": w["norm_q"], "self_attn.norm_k.weight": w["norm_k"],
        "norm3.weight": w["norm3.weight"], "norm3.bias": w["norm3.bias"],
        "cross_attn.q.weight": w["cq.weight"], "cross_attn.q.bias": w["cq.bias"],
        "cross_attn.k.weight": w["ckv.weight"][:C], "cross_attn.v.weight": w["ckv.weight"][C:],
        "cross_attn.k.bias": w["ckv.bias"][:C], "cross_attn.v.bias": w["ckv.bias"][C:],
        "cross_attn.o.weight": w["co.weight"], "cross_attn.o.bias": w["co.bias"],
        "cross_attn.norm_q.weight": w["cnorm_q"], "cross_attn.norm_k.weight": w["cnorm_k"],
        "ffn.0.weight": w["ffn1.weight"], "ffn.0.bias": w["ffn1.bias"],
        "ffn.2.weight": w["ffn2.weight"], "ffn.2.bias": w["ffn2.bias"], "modulation": w["modulation"],
    }
    ref = oracle.wan_block(x, e, params, grid, ctx.float(), heads)
    out = blk(x.to(cuda), e.to(cuda), grid, ctx.to(cuda), B200AttnBackend("b200"))
    err, cos = _close(out, ref)
    assert err <= 3e-2 and cos >= 0.999, (err, cos)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rescale", [False, True])
def test_cfg_combine(cuda, dtype, rescale):
    from chitudiffusion_b200 import ops

    gen = torch.Generator().manual_seed(3)
    cond = torch.randn(2, 777, 64, generator=gen).to(dtype)
    uncond = torch.randn(2, 777, 64, generator=gen).to(dtype)
    out = ops.cfg_combine(cond.to(cuda), uncond.to(cuda), 4.0, rescale)
    comb = uncond + 4.0 * (cond - uncond)
    ref = comb * (torch.norm(cond, dim=-1, keepdim=True) / torch.norm(comb, dim=-1, keepdim=True)) if rescale else comb
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert out.dtype == dtype and torch.allclose(out.float().cpu(), ref.float(), atol=tol, rtol=tol)
