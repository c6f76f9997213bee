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


def _flux_inputs(dim, n_txt, side, heads):
    from chitudiffusion_b200 import pre_attention

    gen = torch.Generator().manual_seed(21)
    n_img = side * side
    img = torch.randn(2, n_img, dim, generator=gen).to(torch.bfloat16)
    txt = torch.randn(2, n_txt, dim, generator=gen).to(torch.bfloat16)
    temb = torch.randn(2, dim, generator=gen).to(torch.bfloat16)
    ids = torch.zeros(n_txt + n_img, 3)
    ids[n_txt:, 1] = torch.arange(side).repeat_interleave(side)
    ids[n_txt:, 2] = torch.arange(side).repeat(side)
    cos, sin = oracle.axis_rope_table(ids, (16, 56, 56))
    table = pre_attention.axis_rope_table(ids, (16, 56, 56))
    return img, txt, temb, cos, sin, table


def _randomise(blk, seed):
    """Non-trivial biases and norm weights (random_init leaves them at 0 / 1)."""
    gen = torch.Generator().manual_seed(seed)
    for name, t in blk.w.items():
        if name.endswith(".bias"):
            t.copy_((0.05 * torch.randn(t.shape, generator=gen)).to(t.dtype))
        elif "norm_" in name:
            t.copy_(1.0 + 0.1 * torch.randn(t.shape, generator=gen))


def test_flux_double_block_against_oracle(cuda):
    from chitudiffusion_b200 import B200AttnBackend
    from chitudiffusion_b200.flux_dit import FluxDoubleBlock

    dim, heads = 256, 2
    img, txt, temb, cos, sin, table = _flux_inputs(dim, 24, 12, heads)
    blk = FluxDoubleBlock.random_init(dim, heads, cuda, seed=9, std=0.05)
    _randomise(blk, 4)
    w = {k: v.float().cpu() for k, v in blk.w.items()}
    C = dim
    p = {}
    for s, mod, qkv, nq, nk, out, ff in (
            ("img", "norm1", ("attn.to_q", "attn.to_k", "attn.to_v"), "attn.norm_q", "attn.norm_k", "attn.to_out.0", "ff"),
            ("txt", "norm1_context", ("attn.add_q_proj", "attn.add_k_proj", "attn.add_v_proj"), "attn.norm_added_q",
             "attn.norm_added_k", "attn.to_add_out", "ff_context")):
        p[mod + ".linear.weight"], p[mod + ".linear.bias"] = w[f"{s}.mod.weight"], w[f"{s}.mod.bias"]
        for i, n in enumerate(qkv):
            p[n + ".weight"], p[n + ".bias"] = w[f"{s}.qkv.weight"][i * C:(i + 1) * C], w[f"{s}.qkv.bias"][i * C:(i + 1) * C]
        p[nq + ".weight"], p[nk + ".weight"] = w[f"{s}.norm_q"], w[f"{s}.norm_k"]
        p[out + ".weight"], p[out + ".bias"] = w[f"{s}.out.weight"], w[f"{s}.out.bias"]
        p[ff + ".net.0.proj.weight"], p[ff + ".net.0.proj.bias"] = w[f"{s}.ff1.weight"], w[f"{s}.ff1.bias"]
        p[ff + ".net.2.weight"], p[ff + ".net.2.bias"] = w[f"{s}.ff2.weight"], w[f"{s}.ff2.bias"]
    ref_txt, ref_img = oracle.flux_double_block(img.float(), txt.float(), temb.float(), p, heads, cos, sin)
    # the from_reference_params route must rebuild the same block
    blk2 = FluxDoubleBlock.from_reference_params(p, heads, cuda)
    for b in (blk, blk2):
        o_txt, o_img = b(img.to(cuda).clone(), txt.to(cuda).clone(), temb.to(cuda), table.to(cuda), B200AttnBackend("b200"))
        for out, ref in ((o_txt, ref_txt), (o_img, ref_img)):
            err, cos_sim = _close(out, ref)
            assert err <= 3e-2 and cos_sim >= 0.999, (err, cos_sim)


def test_flux_single_block_against_oracle(cuda):
    from chitudiffusion_b200 import B200AttnBackend
    from chitudiffusion_b200.flux_dit import FluxSingleBlock

    dim, heads = 256, 2
    img, txt, temb, cos, sin, table = _flux_inputs(dim, 24, 12, heads)
    x = torch.cat([txt, img], 1)
    blk = FluxSingleBlock.random_init(dim, heads, cuda, seed=10, std=0.05)
    _randomise(blk, 5)
    w = {k: v.float().cpu() for k, v in blk.w.items()}
    C = dim
    p = {"norm.linear.weight": w["mod.weight"], "norm.linear.bias": w["mod.bias"], "proj_mlp.weight": w["mlp.weight"],
         "proj_mlp.bias": w["mlp.bias"], "attn.norm_q.weight": w["norm_q"], "attn.norm_k.weight": w["norm_k"],
         "proj_out.weight": torch.cat([w["out_attn.weight"], w["out_mlp.weight"]], 1), "proj_out.bias": w["out.bias"]}
    for i, n in enumerate(("attn.to_q", "attn.to_k", "attn.to_v")):
        p[n + ".weight"], p[n + ".bias"] = w["qkv.weight"][i * C:(i + 1) * C], w["qkv.bias"][i * C:(i + 1) * C]
    ref = oracle.flux_single_block(x.float(), temb.float(), p, heads, cos, sin)
    blk2 = FluxSingleBlock.from_reference_params(p, heads, cuda)
    for b in (blk, blk2):
        out = b(x.to(cuda).clone(), temb.to(cuda), table.to(cuda), B200AttnBackend("b200"))
        err, cos_sim = _close(out, ref)
        assert err <= 3e-2 and cos_sim >= 0.999, (err, cos_sim)


def _qwen_inputs(dim, n_txt, n_img, heads):
    gen = torch.Generator().manual_seed(33)
    img = torch.randn(2, n_img, dim, generator=gen).to(torch.bfloat16)
    txt = torch.randn(2, n_txt, dim, generator=gen).to(torch.bfloat16)
    temb = torch.randn(2, dim, generator=gen).to(torch.bfloat16)
    half = dim // heads // 2
    ang_i = torch.randn(n_img, half, generator=gen, dtype=torch.float64)
    ang_t = torch.randn(n_txt, half, generator=gen, dtype=torch.float64)
    rotary = (torch.polar(torch.ones_like(ang_i), ang_i), torch.polar(torch.ones_like(ang_t), ang_t))
    return img, txt, temb, rotary


def test_qwen_double_block_and_processor_against_oracle(cuda):
    """The Qwen-Image MMDiT block (and the attention processor inside it) against the fp32 restatement; the block's
    definition lives in the un-vendored diffusers, so this parity is unpinned - the processor's call contract is the
    reference's own."""
    from chitudiffusion_b200 import B200AttnBackend
    from chitudiffusion_b200.qwen import B200QwenAttnProcessor, QwenDoubleBlock, slice_rotary_table
    from chitudiffusion_b200.pre_attention import table_from_complex

    dim, heads = 256, 2
    img, txt, temb, rotary = _qwen_inputs(dim, 20, 150, heads)
    blk = QwenDoubleBlock.random_init(dim, heads, cuda, seed=12, std=0.05)
    gen = torch.Generator().manual_seed(6)
    for name, t in blk.p.items():
        if name.endswith(".bias"):
            t.copy_((0.05 * torch.randn(t.shape, generator=gen)).to(t.dtype))
        elif "norm" in name:
            t.copy_(1.0 + 0.1 * torch.randn(t.shape, generator=gen))
    p = {k: v.float().cpu() for k, v in blk.p.items()}
    ref_txt, ref_img = oracle.qwen_double_block(img.float(), txt.float(), temb.float(), p, heads, rotary)
    proc = B200QwenAttnProcessor(B200AttnBackend("b200"))
    blk2 = QwenDoubleBlock.from_reference(p, heads, cuda)
    rot_dev = tuple(r.to(cuda) for r in rotary)
    for b in (blk, blk2):
        o_txt, o_img = b(img.to(cuda).clone(), txt.to(cuda).clone(), temb.to(cuda), rot_dev, proc)
        for out, ref in ((o_txt, ref_txt), (o_img, ref_img)):
            err, cos_sim = _close(out, ref)
            assert err <= 3e-2 and cos_sim >= 0.999, (err, cos_sim)
    # rows of the image rotary table taken at an offset, zero past the end (what a rank with a padded shard gets)
    t = table_from_complex(rotary[0])
    got = slice_rotary_table(t, 140, 16)
    assert torch.equal(got[:10], t[140:150]) and not got[10:].any()
    want = oracle.slice_rotary_freqs(rotary[0], 140, 16)
    assert torch.equal(got, table_from_complex(want))
    with pytest.raises(ValueError):
        proc(blk.attn, img.to(cuda), None)
    with pytest.raises(NotImplementedError):
        proc(blk.attn, img.to(cuda), txt.to(cuda), attention_mask=torch.ones(1))
