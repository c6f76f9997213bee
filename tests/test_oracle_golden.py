"""The CPU oracle replayed against vectors produced by the reference's own code.

Fixtures: tests/golden/hotpath_golden.pt, written by tests/golden/make_golden.py
(which imports and runs the reference).  These tests need no reference tree.
"""

import torch

import oracle


def test_sdpa_matches_reference_backend(golden):
    for name in ("sdpa_square", "sdpa_ragged", "sdpa_scale", "sdpa_d64"):
        c = golden[name]
        out, lse = oracle.sdpa_fp32(c["q"], c["k"], c["v"], c["scale"], return_lse=True)
        assert out.shape == c["out"].shape and out.is_contiguous()
        assert torch.allclose(out, c["out"], atol=2e-6, rtol=1e-5), name
        assert lse.shape == (c["q"].shape[0], c["q"].shape[2], c["q"].shape[1])


def test_sdpa_chunking_is_invisible(golden):
    c = golden["sdpa_ragged"]
    a = oracle.sdpa_fp32(c["q"], c["k"], c["v"], chunk=4)
    b = oracle.sdpa_fp32(c["q"], c["k"], c["v"], chunk=4096)
    assert torch.allclose(a, b, atol=1e-6)


def test_lse_merge_chain(golden):
    for name in ("lse_merge", "lse_merge_bf16"):
        c = golden[name]
        o, l = None, None
        for bo, bl in zip(c["outs"], c["lses"]):
            o, l = oracle.update_out_and_lse(o, l, bo, bl)
        assert o.dtype == torch.float32 and l.shape == c["lse"].shape
        assert torch.allclose(o, c["out"], atol=1e-6)
        assert torch.allclose(l, c["lse"], atol=1e-6)


def test_lse_merge_equals_full_attention():
    torch.manual_seed(3)
    q = torch.randn(1, 19, 2, 32)
    k = torch.randn(1, 50, 2, 32)
    v = torch.randn(1, 50, 2, 32)
    full, full_lse = oracle.sdpa_fp32(q, k, v, return_lse=True)
    parts = [oracle.sdpa_fp32(q, k[:, a:b], v[:, a:b], return_lse=True) for a, b in ((0, 7), (7, 30), (30, 50))]
    out, lse = oracle.merge_partials([p[0] for p in parts], [p[1] for p in parts])
    assert torch.allclose(out, full, atol=2e-6)
    assert torch.allclose(lse, full_lse, atol=2e-6)


def test_wan_rms_norm(golden):
    for name in ("wan_norm_fp32", "wan_norm_bf16"):
        c = golden[name]
        y = oracle.wan_rms_norm(c["x"], c["weight"], c["eps"])
        assert y.dtype == c["out"].dtype
        assert torch.equal(y, c["out"]), name


def test_wan_rope(golden):
    freqs = oracle.wan_rope_table(128)
    for name in ("wan_rope", "wan_rope_bf16"):
        c = golden[name]
        y = oracle.wan_rope_apply(c["x"], c["grid"], freqs)
        assert y.dtype == torch.float32
        assert torch.equal(y, c["out"]), name


def test_wan_rope_with_cp(golden):
    c = golden["wan_rope_cp"]
    freqs = oracle.wan_rope_table(128)
    for r, (x, ref) in enumerate(zip(c["xs"], c["outs"])):
        y = oracle.wan_rope_apply_with_cp(x, c["grid"], freqs, c["cp_size"], r)
        assert torch.equal(y, ref)


def test_wan_layer_end_to_end(golden):
    c = golden["wan_layer"]
    heads = c["heads"]
    d = c["x"].shape[-1] // heads
    freqs = oracle.wan_rope_table(d)
    ones = torch.ones(c["x"].shape[-1])
    q, k, v = oracle.wan_self_attention_pre(c["q_proj"], c["k_proj"], c["v_proj"], ones, ones, heads, c["grid"], freqs)
    assert q.dtype == torch.bfloat16
    # the reference module runs SDPA on the bf16-rounded tensors
    o = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    ).transpose(1, 2)
    y = o.to(torch.float32).flatten(2) @ c["wo"].t()
    assert torch.allclose(y, c["out"], atol=1e-6)


def test_pad_split(golden):
    c = golden["pad_split"]
    parts = oracle.split_sequence_padding(c["x"], c["n"], c["dim"])
    assert len(parts) == len(c["parts"])
    for a, b in zip(parts, c["parts"]):
        assert torch.equal(a, b)


def test_wan_block_matches_reference_block():
    """The restated DiT block against the output of the reference's WanAttentionBlock (fixture made by
    tests/golden/make_golden_block.py)."""
    import os

    g = torch.load(os.path.join(os.path.dirname(__file__), "golden", "wan_block_golden.pt"), weights_only=False)
    params = {k: v.float() for k, v in g["params"].items()}
    out = oracle.wan_block(g["x"].float(), g["e"].float(), params, g["grid"][0].tolist(), g["context"].float(),
                           g["heads"], self_attn_bf16=True)
    assert out.dtype == torch.float32 and out.shape == g["out"].shape
    assert (out - g["out"]).abs().max().item() <= 2e-5
    # the all-fp32 form differs from it only by the bf16 rounding of the self-attention operands
    out32 = oracle.wan_block(g["x"].float(), g["e"].float(), params, g["grid"][0].tolist(), g["context"].float(),
                             g["heads"])
    assert (out32 - g["out"]).abs().max().item() <= 2e-2
