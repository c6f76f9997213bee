"""Generate tests/golden/wan_block_golden.pt by EXECUTING the reference's ``WanAttentionBlock``.

Run where the reference tree is mounted (CHITU_REFERENCE_ROOT points at it):

    python tests/golden/make_golden_block.py

The block (chitu_diffusion/models/model_wan.py:286-366) runs on CPU with fp32 weights.  Two
settings make that possible without touching its code:

* ``wan_attention.FLASH_ATTN_2_AVAILABLE / FLASH_ATTN_3_AVAILABLE = False`` selects the reference's own
  ``scaled_dot_product_attention`` branch (modules/attention/wan_attention.py:160-179) - the flash
  branch needs a GPU;
* the cross-attention's call ``attention(q, k, v, k_lens=...)`` is given the function's own ``dtype``
  argument as float32 (its default, bfloat16, returns a bf16 tensor that the fp32 ``o`` projection
  rejects outside autocast).

Weights and inputs are bf16-representable values so that the fixture stores them losslessly in bf16.
"""

import functools
import importlib
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))

from oracle import ref_import  # noqa: E402


def bf16_values(t):
    return t.to(torch.bfloat16).to(torch.float32)


def main():
    ns = ref_import.load()
    wan = ns.model_wan
    wan_attention = importlib.import_module("chitu_diffusion.modules.attention.wan_attention")
    wan_attention.FLASH_ATTN_2_AVAILABLE = False
    wan_attention.FLASH_ATTN_3_AVAILABLE = False
    wan.attention = functools.partial(wan_attention.attention, dtype=torch.float32)

    gen = torch.Generator().manual_seed(2024)
    dim, heads, ffn, text = 128, 1, 256, 8
    grid = torch.tensor([[2, 3, 4]])
    L = 24
    backend = ns.DiffusionAttnBackend("torch_sdpa")
    block = wan.WanAttentionBlock(backend, None, "t2v_cross_attn", dim, ffn, heads, (-1, -1), True, True, 1e-6)
    with torch.no_grad():
        for name, prm in block.named_parameters():
            if name.endswith("norm_q.weight") or name.endswith("norm_k.weight") or name == "norm3.weight":
                prm.copy_(bf16_values(1.0 + 0.1 * torch.randn(prm.shape, generator=gen)))
            elif name.endswith(".bias") or name == "modulation":
                prm.copy_(bf16_values(0.1 * torch.randn(prm.shape, generator=gen)))
            else:
                prm.copy_(bf16_values(0.05 * torch.randn(prm.shape, generator=gen)))
        x = bf16_values(torch.randn(1, L, dim, generator=gen))
        e = bf16_values(0.3 * torch.randn(1, 6, dim, generator=gen))
        context = bf16_values(torch.randn(1, text, dim, generator=gen))
        freqs = torch.cat([wan.rope_params(1024, dim // heads - 4 * (dim // heads // 6)),
                           wan.rope_params(1024, 2 * (dim // heads // 6)),
                           wan.rope_params(1024, 2 * (dim // heads // 6))], dim=1)
        out = block(x, e, torch.tensor([L]), grid, freqs, context, None)
    g = dict(
        dim=dim, heads=heads, ffn=ffn, grid=grid, x=x.to(torch.bfloat16), e=e.to(torch.bfloat16),
        context=context.to(torch.bfloat16), out=out.clone(),
        params={k: v.detach().to(torch.bfloat16) for k, v in block.named_parameters()},
    )
    path = os.path.join(HERE, "wan_block_golden.pt")
    torch.save(g, path)
    print("wrote", path, os.path.getsize(path), "bytes; out", tuple(out.shape), out.dtype, float(out.abs().max()))


if __name__ == "__main__":
    main()
