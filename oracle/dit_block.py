"""CPU restatement of the Wan DiT block around the attention hot path.

TEST INFRASTRUCTURE ONLY - imported by tests/, the smoke check and the CPU legs of bench.py.

Follows ``WanAttentionBlock.forward`` (chitu_diffusion/models/model_wan.py:321-366):

    e_0..e_5 = (modulation + e).chunk(6)                              fp32          (:339-341)
    y = self_attn(LayerNorm(x) * (1 + e_1) + e_0);  x = x + y * e_2                 (:344-348)
    x = x + cross_attn(LayerNorm_affine(x), context)                                (:352)
    y = ffn(LayerNorm(x) * (1 + e_4) + e_3);        x = x + y * e_5                 (:353-355)

with ``WanLayerNorm`` (no affine unless ``cross_attn_norm``; computed in fp32, :68-78),
``WanSelfAttention`` (:141-208), ``WanT2VCrossAttention`` (:211-232: RMSNorm on q and k, no rotary,
attention over the text tokens) and the FFN ``Linear -> GELU(tanh) -> Linear`` (:312-314).

``self_attn_bf16=True`` reproduces where the reference module itself rounds on a CPU run: q/k/v of the
self-attention are cast to bf16 (``half()``, :80-81,198-200) and SDPA runs on bf16 tensors (the
golden fixture is made that way; its cross-attention runs in fp32, see tests/golden/make_golden_block.py).
``False`` keeps everything in fp32 - the accuracy reference for the GPU block.
"""

from __future__ import annotations

from typing import Dict, Sequence

import torch
import torch.nn.functional as F

from .reference_math import wan_rms_norm, wan_rope_table, wan_self_attention_pre


def layer_norm_fp32(x: torch.Tensor, eps: float, weight=None, bias=None) -> torch.Tensor:
    """``WanLayerNorm.forward``: ``LayerNorm(x.float()).type_as(x)`` (model_wan.py:68-78)."""
    return F.layer_norm(x.float(), (x.shape[-1],), weight, bias, eps).type_as(x)


def _sdpa(q, k, v, low_precision: bool):
    if low_precision:
        q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    else:
        q, k, v = (t.float() for t in (q, k, v))
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    return o.transpose(1, 2).contiguous()


def wan_block(x: torch.Tensor, e: torch.Tensor, p: Dict[str, torch.Tensor], grid: Sequence[int],
              context: torch.Tensor, num_heads: int, eps: float = 1e-6, self_attn_bf16: bool = False) -> torch.Tensor:
    """One Wan T2V block.  ``x [B,L,C]`` fp32, ``e [B,6,C]`` fp32, ``context [B,T,C]``; ``p`` holds the weights
    under the reference's parameter names (``self_attn.q.weight``, ..., ``ffn.0.weight``, ``modulation``)."""
    B, L, C = x.shape
    D = C // num_heads
    lin = lambda t, name: F.linear(t, p[name + ".weight"], p[name + ".bias"])  # noqa: E731
    mod = (p["modulation"].float() + e.float()).chunk(6, dim=1)  # six [B,1,C]

    # self-attention
    h = layer_norm_fp32(x, eps).float() * (1 + mod[1]) + mod[0]
    freqs = wan_rope_table(D)
    q, k, v = wan_self_attention_pre(
        lin(h, "self_attn.q"), lin(h, "self_attn.k"), lin(h, "self_attn.v"), p["self_attn.norm_q.weight"],
        p["self_attn.norm_k.weight"], num_heads, [list(grid)] * B, freqs, eps, round_bf16=self_attn_bf16)
    y = lin(_sdpa(q, k, v, self_attn_bf16).to(x.dtype).flatten(2), "self_attn.o")
    x = x + y * mod[2]

    # cross-attention over the text tokens
    h = layer_norm_fp32(x, eps, p.get("norm3.weight"), p.get("norm3.bias"))
    q = wan_rms_norm(lin(h, "cross_attn.q"), p["cross_attn.norm_q.weight"], eps).view(B, L, num_heads, D)
    k = wan_rms_norm(lin(context, "cross_attn.k"), p["cross_attn.norm_k.weight"], eps).view(B, -1, num_heads, D)
    v = lin(context, "cross_attn.v").view(B, -1, num_heads, D)
    x = x + lin(_sdpa(q, k, v, False).to(x.dtype).flatten(2), "cross_attn.o")

    # feed-forward
    h = layer_norm_fp32(x, eps).float() * (1 + mod[4]) + mod[3]
    y = lin(F.gelu(lin(h, "ffn.0"), approximate="tanh"), "ffn.2")
    return x + y * mod[5]
