"""CPU restatement (fp32) of the Flux double- and single-stream blocks around the joint attention.

TEST INFRASTRUCTURE ONLY.  PARITY UNPINNED: the block forwards are in the reference tree
(``FluxTransformerBlock.forward`` / ``FluxSingleTransformerBlock.forward``,
chitu_diffusion/models/model_flux1.py:90-116,180-236) and so is the attention processor
(``ChituFluxAttnProcessor2_0.__call__``, chitu_diffusion/modules/attention/flux_attention.py:96-171),
but the layers they are built from come from the un-vendored ``diffusers==0.36.0``
(``requirements.txt:1``) and the reference holds no vectors for them.  Those layers are restated
from their published definitions:

* ``AdaLayerNormZero``: ``emb = Linear(SiLU(temb))`` split into shift/scale/gate for the attention
  and for the MLP; ``x -> LayerNorm(x, eps=1e-6, no affine) * (1 + scale) + shift``;
  ``AdaLayerNormZeroSingle`` is the three-chunk form;
* ``Attention(qk_norm="rms_norm", eps=1e-6)``: per-head RMSNorm with a learned weight on q and k
  (separate weights for the text stream's added projections);
* ``FeedForward(activation_fn="gelu-approximate")``: ``Linear(C, 4C) -> GELU(tanh) -> Linear(4C, C)``;
* ``apply_rotary_emb``: rotation of adjacent pairs by per-token angles.

Parameter names are the reference modules' own (``norm1.linear.weight``, ``attn.to_q.weight``, ...).
"""

from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.nn.functional as F

from .reference_math import apply_rope_interleaved, per_head_rms_norm, sdpa_fp32


def _lin(t, p, name):
    return F.linear(t, p[name + ".weight"], p.get(name + ".bias"))


def _ada_chunks(temb, p, name, n):
    return _lin(F.silu(temb), p, name + ".linear").chunk(n, dim=1)


def _ln(x):
    return F.layer_norm(x, (x.shape[-1],), None, None, 1e-6)


def _heads(t, H):
    B, S, C = t.shape
    return t.view(B, S, H, C // H)


def flux_double_block(img: torch.Tensor, txt: torch.Tensor, temb: torch.Tensor, p: Dict[str, torch.Tensor], H: int,
                      cos: torch.Tensor, sin: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(txt_out, img_out)``; ``cos`` / ``sin`` are ``[S_txt + S_img, D/2]`` for the joint sequence (text first)."""
    sh_a, sc_a, g_a, sh_m, sc_m, g_m = _ada_chunks(temb, p, "norm1", 6)
    csh_a, csc_a, cg_a, csh_m, csc_m, cg_m = _ada_chunks(temb, p, "norm1_context", 6)
    hi = _ln(img) * (1 + sc_a[:, None]) + sh_a[:, None]
    ht = _ln(txt) * (1 + csc_a[:, None]) + csh_a[:, None]
    q = per_head_rms_norm(_heads(_lin(hi, p, "attn.to_q"), H), p["attn.norm_q.weight"])
    k = per_head_rms_norm(_heads(_lin(hi, p, "attn.to_k"), H), p["attn.norm_k.weight"])
    v = _heads(_lin(hi, p, "attn.to_v"), H)
    tq = per_head_rms_norm(_heads(_lin(ht, p, "attn.add_q_proj"), H), p["attn.norm_added_q.weight"])
    tk = per_head_rms_norm(_heads(_lin(ht, p, "attn.add_k_proj"), H), p["attn.norm_added_k.weight"])
    tv = _heads(_lin(ht, p, "attn.add_v_proj"), H)
    q = apply_rope_interleaved(torch.cat([tq, q], 1), cos, sin)
    k = apply_rope_interleaved(torch.cat([tk, k], 1), cos, sin)
    o = sdpa_fp32(q, k, torch.cat([tv, v], 1)).flatten(2)
    n_txt = txt.shape[1]
    img = img + g_a[:, None] * _lin(o[:, n_txt:], p, "attn.to_out.0")
    txt = txt + cg_a[:, None] * _lin(o[:, :n_txt], p, "attn.to_add_out")
    h = _ln(img) * (1 + sc_m[:, None]) + sh_m[:, None]
    img = img + g_m[:, None] * _lin(F.gelu(_lin(h, p, "ff.net.0.proj"), approximate="tanh"), p, "ff.net.2")
    h = _ln(txt) * (1 + csc_m[:, None]) + csh_m[:, None]
    txt = txt + cg_m[:, None] * _lin(F.gelu(_lin(h, p, "ff_context.net.0.proj"), approximate="tanh"), p,
                                     "ff_context.net.2")
    return txt, img


def flux_single_block(x: torch.Tensor, temb: torch.Tensor, p: Dict[str, torch.Tensor], H: int, cos: torch.Tensor,
                      sin: torch.Tensor) -> torch.Tensor:
    """``x`` is the joint ``[text, image]`` stream."""
    shift, scale, gate = _ada_chunks(temb, p, "norm", 3)
    h = _ln(x) * (1 + scale[:, None]) + shift[:, None]
    mlp = F.gelu(_lin(h, p, "proj_mlp"), approximate="tanh")
    q = apply_rope_interleaved(per_head_rms_norm(_heads(_lin(h, p, "attn.to_q"), H), p["attn.norm_q.weight"]), cos, sin)
    k = apply_rope_interleaved(per_head_rms_norm(_heads(_lin(h, p, "attn.to_k"), H), p["attn.norm_k.weight"]), cos, sin)
    o = sdpa_fp32(q, k, _heads(_lin(h, p, "attn.to_v"), H)).flatten(2)
    return x + gate[:, None] * _lin(torch.cat([o, mlp], dim=2), p, "proj_out")
