"""CPU restatement (fp32) of the Qwen-Image MMDiT block and of its attention processor.

TEST INFRASTRUCTURE ONLY.  PARITY UNPINNED for the block: ``QwenImageTransformerBlock`` lives in the
un-vendored ``diffusers`` (the reference only installs its own attention processor into it,
chitu_diffusion/runtime/adapter/qwen_image.py:293-303).  Restated from its published definition:

* ``img_mod`` / ``txt_mod`` = ``Linear(SiLU(temb))`` -> 6 C values, first half for the attention, second
  half for the MLP, each half ``(shift, scale, gate)``; ``x -> LayerNorm(x, eps 1e-6, no affine) * (1 + scale)
  + shift``; residual ``x + gate * f(x)``;
* joint attention over ``[text, image]`` with per-head RMSNorm (learned weight) on q and k of both
  streams, and the rotary embedding in the complex form (``use_real=False``): adjacent channel pairs
  multiplied by ``freqs[s, j]``;
* ``FeedForward(gelu-approximate)``.

The processor part follows the reference's own file line by line in meaning
(chitu_diffusion/modules/attention/qwen_image_attention.py:60-284): six producers, image rotary rows
taken at ``image_offset`` with zero rows past the end of the table (:26-34), joint order text first.
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

from .reference_math import per_head_rms_norm, sdpa_fp32


def slice_rotary_freqs(freqs: torch.Tensor, offset: int, length: int) -> torch.Tensor:
    avail = max(0, freqs.shape[0] - offset)
    part = freqs.narrow(0, offset, min(length, avail)) if avail > 0 else freqs[:0]
    if part.shape[0] == length:
        return part
    pad = torch.zeros((length - part.shape[0],) + tuple(freqs.shape[1:]), dtype=freqs.dtype)
    return torch.cat([part, pad], dim=0)


def apply_rotary_complex(x: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """``[B, S, H, D]`` real, ``freqs [S, D/2]`` complex: adjacent pairs as complex numbers times ``freqs``."""
    xc = torch.view_as_complex(x.to(torch.float64).reshape(*x.shape[:-1], -1, 2))
    out = torch.view_as_real(xc * freqs.to(torch.complex128)[None, :, None, :]).flatten(3)
    return out.to(torch.float32)


def _lin(t, p, name):
    return F.linear(t, p[name + ".weight"], p.get(name + ".bias"))


def _heads(t, H):
    B, S, C = t.shape
    return t.view(B, S, H, C // H)


def qwen_streams(hi, ht, p: Dict[str, torch.Tensor], H: int, rotary, image_offset: Optional[int] = None):
    """The six producer outputs ``(txt_q, txt_k, txt_v, img_q, img_k, img_v)`` of the processor."""
    iq = per_head_rms_norm(_heads(_lin(hi, p, "attn.to_q"), H), p["attn.norm_q.weight"])
    ik = per_head_rms_norm(_heads(_lin(hi, p, "attn.to_k"), H), p["attn.norm_k.weight"])
    iv = _heads(_lin(hi, p, "attn.to_v"), H)
    tq = per_head_rms_norm(_heads(_lin(ht, p, "attn.add_q_proj"), H), p["attn.norm_added_q.weight"])
    tk = per_head_rms_norm(_heads(_lin(ht, p, "attn.add_k_proj"), H), p["attn.norm_added_k.weight"])
    tv = _heads(_lin(ht, p, "attn.add_v_proj"), H)
    if rotary is not None:
        img_f, txt_f = rotary
        if image_offset is not None:
            img_f = slice_rotary_freqs(img_f, image_offset, hi.shape[1])
        iq, ik = apply_rotary_complex(iq, img_f), apply_rotary_complex(ik, img_f)
        tq, tk = apply_rotary_complex(tq, txt_f), apply_rotary_complex(tk, txt_f)
    return tq, tk, tv, iq, ik, iv


def qwen_attention(hi, ht, p, H, rotary) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(img_attn_output, txt_attn_output)`` of the processor on one device (joint order: text first)."""
    tq, tk, tv, iq, ik, iv = qwen_streams(hi, ht, p, H, rotary)
    o = sdpa_fp32(torch.cat([tq, iq], 1), torch.cat([tk, ik], 1), torch.cat([tv, iv], 1)).flatten(2)
    n_txt = ht.shape[1]
    return _lin(o[:, n_txt:], p, "attn.to_out.0"), _lin(o[:, :n_txt], p, "attn.to_add_out")


def qwen_double_block(img, txt, temb, p: Dict[str, torch.Tensor], H: int, rotary) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(txt_out, img_out)``."""
    def ln(x):
        return F.layer_norm(x, (x.shape[-1],), None, None, 1e-6)

    def mods(name):
        m1, m2 = _lin(F.silu(temb), p, name).chunk(2, dim=-1)
        return m1.chunk(3, dim=-1), m2.chunk(3, dim=-1)

    (ish1, isc1, ig1), (ish2, isc2, ig2) = mods("img_mod.1")
    (tsh1, tsc1, tg1), (tsh2, tsc2, tg2) = mods("txt_mod.1")
    hi = ln(img) * (1 + isc1[:, None]) + ish1[:, None]
    ht = ln(txt) * (1 + tsc1[:, None]) + tsh1[:, None]
    io, to = qwen_attention(hi, ht, p, H, rotary)
    img = img + ig1[:, None] * io
    txt = txt + tg1[:, None] * to
    h = ln(img) * (1 + isc2[:, None]) + ish2[:, None]
    img = img + ig2[:, None] * _lin(F.gelu(_lin(h, p, "img_mlp.net.0.proj"), approximate="tanh"), p, "img_mlp.net.2")
    h = ln(txt) * (1 + tsc2[:, None]) + tsh2[:, None]
    txt = txt + tg2[:, None] * _lin(F.gelu(_lin(h, p, "txt_mlp.net.0.proj"), approximate="tanh"), p, "txt_mlp.net.2")
    return txt, img
