"""CPU emulation of the 8-bit attention variant (per-block INT8 QK^T, E4M3 PV, fp32 accumulate).

TEST INFRASTRUCTURE ONLY - never imported by the product package.

The reference delegates this path to the third-party wheel ``sageattention`` (git dependency
``thu-ml/SageAttention`` without a commit pin, chitu_diffusion/modules/attention/
diffusion_attn_backend.py:242-268), which is neither vendored nor installable here: PARITY UNPINNED.
This file restates the published SageAttention recipe in the exact tiling of the CUDA kernel so
that the kernel can be checked product by product:

* K is centred over the tokens per (batch, head, channel);
* Q is multiplied by ``softmax_scale * log2(e)`` and quantised to INT8 with one scale per block of
  128 tokens, K with one scale per block of 64 tokens (``scale = max|x| / 127``);
* V is quantised to E4M3 with one scale per (batch, head, channel) (``max|v| -> 448``);
* per 128-key step: integer scores, base-2 online softmax with the lazy-rescale rule of the kernel
  (threshold 4, stored probabilities ``2^(s - m + 4)`` rounded to E4M3), fp32 accumulation.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

SHIFT, THRESHOLD = 4.0, 4.0


def _block_quant(x: torch.Tensor, block: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [B,S,H,D] fp32 -> (int8 values as fp32, scales [B,H,nblk]) with one scale per token block."""
    B, S, H, D = x.shape
    nblk = -(-S // block)
    pad = nblk * block - S
    xp = torch.cat([x, x.new_zeros(B, pad, H, D)], dim=1) if pad else x
    blocks = xp.view(B, nblk, block, H, D)
    amax = blocks.abs().amax(dim=(2, 4))  # [B,nblk,H]
    scale = amax.clamp_min(1e-8) / 127.0
    q = torch.round(blocks / scale[:, :, None, :, None]).clamp_(-127, 127)
    return q.view(B, nblk * block, H, D)[:, :S], scale.permute(0, 2, 1).contiguous()


def quantise(q, k, v, softmax_scale: Optional[float] = None):
    D = q.shape[-1]
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    qf = q.float() * (scale * 1.4426950408889634)
    kmean = k.float().mean(dim=1, keepdim=True)
    kf = k.float() - kmean
    q8, q_sc = _block_quant(qf, 128)
    k8, k_sc = _block_quant(kf, 64)
    v_amax = v.float().abs().amax(dim=1)  # [B,H,D]
    v8 = (v.float() * (448.0 / v_amax.clamp_min(1e-8))[:, None]).to(torch.float8_e4m3fn).float()
    q_corr = (qf * kmean).sum(-1).permute(0, 2, 1).contiguous()  # [B,H,Sq]
    return q8, q_sc, k8, k_sc, v8, v_amax, q_corr


def attention_q8(q, k, v, softmax_scale: Optional[float] = None, return_lse: bool = False):
    """Emulation of ``chitu_b200_attn_fwd_q8``; returns ``out [B,Sq,H,D]`` fp32 (and ``lse [B,H,Sq]``)."""
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    q8, q_sc, k8, k_sc, v8, v_amax, q_corr = quantise(q, k, v, softmax_scale)
    qh = q8.permute(0, 2, 1, 3)  # [B,H,Sq,D]
    kh = k8.permute(0, 2, 1, 3)
    vh = v8.permute(0, 2, 1, 3)
    row_sc = q_sc.repeat_interleave(128, dim=2)[:, :, :Sq]  # [B,H,Sq]
    col_sc = k_sc.repeat_interleave(64, dim=2)[:, :, :Sk]  # [B,H,Sk]
    m = torch.full((B, H, Sq), -float("inf"))
    l = torch.zeros(B, H, Sq)
    o = torch.zeros(B, H, Sq, D)
    for j0 in range(0, Sk, 128):
        j1 = min(Sk, j0 + 128)
        s_int = torch.matmul(qh, kh[:, :, j0:j1].transpose(-1, -2))  # exact small integers in fp32
        x = s_int * row_sc[..., None] * col_sc[:, :, None, j0:j1]
        mx = x.amax(dim=-1)
        if j0 == 0:
            m = mx
        else:
            need = (mx - m) > THRESHOLD
            f = torch.where(need, torch.exp2(m - mx), torch.ones_like(m))
            o = o * f[..., None]
            l = l * f
            m = torch.where(need, mx, m)
        p = torch.exp2(x - m[..., None] + SHIFT)
        l = l + p.sum(-1)
        p8 = p.clamp(max=448.0).to(torch.float8_e4m3fn).float()
        o = o + torch.matmul(p8, vh[:, :, j0:j1])
    out = o / (l[..., None] * 448.0) * v_amax[:, :, None, :]
    out = out.permute(0, 2, 1, 3).contiguous()
    if return_lse:
        return out, (m - SHIFT + torch.log2(l) + q_corr) * math.log(2.0)
    return out
