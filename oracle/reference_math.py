"""CPU restatement of the arithmetic on ChituDiffusion's attention hot path.

TEST INFRASTRUCTURE ONLY - never imported by the product package.

Each function cites the reference file:line it follows (paths are relative to
the reference project root).  Tensors use the reference's layouts:
``q, k, v, out`` are ``[B, S, H, D]``; the block log-sum-exp is ``[B, H, S]``.
"""

from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch

# --------------------------------------------------------------------------- #
# attention core
# --------------------------------------------------------------------------- #


def sdpa_fp32(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    softmax_scale: Optional[float] = None,
    return_lse: bool = False,
    chunk: int = 2048,
):
    """Non-causal, mask-free scaled-dot-product attention in fp32.

    Follows chitu_diffusion/modules/attention/diffusion_attn_backend.py:270-315
    (``_fwd_torch_sdpa``): inputs ``[B,S,H,D]`` are viewed as ``[B,H,S,D]``,
    ``softmax(scale * q k^T) v`` with ``scale`` defaulting to ``D**-0.5``, and
    the result is returned as a contiguous ``[B,Sq,H,D]`` tensor.  The
    log-sum-exp mirrors what ``aten::_scaled_dot_product_flash_attention``
    returns at :296-303: natural log of ``sum_j exp(scale * q.k_j)``, shape
    ``[B,H,Sq]``, fp32.

    Query rows are processed in chunks so that the ``Sq x Sk`` score matrix of
    the long video shapes never has to exist at once.
    """
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    qf = q.detach().to(torch.float32).permute(0, 2, 1, 3)  # [B,H,Sq,D]
    kf = k.detach().to(torch.float32).permute(0, 2, 3, 1)  # [B,H,D,Sk]
    vf = v.detach().to(torch.float32).permute(0, 2, 1, 3)  # [B,H,Sk,D]
    out = torch.empty(B, H, Sq, D, dtype=torch.float32)
    lse = torch.empty(B, H, Sq, dtype=torch.float32)
    if Sk == 0:
        out.zero_()
        lse.fill_(-float("inf"))
    for s0 in range(0, Sq, chunk):
        if Sk == 0:
            break
        s1 = min(Sq, s0 + chunk)
        scores = torch.matmul(qf[:, :, s0:s1], kf) * scale  # [B,H,c,Sk]
        row_lse = torch.logsumexp(scores, dim=-1)
        probs = torch.exp(scores - row_lse.unsqueeze(-1))
        out[:, :, s0:s1] = torch.matmul(probs, vf)
        lse[:, :, s0:s1] = row_lse
    out = out.permute(0, 2, 1, 3).contiguous()
    if return_lse:
        return out, lse
    return out


def sdpa_reference_call(q, k, v, softmax_scale: Optional[float] = None) -> torch.Tensor:
    """The exact library call the reference's torch-SDPA backend makes, on CPU tensors.

    Follows chitu_diffusion/modules/attention/diffusion_attn_backend.py:283-285,305-315:
    ``[B,S,H,D]`` -> ``transpose(1, 2)`` views -> ``F.scaled_dot_product_attention(attn_mask=None,
    dropout_p=0, is_causal=False, scale=softmax_scale)`` -> ``transpose(1, 2).contiguous()``.  This is
    the form timed as the CPU baseline (torch's fused CPU kernel); :func:`sdpa_fp32` is the explicit
    form that also yields the log-sum-exp.
    """
    out = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=None, dropout_p=0.0, is_causal=False,
        scale=softmax_scale,
    )
    return out.transpose(1, 2).contiguous()


# --------------------------------------------------------------------------- #
# Wan pre-attention: full-width RMSNorm + 3-axis complex RoPE
# --------------------------------------------------------------------------- #


def wan_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Wan's QK-RMSNorm: statistics over the WHOLE channel dim (all heads).

    Follows chitu_diffusion/models/model_wan.py:49-65.  Rounding order matters:
    the normalised value is computed in fp32, rounded back to ``x``'s dtype,
    and only then multiplied by the weight (whose product follows torch type
    promotion, e.g. bf16 * fp32 -> fp32).
    """
    xf = x.to(torch.float32)
    rstd = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * rstd).to(x.dtype) * weight


def wan_rope_params(max_seq_len: int, dim: int, theta: float = 10000.0) -> torch.Tensor:
    """Unit complex128 table ``[max_seq_len, dim/2]`` of ``exp(i * pos * theta^(-2j/dim))``.

    Follows chitu_diffusion/models/model_wan.py:37-45.
    """
    if dim % 2:
        raise ValueError("rope dim must be even")
    expo = torch.arange(0, dim, 2, dtype=torch.float64) / dim
    inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64), expo)
    ang = torch.outer(torch.arange(max_seq_len, dtype=torch.float64), inv)
    return torch.polar(torch.ones_like(ang), ang)


def wan_rope_table(head_dim: int, max_seq_len: int = 1024, theta: float = 10000.0) -> torch.Tensor:
    """The concatenated t/h/w table Wan builds once per model.

    Follows chitu_diffusion/models/model_wan.py:513-518: three tables with real
    dims ``d - 4*(d//6)``, ``2*(d//6)``, ``2*(d//6)`` joined along dim 1, giving
    ``[1024, d/2]`` complex entries (22 + 21 + 21 pairs at d = 128).
    """
    d = head_dim
    return torch.cat(
        [
            wan_rope_params(max_seq_len, d - 4 * (d // 6), theta),
            wan_rope_params(max_seq_len, 2 * (d // 6), theta),
            wan_rope_params(max_seq_len, 2 * (d // 6), theta),
        ],
        dim=1,
    )


def _wan_token_freqs(grid: Sequence[int], freqs: torch.Tensor, pairs: int) -> torch.Tensor:
    """Per-token complex multipliers ``[f*h*w, pairs]`` for a (f, h, w) grid.

    Token n sits at ``f = n // (h*w)``, ``h = (n // w) % h``, ``w = n % w``
    (row-major expansion, chitu_diffusion/models/model_wan.py:98-102); the pair
    axis is split ``[pairs - 2*(pairs//3), pairs//3, pairs//3]`` for t/h/w (:88).
    """
    f, h, w = (int(g) for g in grid)
    n_h = pairs // 3
    n_t = pairs - 2 * n_h
    ft, fh, fw = freqs[:, :n_t], freqs[:, n_t : n_t + n_h], freqs[:, n_t + n_h : n_t + 2 * n_h]
    n = torch.arange(f * h * w)
    idx_t = n // (h * w)
    idx_h = (n // w) % h
    idx_w = n % w
    return torch.cat([ft[idx_t], fh[idx_h], fw[idx_w]], dim=1)


def wan_rope_apply(x: torch.Tensor, grid_sizes, freqs: torch.Tensor) -> torch.Tensor:
    """3-axis rotary embedding on interleaved pairs, float64 complex arithmetic.

    Follows chitu_diffusion/models/model_wan.py:83-110.  ``x`` is ``[B,S,H,D]``;
    adjacent elements ``(x[2j], x[2j+1])`` form one complex number that is
    multiplied by the token's multiplier; tokens past ``f*h*w`` pass through
    unchanged; the result is fp32.
    """
    B, S, H, D = x.shape
    pairs = D // 2
    grids = grid_sizes.tolist() if hasattr(grid_sizes, "tolist") else list(grid_sizes)
    rows = []
    for b, grid in enumerate(grids):
        mult = _wan_token_freqs(grid, freqs, pairs)  # [n, pairs] complex128
        n = mult.shape[0]
        xc = torch.view_as_complex(x[b, :n].to(torch.float64).reshape(n, H, pairs, 2))
        rot = torch.view_as_real(xc * mult[:, None, :]).reshape(n, H, D)
        rows.append(torch.cat([rot, x[b, n:].to(torch.float64)], dim=0))
    return torch.stack(rows).to(torch.float32)


def wan_rope_apply_with_cp(
    x: torch.Tensor, grid_sizes, freqs: torch.Tensor, cp_size: int, cp_rank: int
) -> torch.Tensor:
    """Rank-local rotary embedding under context parallelism.

    Follows chitu_diffusion/modules/utils/wan/__init__.py:17-67: the full
    per-token multiplier table is padded with ones up to ``s * cp_size`` and
    this rank takes rows ``[cp_rank*s, (cp_rank+1)*s)`` of it, where ``s`` is
    the local sequence length.
    """
    B, s, H, D = x.shape
    pairs = D // 2
    grids = grid_sizes.tolist() if hasattr(grid_sizes, "tolist") else list(grid_sizes)
    rows = []
    for b, grid in enumerate(grids):
        mult = _wan_token_freqs(grid, freqs, pairs)
        pad = s * cp_size - mult.shape[0]
        if pad > 0:
            mult = torch.cat([mult, torch.ones(pad, pairs, dtype=mult.dtype)], dim=0)
        mult = mult[cp_rank * s : (cp_rank + 1) * s]
        xc = torch.view_as_complex(x[b].to(torch.float64).reshape(s, H, pairs, 2))
        rows.append(torch.view_as_real(xc * mult[:, None, :]).reshape(s, H, D))
    return torch.stack(rows).to(torch.float32)


def wan_self_attention_pre(
    xq: torch.Tensor,
    xk: torch.Tensor,
    xv: torch.Tensor,
    wq: torch.Tensor,
    wk: torch.Tensor,
    num_heads: int,
    grid_sizes,
    freqs: torch.Tensor,
    eps: float = 1e-6,
    cp_size: int = 1,
    cp_rank: int = 0,
    round_bf16: bool = True,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Projection outputs ``[B,S,C]`` -> the (q, k, v) handed to the backend.

    Follows chitu_diffusion/models/model_wan.py:152-156,194-200: RMSNorm on the
    flat channel dim, head split, rotary embedding, then ``half()`` (a bf16 cast
    for non-half inputs, :80-81).  ``round_bf16=False`` keeps fp32 (the
    "all-fp32" variant the acceptance tolerance is quoted against).
    """
    B, S, C = xq.shape
    D = C // num_heads
    q = wan_rms_norm(xq, wq, eps).view(B, S, num_heads, D)
    k = wan_rms_norm(xk, wk, eps).view(B, S, num_heads, D)
    v = xv.view(B, S, num_heads, D)
    if cp_size > 1:
        q = wan_rope_apply_with_cp(q, grid_sizes, freqs, cp_size, cp_rank)
        k = wan_rope_apply_with_cp(k, grid_sizes, freqs, cp_size, cp_rank)
    else:
        q = wan_rope_apply(q, grid_sizes, freqs)
        k = wan_rope_apply(k, grid_sizes, freqs)
    if round_bf16:
        q, k = q.to(torch.bfloat16), k.to(torch.bfloat16)
        v = v if v.dtype in (torch.float16, torch.bfloat16) else v.to(torch.bfloat16)
    return q, k, v


# --------------------------------------------------------------------------- #
# Flux / Qwen pre-attention: per-head RMSNorm + axis RoPE   (parity unpinned)
# --------------------------------------------------------------------------- #


def per_head_rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm over the head dim of ``[B,S,H,D]`` (Flux / Qwen QK-norm).

    The reference delegates this to ``diffusers`` (``Attention(qk_norm=
    "rms_norm", eps=1e-6)``, chitu_diffusion/models/model_flux1.py:77-88); that
    package is not vendored, so this is the published definition
    ``x * rsqrt(mean_D(x^2) + eps) * w`` with fp32 statistics.  PARITY UNPINNED.
    """
    xf = x.to(torch.float32)
    y = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.to(torch.float32)
    return y


def axis_rope_table(ids: torch.Tensor, axes_dims: Sequence[int], theta: float = 10000.0):
    """cos/sin tables ``[S, sum(axes_dims)/2]`` (fp64) from integer position ids ``[S, n_axes]``.

    Axis ``a`` contributes ``axes_dims[a]/2`` pairs with angle
    ``ids[:, a] * theta^(-2j/axes_dims[a])``; Flux uses axes dims (16, 56, 56),
    text ids all zero (chitu_diffusion/modules/encoders/clip_t5.py:88) and image
    ids ``(0, row, col)`` (chitu_diffusion/modules/utils/flux/__init__.py:70-75).
    The table construction itself is diffusers' ``FluxPosEmbed``: PARITY UNPINNED.
    """
    cols = []
    for a, dim in enumerate(axes_dims):
        expo = torch.arange(0, dim, 2, dtype=torch.float64) / dim
        inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64), expo)
        cols.append(torch.outer(ids[:, a].to(torch.float64), inv))
    ang = torch.cat(cols, dim=1)
    return torch.cos(ang), torch.sin(ang)


def apply_rope_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate adjacent pairs ``(x[2j], x[2j+1])`` of ``[B,S,H,D]`` by per-token angles.

    The pairing is the same interleaved one the two in-tree exemplars use
    (chitu_diffusion/models/model_wan.py:96-105 and
    chitu_diffusion/modules/attention/z_image_attention.py:87-93).  fp64 math,
    fp32 result.
    """
    B, S, H, D = x.shape
    xd = x.to(torch.float64).reshape(B, S, H, D // 2, 2)
    c = cos[None, :, None, :]
    s = sin[None, :, None, :]
    re = xd[..., 0] * c - xd[..., 1] * s
    im = xd[..., 0] * s + xd[..., 1] * c
    return torch.stack([re, im], dim=-1).reshape(B, S, H, D).to(torch.float32)


# --------------------------------------------------------------------------- #
# log-sum-exp combine of partial attention results
# --------------------------------------------------------------------------- #


def update_out_and_lse(
    out: Optional[torch.Tensor],
    lse: Optional[torch.Tensor],
    block_out: torch.Tensor,
    block_lse: torch.Tensor,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Fold one partial result into the running (out, lse).

    Follows chitu_diffusion/runtime/parallel_utils.py:59-97.  ``out`` is
    ``[B,S,H,D]`` fp32, ``lse`` is ``[B,S,H,1]`` fp32, ``block_lse`` arrives as
    ``[B,H,S]``.  First block: copy.  Later blocks:
    ``out <- out - sigmoid(lse_b - lse) * (out - out_b)``,
    ``lse <- lse - logsigmoid(lse - lse_b)``.
    """
    b_out = block_out.to(torch.float32)
    b_lse = block_lse.to(torch.float32).transpose(-2, -1).unsqueeze(-1)
    if out is None:
        return b_out, b_lse
    new_out = out - torch.sigmoid(b_lse - lse) * (out - b_out)
    new_lse = lse - torch.nn.functional.logsigmoid(lse - b_lse)
    return new_out, new_lse


def merge_partials(outs: List[torch.Tensor], lses: List[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sequentially merge N partials; returns ``out [B,S,H,D]`` fp32 and ``lse [B,H,S]`` fp32."""
    out, lse = None, None
    for o, l in zip(outs, lses):
        out, lse = update_out_and_lse(out, lse, o, l)
    return out, lse.squeeze(-1).transpose(-1, -2).contiguous()


# --------------------------------------------------------------------------- #
# sequence padding used when the token count does not divide the CP size
# --------------------------------------------------------------------------- #


def split_sequence_padding(t: torch.Tensor, parts: int, dim: int = 0) -> List[torch.Tensor]:
    """Zero-pad ``dim`` up to a multiple of ``parts`` and split into equal shards.

    Follows chitu_diffusion/runtime/parallel_utils.py:11-32.
    """
    size = t.size(dim)
    shard = -(-size // parts)
    pad = shard * parts - size
    if pad:
        shape = list(t.shape)
        shape[dim] = pad
        t = torch.cat([t, torch.zeros(shape, dtype=t.dtype)], dim=dim)
    return list(torch.split(t, shard, dim=dim))
