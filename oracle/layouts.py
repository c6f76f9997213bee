"""Single-process simulators of the context-parallel data movement.

TEST INFRASTRUCTURE ONLY - never imported by the product package.

Every function takes a Python list with one CPU tensor per rank and performs,
as pure index shuffles plus calls of a per-rank attention callable, what the
reference's wrapper does with NCCL collectives.  This lets every rank map,
chunk order, valid-length rule and merge order be checked without GPUs or
process groups.  ``attn(q, k, v, return_lse) -> (out [B,Sq,H,D], lse [B,H,Sq] | None)``.
"""

from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch

from .reference_math import sdpa_fp32, update_out_and_lse


def _default_attn(q, k, v, return_lse):
    if return_lse:
        return sdpa_fp32(q, k, v, return_lse=True)
    return sdpa_fp32(q, k, v), None


# --------------------------------------------------------------------------- #
# rank maps
# --------------------------------------------------------------------------- #


def cfg_rank_lists(world: int, cfg_size: int) -> List[List[int]]:
    """CFG groups: singletons, or pairs ``[i, i + world/2]``.

    Follows chitu_diffusion/core/distributed/parallel_state.py:329-345.
    """
    if cfg_size == 1:
        return [[r] for r in range(world)]
    if cfg_size != 2:
        raise ValueError("CFG size can only be 1 or 2")
    half = world // 2
    return [[i, i + half] for i in range(half)]


def cp_rank_lists(world: int, cfg_size: int) -> List[List[int]]:
    """CP groups: all ranks, or the two halves when CFG parallelism is on.

    Follows chitu_diffusion/core/distributed/parallel_state.py:347-362.
    """
    if cfg_size == 2:
        half = world // 2
        return [list(range(half)), list(range(half, world))]
    return [list(range(world))]


def up_rank_lists(world: int, cfg_size: int, up_size: int) -> List[List[int]]:
    """Ulysses groups: consecutive ``up_size`` slices of every CP group.

    Follows chitu_diffusion/core/distributed/parallel_state.py:364-399.
    """
    out = []
    for ranks in cp_rank_lists(world, cfg_size):
        for i in range(0, len(ranks), up_size):
            out.append(ranks[i : i + up_size])
    return out


# --------------------------------------------------------------------------- #
# Ulysses all-to-all as an index shuffle
# --------------------------------------------------------------------------- #


def ulysses_scatter_heads(xs: Sequence[torch.Tensor]) -> List[torch.Tensor]:
    """``[B,s,H,D]`` per rank -> ``[B,U*s,H/U,D]`` per rank (scatter heads, gather sequence).

    Follows chitu_diffusion/core/distributed/comm_group.py:363-371: rank ``r``
    ends up with head slice ``[r*H/U, (r+1)*H/U)`` of every rank's tokens, and
    the gathered sequence is rank-major (rank 0's tokens first).
    """
    U = len(xs)
    H = xs[0].shape[2]
    if H % U:
        raise ValueError(f"head dim {H} must be divisible by CP size {U}")
    hc = H // U
    return [torch.cat([x[:, :, r * hc : (r + 1) * hc] for x in xs], dim=1).contiguous() for r in range(U)]


def ulysses_gather_heads(ys: Sequence[torch.Tensor]) -> List[torch.Tensor]:
    """``[B,U*s,h,D]`` per rank -> ``[B,s,U*h,D]`` per rank (scatter sequence, gather heads).

    Follows chitu_diffusion/core/distributed/comm_group.py:372-380.
    """
    U = len(ys)
    S = ys[0].shape[1]
    if S % U:
        raise ValueError(f"sequence dim {S} must be divisible by CP size {U}")
    sc = S // U
    return [torch.cat([y[:, r * sc : (r + 1) * sc] for y in ys], dim=2).contiguous() for r in range(U)]


def _scatter_lse(ls: Sequence[torch.Tensor]) -> List[torch.Tensor]:
    """LSE ``[B,h,U*s]`` per rank -> ``[B,U*h,s]`` per rank (scatter dim 2, gather dim 1).

    Follows the list-based exchange at diffusion_attn_backend.py:828 /
    comm_group.py:335-338.
    """
    U = len(ls)
    sc = ls[0].shape[2] // U
    return [torch.cat([l[:, :, r * sc : (r + 1) * sc] for l in ls], dim=1).contiguous() for r in range(U)]


# --------------------------------------------------------------------------- #
# whole-wrapper simulators
# --------------------------------------------------------------------------- #


def simulate_ucp(
    qs: Sequence[torch.Tensor],
    ks: Sequence[torch.Tensor],
    vs: Sequence[torch.Tensor],
    up: int,
    attn: Callable = _default_attn,
) -> List[torch.Tensor]:
    """Ulysses x ring attention over ``P = len(qs)`` ranks; returns local outputs.

    Follows chitu_diffusion/modules/attention/diffusion_attn_backend.py:744-837:
    ``U = min(P, up)``, ``R = P // U``; Ulysses groups are consecutive U-sized
    slices; at every ring step rank ``r`` sends its current K/V to ``(r-U) % P``
    and receives from ``(r+U) % P``; each block result is exchanged back to the
    local layout and folded with the LSE merge.  With ``R > 1`` the result is
    fp32, as in the reference.
    """
    P = len(qs)
    U = P if P <= up else up
    R = P // U
    q, k, v = list(qs), list(ks), list(vs)
    groups = [list(range(g, g + U)) for g in range(0, P, U)]
    if U > 1:
        for g in groups:
            for name, buf in (("q", q), ("k", k), ("v", v)):
                res = ulysses_scatter_heads([buf[r] for r in g])
                for r, t in zip(g, res):
                    buf[r] = t
    out: List[Optional[torch.Tensor]] = [None] * P
    lse: List[Optional[torch.Tensor]] = [None] * P
    for step in range(R):
        blk = [attn(q[r], k[r], v[r], R > 1) for r in range(P)]
        f_out = [b[0] if R == 1 else b[0].to(torch.float32) for b in blk]
        f_lse = [b[1] for b in blk]
        if step + 1 != R:
            k = [k[(r + U) % P] for r in range(P)]
            v = [v[(r + U) % P] for r in range(P)]
        if U > 1:
            for g in groups:
                res = ulysses_gather_heads([f_out[r] for r in g])
                for r, t in zip(g, res):
                    f_out[r] = t
                if R > 1:
                    resl = _scatter_lse([f_lse[r] for r in g])
                    for r, t in zip(g, resl):
                        f_lse[r] = t
        for r in range(P):
            if R == 1:
                out[r] = f_out[r]
            else:
                out[r], lse[r] = update_out_and_lse(out[r], lse[r], f_out[r], f_lse[r])
    return out  # type: ignore[return-value]


def simulate_agcp(
    qs: Sequence[torch.Tensor],
    ks: Sequence[torch.Tensor],
    vs: Sequence[torch.Tensor],
    attn: Callable = _default_attn,
) -> List[torch.Tensor]:
    """All-gather-KV attention: local Q against the rank-ordered full K/V.

    Follows chitu_diffusion/modules/attention/diffusion_attn_backend.py:581-597,739-742.
    """
    k_full = torch.cat(list(ks), dim=1)
    v_full = torch.cat(list(vs), dim=1)
    return [attn(q, k_full, v_full, False)[0] for q in qs]


def simulate_full_txt(
    txt_q: torch.Tensor,
    txt_k: torch.Tensor,
    txt_v: torch.Tensor,
    img_qs: Sequence[torch.Tensor],
    img_ks: Sequence[torch.Tensor],
    img_vs: Sequence[torch.Tensor],
    image_seq_len: int,
    up: int,
    cp_backend: str = "ucp",
    attn: Callable = _default_attn,
) -> List[Tuple[torch.Tensor, torch.Tensor]]:
    """Replicated-text + sharded-image attention (Qwen-Image layout).

    Follows chitu_diffusion/modules/attention/diffusion_attn_backend.py:839-984.
    Returns, per rank, ``(text output for all heads, local image output)``.
    """
    P = len(img_qs)
    txt_len = txt_q.shape[1]
    if cp_backend == "agcp":
        k_img = torch.cat(list(img_ks), dim=1)[:, :image_seq_len]
        v_img = torch.cat(list(img_vs), dim=1)[:, :image_seq_len]
        k = torch.cat([txt_k, k_img], dim=1)
        v = torch.cat([txt_v, v_img], dim=1)
        res = []
        for r in range(P):
            o = attn(torch.cat([txt_q, img_qs[r]], dim=1), k, v, False)[0]
            res.append((o[:, :txt_len], o[:, txt_len:]))
        return res

    U = P if P <= up else up
    R = P // U
    groups = [list(range(g, g + U)) for g in range(0, P, U)]
    iq, ik, iv = list(img_qs), list(img_ks), list(img_vs)
    local_len0 = iq[0].shape[1]
    tq, tk, tv = [txt_q] * P, [txt_k] * P, [txt_v] * P
    if U > 1:
        for g in groups:
            for buf in (iq, ik, iv):
                res = ulysses_scatter_heads([buf[r] for r in g])
                for r, t in zip(g, res):
                    buf[r] = t
        for r in range(P):
            ur = r % U
            tq[r] = torch.tensor_split(txt_q, U, 2)[ur].contiguous()
            tk[r] = torch.tensor_split(txt_k, U, 2)[ur].contiguous()
            tv[r] = torch.tensor_split(txt_v, U, 2)[ur].contiguous()
    block_seq = ik[0].shape[1]
    local_img_len = iq[0].shape[1]
    out: List[Optional[torch.Tensor]] = [None] * P
    lse: List[Optional[torch.Tensor]] = [None] * P
    cur_k, cur_v = ik, iv
    for step in range(R):
        for r in range(P):
            owner = (r // U + step) % R
            start = owner * block_seq
            valid = max(0, min(cur_k[r].shape[1], image_seq_len - start))
            if step == 0:
                bk = torch.cat([tk[r], cur_k[r][:, :valid]], dim=1)
                bv = torch.cat([tv[r], cur_v[r][:, :valid]], dim=1)
            else:
                bk, bv = cur_k[r][:, :valid], cur_v[r][:, :valid]
            if bk.shape[1] > 0:
                q = torch.cat([tq[r], iq[r]], dim=1)
                bo, bl = attn(q, bk, bv, R > 1)
                if R == 1:
                    out[r] = bo
                else:
                    out[r], lse[r] = update_out_and_lse(out[r], lse[r], bo, bl)
        if step + 1 != R:
            cur_k = [cur_k[(r + U) % P] for r in range(P)]
            cur_v = [cur_v[(r + U) % P] for r in range(P)]
    res: List[Optional[Tuple[torch.Tensor, torch.Tensor]]] = [None] * P
    for g in groups:
        t_outs = [out[r][:, :txt_len] for r in g]
        i_outs = [out[r][:, txt_len : txt_len + local_img_len] for r in g]
        if U > 1:
            i_outs = [t[:, :local_len0] for t in ulysses_gather_heads(i_outs)]
            t_full = torch.cat(t_outs, dim=2).contiguous()
            t_outs = [t_full] * U
        for r, to, io in zip(g, t_outs, i_outs):
            res[r] = (to, io)
    return res  # type: ignore[return-value]
