"""Ring attention with reusable attention states (the mechanism of DiTango's state reuse).

The reference's DiTango runtime (chitu_diffusion/ditango/runtime.py:23-668) runs ring attention over the
context-parallel group and, on most denoising steps, skips part of the ring: for a skipped source block it
neither fetches the block's K/V nor computes on it, but merges the ``(out, lse)`` state it computed for
that block at an earlier step (chitu_diffusion/ditango/state.py:9-34; selective pattern,
runtime.py:59-79; reuse and merge, :632-668).  States compose associatively and commutatively, so the
result is the log-sum-exp merge of fresh and stale states in any order.

This module is that mechanism and nothing of the policy: the caller passes, per call, which source blocks
are fresh (``plan[t]`` for the block of rank ``(r + t) % P``; ``plan[0]``, the local block, must be fresh).
Every rank of the group must pass the same plan - a fresh block is one send and one receive.  The
reference's planner (curvature-based schedules, state-alignment correction) is not mirrored.

Blocks are attended with the backend passed in (the b200 kernel on GPUs) and merged with the log-sum-exp
combine kernel, or with the merger the caller injects (CPU tests).
"""

from __future__ import annotations

from typing import Callable, Dict, Optional, Sequence, Tuple

import torch

from .comm import CommGroup, get_cp_group


class CachedRingAttention:
    def __init__(self, attn_backend, group: Optional[CommGroup] = None, layer_id: int = 0,
                 merger_factory: Optional[Callable[[], object]] = None) -> None:
        from .context_parallel import _KernelMerger

        self.attn = getattr(attn_backend, "attn", attn_backend)
        self.group = group if group is not None else get_cp_group()
        self.layer_id = int(layer_id)
        self._merger_factory = merger_factory or _KernelMerger
        # (tag, source offset) -> (block_out [B, s, H, D], block_lse [B, H, s]) of the step that computed it
        self._states: Dict[Tuple[str, int], Tuple[torch.Tensor, torch.Tensor]] = {}
        self.stats = {"fresh_blocks": 0, "reused_blocks": 0}

    def clear(self) -> None:
        self._states.clear()

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, plan: Optional[Sequence[bool]] = None,
                 tag: str = "cond", softmax_scale: Optional[float] = None) -> torch.Tensor:
        """``q, k, v [B, s, H, D]`` (this rank's rows); returns the merged fp32 ``[B, s, H, D]``.

        ``plan[t]`` true: fetch the K/V of rank ``(r + t) % P`` and attend them now (the state is kept);
        false: reuse the state kept for that block under ``tag``.  ``None``: everything fresh.
        """
        g = self.group
        P, r = g.group_size, g.rank_in_group
        plan = [True] * P if plan is None else [bool(x) for x in plan]
        if len(plan) != P:
            raise ValueError(f"plan needs one entry per rank of the group ({P}), got {len(plan)}")
        if not plan[0]:
            raise ValueError("the local block (plan[0]) is always computed")
        for t in range(1, P):
            if not plan[t] and (tag, t) not in self._states:
                raise RuntimeError(f"no state kept for source offset {t} under tag {tag!r}: it must be fresh once first")
        # post every transfer of the call at once: my K/V to rank r - t, the block of rank r + t to me
        incoming = {}
        k, v = k.contiguous(), v.contiguous()
        for t in range(1, P):
            if plan[t]:
                g.p2p_isend(k, (r - t) % P)
                g.p2p_isend(v, (r - t) % P)
                incoming[t] = (g.p2p_irecv(k.shape, k.dtype, (r + t) % P), g.p2p_irecv(v.shape, v.dtype, (r + t) % P))
        if incoming:
            g.p2p_commit()
        merger = self._merger_factory()
        out, lse, _ = self.attn(q, k, v, softmax_scale=softmax_scale, causal=False, return_attn_probs=True)
        merger.add(out, lse)
        self.stats["fresh_blocks"] += 1
        if incoming:
            g.p2p_wait()
        for t in range(1, P):
            if plan[t]:
                bk, bv = incoming[t]
                out, lse, _ = self.attn(q, bk, bv, softmax_scale=softmax_scale, causal=False, return_attn_probs=True)
                self._states[(tag, t)] = (out, lse)
                self.stats["fresh_blocks"] += 1
            else:
                out, lse = self._states[(tag, t)]
                self.stats["reused_blocks"] += 1
            merger.add(out, lse)
        return merger.result()


__all__ = ["CachedRingAttention"]
