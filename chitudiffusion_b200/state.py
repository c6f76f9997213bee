"""Attention state: the composable ``(out, lse)`` pair that partitioned attention merges and caches.

Mirror of ``AttentionState`` (chitu_diffusion/ditango/state.py:9-34), the medium of the reference's
cached-ring-state scheme: ``out [B, S, H, D]`` fp32 and ``lse [B, S, H, 1]`` fp32 in the layouts of
``update_out_and_lse`` (chitu_diffusion/runtime/parallel_utils.py:59-97).  ``update`` folds a block
result in with the log-sum-exp combine kernel (in place after the first block); ``merge`` composes
two states; ``corrected`` applies additive deltas, as the reference's state-alignment correction does.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import ops


@dataclass
class AttentionState:
    out: Optional[torch.Tensor] = None
    lse: Optional[torch.Tensor] = None

    def is_empty(self) -> bool:
        return self.lse is None

    def update(self, block_out: torch.Tensor, block_lse: torch.Tensor) -> None:
        """``block_out [B, S, H, D]`` (16-bit or fp32), ``block_lse [B, H, S]`` fp32 - a backend's two results."""
        first = self.is_empty()
        if first:
            B, S, H, _ = block_out.shape
            self.out = torch.empty(block_out.shape, dtype=torch.float32, device=block_out.device)
            self.lse = torch.empty((B, S, H, 1), dtype=torch.float32, device=block_out.device)
        ops.lse_combine(self.out, self.lse, block_out, block_lse, first=first)

    def corrected(self, out_delta: torch.Tensor, lse_delta: torch.Tensor) -> "AttentionState":
        if self.is_empty() or self.out is None:
            return AttentionState()
        return AttentionState(
            out=self.out + out_delta.to(device=self.out.device, dtype=self.out.dtype),
            lse=self.lse + lse_delta.to(device=self.lse.device, dtype=self.lse.dtype),
        )

    @staticmethod
    def merge(state1: "AttentionState", state2: "AttentionState") -> "AttentionState":
        """``state1 (+) state2`` accumulated into ``state1`` (which may be empty)."""
        if state2.is_empty():
            return state1
        # the combine kernel reads a block's lse as [B, H, S]
        state1.update(state2.out, state2.lse.squeeze(-1).transpose(-1, -2).contiguous())
        return state1


__all__ = ["AttentionState"]
