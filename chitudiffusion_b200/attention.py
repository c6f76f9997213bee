"""Per-rank attention backend with the reference's callable contract.

Mirrors ``DiffusionAttnBackend`` (chitu_diffusion/modules/attention/
diffusion_attn_backend.py:45-207): ``backend(q, k, v, ...) -> (out, lse | None,
None)`` on ``[B, S, H, D]`` tensors, an ``impl`` string attribute, the same
keyword names and the same exceptions for unsupported features.  The work is
done by the sm_100a kernel in libchitu_b200.so; nothing falls back to torch.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib, ops

BACKEND_NAME = "b200"
QUANT_BACKEND_NAME = "b200_q8"
_ALIASES = {"b200": "b200", "b200_attn": "b200", "chitu_b200": "b200", "tcgen05": "b200",
            "b200_q8": "b200_q8", "b200_sage": "b200_q8", "b200_int8": "b200_q8"}


class B200AttnBackend:
    """Drop-in for ``DiffusionAttnBackend`` selected by ``infer.attn_type: b200``."""

    def __init__(self, attn_type: str = BACKEND_NAME) -> None:
        name = _ALIASES.get(str(attn_type or BACKEND_NAME).strip().lower())
        if name is None:
            raise RuntimeError(
                f"Requested attention backend '{attn_type}' is not available. Availability: {self.availability_report()}."
            )
        _lib.load()  # raises if the CUDA library has not been built
        self.impl = name

    @staticmethod
    def availability_report() -> str:
        import os

        return f"b200={os.path.exists(_lib.LIB_PATH)}"

    def __call__(
        self,
        q: torch.Tensor,
        k: torch.Tensor,
        v: torch.Tensor,
        cu_seqlens_q: Optional[torch.Tensor] = None,
        cu_seqlens_k: Optional[torch.Tensor] = None,
        max_seqlen_q: Optional[int] = None,
        max_seqlen_k: Optional[int] = None,
        dropout_p: float = 0.0,
        softmax_scale: Optional[float] = None,
        causal: bool = False,
        window_size: Tuple[int, int] = (-1, -1),
        deterministic: bool = False,
        return_attn_probs: bool = False,
    ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
        if cu_seqlens_q is not None or cu_seqlens_k is not None:
            raise NotImplementedError("b200 backend does not support varlen attention.")
        if causal:
            raise NotImplementedError("b200 backend implements non-causal DiT attention only.")
        if dropout_p:
            raise NotImplementedError("b200 backend does not support dropout.")
        if tuple(window_size) != (-1, -1):
            raise NotImplementedError("b200 backend does not support sliding-window attention.")
        if self.impl == QUANT_BACKEND_NAME:
            # per-block INT8 QK^T / E4M3 PV, the role SageAttention plays in the reference
            # (diffusion_attn_backend.py:242-268); like there, ring CP refuses it (no LSE merge of 8-bit partials)
            out, lse = ops.attn_fwd_q8(q, k, v, softmax_scale=softmax_scale, return_lse=return_attn_probs)
        else:
            out, lse = ops.attn_fwd(q, k, v, softmax_scale=softmax_scale, return_lse=return_attn_probs)
        # a bounded device wait that ran out in an earlier call surfaces here as an exception
        ops.poll_status(q.device)
        return out, lse, None
