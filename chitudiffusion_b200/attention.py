"""Per-rank attention backend with the reference's callable contract.

Mirrors ``DiffusionAttnBackend`` (chitu_diffusion/modules/attention/
diffusion_attn_backend.py:45-207): ``backend(q, k, v, ...) -> (out, lse | None,
None)`` on ``[B, S, H, D]`` tensors, an ``impl`` string attribute, the same
keyword names and the same exceptions for unsupported features.  The work is
done by the sm_100a kernel in libchitu_b200.so; nothing falls back to torch.
"""

from __future__ import annotations

import os
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
        # measurement hook: set to a list and every attention launch appends its (start, end) CUDA events
        self.event_log = None
        # query transform inside the attention kernel instead of the pre-pass (see attention_from_projections)
        self.q_in_kernel = False

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
        ev = self._event_start()
        if self.impl == QUANT_BACKEND_NAME:
            # per-block INT8 QK^T / E4M3 PV, the role SageAttention plays in the reference
            # (diffusion_attn_backend.py:242-268); like there, ring CP refuses it (no LSE merge of 8-bit partials)
            out, lse = ops.attn_fwd_q8(q, k, v, softmax_scale=softmax_scale, return_lse=return_attn_probs)
        else:
            out, lse = ops.attn_fwd(q, k, v, softmax_scale=softmax_scale, return_lse=return_attn_probs)
        self._event_stop(ev)
        # a bounded device wait that ran out in an earlier call surfaces here as an exception
        ops.poll_status(q.device)
        return out, lse, None

    def _event_start(self):
        if self.event_log is None:
            return None
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        return ev

    def _event_stop(self, start) -> None:
        if start is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self.event_log.append((start, end))

    # ------------------------------------------------------------------ projections in, attention out
    def attention_from_projections(self, jobs, v_proj: torch.Tensor, *, row_offset: int = 0, last: bool = True,
                                   softmax_scale: Optional[float] = None, **batch_args) -> Optional[torch.Tensor]:
        """Pre-attention transform and attention of one layer; same contract as
        ``B200ContextParallel.attention_from_projections`` (so model code calls one name on one or many GPUs).

        Two placements of q's transform exist and give bit-identical results.  Default: q and k both go
        through the pre-pass kernel (one launch).  With ``CHITU_B200_Q_PRELOAD=fused`` (or
        ``self.q_in_kernel = True``) a layer that arrives in ONE piece has its query transform done INSIDE the
        attention kernel: only k goes through the pre-pass, q is read once - raw - by the attention
        kernel's own tile copies and normalised / rotated in shared memory.  Measured on B200 at the Flux
        shape the in-kernel form saves 31 us of pre-pass per layer and costs 38 us of attention prologue
        (each CTA fetches 128 KB of rotary factors while its K/V ring is filling), so the pre-pass is the
        default; ``bench.py`` prints both.  Layers that arrive in row pieces (Flux's separately projected
        text and image streams) are transformed piece by piece into joint tensors.
        """
        from .pre_attention import transform_pieces

        pieces = getattr(self, "_pending_pieces", None) or []
        pieces.append((jobs, v_proj, row_offset, dict(batch_args)))
        self._pending_pieces = pieces
        if not last:
            return None
        self._pending_pieces = []
        dtype = batch_args.get("out_dtype", torch.bfloat16)
        x0 = jobs[0]["x"]
        fuse = (len(pieces) == 1 and row_offset == 0 and self.impl == BACKEND_NAME and x0.dtype == dtype
                and v_proj.dtype == dtype
                and (self.q_in_kernel or os.environ.get("CHITU_B200_Q_PRELOAD", "prepass") == "fused"))
        if not fuse:
            q, k, v = transform_pieces(pieces, dtype)
            return self(q, k, v, softmax_scale=softmax_scale)[0]
        B, S, C = x0.shape
        H = int(batch_args["num_heads"])
        D = C // H
        args = {key: val for key, val in batch_args.items() if key != "out_dtype"}
        q_job, k_job = jobs
        k_jobs = [dict(k_job)]
        rstd = None
        if int(q_job.get("norm_mode", 2)) == 0:
            # full-width statistic of q: a statistics-only job in the same launch as k's transform
            rstd = torch.empty((B, S), dtype=torch.float32, device=x0.device)
            k_jobs.append(dict(x=q_job["x"], weight=q_job.get("weight"), norm_mode=0, rope_mode=k_job.get("rope_mode", 0),
                               rstd_out=rstd))
        k = ops.qk_norm_rope_batch(k_jobs, out_dtype=dtype, **args)[0]
        q_pre = dict(norm_mode=q_job.get("norm_mode", 2), rope_mode=q_job.get("rope_mode", 0), weight=q_job.get("weight"),
                     rstd=rstd, eps=args.get("eps", 1e-6), rope_table=args.get("rope_table"), grid=args.get("grid", (0, 0, 0)),
                     axis_split=args.get("axis_split", (0, 0)), pos_offset=args.get("pos_offset", 0),
                     round_mid=args.get("round_mid", True))
        ev = self._event_start()
        out, _ = ops.attn_fwd(x0.view(B, S, H, D) if x0.is_contiguous() else x0.unflatten(2, (H, D)), k,
                              v_proj.unflatten(2, (H, D)) if v_proj.dim() == 3 else v_proj,
                              softmax_scale=softmax_scale, q_pre=q_pre)
        self._event_stop(ev)
        ops.poll_status(x0.device)
        return out
