"""Replicated-text + sharded-image context-parallel attention core.

Mirror of ``ImageContextParallelAttention`` (chitu_diffusion/modules/attention/image_cp_attention.py:81-505):
one instance is shared by every attention block of a model; ``enable(group)`` arms it; ``attention``
takes the replicated text Q/K/V and this rank's image shard and returns ``(text output for all
heads, local image output)``.  The four exchanges are the ones of the generic wrapper, so this
class only resolves the mode into a layout and hands over to ``B200ContextParallel``:

    agkv            all-gather of the image K/V (:637-653)            -> cp_backend "agcp"
    ulysses         head / sequence all-to-all over the group (:740-769; falls back to agkv when the
                    head count does not divide, :474-483)             -> Ulysses degree = cp_size
    ring, ring_graph  K/V rotation, send to r-1, receive from r+1, text K/V joined at step 0
                    (:883-943)                                        -> Ulysses degree 1
    unified         Ulysses inside ``ulysses_size`` sub-groups x ring across them, pure ring when
                    the degree does not divide cp_size (:945-1065)    -> Ulysses degree = ulysses_size

The reference's optional FP8 transfer of K/V and its cross-step K/V cache (environment switches,
:131-157) change the numerics of the exchange and are not mirrored.
"""

from __future__ import annotations

import time
from typing import Dict, Optional, Tuple

import torch

from .context_parallel import B200ContextParallel

_VALID_MODES = {"agkv", "ulysses", "ring", "ring_graph", "unified"}


class B200ImageContextParallel:
    def __init__(self, attn_backend, *, mode: str = "agkv", profile: bool = False, use_cudagraph: bool = True,
                 ulysses_size: int = 1, merger_factory=None) -> None:
        # a CP wrapper is unwrapped to the raw kernel so that CP is applied exactly once, here
        self.attn_backend = getattr(attn_backend, "attn", attn_backend)
        mode = str(mode).strip().lower()
        if mode not in _VALID_MODES:
            raise ValueError(f"CP mode must be one of {sorted(_VALID_MODES)}, got {mode!r}.")
        self.mode = mode
        self.profile = bool(profile)
        self.use_cudagraph = bool(use_cudagraph)
        self.ulysses_size = max(1, int(ulysses_size))
        self._merger_factory = merger_factory
        self._group = None
        self._enabled = False
        self._wrappers: Dict[Tuple[int, str], B200ContextParallel] = {}
        self._cur_step: Optional[int] = None
        self.reset_stats()

    # ------------------------------------------------------------------ switches
    def enable(self, group) -> None:
        self._group = group
        self._enabled = True

    def disable(self) -> None:
        self._enabled = False

    @property
    def enabled(self) -> bool:
        return self._enabled and self._group is not None and self._group.group_size > 1

    @property
    def group(self):
        return self._group

    @property
    def supports_fused_overlap(self) -> bool:
        return self.enabled and torch.cuda.is_available() and not self.profile and self.mode in ("agkv", "ulysses")

    def begin_forward(self, step: int, total_steps: int, cfg_tag: str = "cond") -> None:
        """Step bookkeeping of the reference's K/V cache schedule; kept for call compatibility."""
        self._cur_step, self._cur_total, self._cur_tag = step, total_steps, cfg_tag

    # ------------------------------------------------------------------ statistics
    def reset_stats(self) -> None:
        self._stats = {"calls": 0, "total_ms": 0.0}

    def stats(self) -> dict:
        out = dict(self._stats)
        out["mode"] = self.mode
        out["avg_ms"] = out["total_ms"] / out["calls"] if out["calls"] and self.profile else None
        return out

    # ------------------------------------------------------------------ layout resolution
    def _layout(self, heads: int) -> Tuple[int, str]:
        """``(ulysses_degree, cp_backend)`` for the current mode, group size and head count."""
        cp = self._group.group_size
        if self.mode == "agkv":
            return cp, "agcp"
        if self.mode == "ulysses":
            return (cp, "ucp") if heads % cp == 0 else (cp, "agcp")
        if self.mode in ("ring", "ring_graph"):
            return 1, "ucp"
        u = min(self.ulysses_size, cp)
        if cp % u != 0 or heads % u != 0:
            u = 1
        return u, "ucp"

    def _wrapper(self, heads: int) -> B200ContextParallel:
        key = self._layout(heads)
        w = self._wrappers.get(key)
        if w is None:
            kw = {} if self._merger_factory is None else {"merger_factory": self._merger_factory}
            w = B200ContextParallel(self.attn_backend, key[0], cp_backend=key[1], group=self._group, **kw)
            self._wrappers[key] = w
        return w

    # ------------------------------------------------------------------ attention
    def attention(self, txt_q, txt_k, txt_v, img_q, img_k, img_v) -> Tuple[torch.Tensor, torch.Tensor]:
        """``txt_* [B, S_txt, H, D]`` replicated, ``img_* [B, S_img_local, H, D]`` this rank's shard."""
        if self._group is None:
            raise RuntimeError("enable(group) must be called before attention()")
        t0 = None
        if self.profile:
            if img_q.is_cuda:
                torch.cuda.synchronize(img_q.device)
            t0 = time.perf_counter()
        txt_out, img_out = self._wrapper(img_q.shape[2]).cp_attn_with_full_txt(txt_q, txt_k, txt_v, img_q, img_k, img_v)
        if txt_out.dtype != img_q.dtype:  # merged ring results are fp32; this API hands back the compute dtype
            txt_out, img_out = txt_out.to(img_q.dtype), img_out.to(img_q.dtype)
        self._stats["calls"] += 1
        if t0 is not None:
            if img_q.is_cuda:
                torch.cuda.synchronize(img_q.device)
            self._stats["total_ms"] += (time.perf_counter() - t0) * 1e3
        return txt_out.contiguous(), img_out.contiguous()

    def _attention_from_packed(self, q, k, v, img_len: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """``[image_shard, text]`` packed along the sequence (:253-258)."""
        return self.attention(q[:, img_len:], k[:, img_len:], v[:, img_len:], q[:, :img_len], k[:, :img_len],
                              v[:, :img_len])
