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

Two optional approximations of the reference's all-gather mode, switched by the same environment
variables (:131-157), are mirrored for the ``agkv`` mode (they change the result, as they do there):

    CHITU_CP_FP8_KV=1     the image K/V of the OTHER ranks travel as e4m3 bytes with one fp32 scale per head
                          and rank and are dequantised on arrival; this rank's own shard stays exact (:376-420)
    CHITU_CP_KV_CACHE=1   cross-step cache: after ``begin_forward(step, total, tag)`` the gathered image K/V of
                          every (tag, layer) is kept; on "stale" steps - not among the first
                          CHITU_CP_KV_CACHE_WARMUP (8), not among the last CHITU_CP_KV_CACHE_TAIL (3), not a
                          multiple of CHITU_CP_KV_CACHE_INTERVAL (4) - nothing is gathered: the cached tensors
                          are reused with this rank's fresh shard spliced in (:167-205)

The producer-callback entries (``attention_fused``, ``cp_attn_with_full_txt_fused``,
``attention_fused_packed``, :508-635) run the producers and take the same paths: the overlap they buy
in the reference comes here from the exchange kernels themselves.
"""

from __future__ import annotations

import os
import time
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from .context_parallel import B200ContextParallel

_VALID_MODES = {"agkv", "ulysses", "ring", "ring_graph", "unified"}
_FP8_MAX = 448.0  # largest e4m3 magnitude


def quantize_fp8_per_head(x: torch.Tensor):
    """``[B, S, H, D]`` -> (e4m3 payload viewed as uint8, fp32 scale ``[1, 1, H, 1]``); restates :61-73."""
    amax = x.abs().to(torch.float32).amax(dim=(0, 1, 3), keepdim=True).clamp_min(1e-12)
    scale = amax / _FP8_MAX
    q = (x.to(torch.float32) / scale).clamp_(-_FP8_MAX, _FP8_MAX).to(torch.float8_e4m3fn)
    return q.view(torch.uint8), scale


def dequantize_fp8(x_u8: torch.Tensor, scale: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    return (x_u8.view(torch.float8_e4m3fn).to(torch.float32) * scale).to(out_dtype)


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
        self._fp8_kv = os.environ.get("CHITU_CP_FP8_KV", "0") == "1"
        self._kvcache_enabled = os.environ.get("CHITU_CP_KV_CACHE", "0") == "1"
        self._kvcache_warmup = int(os.environ.get("CHITU_CP_KV_CACHE_WARMUP", "8"))
        self._kvcache_interval = max(1, int(os.environ.get("CHITU_CP_KV_CACHE_INTERVAL", "4")))
        self._kvcache_tail = int(os.environ.get("CHITU_CP_KV_CACHE_TAIL", "3"))
        self._kvcache: Dict[tuple, tuple] = {}
        self._cur_step: Optional[int] = None
        self._cur_total: Optional[int] = None
        self._cur_tag = "cond"
        self._layer_idx = 0
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
        """Announce the denoising step before a transformer forward (:167-178): the K/V cache decides fresh or
        stale from it and keys its entries per (tag, layer).  Nothing happens while the cache is off."""
        if not self._kvcache_enabled:
            return
        if step == 0 and cfg_tag == "cond":
            self._kvcache.clear()
        self._cur_step, self._cur_total, self._cur_tag = int(step), int(total_steps), str(cfg_tag)
        self._layer_idx = 0

    def _kvcache_is_fresh(self) -> bool:
        s, n = self._cur_step, self._cur_total
        if s is None or s < self._kvcache_warmup:
            return True
        if n is not None and s >= n - self._kvcache_tail:
            return True
        return s % self._kvcache_interval == 0

    # ------------------------------------------------------------------ the all-gather mode's approximations
    def all_gather_seq(self, tensor: torch.Tensor) -> torch.Tensor:
        return self._group.all_gather_sequence(tensor)

    def all_gather_seq_fp8(self, tensor: torch.Tensor) -> torch.Tensor:
        """Sequence all-gather with the other ranks' shards travelling as e4m3 bytes + per-head scales (:376-420)."""
        g = self._group
        payload, scale = quantize_fp8_per_head(tensor)
        payload, scale = payload.contiguous(), scale.contiguous()
        bytes_in = [torch.empty_like(payload) for _ in range(g.group_size)]
        scales_in = [torch.empty_like(scale) for _ in range(g.group_size)]
        pg = g.gpu_group if tensor.is_cuda else g.cpu_group
        dist.all_gather(scales_in, scale, group=pg)
        dist.all_gather(bytes_in, payload, group=pg)
        parts = [dequantize_fp8(b, sc, tensor.dtype) for b, sc in zip(bytes_in, scales_in)]
        parts[g.rank_in_group] = tensor  # the local shard never left the device: keep it exact
        return torch.cat(parts, dim=1)

    def _agkv_gather_cached(self, layer: int, img_k: torch.Tensor, img_v: torch.Tensor):
        key = (self._cur_tag, layer)
        if self._kvcache_is_fresh() or key not in self._kvcache:
            full_k, full_v = self.all_gather_seq(img_k), self.all_gather_seq(img_v)
            self._kvcache[key] = (full_k.detach(), full_v.detach())
            return full_k, full_v
        cached_k, cached_v = self._kvcache[key]
        n = img_k.shape[1]
        lo = self._group.rank_in_group * n
        full_k = torch.cat([cached_k[:, :lo], img_k, cached_k[:, lo + n:]], dim=1)
        full_v = torch.cat([cached_v[:, :lo], img_v, cached_v[:, lo + n:]], dim=1)
        return full_k, full_v

    def _attn_agkv_approx(self, txt_q, txt_k, txt_v, img_q, img_k, img_v):
        """All-gather mode with the cache or the FP8 transfer switched on (:637-653): local queries
        ``[image shard, text]`` against ``[all image keys, text keys]`` on the raw kernel."""
        n = img_q.shape[1]
        if self._kvcache_enabled and self._cur_step is not None:
            layer = self._layer_idx
            self._layer_idx += 1
            full_k, full_v = self._agkv_gather_cached(layer, img_k, img_v)
        else:
            full_k, full_v = self.all_gather_seq_fp8(img_k), self.all_gather_seq_fp8(img_v)
        q = torch.cat([img_q, txt_q], dim=1).contiguous()
        k = torch.cat([full_k, txt_k], dim=1).contiguous()
        v = torch.cat([full_v, txt_v], dim=1).contiguous()
        out = self.attn_backend(q, k, v, causal=False)[0]
        return out[:, n:], out[:, :n]

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
        approx = (self._kvcache_enabled and self._cur_step is not None) or self._fp8_kv
        if approx and self._layout(img_q.shape[2])[1] == "agcp":
            txt_out, img_out = self._attn_agkv_approx(txt_q, txt_k, txt_v, img_q, img_k, img_v)
        else:
            txt_out, img_out = self._wrapper(img_q.shape[2]).cp_attn_with_full_txt(txt_q, txt_k, txt_v, img_q, img_k,
                                                                                   img_v)
        if txt_out.dtype != img_q.dtype:  # merged ring results are fp32; this API hands back the compute dtype
            txt_out, img_out = txt_out.to(img_q.dtype), img_out.to(img_q.dtype)
        self._stats["calls"] += 1
        if t0 is not None:
            if img_q.is_cuda:
                torch.cuda.synchronize(img_q.device)
            self._stats["total_ms"] += (time.perf_counter() - t0) * 1e3
        return txt_out.contiguous(), img_out.contiguous()

    # ------------------------------------------------------------------ producer-callback forms
    @torch.compiler.disable
    def attention_fused(self, *, produce_img_q, produce_img_k, produce_img_v, produce_txt_q, produce_txt_k,
                        produce_txt_v, num_heads: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Projection-aware entry (:508-568): each callable returns ``[B, S, H, D]``; image producers run first."""
        img_q, img_k, img_v = produce_img_q(), produce_img_k(), produce_img_v()
        txt_q, txt_k, txt_v = produce_txt_q(), produce_txt_k(), produce_txt_v()
        return self.attention(txt_q, txt_k, txt_v, img_q, img_k, img_v)

    @torch.compiler.disable
    def cp_attn_with_full_txt_fused(self, *, produce_txt_q, produce_txt_k, produce_txt_v, produce_img_q,
                                    produce_img_k, produce_img_v, num_heads: Optional[int] = None, **_: object):
        """Name of the same entry on ``DiffusionAttention_with_CP`` (:570-592)."""
        return self.attention_fused(produce_img_q=produce_img_q, produce_img_k=produce_img_k,
                                    produce_img_v=produce_img_v, produce_txt_q=produce_txt_q,
                                    produce_txt_k=produce_txt_k, produce_txt_v=produce_txt_v, num_heads=num_heads)

    @torch.compiler.disable
    def attention_fused_packed(self, *, img_len: int, produce_q, produce_k, produce_v,
                               num_heads: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """Producers of packed ``[image shard, text]`` tensors (single-stream models, :594-635)."""
        return self._attention_from_packed(produce_q(), produce_k(), produce_v(), img_len)

    def _attention_from_packed(self, q, k, v, img_len: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """``[image_shard, text]`` packed along the sequence (:253-258)."""
        return self.attention(q[:, img_len:], k[:, img_len:], v[:, img_len:], q[:, :img_len], k[:, :img_len],
                              v[:, :img_len])
