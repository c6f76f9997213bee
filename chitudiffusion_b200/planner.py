"""Resolve the DiT parallel plan and wrap the attention backend accordingly.

Mirrors chitu_diffusion/parallel/{state,planner,dit}.py: ``DitParallelPlan(cfg_size, cp_size,
up, cp_backend)``, ``ParallelPlanner.resolve_cp_backend`` (``auto`` picks all-gather-KV when
``cp_size <= 4`` and at least 20 % of device memory is free, else Ulysses/ring) and
``wrap_attention_backend_for_dit_parallel``.  The knobs arrive as
``args.infer.diffusion.{cfg_size, cp_size, up, cp_backend, ring_cudagraph}``, which is what
``chitu run`` derives from ``parallel.cfp``, ``parallel.up`` and ``infer.cp_backend``
(chitu_diffusion/cli.py:157-161,229-245).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

SUPPORTED_CP_BACKENDS = {"auto", "agcp", "ucp"}


@dataclass
class DitParallelPlan:
    cfg_size: int = 1
    cp_size: int = 1
    up: int = 1
    cp_backend: str = "none"

    @property
    def enabled(self) -> bool:
        return self.cp_size > 1 or self.cfg_size > 1

    @property
    def uses_agcp(self) -> bool:
        return self.cp_backend == "agcp"

    @property
    def uses_ucp(self) -> bool:
        return self.cp_backend == "ucp"


@dataclass
class ParallelPlan:
    dit: DitParallelPlan = field(default_factory=DitParallelPlan)


class ParallelPlanner:
    def __init__(self, args: Any, model_adapter: Any = None):
        self.args = args
        self.model_adapter = model_adapter

    def build(self) -> ParallelPlan:
        diffusion = self.args.infer.diffusion
        cp_size = int(getattr(diffusion, "cp_size", 1))
        cfg_size = int(getattr(diffusion, "cfg_size", 1))
        up = int(getattr(diffusion, "up", 1))
        requested = str(getattr(diffusion, "cp_backend", "auto") or "auto").strip().lower()
        resolved = self.resolve_cp_backend(requested, cp_size=cp_size, up=up)
        return ParallelPlan(dit=DitParallelPlan(cfg_size=cfg_size, cp_size=cp_size, up=up,
                                                cp_backend=resolved if cp_size > 1 else "none"))

    def resolve_cp_backend(self, requested: str, *, cp_size: int, up: int) -> str:
        mode = str(requested or "auto").strip().lower()
        if mode not in SUPPORTED_CP_BACKENDS:
            raise ValueError(f"infer.diffusion.cp_backend must be one of auto, agcp, ucp; got {requested!r}.")
        if cp_size <= 1:
            return "none"
        if mode != "auto":
            return mode
        if not torch.cuda.is_available():
            return "ucp"
        try:
            free_mem, total_mem = torch.cuda.mem_get_info()
        except Exception:
            return "ucp"
        return "agcp" if cp_size <= 4 and free_mem / max(total_mem, 1) >= 0.20 else "ucp"


def build_parallel_plan(args: Any, model_adapter: Any = None) -> ParallelPlan:
    return ParallelPlanner(args, model_adapter=model_adapter).build()


def wrap_attention_backend_for_dit_parallel(attn: Any, args: Any, plan: ParallelPlan) -> Any:
    """Return ``attn`` itself for one rank, else the context-parallel wrapper around it."""
    if plan.dit.cp_size <= 1:
        return attn
    from .context_parallel import B200ContextParallel

    return B200ContextParallel(
        attn,
        plan.dit.up,
        ring_cudagraph=getattr(args.infer.diffusion, "ring_cudagraph", False),
        cp_backend=plan.dit.cp_backend,
    )
