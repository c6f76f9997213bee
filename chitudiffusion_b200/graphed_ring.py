"""Stand-alone ring attention over one process group, optionally replayed from a CUDA graph.

Mirror of ``GraphedRingAttention`` (chitu_diffusion/modules/attention/graphed_ring_attention.py:166-323):
same constructor and call signature, one instance per attention site, graph keyed by shapes, dtype
and scale, static input copies + replay + clone.  The reference rotates K/V with NCCL send/recv
(send to the next rank, receive from the previous one, :196-198); here every rank publishes its K/V
block in peer-mapped memory and step ``t`` pulls the block of rank ``(r - t) % P`` - the block that
rotation delivers at step ``t`` - with the copy engines while the attention kernel works on the
previous block (``peer.PeerRing``).  K/V with fewer heads than Q (GQA / MQA) are broadcast to Q's
head count before the kernel call, as at :245-248.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist


class _GroupView:
    """The three attributes ``PeerRing`` needs, for a raw ``ProcessGroup``."""

    def __init__(self, pg, size: int, rank: int, ranks: List[int]):
        self.gpu_group, self.group_size, self.rank_in_group, self.rank_list = pg, size, rank, ranks


def _resolve_group(group) -> Tuple[Optional["dist.ProcessGroup"], int, int, List[int]]:
    """``(process_group, world_size, rank_in_group, global ranks)`` for a CommGroup, a raw
    ``ProcessGroup`` or ``None`` (the CP group if one exists, else WORLD, else a single rank)."""
    if hasattr(group, "gpu_group") and hasattr(group, "rank_list"):
        if group.group_size == 1 or group.gpu_group is None:
            return None, 1, 0, [0]
        return group.gpu_group, int(group.group_size), int(group.rank_in_group), list(group.rank_list)
    if group is None:
        try:
            from .comm import get_cp_group

            return _resolve_group(get_cp_group())
        except Exception:
            pass
    if not (dist.is_available() and dist.is_initialized()):
        return None, 1, 0, [0]
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    peers = [dist.get_global_rank(group, i) for i in range(world)] if group is not None else list(range(world))
    return group, world, rank, peers


class B200GraphedRingAttention:
    """``attn(q, k, v, softmax_scale=None, causal=False) -> out`` for this rank's query shard."""

    def __init__(self, group=None, *, kernel: str = "auto", use_cuda_graph: bool = True, warmup_iters: int = 3,
                 backend=None) -> None:
        if kernel not in ("auto", "b200"):
            raise ValueError(f"Unknown kernel '{kernel}'. Choose from ['b200'] or 'auto'.")
        self.pg, self.world_size, self.rank_in_group, self._peers = _resolve_group(group)
        self.kernel_name = "b200"
        self.use_cuda_graph = use_cuda_graph
        self.warmup_iters = max(1, int(warmup_iters))
        if backend is None:
            from .attention import B200AttnBackend

            backend = B200AttnBackend("b200")
        self.backend = backend
        self._rings: Dict[tuple, object] = {}
        self._graph_cache: Dict[tuple, dict] = {}

    def reset_graph_cache(self) -> None:
        """Drop all captured graphs and their static buffers."""
        self._graph_cache.clear()

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, softmax_scale: Optional[float] = None,
                 causal: bool = False) -> torch.Tensor:
        if causal:
            raise NotImplementedError(
                "Causal ring attention requires a zig-zag load-balanced partition and per-step masking, "
                "which this module does not implement."
            )
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** -0.5
        if k.shape[-2] != q.shape[-2]:  # GQA / MQA: broadcast K/V heads to the query heads
            rep = q.shape[-2] // k.shape[-2]
            k, v = k.repeat_interleave(rep, dim=-2), v.repeat_interleave(rep, dim=-2)
        if self.world_size == 1:
            return self.backend(q, k, v, softmax_scale=float(softmax_scale))[0].to(q.dtype)
        if not q.is_cuda:
            raise RuntimeError("B200GraphedRingAttention has no CPU path")
        if self.world_size > 8:
            raise NotImplementedError("the peer-memory ring supports at most 8 GPUs of one node")
        if self.use_cuda_graph:
            return self._ring_graphed(q, k, v, float(softmax_scale))
        return self._ring_eager(q, k, v, float(softmax_scale))

    # ------------------------------------------------------------------ internals
    def _ring(self, q: torch.Tensor):
        from .context_parallel import _KernelMerger
        from .peer import PeerRing

        B, s, H, D = q.shape
        key = (B, s, H, D, q.dtype, str(q.device))
        ring = self._rings.get(key)
        if ring is None:
            view = _GroupView(self.pg, self.world_size, self.rank_in_group, self._peers)
            ring = PeerRing(view, 1, B, s, H, D, q.dtype, q.device, mode="ring", merger_factory=_KernelMerger,
                            direction=-1)
            self._rings[key] = ring
        return ring

    def _ring_eager(self, q, k, v, scale: float) -> torch.Tensor:
        ring = self._ring(q)
        ring.scatter_plain(k, "k")
        ring.scatter_plain(v, "v")
        return ring.attention(scale, q=q).to(q.dtype)

    def _ring_graphed(self, q, k, v, scale: float) -> torch.Tensor:
        key = (tuple(q.shape), tuple(k.shape), tuple(v.shape), q.dtype, scale)
        entry = self._graph_cache.get(key)
        if entry is None:
            sq, sk, sv = q.clone(), k.clone(), v.clone()
            cur = torch.cuda.current_stream(q.device)
            side = torch.cuda.Stream(device=q.device)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                for _ in range(self.warmup_iters):
                    self._ring_eager(sq, sk, sv, scale)
            cur.wait_stream(side)
            torch.cuda.synchronize(q.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_out = self._ring_eager(sq, sk, sv, scale)
            torch.cuda.synchronize(q.device)
            entry = dict(graph=graph, q=sq, k=sk, v=sv, out=static_out)
            self._graph_cache[key] = entry
        entry["q"].copy_(q)
        entry["k"].copy_(k)
        entry["v"].copy_(v)
        entry["graph"].replay()
        return entry["out"].clone()
