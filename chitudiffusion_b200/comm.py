"""Communication groups for CFG / context / Ulysses parallelism.

Mirrors the comm-group surface the reference's attention code relies on
(chitu_diffusion/core/distributed/comm_group.py:64-110,305-384 and
chitu_diffusion/core/distributed/parallel_state.py:312-431): ``CommGroup`` with
``gpu_group, cpu_group, rank_list, rank_in_group, group_size, device,
all_to_all(), p2p_*()``, and the lookups ``get_cp_group() / get_up_group(size) /
get_cfg_group()``.  One process per GPU, ``torch.distributed`` underneath: NCCL
over NVLink for CUDA tensors, gloo for host objects and for CPU-rank tests of
the layout logic.

Differences from the reference that do not change results: the packed
all-to-all skips the unpack copy when it is a pure view (batch 1), receives
directly into caller-owned buffers, and layout copies of CUDA tensors go
through the library's 16-byte strided-copy kernel.
"""

from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

_GROUP_CACHE: Dict[Tuple[Tuple[int, ...], str], object] = {}


def _layout_copy(src_view: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """Materialise a permuted view into a contiguous buffer.

    CUDA tensors go through the library's 16-byte vector kernel and must satisfy its alignment rules
    (rows and strides multiples of 16 bytes) - there is no silent second path on the GPU.  Host tensors
    (the gloo ranks that test the layout logic) are copied by torch.
    """
    if src_view.is_cuda:
        from . import ops

        es = src_view.element_size()
        ok = (src_view.dim() == 5 and src_view.stride(4) == 1 and (src_view.shape[4] * es) % 16 == 0
              and all((s * es) % 16 == 0 for s in src_view.stride()[:4])
              and src_view.data_ptr() % 16 == 0 and dst.data_ptr() % 16 == 0)
        if not ok:
            raise ValueError("all-to-all layout copy needs 16-byte aligned rows and strides "
                             f"(shape {tuple(src_view.shape)}, strides {tuple(src_view.stride())}, {src_view.dtype})")
        return ops.strided_copy(src_view, dst)
    dst.copy_(src_view)
    return dst


def _new_group(ranks: Sequence[int], backend: str):
    key = (tuple(ranks), backend)
    if key not in _GROUP_CACHE:
        _GROUP_CACHE[key] = dist.new_group(list(ranks), backend=backend)
    return _GROUP_CACHE[key]


class CommGroup:
    """One communicator per listed rank subset; this process belongs to exactly one of them."""

    def __init__(self, rank_lists: Sequence[Sequence[int]], global_rank: int, local_rank: int,
                 device: Optional[torch.device] = None):
        self.global_rank = global_rank
        self.local_rank = local_rank
        default_backend = dist.get_backend()
        use_cuda = torch.cuda.is_available() and "nccl" in str(default_backend)
        self.device = device if device is not None else (
            torch.device(f"cuda:{local_rank}") if use_cuda else torch.device("cpu")
        )
        mine = [i for i, rl in enumerate(rank_lists) if global_rank in rl]
        if len(mine) == 0:
            raise ValueError("every rank must appear in exactly one sub-group (use singleton groups for idle ranks)")
        if len(mine) > 1:
            raise ValueError("One rank can not participate in multiple sub-groups.")
        self.gpu_group = None
        self.cpu_group = None
        # every rank must create every group, in the same order
        for i, rl in enumerate(rank_lists):
            if len(rl) == 1:
                continue
            g = _new_group(rl, "nccl" if use_cuda else "gloo")
            c = _new_group(rl, "gloo") if use_cuda else g
            if i == mine[0]:
                self.gpu_group, self.cpu_group = g, c
        self.rank_list = list(rank_lists[mine[0]])
        self.rank_in_group = self.rank_list.index(global_rank)
        self.group_size = len(self.rank_list)
        self.p2p_ops: List[dist.P2POp] = []
        self.p2p_reqs = None

    # ------------------------------------------------------------------ ring p2p
    def p2p_isend(self, tensor: torch.Tensor, dst: int) -> None:
        self.p2p_ops.append(dist.P2POp(dist.isend, tensor, self.rank_list[dst], self.gpu_group))

    def p2p_irecv(self, size, dtype: torch.dtype, src: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        tensor = out if out is not None else torch.empty(size, dtype=dtype, device=self.device)
        self.p2p_ops.append(dist.P2POp(dist.irecv, tensor, self.rank_list[src], self.gpu_group))
        return tensor

    def p2p_commit(self) -> None:
        assert self.p2p_reqs is None
        self.p2p_reqs = dist.batch_isend_irecv(self.p2p_ops)

    def p2p_wait(self) -> None:
        for req in self.p2p_reqs or []:
            req.wait()
        self.p2p_ops.clear()
        self.p2p_reqs = None

    # ------------------------------------------------------------------ Ulysses all-to-all
    def all_to_all(self, input_: torch.Tensor, scatter_dim: int = 2, gather_dim: int = 1) -> torch.Tensor:
        """``[B,s,H,D] -> [B,U*s,H/U,D]`` (scatter 2, gather 1) or the reverse (scatter 1, gather 2).

        Index order follows chitu_diffusion/core/distributed/comm_group.py:363-380: the gathered
        sequence is rank-major, head slices are contiguous per rank.  Other dims (the 3-d LSE
        exchange) take the list form like the reference's fallback at :335-338.
        """
        U = self.group_size
        if U == 1:
            return input_
        if input_.dim() == 4 and (scatter_dim, gather_dim) == (2, 1):
            b, s, h, d = input_.shape
            if h % U:
                raise ValueError(f"head dim {h} must be divisible by CP size {U}")
            hc = h // U
            send = torch.empty((U, b, s, 1, hc * d), dtype=input_.dtype, device=input_.device)
            x = input_ if input_.stride(3) == 1 and input_.stride(2) == d else input_.contiguous()
            _layout_copy(x.as_strided((U, b, s, 1, hc * d), (hc * x.stride(2), x.stride(0), x.stride(1), 0, 1),
                                      x.storage_offset()), send)
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=self.gpu_group)
            recv = recv.view(U, b, s, hc, d)
            if b == 1:
                return recv.view(1, U * s, hc, d)
            out = torch.empty((b, U, s, 1, hc * d), dtype=input_.dtype, device=input_.device)
            _layout_copy(recv.view(U, b, s, 1, hc * d).permute(1, 0, 2, 3, 4), out)
            return out.view(b, U * s, hc, d)
        if input_.dim() == 4 and (scatter_dim, gather_dim) == (1, 2):
            b, s, h, d = input_.shape
            if s % U:
                raise ValueError(f"sequence dim {s} must be divisible by CP size {U}")
            sc = s // U
            x = input_.contiguous()
            if b == 1:
                send = x.view(U, 1, sc, h, d)
            else:
                send = torch.empty((U, b, sc, 1, h * d), dtype=x.dtype, device=x.device)
                _layout_copy(x.view(b, U, sc, 1, h * d).permute(1, 0, 2, 3, 4), send)
            recv = torch.empty((U, b, sc, 1, h * d), dtype=x.dtype, device=x.device)
            dist.all_to_all_single(recv, send.view(U, b, sc, 1, h * d), group=self.gpu_group)
            out = torch.empty((b, sc, U, 1, h * d), dtype=x.dtype, device=x.device)
            _layout_copy(recv.permute(1, 2, 0, 3, 4), out)
            return out.view(b, sc, U * h, d)
        pieces = [t.contiguous() for t in torch.tensor_split(input_, U, scatter_dim)]
        stacked = torch.stack(pieces)
        got = torch.empty_like(stacked)
        dist.all_to_all_single(got, stacked, group=self.gpu_group)
        return torch.cat(list(got.unbind(0)), dim=gather_dim).contiguous()

    def all_gather_sequence(self, tensor: torch.Tensor) -> torch.Tensor:
        """``[B,s,H,D]`` per rank -> rank-ordered ``[B,P*s,H,D]`` (one collective, no list / cat copies)."""
        P = self.group_size
        if P == 1:
            return tensor
        x = tensor.contiguous()
        b = x.shape[0]
        buf = torch.empty((P * b,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(buf, x, group=self.gpu_group)  # concatenated on dim 0 == stacked [P, b, ...]
        buf = buf.view((P,) + tuple(x.shape))
        if b == 1:
            return buf.view(1, P * x.shape[1], *x.shape[2:])
        return buf.transpose(0, 1).reshape(b, P * x.shape[1], *x.shape[2:])

    def barrier(self) -> None:
        if self.group_size > 1:
            dist.barrier(group=self.cpu_group)


# --------------------------------------------------------------------------- #
# process-wide parallel state (CFG / CP / UP groups)
# --------------------------------------------------------------------------- #

_CFG_GROUP: Optional[CommGroup] = None
_CP_GROUP: Optional[CommGroup] = None
_UP_GROUPS: Optional[Dict[int, CommGroup]] = None


def cfg_rank_lists(world: int, cfg_size: int) -> List[List[int]]:
    if cfg_size == 1:
        return [[r] for r in range(world)]
    if cfg_size != 2:
        raise ValueError("CFG size can only be 1 or 2")
    if world % 2:
        raise ValueError("World size must be even for CFG parallelism")
    half = world // 2
    return [[i, i + half] for i in range(half)]


def cp_rank_lists(world: int, cfg_size: int) -> List[List[int]]:
    if cfg_size == 2:
        half = world // 2
        return [list(range(half)), list(range(half, world))]
    return [list(range(world))]


def up_rank_lists(world: int, cfg_size: int, up_size: int) -> List[List[int]]:
    lists = []
    for ranks in cp_rank_lists(world, cfg_size):
        for i in range(0, len(ranks), up_size):
            lists.append(ranks[i : i + up_size])
    return lists


def initialize_diffusion_parallel_groups(cfg_size: int, cp_size: int, up: int = 8) -> None:
    """Create the CFG, CP and Ulysses groups.

    Rank maps follow chitu_diffusion/core/distributed/parallel_state.py:329-431: CFG pairs
    ``[i, i + W/2]``; the CP group is all ranks, or each half when ``cfg_size == 2``; Ulysses
    groups are consecutive slices of every CP group for sizes ``min(up, cp)`` and half of it.
    """
    global _CFG_GROUP, _CP_GROUP, _UP_GROUPS
    if _CP_GROUP is not None:
        raise RuntimeError("parallel groups already initialised")
    rank = dist.get_rank()
    world = dist.get_world_size()
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    if cfg_size * cp_size != world:
        raise ValueError(f"cfg_size ({cfg_size}) * cp_size ({cp_size}) must equal the world size ({world})")
    _CFG_GROUP = CommGroup(cfg_rank_lists(world, cfg_size), rank, local_rank)
    _CP_GROUP = CommGroup(cp_rank_lists(world, cfg_size), rank, local_rank)
    _UP_GROUPS = {}
    top = min(up, cp_size)
    for size in (top, top // 2):
        if size == 0 or size in _UP_GROUPS or cp_size % size or size > up:
            continue
        _UP_GROUPS[size] = CommGroup(up_rank_lists(world, cfg_size, size), rank, local_rank)


def destroy_diffusion_parallel_groups() -> None:
    global _CFG_GROUP, _CP_GROUP, _UP_GROUPS
    _CFG_GROUP = _CP_GROUP = _UP_GROUPS = None
    for group in _GROUP_CACHE.values():
        try:
            dist.destroy_process_group(group)
        except Exception:  # the default group is already gone at interpreter shutdown
            pass
    _GROUP_CACHE.clear()


def get_cp_group() -> CommGroup:
    if _CP_GROUP is None:
        raise RuntimeError("parallel groups not initialised")
    return _CP_GROUP


def get_cfg_group() -> CommGroup:
    if _CFG_GROUP is None:
        raise RuntimeError("parallel groups not initialised")
    return _CFG_GROUP


def get_up_group(size: int) -> CommGroup:
    if _UP_GROUPS is None or size not in _UP_GROUPS:
        raise ValueError(f"UP group of size {size} not initialized.")
    return _UP_GROUPS[size]
