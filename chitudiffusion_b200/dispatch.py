"""Token dispatch / gather either side of a context-parallel DiT forward, and the CFG-parallel combine.

Host-side mirror of ``SequencePadder`` (chitu_diffusion/runtime/parallel_utils.py:7-57),
``ContextParallelDispatcher`` and ``CfgDispatcher`` (chitu_diffusion/runtime/generator.py:134-209):
same method names and argument meaning.  The split is a view-level operation; the gather lands in
one ``[B, P*s, ...]`` buffer (no list + cat copy); the guidance combine after the CFG all-gather is
one kernel.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from . import ops
from .comm import CommGroup, get_cfg_group, get_cp_group


class SequencePadder:
    """Zero-pad a dim to a multiple of the split count, remember the original extent by name."""

    _padding_info: Dict[str, dict] = {}

    @staticmethod
    def split_sequence_padding(tensor: torch.Tensor, split_num: int, split_dim: int = 0,
                               name: Optional[str] = None) -> List[torch.Tensor]:
        size = tensor.size(split_dim)
        padded = (size + split_num - 1) // split_num * split_num
        if name is not None:
            SequencePadder._padding_info[name] = {"original_size": size, "padded_size": padded, "split_dim": split_dim}
        if padded != size:
            shape = list(tensor.shape)
            shape[split_dim] = padded - size
            tensor = torch.cat([tensor, torch.zeros(shape, dtype=tensor.dtype, device=tensor.device)], dim=split_dim)
        return list(torch.chunk(tensor, split_num, dim=split_dim))

    @staticmethod
    def remove_sequence_padding_and_concat(tensor_list: List[torch.Tensor], gather_dim: int = 0,
                                           name: Optional[str] = None) -> torch.Tensor:
        tensor = torch.cat(tensor_list, dim=gather_dim)
        if name is None and SequencePadder._padding_info:
            name = next(iter(SequencePadder._padding_info))
        info = SequencePadder._padding_info.get(name)
        if info is None:
            return tensor
        return tensor.narrow(gather_dim, 0, info["original_size"])


class ContextParallelDispatcher:
    """Split the token sequence over the CP group before a forward, gather the result after it."""

    def __init__(self, group: Optional[CommGroup] = None):
        self.group = group if group is not None else get_cp_group()
        self.cp_size = self.group.group_size
        self.rank = self.group.global_rank
        self.local_rank = self.group.local_rank
        self.rank_in_group = self.group.rank_in_group
        # when True the caller keeps rank-local latents across scheduler steps: no split, no gather
        self.local_latent_mode = False

    def dispatch(self, tokens: torch.Tensor, name: str = "x") -> torch.Tensor:
        return self.dispatch_sequence_dim(tokens, 1, name)

    def dispatch_sequence_dim0(self, tensor: torch.Tensor, name: str) -> torch.Tensor:
        return self.dispatch_sequence_dim(tensor, 0, name)

    def dispatch_sequence_dim(self, tensor: torch.Tensor, split_dim: int, name: str) -> torch.Tensor:
        return SequencePadder.split_sequence_padding(tensor, self.cp_size, split_dim, name)[self.rank_in_group]

    def dispatch_id_sequence(self, tensor: torch.Tensor, name: str) -> torch.Tensor:
        return self.dispatch_sequence_dim(tensor, 1 if tensor.ndim >= 3 else 0, name)

    def gather(self, tokens: torch.Tensor, name: str = "x") -> torch.Tensor:
        """All-gather along dim 1 in rank order and drop the padding recorded under ``name``."""
        if self.cp_size == 1:
            full = tokens
        else:
            full = self.group.all_gather_sequence(tokens)
        info = SequencePadder._padding_info.get(name)
        return full if info is None else full.narrow(1, 0, info["original_size"])


class CfgDispatcher:
    """The two CFG branches run on the two ranks of the CFG group; each step ends with their exchange."""

    def __init__(self, group: Optional[CommGroup] = None):
        self.group = group if group is not None else get_cfg_group()
        self.rank = self.group.global_rank
        self.local_rank = self.group.local_rank

    def all_gather_cfg_noise_preds(self, local_noise_pred: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """``(cond, uncond)``: rank 0 of the group computes the conditional branch."""
        local = local_noise_pred.contiguous()
        both = torch.empty((2,) + tuple(local.shape), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(both.view(-1), local.view(-1), group=self.group.gpu_group)
        return both[0], both[1]

    def guided_noise_pred(self, local_noise_pred: torch.Tensor, guidance_scale: float,
                          rescale: bool = False) -> torch.Tensor:
        """Exchange + ``uncond + s * (cond - uncond)`` (optionally norm-rescaled over the last dim) in one kernel."""
        cond, uncond = self.all_gather_cfg_noise_preds(local_noise_pred)
        if cond.is_cuda:
            return ops.cfg_combine(cond, uncond, guidance_scale, rescale)
        out = uncond + guidance_scale * (cond - uncond)  # host tensors: the group test path (gloo)
        if rescale:
            out = out * (torch.norm(cond, dim=-1, keepdim=True) / torch.norm(out, dim=-1, keepdim=True))
        return out
