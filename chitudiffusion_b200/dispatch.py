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

    def dispatch_flux_rotary_emb(self, rotary_emb, text_seq_len: int):
        """Rank-local rows of a precomputed joint ``(cos, sin)`` rotary pair (generator.py:204-235).

        The joint sequence is ``[text | image]``; text rows and image rows are sharded separately
        (each zero-padded to a multiple of the CP size) and re-joined, so that rank ``r`` holds the rows
        of its text shard followed by the rows of its image shard - the order its tokens have after
        :meth:`dispatch` of the two streams.  The sequence dim of each tensor is the first one whose
        extent equals the joint length recorded by the last wrapped forward (dim 0 otherwise).
        """
        if rotary_emb is None or not isinstance(rotary_emb, (tuple, list)):
            return rotary_emb
        joint = getattr(self, "_last_text_seq_len", text_seq_len) + getattr(self, "_last_image_seq_len", -1)
        parts = []
        for i, t in enumerate(rotary_emb):
            dim = next((d for d, n in enumerate(t.shape) if n == joint), 0)
            n_img = t.shape[dim] - text_seq_len
            txt = self.dispatch_sequence_dim(t.narrow(dim, 0, text_seq_len), dim, f"flux_rotary_text_{i}")
            img = self.dispatch_sequence_dim(t.narrow(dim, text_seq_len, n_img), dim, f"flux_rotary_image_{i}")
            parts.append(torch.cat([txt, img], dim=dim))
        return tuple(parts)

    def wrap_model_compute(self, model_compute):
        """Sequence-parallel form of a DiT's ``model_compute(tokens, **kwargs)`` (generator.py:237-283).

        Replicated mode (default): the latent tokens are split before the call and the output is
        gathered after it.  With ``local_latent_mode`` the caller already holds the rank-local shard
        (split once before the denoising loop, gathered once before decoding): tokens go in and come
        out untouched, and only the cheap per-call shards are taken - text states, position ids,
        ``seq_lens``.  A precomputed joint rotary pair cannot be sharded in that mode (the full image
        length is not in hand), which is refused like in the reference.
        """

        def compute(tokens: torch.Tensor, **kwargs):
            local = self.local_latent_mode
            n_img = tokens.size(1)
            if not local:
                tokens = self.dispatch(tokens, name="hidden_states")
            if "seq_lens" in kwargs:
                kwargs["seq_lens"] = torch.tensor([tokens.size(1)])
            n_txt = None
            enc = kwargs.get("encoder_hidden_states")
            if enc is not None:
                n_txt = enc.size(1)
                self._last_text_seq_len = n_txt
                self._last_image_seq_len = n_img * self.cp_size if local else n_img
                kwargs["encoder_hidden_states"] = self.dispatch(enc, name="encoder_hidden_states")
            for key in ("txt_ids", "img_ids"):
                if kwargs.get(key) is not None:
                    kwargs[key] = self.dispatch_id_sequence(kwargs[key], name=key)
            if kwargs.get("image_rotary_emb") is not None and n_txt is not None:
                if local:
                    raise NotImplementedError(
                        "Parallel-sampler local-latent mode does not support precomputed "
                        "image_rotary_emb yet; rotary must be derived from sharded img_ids.")
                kwargs["image_rotary_emb"] = self.dispatch_flux_rotary_emb(kwargs["image_rotary_emb"], n_txt)
            out = model_compute(tokens, **kwargs)
            return out if local else self.gather(out, name="hidden_states")

        return compute

    def wrap_model_compute_with_cp(self, models) -> None:
        """Replace ``model.model_compute`` of every listed model by its sequence-parallel form."""
        for model in models:
            model.model_compute = self.wrap_model_compute(model.model_compute)


class CfgDispatcher:
    """The two CFG branches run on the two ranks of the CFG group; each step ends with their exchange."""

    def __init__(self, group: Optional[CommGroup] = None, combine=None):
        self.group = group if group is not None else get_cfg_group()
        self.rank = self.group.global_rank
        self.local_rank = self.group.local_rank
        # the guidance arithmetic: the library's kernel unless a test of the group logic injects its own
        self._combine = combine if combine is not None else ops.cfg_combine

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
        return self._combine(cond, uncond, guidance_scale, rescale)
