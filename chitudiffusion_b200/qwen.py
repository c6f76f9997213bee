"""Qwen-Image joint text/image attention: processor mirror and MMDiT block on the b200 kernels.

``B200QwenAttnProcessor`` mirrors ``QwenImageChituAttnProcessor``
(chitu_diffusion/modules/attention/qwen_image_attention.py:18-284): same constructor argument, same
``__call__(attn, hidden_states, encoder_hidden_states, encoder_hidden_states_mask, attention_mask,
image_rotary_emb, qwen_cp_info) -> (img_attn_output, txt_attn_output)``, the same six producers
(image / text x q / k / v), the rotary rows of the image stream sliced by ``qwen_cp_info["image_offset"]``
with ZERO rows past the end of the table (:26-34,84-87), text replicated and image tokens sharded under
context parallelism (``cp_attn_with_full_txt`` / ``cp_attn_with_full_txt_fused``), joint ``[text, image]``
attention otherwise.  What differs: per-head RMSNorm, rotary embedding and the 16-bit cast of q and k run
as ONE kernel launch per stream (the reference chains a norm module, a complex multiply in fp32 and two
casts per tensor), and the single-GPU joint tensors are written in place instead of concatenated.

The layers themselves (projections, norm weights, output projections) stay the caller's: ``attn`` is the
model's attention module (``to_q, to_k, to_v, add_q_proj, add_k_proj, add_v_proj, norm_q, norm_k,
norm_added_q, norm_added_k, to_out, to_add_out, heads``), as in the reference.  The rotary pair is
``(img_freqs, txt_freqs)``, complex ``[S, D/2]`` (``use_real=False`` form, :87) or already converted
``[S, D/2, 2]`` (cos, sin) tables.

``QwenDoubleBlock`` is the MMDiT block around it (the reference wraps the un-vendored diffusers block,
chitu_diffusion/runtime/adapter/qwen_image.py:214-281): two modulated streams, joint attention, gated
residuals, GELU-tanh MLPs - the same kernels as the Flux double block, with Qwen's own chunk order.
"""

from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

from . import ops
from .pre_attention import table_from_complex


def slice_rotary_table(table: torch.Tensor, offset: int, length: int) -> torch.Tensor:
    """Rows ``[offset, offset + length)`` of a ``[S, D/2, 2]`` (cos, sin) table; rows past the end are zero
    (``_slice_rotary_freqs``, qwen_image_attention.py:26-34: padded tokens get zero rotary factors)."""
    avail = max(0, table.shape[0] - offset)
    part = table.narrow(0, offset, min(length, avail)) if avail > 0 else table[:0]
    if part.shape[0] == length:
        return part.contiguous()
    pad = torch.zeros((length - part.shape[0],) + tuple(table.shape[1:]), dtype=table.dtype, device=table.device)
    return torch.cat([part, pad], dim=0)


def _as_table(freqs: torch.Tensor, device) -> torch.Tensor:
    if freqs.is_complex():
        return table_from_complex(freqs, device)
    return freqs.to(device=device, dtype=torch.float32).contiguous()


class B200QwenAttnProcessor:
    """Drop-in for ``QwenImageChituAttnProcessor``."""

    def __init__(self, attn_backend):
        self.attn_backend = attn_backend
        self.base_attn_backend = getattr(attn_backend, "attn", attn_backend)
        self._tables: Dict[tuple, torch.Tensor] = {}

    def _table(self, freqs: torch.Tensor, device, offset: Optional[int], length: int) -> torch.Tensor:
        key = (freqs.data_ptr(), tuple(freqs.shape), freqs._version, str(device), offset, length)
        t = self._tables.get(key)
        if t is None:
            t = _as_table(freqs, device)
            if offset is not None:
                t = slice_rotary_table(t, offset, length)
            if len(self._tables) > 64:
                self._tables.clear()
            self._tables[key] = t
        return t

    @staticmethod
    def _weight(norm) -> Optional[torch.Tensor]:
        return None if norm is None else getattr(norm, "weight", None)

    def _stream(self, x, proj_q, proj_k, proj_v, norm_q, norm_k, heads: int, table: Optional[torch.Tensor],
                outs=None, row_offset: int = 0):
        """q, k (per-head RMSNorm + rotary, one launch) and v of one stream; ``outs`` = joint tensors to fill in place."""
        B, S, _ = x.shape
        q_proj, k_proj, v_proj = proj_q(x), proj_k(x), proj_v(x)
        C = q_proj.shape[-1]
        D = C // heads
        eps = float(getattr(norm_q, "eps", 1e-6) or 1e-6)
        nm = 1 if norm_q is not None else 2
        jobs = [dict(x=q_proj, weight=self._weight(norm_q), norm_mode=nm, rope_mode=2 if table is not None else 0),
                dict(x=k_proj, weight=self._weight(norm_k), norm_mode=1 if norm_k is not None else 2,
                     rope_mode=2 if table is not None else 0)]
        if jobs[0]["norm_mode"] != jobs[1]["norm_mode"]:
            raise NotImplementedError("q and k of a stream are normalised the same way")
        dtype = q_proj.dtype if q_proj.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16
        if outs is None:
            q, k = ops.qk_norm_rope_batch(jobs, heads, eps, table, out_dtype=dtype, round_mid=False)
            v = v_proj.view(B, S, heads, D)
            return q, k, (v if v.dtype == dtype else v.to(dtype))
        Sj = outs[0].shape[1]
        for j, t in zip(jobs, outs[:2]):
            j["out"] = t[:, row_offset:]
        if v_proj.dtype == q_proj.dtype:
            jobs.append(dict(x=v_proj, norm_mode=2, rope_mode=0, out=outs[2][:, row_offset:]))
        else:
            outs[2][:, row_offset:row_offset + S].copy_(v_proj.view(B, S, heads, D))
        ops.qk_norm_rope_batch(jobs, heads, eps, table, out_strides=(Sj * C, C, 0, D), heads_per_group=heads,
                               out_dtype=outs[0].dtype, round_mid=False)
        return None

    def __call__(self, attn, hidden_states: torch.Tensor, encoder_hidden_states: torch.Tensor = None,
                 encoder_hidden_states_mask: torch.Tensor = None, attention_mask: Optional[torch.Tensor] = None,
                 image_rotary_emb: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                 qwen_cp_info: Optional[dict] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        if encoder_hidden_states is None:
            raise ValueError("QwenImageChituAttnProcessor requires encoder_hidden_states.")
        if attention_mask is not None:
            raise NotImplementedError("Qwen-Image Chitu attention backend does not support attention_mask yet.")
        H = attn.heads
        dev = hidden_states.device
        n_img, n_txt = hidden_states.shape[1], encoder_hidden_states.shape[1]
        img_table = txt_table = None
        if image_rotary_emb is not None:
            img_freqs, txt_freqs = image_rotary_emb
            offset = int(qwen_cp_info.get("image_offset", 0)) if qwen_cp_info is not None else None
            img_table = self._table(img_freqs, dev, offset, n_img)
            txt_table = self._table(txt_freqs, dev, None, n_txt)
        img = (hidden_states, attn.to_q, attn.to_k, attn.to_v, attn.norm_q, attn.norm_k, H, img_table)
        txt = (encoder_hidden_states, attn.add_q_proj, attn.add_k_proj, attn.add_v_proj, attn.norm_added_q,
               attn.norm_added_k, H, txt_table)

        def finish(txt_o, img_o):
            dt = hidden_states.dtype
            img_o = attn.to_out[0](img_o.flatten(2, 3).to(dt).contiguous())
            if len(attn.to_out) > 1:
                img_o = attn.to_out[1](img_o)
            return img_o, attn.to_add_out(txt_o.flatten(2, 3).to(dt).contiguous())

        if qwen_cp_info is not None and hasattr(self.attn_backend, "cp_attn_with_full_txt"):
            from .comm import get_cp_group

            image_seq_len = int(qwen_cp_info.get("image_seq_len", n_img * get_cp_group().group_size))
            overlap = (hidden_states.is_cuda and hasattr(self.attn_backend, "cp_attn_with_full_txt_fused")
                       and os.environ.get("CHITU_CP_OVERLAP_QKV", "0") == "1"
                       and (not hasattr(self.attn_backend, "supports_fused_overlap")
                            or self.attn_backend.supports_fused_overlap(num_heads=H)))
            if overlap:
                made: Dict[str, tuple] = {}

                def stream(name):
                    if name not in made:
                        made[name] = self._stream(*(img if name == "img" else txt))
                    return made[name]

                t_o, i_o = self.attn_backend.cp_attn_with_full_txt_fused(
                    produce_txt_q=lambda: stream("txt")[0], produce_txt_k=lambda: stream("txt")[1],
                    produce_txt_v=lambda: stream("txt")[2], produce_img_q=lambda: stream("img")[0],
                    produce_img_k=lambda: stream("img")[1], produce_img_v=lambda: stream("img")[2],
                    image_seq_len=image_seq_len, causal=False, num_heads=H)
                return finish(t_o, i_o)
            iq, ik, iv = self._stream(*img)
            tq, tk, tv = self._stream(*txt)
            t_o, i_o = self.attn_backend.cp_attn_with_full_txt(tq, tk, tv, iq, ik, iv, image_seq_len=image_seq_len,
                                                               causal=False)
            return finish(t_o, i_o)
        if qwen_cp_info is not None:
            # a backend without the replicated-text entry: gather the image keys / values, drop the padding
            from .comm import get_cp_group

            group = get_cp_group()
            image_seq_len = int(qwen_cp_info.get("image_seq_len", n_img * group.group_size))
            iq, ik, iv = self._stream(*img)
            tq, tk, tv = self._stream(*txt)
            ik = group.all_gather_sequence(ik)[:, :image_seq_len]
            iv = group.all_gather_sequence(iv)[:, :image_seq_len]
            o = self.base_attn_backend(torch.cat([tq, iq], 1), torch.cat([tk, ik], 1), torch.cat([tv, iv], 1),
                                       causal=False)[0]
            return finish(o[:, :n_txt], o[:, n_txt:])
        # one GPU: both streams are written straight into the joint [text, image] tensors
        B = hidden_states.shape[0]
        D = attn.to_q.weight.shape[0] // H
        dtype = hidden_states.dtype if hidden_states.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16
        joint = tuple(torch.empty((B, n_txt + n_img, H, D), dtype=dtype, device=dev) for _ in range(3))
        self._stream(*txt, outs=joint, row_offset=0)
        self._stream(*img, outs=joint, row_offset=n_txt)
        o = self.attn_backend(*joint, causal=False)[0]
        return finish(o[:, :n_txt], o[:, n_txt:])


class _Linear:
    """A weight + bias pair callable like ``nn.Linear`` (the blocks below hold plain tensors)."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.weight, self.bias = weight, bias

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return F.linear(x, self.weight, self.bias)


class _Norm:
    def __init__(self, weight: torch.Tensor, eps: float = 1e-6):
        self.weight, self.eps = weight, eps


class QwenJointAttention:
    """The attribute surface of the model's attention module that the processor reads."""

    def __init__(self, p: Dict[str, torch.Tensor], heads: int, prefix: str = "attn."):
        def lin(name):
            return _Linear(p[prefix + name + ".weight"], p.get(prefix + name + ".bias"))

        self.heads = heads
        self.head_dim = p[prefix + "to_q.weight"].shape[0] // heads
        self.to_q, self.to_k, self.to_v = lin("to_q"), lin("to_k"), lin("to_v")
        self.add_q_proj, self.add_k_proj, self.add_v_proj = lin("add_q_proj"), lin("add_k_proj"), lin("add_v_proj")
        self.norm_q, self.norm_k = _Norm(p[prefix + "norm_q.weight"]), _Norm(p[prefix + "norm_k.weight"])
        self.norm_added_q = _Norm(p[prefix + "norm_added_q.weight"])
        self.norm_added_k = _Norm(p[prefix + "norm_added_k.weight"])
        self.to_out = [lin("to_out.0")]
        self.to_add_out = lin("to_add_out")


class QwenDoubleBlock:
    """One Qwen-Image MMDiT block: ``(img, txt, temb) -> (txt, img)``, 16-bit residual streams updated in place."""

    def __init__(self, dim: int, num_heads: int, device: torch.device, dtype: torch.dtype = torch.bfloat16,
                 eps: float = 1e-6):
        self.dim, self.num_heads, self.device, self.dtype, self.eps = dim, num_heads, device, dtype, eps
        self.p: Dict[str, torch.Tensor] = {}
        self.attn: Optional[QwenJointAttention] = None

    @staticmethod
    def param_shapes(dim: int, num_heads: int) -> Dict[str, tuple]:
        D = dim // num_heads
        shapes = {}
        for s, mod, ff in (("img", "img_mod.1", "img_mlp"), ("txt", "txt_mod.1", "txt_mlp")):
            shapes[mod + ".weight"], shapes[mod + ".bias"] = (6 * dim, dim), (6 * dim,)
            shapes[ff + ".net.0.proj.weight"], shapes[ff + ".net.0.proj.bias"] = (4 * dim, dim), (4 * dim,)
            shapes[ff + ".net.2.weight"], shapes[ff + ".net.2.bias"] = (dim, 4 * dim), (dim,)
        for name in ("to_q", "to_k", "to_v", "add_q_proj", "add_k_proj", "add_v_proj", "to_out.0", "to_add_out"):
            shapes[f"attn.{name}.weight"], shapes[f"attn.{name}.bias"] = (dim, dim), (dim,)
        for name in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            shapes[f"attn.{name}.weight"] = (D,)
        return shapes

    @classmethod
    def random_init(cls, dim: int, num_heads: int, device: torch.device, seed: int = 0, std: float = 0.02):
        blk = cls(dim, num_heads, device)
        gen = torch.Generator(device=device).manual_seed(seed)
        for name, shape in cls.param_shapes(dim, num_heads).items():
            if "norm" in name:
                blk.p[name] = torch.ones(shape, device=device, dtype=torch.float32)
            elif name.endswith(".bias"):
                blk.p[name] = torch.zeros(shape, device=device, dtype=blk.dtype)
            else:
                blk.p[name] = (torch.randn(shape, generator=gen, device=device) * std).to(blk.dtype)
        blk.attn = QwenJointAttention(blk.p, num_heads)
        return blk

    @classmethod
    def from_reference(cls, p: Dict[str, torch.Tensor], num_heads: int, device: torch.device,
                       dtype: torch.dtype = torch.bfloat16):
        """From a parameter dict with the model's own names (``img_mod.1.weight``, ``attn.to_q.weight``, ...)."""
        blk = cls(p["attn.to_q.weight"].shape[0], num_heads, device, dtype)
        for name, t in p.items():
            blk.p[name] = t.to(device=device, dtype=torch.float32 if "norm" in name else dtype).contiguous()
        blk.attn = QwenJointAttention(blk.p, num_heads)
        return blk

    def forward(self, img: torch.Tensor, txt: torch.Tensor, temb: torch.Tensor, rotary, processor: B200QwenAttnProcessor,
                qwen_cp_info: Optional[dict] = None):
        p, C = self.p, self.dim
        B = img.shape[0]

        def mods(name):
            e = F.linear(F.silu(temb), p[name + ".weight"], p[name + ".bias"]).float().view(B, 2, 3, C)
            return e[:, 0], e[:, 1]  # (shift, scale, gate) of the attention half and of the MLP half

        (i1, i2), (t1, t2) = mods("img_mod.1"), mods("txt_mod.1")
        hi = ops.layernorm_modulate(img, i1[:, 1], i1[:, 0], add_one=True, eps=self.eps, out_dtype=self.dtype)
        ht = ops.layernorm_modulate(txt, t1[:, 1], t1[:, 0], add_one=True, eps=self.eps, out_dtype=self.dtype)
        img_o, txt_o = processor(self.attn, hi, ht, None, None, rotary, qwen_cp_info)
        ops.gate_residual(img, img_o.contiguous(), i1[:, 2])
        ops.gate_residual(txt, txt_o.contiguous(), t1[:, 2])
        for x, m, ff in ((img, i2, "img_mlp"), (txt, t2, "txt_mlp")):
            h = ops.layernorm_modulate(x, m[:, 1], m[:, 0], add_one=True, eps=self.eps, out_dtype=self.dtype)
            u = torch._addmm_activation(p[ff + ".net.0.proj.bias"], h.view(-1, C), p[ff + ".net.0.proj.weight"].t(),
                                        use_gelu=True)
            ops.gate_residual(x, F.linear(u, p[ff + ".net.2.weight"], p[ff + ".net.2.bias"]).view(B, -1, C), m[:, 2])
        return txt, img

    __call__ = forward


class QwenDiTStack:
    """``n_blocks`` random-init MMDiT blocks sharing one attention processor."""

    def __init__(self, n_blocks: int, dim: int, num_heads: int, device: torch.device, attn_backend, seed: int = 0):
        self.blocks = [QwenDoubleBlock.random_init(dim, num_heads, device, seed=seed * 1000 + i) for i in range(n_blocks)]
        self.processor = B200QwenAttnProcessor(attn_backend)

    def forward(self, img, txt, temb, rotary, qwen_cp_info: Optional[dict] = None):
        for blk in self.blocks:
            txt, img = blk(img, txt, temb, rotary, self.processor, qwen_cp_info)
        return txt, img

    __call__ = forward
