"""Flux double- and single-stream blocks around the joint attention: library GEMMs + this package's kernels.

Host-side mirror of ``FluxTransformerBlock`` and ``FluxSingleTransformerBlock``
(chitu_diffusion/models/model_flux1.py:48-236) with the attention processor
``ChituFluxAttnProcessor2_0`` (chitu_diffusion/modules/attention/flux_attention.py:96-171) for
inference, 16-bit residual streams as in the reference:

    double block, per stream (image / text):
        shift, scale, gate (attention and MLP) = Linear(SiLU(temb))       tiny GEMM
        h = LayerNorm(x) * (1 + scale) + shift                             layernorm_modulate kernel
        q, k, v = h W_qkv                                                  one GEMM (the reference's three)
        per-head RMSNorm + rotary, written at the stream's rows of the joint [text, image] q / k / v
                                                                           qk_norm_rope kernel, one launch per stream
        o = attention(q, k, v)                                             attention kernel (or its CP wrapper)
        x += gate * (o_stream W_out) ;  x += gate_mlp * MLP(LayerNorm(x) * (1 + scale_mlp) + shift_mlp)
    single block on the joint stream:
        h = LayerNorm(x) * (1 + scale) + shift ;  q, k, v = h W_qkv ;  m = GELU_tanh(h W_mlp)  (epilogue)
        x += gate * (o W_out[:, :C] + m W_out[:, C:])                      two accumulating GEMMs, no concat

GEMMs are plain library calls; there is no CPU path.
"""

from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.nn.functional as F

from . import ops


def _mod(temb: torch.Tensor, w: torch.Tensor, b: torch.Tensor, n: int):
    """``Linear(SiLU(temb))`` as fp32 ``[B, n, C]`` (shift / scale / gate vectors for the kernels)."""
    e = F.linear(F.silu(temb), w, b).float()
    return e.view(e.shape[0], n, -1)


def _pre_attention(qkv: torch.Tensor, H: int, wq: torch.Tensor, wk: torch.Tensor, table: torch.Tensor, pos_offset: int,
                   joint: Tuple[torch.Tensor, torch.Tensor, torch.Tensor], eps: float) -> None:
    """Norm + rotary of one stream's q and k and the copy of its v into rows ``[pos_offset, pos_offset + S)`` of the
    joint ``[B, S_joint, H, D]`` tensors: one launch."""
    B, S, C3 = qkv.shape
    C = C3 // 3
    D = C // H
    Sj = joint[0].shape[1]
    jobs = [
        dict(x=qkv[..., :C], weight=wq, norm_mode=1, rope_mode=2, out=joint[0][:, pos_offset:]),
        dict(x=qkv[..., C:2 * C], weight=wk, norm_mode=1, rope_mode=2, out=joint[1][:, pos_offset:]),
        dict(x=qkv[..., 2 * C:], norm_mode=2, rope_mode=0, out=joint[2][:, pos_offset:]),
    ]
    ops.qk_norm_rope_batch(jobs, H, eps, table, pos_offset=pos_offset, out_strides=(Sj * C, C, 0, D),
                           heads_per_group=H, out_dtype=qkv.dtype, round_mid=False)


class FluxDoubleBlock:
    def __init__(self, dim: int, num_heads: int, device: torch.device, dtype: torch.dtype = torch.bfloat16,
                 eps: float = 1e-6):
        self.dim, self.num_heads, self.device, self.dtype, self.eps = dim, num_heads, device, dtype, eps
        self.w: Dict[str, torch.Tensor] = {}

    @classmethod
    def random_init(cls, dim: int, num_heads: int, device: torch.device, seed: int = 0, std: float = 0.02):
        blk = cls(dim, num_heads, device)
        gen = torch.Generator(device=device).manual_seed(seed)
        rnd = lambda *s: (torch.randn(*s, generator=gen, device=device) * std).to(blk.dtype)  # noqa: E731
        zeros = lambda n: torch.zeros(n, device=device, dtype=blk.dtype)  # noqa: E731
        ones = lambda n: torch.ones(n, device=device, dtype=torch.float32)  # noqa: E731
        D = dim // num_heads
        for s in ("img", "txt"):
            blk.w.update({
                f"{s}.mod.weight": rnd(6 * dim, dim), f"{s}.mod.bias": zeros(6 * dim),
                f"{s}.qkv.weight": rnd(3 * dim, dim), f"{s}.qkv.bias": zeros(3 * dim),
                f"{s}.norm_q": ones(D), f"{s}.norm_k": ones(D),
                f"{s}.out.weight": rnd(dim, dim), f"{s}.out.bias": zeros(dim),
                f"{s}.ff1.weight": rnd(4 * dim, dim), f"{s}.ff1.bias": zeros(4 * dim),
                f"{s}.ff2.weight": rnd(dim, 4 * dim), f"{s}.ff2.bias": zeros(dim),
            })
        return blk

    @classmethod
    def from_reference_params(cls, p: Dict[str, torch.Tensor], num_heads: int, device: torch.device):
        """From ``FluxTransformerBlock.named_parameters()`` names (q/k/v Linears of a stream are concatenated)."""
        dim = p["attn.to_q.weight"].shape[0]
        blk = cls(dim, num_heads, device)
        lp = lambda t: t.detach().to(device=device, dtype=blk.dtype).contiguous()  # noqa: E731
        fp = lambda t: t.detach().to(device=device, dtype=torch.float32).contiguous()  # noqa: E731
        cat = lambda names, suf: lp(torch.cat([p[f"{n}.{suf}"] for n in names], 0))  # noqa: E731
        names = {"img": dict(mod="norm1.linear", qkv=["attn.to_q", "attn.to_k", "attn.to_v"], nq="attn.norm_q.weight",
                             nk="attn.norm_k.weight", out="attn.to_out.0", ff1="ff.net.0.proj", ff2="ff.net.2"),
                 "txt": dict(mod="norm1_context.linear", qkv=["attn.add_q_proj", "attn.add_k_proj", "attn.add_v_proj"],
                             nq="attn.norm_added_q.weight", nk="attn.norm_added_k.weight", out="attn.to_add_out",
                             ff1="ff_context.net.0.proj", ff2="ff_context.net.2")}
        for s, n in names.items():
            blk.w.update({
                f"{s}.mod.weight": lp(p[n["mod"] + ".weight"]), f"{s}.mod.bias": lp(p[n["mod"] + ".bias"]),
                f"{s}.qkv.weight": cat(n["qkv"], "weight"), f"{s}.qkv.bias": cat(n["qkv"], "bias"),
                f"{s}.norm_q": fp(p[n["nq"]]), f"{s}.norm_k": fp(p[n["nk"]]),
                f"{s}.out.weight": lp(p[n["out"] + ".weight"]), f"{s}.out.bias": lp(p[n["out"] + ".bias"]),
                f"{s}.ff1.weight": lp(p[n["ff1"] + ".weight"]), f"{s}.ff1.bias": lp(p[n["ff1"] + ".bias"]),
                f"{s}.ff2.weight": lp(p[n["ff2"] + ".weight"]), f"{s}.ff2.bias": lp(p[n["ff2"] + ".bias"]),
            })
        return blk

    def forward(self, img: torch.Tensor, txt: torch.Tensor, temb: torch.Tensor, table: torch.Tensor, attn):
        """``img [B, S_img, C]`` and ``txt [B, S_txt, C]`` (16-bit, updated in place), ``temb [B, C]``, ``table`` the
        per-token rotary table of the joint ``[text, image]`` sequence; returns ``(txt, img)``."""
        w, C, H = self.w, self.dim, self.num_heads
        B, n_img, _ = img.shape
        n_txt = txt.shape[1]
        D = C // H
        streams = (("txt", txt, 0), ("img", img, n_txt))
        fused = hasattr(attn, "attention_from_projections")  # context-parallel wrapper: stores go straight into the exchange
        joint = None if fused else tuple(
            torch.empty((B, n_txt + n_img, H, D), dtype=self.dtype, device=img.device) for _ in range(3))
        mods = {}
        o = None
        for s, x, off in streams:
            mods[s] = _mod(temb, w[f"{s}.mod.weight"], w[f"{s}.mod.bias"], 6)
            h = ops.layernorm_modulate(x, mods[s][:, 1], mods[s][:, 0], add_one=True, eps=self.eps, out_dtype=self.dtype)
            qkv = F.linear(h, w[f"{s}.qkv.weight"], w[f"{s}.qkv.bias"])
            if fused:
                jobs = [dict(x=qkv[..., :C], weight=w[f"{s}.norm_q"], norm_mode=1, rope_mode=2),
                        dict(x=qkv[..., C:2 * C], weight=w[f"{s}.norm_k"], norm_mode=1, rope_mode=2)]
                o = attn.attention_from_projections(jobs, qkv[..., 2 * C:], row_offset=off, last=(s == "img"),
                                                    num_heads=H, eps=self.eps, rope_table=table, pos_offset=off,
                                                    out_dtype=self.dtype, round_mid=False)
            else:
                _pre_attention(qkv, H, w[f"{s}.norm_q"], w[f"{s}.norm_k"], table, off, joint, self.eps)
        if not fused:
            o = attn(*joint)[0]
        o = o.reshape(B, n_txt + n_img, C)
        for s, x, off in streams:
            m = mods[s]
            o_s = o[:, off:off + x.shape[1]]
            ops.gate_residual(x, F.linear(o_s, w[f"{s}.out.weight"], w[f"{s}.out.bias"]).contiguous(), m[:, 2])
            h = ops.layernorm_modulate(x, m[:, 4], m[:, 3], add_one=True, eps=self.eps, out_dtype=self.dtype)
            u = torch._addmm_activation(w[f"{s}.ff1.bias"], h.view(-1, C), w[f"{s}.ff1.weight"].t(), use_gelu=True)
            ops.gate_residual(x, F.linear(u, w[f"{s}.ff2.weight"], w[f"{s}.ff2.bias"]).view(B, -1, C), m[:, 5])
        return txt, img

    __call__ = forward


class FluxSingleBlock:
    def __init__(self, dim: int, num_heads: int, device: torch.device, dtype: torch.dtype = torch.bfloat16,
                 eps: float = 1e-6):
        self.dim, self.num_heads, self.device, self.dtype, self.eps = dim, num_heads, device, dtype, eps
        self.w: Dict[str, torch.Tensor] = {}

    @classmethod
    def random_init(cls, dim: int, num_heads: int, device: torch.device, seed: int = 0, std: float = 0.02):
        blk = cls(dim, num_heads, device)
        gen = torch.Generator(device=device).manual_seed(seed)
        rnd = lambda *s: (torch.randn(*s, generator=gen, device=device) * std).to(blk.dtype)  # noqa: E731
        zeros = lambda n: torch.zeros(n, device=device, dtype=blk.dtype)  # noqa: E731
        D = dim // num_heads
        blk.w = {
            "mod.weight": rnd(3 * dim, dim), "mod.bias": zeros(3 * dim),
            "qkv.weight": rnd(3 * dim, dim), "qkv.bias": zeros(3 * dim),
            "mlp.weight": rnd(4 * dim, dim), "mlp.bias": zeros(4 * dim),
            "norm_q": torch.ones(D, device=device), "norm_k": torch.ones(D, device=device),
            "out_attn.weight": rnd(dim, dim), "out_mlp.weight": rnd(dim, 4 * dim), "out.bias": zeros(dim),
        }
        return blk

    @classmethod
    def from_reference_params(cls, p: Dict[str, torch.Tensor], num_heads: int, device: torch.device):
        """From ``FluxSingleTransformerBlock.named_parameters()`` names; ``proj_out`` is split by input columns."""
        dim = p["attn.to_q.weight"].shape[0]
        blk = cls(dim, num_heads, device)
        lp = lambda t: t.detach().to(device=device, dtype=blk.dtype).contiguous()  # noqa: E731
        fp = lambda t: t.detach().to(device=device, dtype=torch.float32).contiguous()  # noqa: E731
        blk.w = {
            "mod.weight": lp(p["norm.linear.weight"]), "mod.bias": lp(p["norm.linear.bias"]),
            "qkv.weight": lp(torch.cat([p["attn.to_q.weight"], p["attn.to_k.weight"], p["attn.to_v.weight"]], 0)),
            "qkv.bias": lp(torch.cat([p["attn.to_q.bias"], p["attn.to_k.bias"], p["attn.to_v.bias"]], 0)),
            "mlp.weight": lp(p["proj_mlp.weight"]), "mlp.bias": lp(p["proj_mlp.bias"]),
            "norm_q": fp(p["attn.norm_q.weight"]), "norm_k": fp(p["attn.norm_k.weight"]),
            "out_attn.weight": lp(p["proj_out.weight"][:, :dim]), "out_mlp.weight": lp(p["proj_out.weight"][:, dim:]),
            "out.bias": lp(p["proj_out.bias"]),
        }
        return blk

    def forward(self, x: torch.Tensor, temb: torch.Tensor, table: torch.Tensor, attn) -> torch.Tensor:
        """``x [B, S, C]`` joint ``[text, image]`` stream (16-bit, updated in place and returned)."""
        w, C, H = self.w, self.dim, self.num_heads
        B, S, _ = x.shape
        D = C // H
        m = _mod(temb, w["mod.weight"], w["mod.bias"], 3)
        h = ops.layernorm_modulate(x, m[:, 1], m[:, 0], add_one=True, eps=self.eps, out_dtype=self.dtype)
        qkv = F.linear(h, w["qkv.weight"], w["qkv.bias"])
        mlp = torch._addmm_activation(w["mlp.bias"], h.view(-1, C), w["mlp.weight"].t(), use_gelu=True)
        jobs = [dict(x=qkv[..., :C], weight=w["norm_q"], norm_mode=1, rope_mode=2),
                dict(x=qkv[..., C:2 * C], weight=w["norm_k"], norm_mode=1, rope_mode=2)]
        if hasattr(attn, "attention_from_projections"):
            o = attn.attention_from_projections(jobs, qkv[..., 2 * C:], num_heads=H, eps=self.eps, rope_table=table,
                                                out_dtype=self.dtype, round_mid=False)
        else:
            q, k = ops.qk_norm_rope_batch(jobs, H, self.eps, table, out_dtype=self.dtype, round_mid=False)
            o = attn(q, k, qkv[..., 2 * C:].view(B, S, H, D))[0]
        y = torch.addmm(w["out.bias"], o.reshape(B * S, C), w["out_attn.weight"].t())
        y = torch.addmm(y, mlp, w["out_mlp.weight"].t())
        ops.gate_residual(x, y.view(B, S, C), m[:, 2])
        return x

    __call__ = forward


class FluxDiTStack:
    """``n_double`` double-stream blocks on (text, image), then ``n_single`` single-stream blocks on their concatenation."""

    def __init__(self, n_double: int, n_single: int, dim: int, num_heads: int, device: torch.device, seed: int = 0):
        self.double = [FluxDoubleBlock.random_init(dim, num_heads, device, seed=seed * 1000 + i) for i in range(n_double)]
        self.single = [FluxSingleBlock.random_init(dim, num_heads, device, seed=seed * 1000 + 500 + i)
                       for i in range(n_single)]

    def forward(self, img: torch.Tensor, txt: torch.Tensor, temb: torch.Tensor, table: torch.Tensor, attn):
        for blk in self.double:
            txt, img = blk(img, txt, temb, table, attn)
        x = torch.cat([txt, img], dim=1)
        for blk in self.single:
            x = blk(x, temb, table, attn)
        return x[:, txt.shape[1]:]

    __call__ = forward
