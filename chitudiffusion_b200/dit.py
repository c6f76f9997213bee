"""Wan DiT block around the attention path: library GEMMs + this package's kernels for everything else.

Host-side mirror of ``WanAttentionBlock`` (chitu_diffusion/models/model_wan.py:286-366) for inference:

    e_0..e_5 = modulation + e                                     (fp32, tiny)
    h = LayerNorm(x) * (1 + e_1) + e_0          -> bf16           layernorm_modulate kernel
    q, k, v = h W_qkv                                              one GEMM (the reference's three Linears)
    q, k = RMSNorm + 3-axis rotary                                 qk_norm_rope kernel (one launch)
    y = attention(q, k, v) W_o ;  x += y * e_2                     attention kernel (+ CP exchange), GEMM,
                                                                   gate_residual kernel
    h = LayerNorm_affine(x) ;  q = RMSNorm(h W_q) ; k, v = ctx W_kv ; x += attention(q, k, v) W_o
    h = LayerNorm(x) * (1 + e_4) + e_3 ;  x += (GELU_tanh(h W_1) W_2) * e_5

The residual stream ``x`` is fp32 (in the reference it becomes fp32 at the first gated residual,
:347-348) and is updated in place; GEMM operands are bf16 with fp32 accumulation (the reference runs
its Linears under bf16 autocast).  GEMMs are plain library calls (``F.linear`` /
``torch._addmm_activation`` for the GELU epilogue); there is no CPU path.
"""

from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch
import torch.nn.functional as F

from . import ops
from .pre_attention import WanPreAttention


class WanBlock:
    """Weights and forward pass of one Wan T2V block (``cross_attn_norm=True``, ``qk_norm=True``)."""

    def __init__(self, dim: int, ffn_dim: int, num_heads: int, device: torch.device, eps: float = 1e-6,
                 dtype: torch.dtype = torch.bfloat16):
        self.dim, self.ffn_dim, self.num_heads, self.head_dim = dim, ffn_dim, num_heads, dim // num_heads
        self.eps, self.device, self.dtype = eps, device, dtype
        self.w: Dict[str, torch.Tensor] = {}

    # ------------------------------------------------------------------ weights
    @classmethod
    def random_init(cls, dim: int, ffn_dim: int, num_heads: int, device: torch.device, seed: int = 0,
                    std: float = 0.02, eps: float = 1e-6) -> "WanBlock":
        """N(0, std^2) matrices, zero biases, unit norm weights, N(0,1)/sqrt(dim) modulation (:317-318)."""
        blk = cls(dim, ffn_dim, num_heads, device, eps)
        gen = torch.Generator(device=device).manual_seed(seed)
        rnd = lambda *shape: (torch.randn(*shape, generator=gen, device=device) * std).to(blk.dtype)  # noqa: E731
        zeros = lambda n: torch.zeros(n, device=device, dtype=blk.dtype)  # noqa: E731
        ones = lambda n: torch.ones(n, device=device, dtype=torch.float32)  # noqa: E731
        blk.w = {
            "qkv.weight": rnd(3 * dim, dim), "qkv.bias": zeros(3 * dim), "o.weight": rnd(dim, dim), "o.bias": zeros(dim),
            "norm_q": ones(dim), "norm_k": ones(dim),
            "norm3.weight": ones(dim), "norm3.bias": torch.zeros(dim, device=device, dtype=torch.float32),
            "cq.weight": rnd(dim, dim), "cq.bias": zeros(dim), "ckv.weight": rnd(2 * dim, dim), "ckv.bias": zeros(2 * dim),
            "co.weight": rnd(dim, dim), "co.bias": zeros(dim), "cnorm_q": ones(dim), "cnorm_k": ones(dim),
            "ffn1.weight": rnd(ffn_dim, dim), "ffn1.bias": zeros(ffn_dim),
            "ffn2.weight": rnd(dim, ffn_dim), "ffn2.bias": zeros(dim),
            "modulation": torch.randn(1, 6, dim, generator=gen, device=device) / dim ** 0.5,
        }
        return blk

    @classmethod
    def from_reference_params(cls, params: Dict[str, torch.Tensor], num_heads: int, device: torch.device,
                              eps: float = 1e-6) -> "WanBlock":
        """Build from a ``WanAttentionBlock.named_parameters()`` mapping (q/k/v Linears are concatenated)."""
        p = {k: v.detach() for k, v in params.items()}
        dim, ffn_dim = p["self_attn.q.weight"].shape[0], p["ffn.0.weight"].shape[0]
        blk = cls(dim, ffn_dim, num_heads, device, eps)
        lp = lambda t: t.to(device=device, dtype=blk.dtype).contiguous()  # noqa: E731
        fp = lambda t: t.to(device=device, dtype=torch.float32).contiguous()  # noqa: E731
        cat = lambda names, suffix: lp(torch.cat([p[f"{n}.{suffix}"] for n in names], dim=0))  # noqa: E731
        blk.w = {
            "qkv.weight": cat(["self_attn.q", "self_attn.k", "self_attn.v"], "weight"),
            "qkv.bias": cat(["self_attn.q", "self_attn.k", "self_attn.v"], "bias"),
            "o.weight": lp(p["self_attn.o.weight"]), "o.bias": lp(p["self_attn.o.bias"]),
            "norm_q": fp(p["self_attn.norm_q.weight"]), "norm_k": fp(p["self_attn.norm_k.weight"]),
            "norm3.weight": fp(p["norm3.weight"]), "norm3.bias": fp(p["norm3.bias"]),
            "cq.weight": lp(p["cross_attn.q.weight"]), "cq.bias": lp(p["cross_attn.q.bias"]),
            "ckv.weight": cat(["cross_attn.k", "cross_attn.v"], "weight"),
            "ckv.bias": cat(["cross_attn.k", "cross_attn.v"], "bias"),
            "co.weight": lp(p["cross_attn.o.weight"]), "co.bias": lp(p["cross_attn.o.bias"]),
            "cnorm_q": fp(p["cross_attn.norm_q.weight"]), "cnorm_k": fp(p["cross_attn.norm_k.weight"]),
            "ffn1.weight": lp(p["ffn.0.weight"]), "ffn1.bias": lp(p["ffn.0.bias"]),
            "ffn2.weight": lp(p["ffn.2.weight"]), "ffn2.bias": lp(p["ffn.2.bias"]),
            "modulation": fp(p["modulation"]),
        }
        return blk

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, e: torch.Tensor, grid: Sequence[int], context: torch.Tensor, attn,
                pre: Optional[WanPreAttention] = None, local_attn=None) -> torch.Tensor:
        """``x [B, L, C]`` fp32 (updated in place and returned), ``e [B, 6, C]`` fp32, ``context [B, T, C]`` 16-bit.

        ``attn`` is the attention callable of the self-attention (the backend, or the context-parallel
        wrapper when ``x`` holds this rank's sequence shard); ``local_attn`` the backend used for the
        cross-attention over the replicated text tokens (default: ``attn.attn`` of a wrapper, else ``attn``).
        """
        w, C, H, D = self.w, self.dim, self.num_heads, self.head_dim
        B, L, _ = x.shape
        if x.dtype != torch.float32 or e.dtype != torch.float32:
            raise ValueError("the residual stream and the modulation input are fp32")
        if pre is None:
            pre = WanPreAttention(H, D, eps=self.eps, device=x.device)
        if local_attn is None:
            local_attn = getattr(attn, "attn", attn)
        mod = w["modulation"] + e  # [B, 6, C] fp32

        # self-attention
        h = ops.layernorm_modulate(x, mod[:, 1], mod[:, 0], add_one=True, eps=self.eps, out_dtype=self.dtype)
        qkv = F.linear(h, w["qkv.weight"], w["qkv.bias"])
        if hasattr(attn, "attention_from_projections"):
            # context-parallel wrapper: norm + rotary + cast are written straight into the exchange
            o = attn.attention_from_projections(pre.jobs(qkv[..., :C], qkv[..., C:2 * C], w["norm_q"], w["norm_k"]),
                                                qkv[..., 2 * C:], **pre.batch_args(L, grid))
        else:
            q, k, v = pre(qkv[..., :C], qkv[..., C:2 * C], qkv[..., 2 * C:], w["norm_q"], w["norm_k"], grid)
            o = attn(q, k, v)[0]
        if o.dtype != self.dtype:  # ring layouts hand back fp32 (the caller casts, model_wan.py:203)
            o = o.to(self.dtype)
        ops.gate_residual(x, F.linear(o.reshape(B, L, C), w["o.weight"], w["o.bias"]), mod[:, 2])

        # cross-attention over the text tokens (no rotary, keys/values from the context)
        h = ops.layernorm_modulate(x, w["norm3.weight"], w["norm3.bias"], eps=self.eps, out_dtype=self.dtype)
        q = ops.qk_norm_rope(F.linear(h, w["cq.weight"], w["cq.bias"]), H, w["cnorm_q"], self.eps, norm_mode=0,
                             rope_mode=0, rope_table=None)
        kv = F.linear(context.to(self.dtype), w["ckv.weight"], w["ckv.bias"])
        k = ops.qk_norm_rope(kv[..., :C], H, w["cnorm_k"], self.eps, norm_mode=0, rope_mode=0, rope_table=None)
        v = kv[..., C:].reshape(B, -1, H, D)
        o = local_attn(q, k, v)[0]
        ops.gate_residual(x, F.linear(o.reshape(B, L, C), w["co.weight"], w["co.bias"]), None)

        # feed-forward: the first GEMM applies bias and tanh-GELU in its epilogue
        h = ops.layernorm_modulate(x, mod[:, 4], mod[:, 3], add_one=True, eps=self.eps, out_dtype=self.dtype)
        u = torch._addmm_activation(w["ffn1.bias"], h.view(B * L, C), w["ffn1.weight"].t(), use_gelu=True)
        y = F.linear(u, w["ffn2.weight"], w["ffn2.bias"]).view(B, L, C)
        ops.gate_residual(x, y, mod[:, 5])
        return x

    __call__ = forward


class WanDiTStack:
    """``n_layers`` random-init blocks sharing one pre-attention object and one attention callable."""

    def __init__(self, n_layers: int, dim: int, ffn_dim: int, num_heads: int, device: torch.device, seed: int = 0,
                 cp_size: int = 1, cp_rank: int = 0):
        self.blocks = [WanBlock.random_init(dim, ffn_dim, num_heads, device, seed=seed * 1000 + i)
                       for i in range(n_layers)]
        self.pre = WanPreAttention(num_heads, dim // num_heads, cp_size=cp_size, cp_rank=cp_rank, device=device)

    def forward(self, x: torch.Tensor, e: torch.Tensor, grid: Sequence[int], context: torch.Tensor, attn,
                local_attn=None) -> torch.Tensor:
        for blk in self.blocks:
            x = blk.forward(x, e, grid, context, attn, self.pre, local_attn)
        return x

    __call__ = forward
