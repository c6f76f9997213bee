"""Pre-attention transforms: QK-RMSNorm + rotary embedding + 16-bit cast in one kernel pass.

Host-side mirror of the pre-attention block of the reference's models:

* Wan: ``WanRMSNorm`` over the full channel dim, ``rope_apply`` / ``rope_apply_with_cp`` on
  interleaved pairs with a three-axis (frame, row, column) position, then ``half()``
  (chitu_diffusion/models/model_wan.py:49-65,83-110,80-81,141-208;
  chitu_diffusion/modules/utils/wan/__init__.py:31-67);
* Flux / Qwen: per-head RMSNorm and axis rotary embedding with per-token position ids
  (chitu_diffusion/modules/attention/flux_attention.py:96-171).

The rotary tables are built once on the host in float64 and kept as fp32 (cos, sin) pairs; the
kernel reads them through L2.
"""

from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

import torch

from . import ops


def wan_axis_split(head_dim: int) -> Tuple[int, int]:
    """(pairs for the frame axis, pairs for the row axis); the column axis takes the rest."""
    pairs = head_dim // 2
    n_h = pairs // 3
    return pairs - 2 * n_h, n_h


def wan_rope_table(head_dim: int, max_len: int = 1024, theta: float = 10000.0,
                   device: Optional[torch.device] = None) -> torch.Tensor:
    """``[max_len, head_dim/2, 2]`` fp32 (cos, sin): Wan's concatenated frame/row/column table.

    The three axes use real dims ``d - 4*(d//6)``, ``2*(d//6)``, ``2*(d//6)``; entry ``[p, j]`` is the
    angle ``p * theta^(-2 j_axis / dim_axis)`` of pair ``j`` at position ``p`` along ITS axis.
    """
    d = head_dim
    cols = []
    for dim in (d - 4 * (d // 6), 2 * (d // 6), 2 * (d // 6)):
        expo = torch.arange(0, dim, 2, dtype=torch.float64) / dim
        inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64), expo)
        cols.append(torch.outer(torch.arange(max_len, dtype=torch.float64), inv))
    ang = torch.cat(cols, dim=1)
    table = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32).contiguous()
    return table.to(device) if device is not None else table


def table_from_complex(freqs: torch.Tensor, device: Optional[torch.device] = None) -> torch.Tensor:
    """Convert the reference's complex ``freqs [max_len, D/2]`` (``WanModel.freqs``) to the kernel's table."""
    t = torch.stack([freqs.real, freqs.imag], dim=-1).to(torch.float32).contiguous()
    return t.to(device) if device is not None else t


def axis_rope_table(ids: torch.Tensor, axes_dims: Sequence[int], theta: float = 10000.0,
                    device: Optional[torch.device] = None) -> torch.Tensor:
    """Per-token ``[S, sum(axes_dims)/2, 2]`` fp32 (cos, sin) from integer position ids ``[S, n_axes]``."""
    cols = []
    ids = ids.detach().cpu()
    for a, dim in enumerate(axes_dims):
        expo = torch.arange(0, dim, 2, dtype=torch.float64) / dim
        inv = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64), expo)
        cols.append(torch.outer(ids[:, a].to(torch.float64), inv))
    ang = torch.cat(cols, dim=1)
    table = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32).contiguous()
    return table.to(device) if device is not None else table


_TABLE_CACHE: Dict[tuple, torch.Tensor] = {}


def rope_apply(x: torch.Tensor, grid_sizes, freqs: torch.Tensor, cp_size: int = 1, cp_rank: int = 0) -> torch.Tensor:
    """Drop-in for the ``rope_impl`` hook of ``WanSelfAttention`` (model_wan.py:139,194-195).

    ``x`` is ``[B, s, H, D]``; returns bf16 (the caller's ``half()`` is then a no-op).  All samples
    must share one grid.  With ``cp_size > 1`` positions start at ``cp_rank * s`` and tokens past the
    grid pass through, as in ``rope_apply_with_cp``.
    """
    grids = grid_sizes.tolist() if hasattr(grid_sizes, "tolist") else [list(g) for g in grid_sizes]
    if any(list(g) != list(grids[0]) for g in grids):
        raise NotImplementedError("b200 rope_apply needs one (f, h, w) grid for the whole batch")
    B, s, H, D = x.shape
    # keyed by the storage the table was built from (address, shape, version), not by id(): ids are
    # reused once a tensor has been freed
    key = (freqs.data_ptr(), tuple(freqs.shape), freqs._version, str(freqs.device), str(x.device))
    table = _TABLE_CACHE.get(key)
    if table is None:
        table = table_from_complex(freqs, x.device)
        _TABLE_CACHE[key] = table
    flat = x.reshape(B, s, H * D)
    return ops.qk_norm_rope(flat, H, None, 0.0, norm_mode=2, rope_mode=1, rope_table=table, grid=grids[0],
                            axis_split=wan_axis_split(D), pos_offset=cp_rank * s if cp_size > 1 else 0)


class WanPreAttention:
    """``(q_proj, k_proj, v_proj) -> (q, k, v)`` for Wan self-attention, one kernel pass per tensor."""

    def __init__(self, num_heads: int, head_dim: int, eps: float = 1e-6, cp_size: int = 1, cp_rank: int = 0,
                 device: Optional[torch.device] = None):
        self.num_heads, self.head_dim, self.eps = num_heads, head_dim, eps
        self.cp_size, self.cp_rank = cp_size, cp_rank
        self.table = wan_rope_table(head_dim, device=device)
        self.split = wan_axis_split(head_dim)

    def one(self, x: torch.Tensor, weight: Optional[torch.Tensor], grid: Sequence[int], **placement) -> torch.Tensor:
        s = x.shape[1]
        return ops.qk_norm_rope(
            x, self.num_heads, weight, self.eps, norm_mode=0, rope_mode=1, rope_table=self.table, grid=grid,
            axis_split=self.split, pos_offset=self.cp_rank * s if self.cp_size > 1 else 0, **placement,
        )

    def jobs(self, q_proj, k_proj, wq, wk):
        return [dict(x=q_proj, weight=wq, norm_mode=0, rope_mode=1), dict(x=k_proj, weight=wk, norm_mode=0, rope_mode=1)]

    def batch_args(self, s: int, grid: Sequence[int]) -> dict:
        return dict(num_heads=self.num_heads, eps=self.eps, rope_table=self.table, grid=grid, axis_split=self.split,
                    pos_offset=self.cp_rank * s if self.cp_size > 1 else 0)

    def __call__(self, q_proj, k_proj, v_proj, wq, wk, grid):
        B, S, C = q_proj.shape
        q, k = ops.qk_norm_rope_batch(self.jobs(q_proj, k_proj, wq, wk), **self.batch_args(S, grid))
        v = v_proj.view(B, S, self.num_heads, self.head_dim)
        if v.dtype not in (torch.bfloat16, torch.float16):
            v = v.to(torch.bfloat16)
        return q, k, v


class JointPreAttention:
    """Per-head RMSNorm + per-token rotary table (Flux / Qwen joint attention)."""

    def __init__(self, num_heads: int, head_dim: int, table: torch.Tensor, eps: float = 1e-6):
        self.num_heads, self.head_dim, self.eps, self.table = num_heads, head_dim, eps, table

    def one(self, x: torch.Tensor, weight: Optional[torch.Tensor], pos_offset: int = 0, **placement) -> torch.Tensor:
        return ops.qk_norm_rope(x, self.num_heads, weight, self.eps, norm_mode=1, rope_mode=2, rope_table=self.table,
                                pos_offset=pos_offset, round_mid=False, **placement)

    def jobs(self, q_proj, k_proj, wq=None, wk=None):
        return [dict(x=q_proj, weight=wq, norm_mode=1, rope_mode=2), dict(x=k_proj, weight=wk, norm_mode=1, rope_mode=2)]

    def batch_args(self, s: int = 0, grid: Sequence[int] = (0, 0, 0), pos_offset: int = 0) -> dict:
        return dict(num_heads=self.num_heads, eps=self.eps, rope_table=self.table, pos_offset=pos_offset,
                    round_mid=False)

    def __call__(self, q_proj, k_proj, v_proj, wq=None, wk=None, pos_offset: int = 0):
        B, S, C = q_proj.shape
        q, k = ops.qk_norm_rope_batch(self.jobs(q_proj, k_proj, wq, wk), **self.batch_args(pos_offset=pos_offset))
        v = v_proj.view(B, S, self.num_heads, self.head_dim)
        if v.dtype not in (torch.bfloat16, torch.float16):
            v = v.to(torch.bfloat16)
        return q, k, v


def transform_pieces(pieces, dtype: torch.dtype = torch.bfloat16):
    """Run the pre-attention jobs of a layer given in row pieces and return contiguous ``(q, k, v)``.

    ``pieces`` is a list of ``(jobs, v_proj, row_offset, batch_args)`` as collected by the
    ``attention_from_projections`` entries: each piece is transformed straight into its rows of the
    joint ``[B, S, H, D]`` tensors (one launch per piece).
    """
    x0 = pieces[0][0][0]["x"]
    B, _, C = x0.shape
    H = int(pieces[0][3]["num_heads"])
    D = C // H
    S = max(off + jb[0]["x"].shape[1] for jb, _, off, _ in pieces)
    if len(pieces) == 1 and pieces[0][2] == 0 and pieces[0][1].dtype == dtype:
        # one piece covering every row: v needs no copy, the attention kernel reads the projection view
        jb, vp, _, args = pieces[0]
        args = {key: val for key, val in args.items() if key != "out_dtype"}
        q, k = ops.qk_norm_rope_batch(jb, out_dtype=dtype, **args)
        return q, k, (vp.unflatten(2, (H, D)) if vp.dim() == 3 else vp)
    q, k, v = (torch.empty((B, S, H, D), dtype=dtype, device=x0.device) for _ in range(3))
    for jb, vp, off, args in pieces:
        n = jb[0]["x"].shape[1]
        args = {key: val for key, val in args.items() if key != "out_dtype"}
        jobs = [dict(j, out=t[:, off:off + n]) for j, t in zip(jb, (q, k))]
        if vp.dtype == x0.dtype:
            jobs.append(dict(x=vp.reshape(B, n, C), norm_mode=2, rope_mode=0, out=v[:, off:off + n]))
        else:
            v[:, off:off + n].copy_(vp.reshape(B, n, H, D))
        ops.qk_norm_rope_batch(jobs, out_strides=(S * C, C, 0, D), heads_per_group=H, out_dtype=dtype, **args)
    return q, k, v
