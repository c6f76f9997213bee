"""Operator-level Python entry points: torch tensors in, C-ABI calls out.

Torch is used for device memory and the current stream only; all arithmetic
happens inside libchitu_b200.so.  Every function raises if the tensors are not
on a CUDA device - there is no CPU path.
"""

from __future__ import annotations

import math
import os
from typing import Optional, Sequence, Tuple

import torch

from . import _lib

_DTYPES = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_FP16, torch.float32: _lib.DTYPE_FP32}

_STATUS_NAMES = {
    1: "TMA producer waited too long for a free K/V stage",
    2: "MMA issuer waited too long for operands",
    3: "softmax warps waited too long for scores",
    4: "epilogue waited too long for the last MMA",
    5: "a bounded flag wait ran out",
}

_status_words = {}

# kernels of this library launched so far by this process (the bench reports the count of a timed region)
launch_count = 0


def _launched(n: int = 1) -> None:
    global launch_count
    launch_count += n


def _stream_ptr(device: torch.device) -> int:
    return int(torch.cuda.current_stream(device).cuda_stream)


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("chitudiffusion_b200 runs on CUDA tensors only (there is no CPU path)")


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 status word that kernels with bounded waits report into."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    word = _status_words.get(key)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
        _status_words[key] = word
    return word


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise and raise if any kernel on `device` reported a timed-out wait."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = status_word(dev)
    code = int(word.item())
    if code != 0:
        word.zero_()
        raise _lib.ChituB200Error(f"device status {code}: {_STATUS_NAMES.get(code, 'unknown')}")


_status_mirrors = {}


def poll_status(device: Optional[torch.device] = None) -> None:
    """Deferred, non-blocking form of :func:`check_status` for the product path.

    Each call first looks at the copy of the status word that the PREVIOUS call sent to pinned host
    memory (if that copy has landed) and raises when it is non-zero, then enqueues a fresh copy behind
    the work just launched.  A timed-out device wait therefore surfaces as an exception one call later
    instead of as silently wrong output, and no call ever synchronises.  ``CHITU_B200_CHECK=1`` makes
    every poll a full synchronising check.  Nothing is enqueued while the stream is being captured.
    """
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if torch.cuda.is_current_stream_capturing():
        return  # event queries and host copies have no place inside a capture
    if os.environ.get("CHITU_B200_CHECK", "0") == "1":
        check_status(dev)
        return
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    mirror = _status_mirrors.get(key)
    if mirror is None:
        mirror = {"host": torch.zeros(1, dtype=torch.int32).pin_memory(), "event": None}
        _status_mirrors[key] = mirror
    ev = mirror["event"]
    if ev is not None and ev.query():
        code = int(mirror["host"][0])
        if code != 0:
            mirror["host"].zero_()
            mirror["event"] = None
            status_word(dev).zero_()
            raise _lib.ChituB200Error(f"device status {code}: {_STATUS_NAMES.get(code, 'unknown')}")
    if ev is None or ev.query():
        mirror["host"].copy_(status_word(dev), non_blocking=True)
        if ev is None:
            ev = torch.cuda.Event()
            mirror["event"] = ev
        ev.record(torch.cuda.current_stream(dev))


def set_flag_wait_cycles(cycles: int) -> int:
    """Clock budget of the cross-GPU flag waits; returns the previous one (see ``chitu_b200_set_flag_wait_cycles``)."""
    return int(_lib.load().chitu_b200_set_flag_wait_cycles(int(cycles)))


_workspaces = {}
_retired_workspaces = []
NUM_SMS = 148


def auto_key_splits(B: int, Sq: int, Sk: int, H: int) -> int:
    """How many key ranges to run as separate CTAs.  A CTA serves 256 query rows of one head; the grid runs in
    waves of one CTA per SM, so the cost of a call is (waves) x (key tiles per CTA, plus about 5 tile steps for
    a CTA's prologue and for parking its partial rows: 216 CTAs x 36 tiles measured 138 us, 432 CTAs x 18 tiles
    143 us) plus about one tile step per range for the merge.  The split that minimises it is taken when it
    saves at least 8 %: it fills small grids (54 CTAs -> 2 ranges).
    ``CHITU_B200_KEY_SPLITS`` overrides."""
    import os

    forced = os.environ.get("CHITU_B200_KEY_SPLITS")
    tiles = -(-Sk // 128)
    if forced:
        return max(1, min(int(forced), tiles, 64))
    ctas = -(-Sq // 256) * H * B

    def cost(n):
        per = -(-tiles // n)
        n_eff = -(-tiles // per)
        waves = -(-ctas * n_eff // NUM_SMS)
        return waves * per if n_eff == 1 else waves * (per + 5.0) + 1.0 * n_eff

    best, best_cost = 1, cost(1)
    for n in range(2, min(tiles, 16) + 1):
        if ctas * n > 512:  # the parked rows (128 KiB per CTA) should stay in L2 until they are merged
            break
        c = cost(n)
        if c < best_cost * 0.92 and c < cost(best):
            best, best_cost = n, c
    return best


def splitkv_workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch for key-split partials, one buffer per (device, stream), grown on demand, zero-filled when
    created (the library keeps per-query-block counters in its first 64 KiB and leaves them zero after each call).

    A buffer that has been handed out may be baked into a captured CUDA graph, so a superseded buffer
    is never freed: it is parked for the life of the process and the larger replacement serves later
    calls.  Streams do not share a buffer (two streams of one GPU may run key-split calls at once).
    Objects that own long-lived graphs (the peer exchanges) allocate their own scratch instead and pass
    it as ``workspace=``.
    """
    dev = torch.device(device)
    key = (dev.index if dev.index is not None else torch.cuda.current_device(),
           int(torch.cuda.current_stream(dev).cuda_stream))
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired_workspaces.append(ws)
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=dev)  # the counters at its head start at zero
        _workspaces[key] = ws
    return ws


def splitkv_workspace_bytes(B: int, Sq: int, H: int, D: int, n_splits: int) -> int:
    """Bytes of scratch a key-split call of this shape needs (0 for one split)."""
    return int(_lib.load().chitu_b200_attn_splitkv_workspace_bytes(B, Sq, H, D, int(n_splits)))


def attn_fwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    softmax_scale: Optional[float] = None,
    return_lse: bool = False,
    out: Optional[torch.Tensor] = None,
    n_splits: Optional[int] = None,
    workspace: Optional[torch.Tensor] = None,
    q_pre: Optional[dict] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """``softmax(scale * q k^T) v`` for ``[B,S,H,128]`` bf16/fp16 tensors of any (16-byte aligned) strides.

    Returns ``(out [B,Sq,H,D] contiguous, lse [B,H,Sq] fp32 | None)``.  ``workspace`` is an optional
    caller-owned uint8 scratch for the key-split partials (see :func:`splitkv_workspace`); its first 64 KiB
    hold counters that must be zero before the first use (``torch.zeros``) and are left zero by every call.  With ``q_pre``
    (keys ``norm_mode, rope_mode, weight, rstd, eps, rope_table, grid, axis_split, pos_offset, round_mid``)
    ``q`` is the raw projection and its pre-attention transform runs inside the kernel
    (``chitu_b200_attn_fwd_qpre``).
    """
    _require_cuda(q, k, v)
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k, v must be [B, S, H, D]")
    B, Sq, H, D = q.shape
    if k.shape != v.shape or k.shape[0] != B or k.shape[2] != H or k.shape[3] != D:
        raise ValueError(f"shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise NotImplementedError("attention kernel takes bf16 or fp16 q/k/v of one dtype")
    Sk = k.shape[1]
    if Sq == 0 or Sk == 0:
        raise ValueError("empty sequence")

    def usable(t):
        return t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0

    q, k, v = (t if usable(t) else t.contiguous() for t in (q, k, v))
    if out is None:
        out = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
    elif out.shape != (B, Sq, H, D) or not out.is_contiguous() or out.dtype != q.dtype:
        raise ValueError("out must be a contiguous [B,Sq,H,D] tensor of q's dtype")
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device) if return_lse else None
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    lib = _lib.load()
    if n_splits is None:
        n_splits = auto_key_splits(B, Sq, Sk, H)
    if q_pre is not None:
        import ctypes

        w, rstd, table = q_pre.get("weight"), q_pre.get("rstd"), q_pre.get("rope_table")
        _require_cuda(w, rstd, table)
        if w is not None:
            w = w.contiguous()
        grid = q_pre.get("grid", (0, 0, 0))
        split = q_pre.get("axis_split", (0, 0))
        desc = _lib.QPre(
            int(q_pre.get("norm_mode", 2)), int(q_pre.get("rope_mode", 0)), 1 if q_pre.get("round_mid", True) else 0,
            _DTYPES[w.dtype] if w is not None else _lib.DTYPE_FP32, w.data_ptr() if w is not None else None,
            rstd.data_ptr() if rstd is not None else None, float(q_pre.get("eps", 1e-6)),
            table.data_ptr() if table is not None else None, int(table.shape[0]) if table is not None else 0,
            int(grid[0]), int(grid[1]), int(grid[2]), int(split[0]), int(split[1]), int(q_pre.get("pos_offset", 0)))
        ws_ptr, ws_bytes = None, 0
        if n_splits > 1:
            need = int(lib.chitu_b200_attn_splitkv_workspace_bytes(B, Sq, H, D, n_splits))
            ws = workspace if workspace is not None else splitkv_workspace(q.device, need)
            ws_ptr, ws_bytes = ws.data_ptr(), ws.numel()
        with torch.cuda.device(q.device):
            rc = lib.chitu_b200_attn_fwd_qpre(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr() if lse is not None else None,
                B, Sq, Sk, H, D, _lib.i64_array(q.stride()), _lib.i64_array(k.stride()), _lib.i64_array(v.stride()),
                scale, _DTYPES[q.dtype], ctypes.byref(desc), int(n_splits), ws_ptr, ws_bytes,
                status_word(q.device).data_ptr(), _stream_ptr(q.device))
        _lib.check(rc, "attn_fwd_qpre")
        _launched(1)
        return out, lse
    with torch.cuda.device(q.device):
        if n_splits > 1:
            need = int(lib.chitu_b200_attn_splitkv_workspace_bytes(B, Sq, H, D, n_splits))
            ws = workspace if workspace is not None else splitkv_workspace(q.device, need)
            if ws.numel() * ws.element_size() < need or ws.device != q.device:
                raise ValueError(f"attn_fwd: workspace must hold {need} bytes on {q.device}")
            rc = lib.chitu_b200_attn_fwd_splitkv(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                lse.data_ptr() if lse is not None else None, B, Sq, Sk, H, D, _lib.i64_array(q.stride()),
                _lib.i64_array(k.stride()), _lib.i64_array(v.stride()), scale, _DTYPES[q.dtype], int(n_splits),
                ws.data_ptr(), ws.numel(), status_word(q.device).data_ptr(), _stream_ptr(q.device),
            )
        else:
            rc = lib.chitu_b200_attn_fwd(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                lse.data_ptr() if lse is not None else None, B, Sq, Sk, H, D, _lib.i64_array(q.stride()),
                _lib.i64_array(k.stride()), _lib.i64_array(v.stride()), scale, _DTYPES[q.dtype],
                status_word(q.device).data_ptr(), _stream_ptr(q.device),
            )
    _lib.check(rc, "attn_fwd")
    _launched(1)
    return out, lse


def attn_fwd_q8(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    softmax_scale: Optional[float] = None,
    return_lse: bool = False,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Quantised attention (INT8 QK^T, E4M3 PV); see ``chitu_b200_attn_fwd_q8``."""
    _require_cuda(q, k, v)
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    if k.shape != v.shape or k.shape[0] != B or k.shape[2] != H or k.shape[3] != D:
        raise ValueError(f"shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)}")
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise NotImplementedError("attention kernel takes bf16 or fp16 q/k/v of one dtype")

    def usable(t):
        return t.stride(3) == 1 and all(s % 4 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0

    q, k, v = (t if usable(t) else t.contiguous() for t in (q, k, v))
    out = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device) if return_lse else None
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    lib = _lib.load()
    need = int(lib.chitu_b200_attn_q8_workspace_bytes(B, Sq, Sk, H))
    ws = torch.empty(need + 256, dtype=torch.uint8, device=q.device)
    base = (ws.data_ptr() + 255) // 256 * 256
    with torch.cuda.device(q.device):
        rc = lib.chitu_b200_attn_fwd_q8(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr() if lse is not None else None,
            B, Sq, Sk, H, D, _lib.i64_array(q.stride()), _lib.i64_array(k.stride()), _lib.i64_array(v.stride()),
            scale, _DTYPES[q.dtype], base, need, status_word(q.device).data_ptr(), _stream_ptr(q.device),
        )
    _lib.check(rc, "attn_fwd_q8")
    _launched(3)
    return out, lse


def lse_combine(
    acc_out: torch.Tensor,
    acc_lse: torch.Tensor,
    block_out: torch.Tensor,
    block_lse: torch.Tensor,
    first: bool,
    final_out: Optional[torch.Tensor] = None,
) -> None:
    """In-place fold of one partial result; see ``chitu_b200_lse_combine``.

    ``acc_out [B,S,H,D] fp32``, ``acc_lse [B,S,H]`` (or ``[B,S,H,1]``) fp32, ``block_out [B,S,H,D]``,
    ``block_lse [B,H,S] fp32``; all contiguous.
    """
    _require_cuda(acc_out, acc_lse, block_out, block_lse, final_out)
    B, S, H, D = block_out.shape
    if acc_out.shape != block_out.shape or acc_out.dtype != torch.float32 or not acc_out.is_contiguous():
        raise ValueError("acc_out must be contiguous fp32 [B,S,H,D]")
    if acc_lse.numel() != B * S * H or acc_lse.dtype != torch.float32 or not acc_lse.is_contiguous():
        raise ValueError("acc_lse must be contiguous fp32 [B,S,H] or [B,S,H,1]")
    if tuple(block_lse.shape) != (B, H, S) or block_lse.dtype != torch.float32:
        raise ValueError("block_lse must be fp32 [B,H,S]")
    block_out = block_out.contiguous()
    block_lse = block_lse.contiguous()
    if final_out is not None and (final_out.shape != block_out.shape or not final_out.is_contiguous()):
        raise ValueError("final_out must be contiguous [B,S,H,D]")
    lib = _lib.load()
    with torch.cuda.device(acc_out.device):
        rc = lib.chitu_b200_lse_combine(
            acc_out.data_ptr(), acc_lse.data_ptr(), block_out.data_ptr(), block_lse.data_ptr(), B, S, H, D,
            _DTYPES[block_out.dtype], 1 if first else 0,
            final_out.data_ptr() if final_out is not None else None,
            _DTYPES[final_out.dtype] if final_out is not None else 0, _stream_ptr(acc_out.device),
        )
    _lib.check(rc, "lse_combine")
    _launched()


def qk_norm_rope(
    x: torch.Tensor,
    num_heads: int,
    weight: Optional[torch.Tensor],
    eps: float,
    norm_mode: int,
    rope_mode: int,
    rope_table: Optional[torch.Tensor],
    grid: Sequence[int] = (0, 0, 0),
    axis_split: Sequence[int] = (0, 0),
    pos_offset: int = 0,
    out: Optional[torch.Tensor] = None,
    out_strides: Optional[Sequence[int]] = None,
    heads_per_group: Optional[int] = None,
    out_dtype: torch.dtype = torch.bfloat16,
    round_mid: bool = True,
    out_ptrs: Optional[Sequence[int]] = None,
) -> Optional[torch.Tensor]:
    """RMSNorm + rotary + 16-bit cast of a projection output ``[B,S,H*D]``; see ``chitu_b200_qk_norm_rope``.

    Without ``out`` a contiguous ``[B,S,H,D]`` tensor is returned.  With ``out`` and ``out_strides``
    ``(b, s, head_group, head_in_group)`` the result is scattered into a caller-owned buffer.
    """
    _require_cuda(x, weight, rope_table, out)
    if x.dim() != 3:
        raise ValueError("x must be [B, S, C]")
    B, S, C = x.shape
    if C % num_heads:
        raise ValueError("channels not divisible by num_heads")
    D = C // num_heads
    if x.stride(2) != 1 or (B > 1 and x.stride(0) != S * x.stride(1)):
        x = x.contiguous()
    if weight is not None:
        weight = weight.contiguous()
        if weight.dtype not in _DTYPES:
            raise ValueError("weight dtype must be bf16, fp16 or fp32")
    if rope_mode != 0:
        if rope_table is None or rope_table.dtype != torch.float32 or not rope_table.is_contiguous():
            raise ValueError("rope_table must be a contiguous fp32 [rows, D/2, 2] tensor")
        if rope_table.shape[-2:] != (D // 2, 2):
            raise ValueError(f"rope_table must be [rows, {D // 2}, 2]")
    if out_ptrs is not None:
        if out is not None or out_strides is None or heads_per_group is None:
            raise ValueError("out_ptrs needs out_strides and heads_per_group, and excludes out")
    elif out is None:
        out = torch.empty((B, S, num_heads, D), dtype=out_dtype, device=x.device)
        out_strides = (S * C, C, 0, D)
        heads_per_group = num_heads
    elif out_strides is None or heads_per_group is None:
        raise ValueError("out needs out_strides and heads_per_group")
    lib = _lib.load()
    import ctypes

    split = (ctypes.c_int * 2)(int(axis_split[0]), int(axis_split[1]))
    common = (
        x.data_ptr(), _DTYPES[x.dtype], x.stride(1), weight.data_ptr() if weight is not None else None,
        _DTYPES[weight.dtype] if weight is not None else _lib.DTYPE_FP32, float(eps), int(norm_mode),
        int(rope_mode), rope_table.data_ptr() if rope_table is not None else None,
        int(rope_table.shape[0]) if rope_table is not None else 0, int(grid[0]), int(grid[1]), int(grid[2]),
        split, int(pos_offset),
    )
    tail = (_lib.i64_array(out_strides), int(heads_per_group), B, S, num_heads, D, 1 if round_mid else 0,
            _stream_ptr(x.device))
    with torch.cuda.device(x.device):
        if out_ptrs is not None:
            rc = lib.chitu_b200_qk_norm_rope_scatter(*common, _lib.ptr_array(out_ptrs), len(out_ptrs),
                                                     _DTYPES[out_dtype], *tail)
        else:
            rc = lib.chitu_b200_qk_norm_rope(*common, out.data_ptr(), _DTYPES[out.dtype], *tail)
    _lib.check(rc, "qk_norm_rope")
    _launched()
    return out


def qk_norm_rope_batch(
    jobs: Sequence[dict],
    num_heads: int,
    eps: float,
    rope_table: Optional[torch.Tensor],
    grid: Sequence[int] = (0, 0, 0),
    axis_split: Sequence[int] = (0, 0),
    pos_offset: int = 0,
    out_strides: Optional[Sequence[int]] = None,
    heads_per_group: Optional[int] = None,
    out_dtype: torch.dtype = torch.bfloat16,
    round_mid: bool = True,
    sync=None,
    stage_only: bool = False,
):
    """Up to three pre-attention jobs (q, k, v) in one launch; see ``chitu_b200_qk_norm_rope_batch``.

    With ``sync`` (a ``_lib.peer_sync_desc`` pair) the launch ends by announcing this rank's rows to its
    peers (``chitu_b200_qk_norm_rope_batch_signal``); with ``stage_only`` as well it only advances the layer
    epoch - its destinations are local, the attention launch's copy CTAs deliver and announce the rows
    (``chitu_b200_qk_norm_rope_batch_stage``).

    Each job is a dict with ``x [B,S,H*D]``, optional ``weight``, ``norm_mode``, ``rope_mode`` and
    either ``out`` (tensor), ``out_ptrs`` (list of device addresses) or neither (a contiguous
    ``[B,S,H,D]`` result is allocated).  All jobs share dtype, shape and placement.  Returns the list
    of output tensors (``None`` for jobs written through ``out_ptrs``).
    """
    import ctypes

    x0 = jobs[0]["x"]
    B, S, C = x0.shape
    D = C // num_heads
    arr = (_lib.NormRopeJob * len(jobs))()
    keep, outs = [], []
    w_dtype = None
    for i, jb in enumerate(jobs):
        x = jb["x"]
        _require_cuda(x, jb.get("weight"), jb.get("out"))
        if x.shape != x0.shape or x.dtype != x0.dtype:
            raise ValueError("batched pre-attention jobs must share shape and dtype")
        if x.stride(2) != 1 or (B > 1 and x.stride(0) != S * x.stride(1)):
            x = x.contiguous()
        w = jb.get("weight")
        if w is not None:
            w = w.contiguous()
            if w_dtype is not None and w.dtype != w_dtype:
                raise ValueError("batched pre-attention jobs must share the weight dtype")
            w_dtype = w.dtype
        out, ptrs, rstd = jb.get("out"), jb.get("out_ptrs"), jb.get("rstd_out")
        if rstd is not None:
            if rstd.dtype != torch.float32 or rstd.numel() != B * S or not rstd.is_contiguous():
                raise ValueError("rstd_out must be a contiguous fp32 tensor of B*S elements")
            out = ptrs = None
            keep.append(rstd)
        arr[i].rstd_out = rstd.data_ptr() if rstd is not None else None
        if ptrs is None and out is None and rstd is None:
            if out_strides is not None:
                raise ValueError("explicit out_strides need out or out_ptrs in every job")
            out = torch.empty((B, S, num_heads, D), dtype=out_dtype, device=x.device)
        keep += [x, w, out]
        arr[i].x = x.data_ptr()
        arr[i].x_row_stride = x.stride(1)
        arr[i].weight = w.data_ptr() if w is not None else None
        arr[i].norm_mode = int(jb.get("norm_mode", 2))
        arr[i].rope_mode = int(jb.get("rope_mode", 0))
        arr[i].out = out.data_ptr() if out is not None else None
        if ptrs is not None:
            pa = _lib.ptr_array(ptrs)
            keep.append(pa)
            arr[i].out_ptrs = ctypes.cast(pa, ctypes.POINTER(ctypes.c_void_p))
            arr[i].n_out_ptrs = len(ptrs)
        else:
            arr[i].n_out_ptrs = 0
        outs.append(out)
    if out_strides is None:
        out_strides, heads_per_group = (S * C, C, 0, D), num_heads
    if rope_table is not None and (rope_table.dtype != torch.float32 or not rope_table.is_contiguous()):
        raise ValueError("rope_table must be a contiguous fp32 [rows, D/2, 2] tensor")
    split = (ctypes.c_int * 2)(int(axis_split[0]), int(axis_split[1]))
    lib = _lib.load()
    args = (
        arr, len(jobs), _DTYPES[x0.dtype], _DTYPES[w_dtype] if w_dtype is not None else _lib.DTYPE_FP32,
        float(eps), rope_table.data_ptr() if rope_table is not None else None,
        int(rope_table.shape[0]) if rope_table is not None else 0, int(grid[0]), int(grid[1]), int(grid[2]),
        split, int(pos_offset), _DTYPES[out_dtype], _lib.i64_array(out_strides), int(heads_per_group),
        B, S, num_heads, D, 1 if round_mid else 0,
    )
    with torch.cuda.device(x0.device):
        if sync is not None:
            import ctypes as _ct

            fn = lib.chitu_b200_qk_norm_rope_batch_stage if stage_only else lib.chitu_b200_qk_norm_rope_batch_signal
            rc = fn(*args, _ct.byref(sync[0]), _stream_ptr(x0.device))
        else:
            rc = lib.chitu_b200_qk_norm_rope_batch(*args, _stream_ptr(x0.device))
    _lib.check(rc, "qk_norm_rope_batch")
    _launched()
    return outs


def strided_copy(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """Copy a 5-d view ``src [n0,n1,n2,n3,row]`` (last dim contiguous) into contiguous ``dst``."""
    _require_cuda(src, dst)
    if src.dim() != 5 or dst.shape != src.shape or not dst.is_contiguous() or src.stride(4) != 1:
        raise ValueError("strided_copy: src must be 5-d with a contiguous last dim, dst contiguous of the same shape")
    es = src.element_size()
    lib = _lib.load()
    with torch.cuda.device(src.device):
        rc = lib.chitu_b200_strided_copy(
            src.data_ptr(), dst.data_ptr(), *[int(n) for n in src.shape[:4]], int(src.shape[4]) * es,
            _lib.i64_array([s * es for s in src.stride()[:4]]), _stream_ptr(src.device),
        )
    _lib.check(rc, "strided_copy")
    _launched()
    return dst


def layernorm_modulate(x: torch.Tensor, mul: Optional[torch.Tensor] = None, add: Optional[torch.Tensor] = None,
                       add_one: bool = False, eps: float = 1e-6, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``LayerNorm(x) * m + a`` for ``x [B, L, C]`` (fp32 or 16-bit); ``mul`` / ``add`` are ``[C]``, ``[1, C]``-like or ``[B, C]``-like
    fp32 (``m = 1 + mul`` with ``add_one``); see ``chitu_b200_layernorm_modulate``."""
    _require_cuda(x)
    if x.dtype not in _DTYPES or x.dim() != 3 or not x.is_contiguous():
        raise ValueError("layernorm_modulate: x must be a contiguous [B, L, C] tensor (fp32, bf16 or fp16)")
    B, L, C = x.shape

    def vec(t):
        if t is None:
            return None, 0
        t = t.reshape(-1, C)
        if t.dtype != torch.float32 or t.shape[0] not in (1, B) or t.stride(1) != 1:
            raise ValueError("layernorm_modulate: mul / add must be fp32 with C channels for 1 or B batches")
        return t, (t.stride(0) if t.shape[0] == B and B > 1 else 0)

    (m, ms), (a, as_) = vec(mul), vec(add)
    out = torch.empty((B, L, C), dtype=out_dtype, device=x.device)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        rc = lib.chitu_b200_layernorm_modulate(
            x.data_ptr(), _DTYPES[x.dtype], out.data_ptr(), _DTYPES[out_dtype], B * L, L, C,
            m.data_ptr() if m is not None else None, ms,
            a.data_ptr() if a is not None else None, as_, int(add_one), float(eps), _stream_ptr(x.device))
    _lib.check(rc, "layernorm_modulate")
    _launched()
    return out


def gate_residual(x: torch.Tensor, y: torch.Tensor, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """In place ``x += y * gate`` (``x [B, L, C]`` fp32 or 16-bit, ``y`` 16-bit, ``gate`` fp32 per batch and channel or None)."""
    _require_cuda(x, y)
    if x.dtype not in _DTYPES or x.dim() != 3 or not x.is_contiguous() or y.shape != x.shape or not y.is_contiguous():
        raise ValueError("gate_residual: x must be contiguous [B, L, C] and y contiguous of the same shape")
    B, L, C = x.shape
    g, gs = None, 0
    if gate is not None:
        g = gate.reshape(-1, C)
        if g.dtype != torch.float32 or g.shape[0] not in (1, B) or g.stride(1) != 1:
            raise ValueError("gate_residual: gate must be fp32 with C channels for 1 or B batches")
        gs = g.stride(0) if g.shape[0] == B and B > 1 else 0
    lib = _lib.load()
    with torch.cuda.device(x.device):
        rc = lib.chitu_b200_gate_residual(x.data_ptr(), _DTYPES[x.dtype], y.data_ptr(), _DTYPES[y.dtype], B * L, L, C,
                                          g.data_ptr() if g is not None else None, gs, _stream_ptr(x.device))
    _lib.check(rc, "gate_residual")
    _launched()
    return x


def cfg_combine(cond: torch.Tensor, uncond: torch.Tensor, scale: float, rescale: bool = False) -> torch.Tensor:
    """``uncond + scale * (cond - uncond)``, with ``rescale`` multiplied row-wise by ``||cond|| / ||result||`` over the last dim."""
    _require_cuda(cond, uncond)
    if cond.shape != uncond.shape or cond.dtype != uncond.dtype or cond.dtype not in _DTYPES:
        raise ValueError("cfg_combine: cond and uncond must share shape and dtype (bf16, fp16 or fp32)")
    cond, uncond = cond.contiguous(), uncond.contiguous()
    out = torch.empty_like(cond)
    C = cond.shape[-1]
    lib = _lib.load()
    with torch.cuda.device(cond.device):
        rc = lib.chitu_b200_cfg_combine(cond.data_ptr(), uncond.data_ptr(), out.data_ptr(), _DTYPES[cond.dtype],
                                        cond.numel() // C, C, float(scale), int(rescale), _stream_ptr(cond.device))
    _lib.check(rc, "cfg_combine")
    _launched()
    return out


def peer_copy_2d(dst_ptr: int, dst_pitch: int, src_ptr: int, src_pitch: int, width: int, rows: int,
                 device: torch.device) -> None:
    """``rows`` pieces of ``width`` bytes between device buffers (either may be peer-mapped), on the copy engines."""
    lib = _lib.load()
    with torch.cuda.device(device):
        rc = lib.chitu_b200_peer_copy_2d(int(dst_ptr), int(dst_pitch), int(src_ptr), int(src_pitch), int(width),
                                         int(rows), _stream_ptr(device))
    _lib.check(rc, "peer_copy_2d")


def scatter_rows(src: torch.Tensor, dst_ptrs: Sequence[int], rows: int, dst_batch_stride_bytes: int,
                 dst_row_stride_bytes: int) -> None:
    """``src [B, n_dest*rows, ...]`` contiguous: row ``(b, i*rows + j)`` goes to ``dst_ptrs[i] + b*batch + j*row`` bytes."""
    _require_cuda(src)
    if not src.is_contiguous() or src.dim() < 3 or src.shape[1] != rows * len(dst_ptrs):
        raise ValueError("scatter_rows: src must be contiguous [B, n_dest*rows, ...]")
    row_bytes = src[0, 0].numel() * src.element_size()
    lib = _lib.load()
    with torch.cuda.device(src.device):
        rc = lib.chitu_b200_scatter_rows(src.data_ptr(), _lib.ptr_array(dst_ptrs), len(dst_ptrs), int(src.shape[0]),
                                         int(rows), int(row_bytes), int(dst_batch_stride_bytes),
                                         int(dst_row_stride_bytes), _stream_ptr(src.device))
    _lib.check(rc, "scatter_rows")
    _launched()


def attn_fwd_scatter(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out_ptrs: Sequence[int],
    rows_per_dest: int,
    dest_batch_stride: int,
    dest_row_stride: int,
    dest_head_offset: int,
    softmax_scale: Optional[float] = None,
    n_splits: Optional[int] = None,
    workspace: Optional[torch.Tensor] = None,
) -> None:
    """Attention whose query row ``r`` is stored to ``out_ptrs[r // rows_per_dest]``; see ``chitu_b200_attn_fwd_scatter``."""
    _require_cuda(q, k, v)
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise NotImplementedError("attention kernel takes bf16 or fp16 q/k/v of one dtype")
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    lib = _lib.load()
    if n_splits is None:
        n_splits = auto_key_splits(B, Sq, Sk, H)
    ws_ptr, ws_bytes = None, 0
    if n_splits > 1:
        need = int(lib.chitu_b200_attn_splitkv_workspace_bytes(B, Sq, H, D, n_splits))
        ws = workspace if workspace is not None else splitkv_workspace(q.device, need)
        if ws.numel() * ws.element_size() < need or ws.device != q.device:
            raise ValueError(f"attn_fwd_scatter: workspace must hold {need} bytes on {q.device}")
        ws_ptr, ws_bytes = ws.data_ptr(), ws.numel()
    with torch.cuda.device(q.device):
        rc = lib.chitu_b200_attn_fwd_scatter(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), _lib.ptr_array(out_ptrs), len(out_ptrs), int(rows_per_dest),
            int(dest_batch_stride), int(dest_row_stride), int(dest_head_offset), None, B, Sq, Sk, H, D,
            _lib.i64_array(q.stride()), _lib.i64_array(k.stride()), _lib.i64_array(v.stride()), scale,
            _DTYPES[q.dtype], int(n_splits), ws_ptr, ws_bytes, status_word(q.device).data_ptr(),
            _stream_ptr(q.device),
        )
    _lib.check(rc, "attn_fwd_scatter")
    _launched(1)


def peer_barrier(flag_ptrs: Sequence[int], rank: int, world: int, device: torch.device) -> None:
    """Enqueue the bounded cross-GPU barrier on the current stream; see ``chitu_b200_peer_barrier``."""
    lib = _lib.load()
    with torch.cuda.device(device):
        rc = lib.chitu_b200_peer_barrier(_lib.ptr_array(flag_ptrs), int(rank), int(world),
                                         status_word(device).data_ptr(), _stream_ptr(device))
    _lib.check(rc, "peer_barrier")
    _launched()


def attn_fwd_exchange(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out_ptrs: Sequence[int],
    rows_per_dest: int,
    dest_batch_stride: int,
    dest_row_stride: int,
    dest_head_offset: int,
    rows_per_src: int,
    sync,
    softmax_scale: Optional[float] = None,
    n_splits: Optional[int] = None,
    workspace: Optional[torch.Tensor] = None,
    prefix_rows: int = 0,
    prefix_ptrs: Optional[Sequence[int]] = None,
    prefix_batch_stride: int = 0,
    prefix_row_stride: int = 0,
    prefix_head_offset: int = 0,
    push=None,
) -> None:
    """:func:`attn_fwd_scatter` over exchange buffers guarded by arrival flags; see ``chitu_b200_attn_fwd_exchange``.
    With ``push`` (a ``_lib.push_desc`` pair) the launch also delivers the staged rows to the peers
    (``chitu_b200_attn_fwd_exchange_push``)."""
    import ctypes

    _require_cuda(q, k, v)
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise NotImplementedError("attention kernel takes bf16 or fp16 q/k/v of one dtype")
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    lib = _lib.load()
    if n_splits is None:
        n_splits = auto_key_splits(B, Sq, Sk, H)
    ws_ptr, ws_bytes = None, 0
    if n_splits > 1:
        need = int(lib.chitu_b200_attn_splitkv_workspace_bytes(B, Sq, H, D, n_splits))
        ws = workspace if workspace is not None else splitkv_workspace(q.device, need)
        if ws.numel() * ws.element_size() < need or ws.device != q.device:
            raise ValueError(f"attn_fwd_exchange: workspace must hold {need} bytes on {q.device}")
        ws_ptr, ws_bytes = ws.data_ptr(), ws.numel()
    if push is not None:
        if prefix_rows:
            raise NotImplementedError("push mode has no replicated prefix")
        with torch.cuda.device(q.device):
            rc = lib.chitu_b200_attn_fwd_exchange_push(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), _lib.ptr_array(out_ptrs), len(out_ptrs),
                int(rows_per_dest), int(dest_batch_stride), int(dest_row_stride), int(dest_head_offset), B, Sq, Sk, H,
                D, _lib.i64_array(q.stride()), _lib.i64_array(k.stride()), _lib.i64_array(v.stride()), scale,
                _DTYPES[q.dtype], int(n_splits), ws_ptr, ws_bytes, int(rows_per_src), ctypes.byref(push[0]),
                ctypes.byref(sync[0]), status_word(q.device).data_ptr(), _stream_ptr(q.device),
            )
        _lib.check(rc, "attn_fwd_exchange_push")
        _launched(1)
        return
    with torch.cuda.device(q.device):
        rc = lib.chitu_b200_attn_fwd_exchange(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), _lib.ptr_array(out_ptrs), len(out_ptrs), int(rows_per_dest),
            int(dest_batch_stride), int(dest_row_stride), int(dest_head_offset), B, Sq, Sk, H, D,
            _lib.i64_array(q.stride()), _lib.i64_array(k.stride()), _lib.i64_array(v.stride()), scale,
            _DTYPES[q.dtype], int(n_splits), ws_ptr, ws_bytes, int(rows_per_src), int(prefix_rows),
            _lib.ptr_array(prefix_ptrs) if prefix_ptrs else None, int(prefix_batch_stride), int(prefix_row_stride),
            int(prefix_head_offset), ctypes.byref(sync[0]),
            status_word(q.device).data_ptr(), _stream_ptr(q.device),
        )
    _lib.check(rc, "attn_fwd_exchange")
    _launched(1)


def set_cluster_merge(enable: bool) -> bool:
    """Merge two key ranges through a thread-block cluster's shared memory (default) or through the workspace;
    returns the previous setting.  ``CHITU_B200_CLUSTER_MERGE=0`` at import time selects the workspace form."""
    return bool(_lib.load().chitu_b200_set_cluster_merge(1 if enable else 0))


def stamp(slots: torch.Tensor, index: int) -> None:
    """Enqueue a launch that writes the GPU's nanosecond timer into ``slots[index]`` (int64 tensor on the GPU);
    works inside a captured graph.  Not counted as a launch of the hot path."""
    if slots.dtype != torch.int64 or not slots.is_cuda or not slots.is_contiguous():
        raise ValueError("stamp: slots must be a contiguous int64 CUDA tensor")
    if not 0 <= index < slots.numel():
        raise IndexError("stamp: index out of range")
    with torch.cuda.device(slots.device):
        rc = _lib.load().chitu_b200_stamp(slots.data_ptr() + 8 * int(index), _stream_ptr(slots.device))
    _lib.check(rc, "stamp")


def push_ctas(B: int, Sq: int, H: int, n_splits: int) -> int:
    """Copy CTAs that push mode would add to an attention launch of this shape on the current device (0: none)."""
    return int(_lib.load().chitu_b200_push_ctas(int(B), int(Sq), int(H), int(n_splits)))


def peer_wait_outputs(sync, device: torch.device) -> None:
    """Enqueue the bounded wait for every rank's output flag; see ``chitu_b200_peer_wait_outputs``."""
    import ctypes

    lib = _lib.load()
    with torch.cuda.device(device):
        rc = lib.chitu_b200_peer_wait_outputs(ctypes.byref(sync[0]), status_word(device).data_ptr(), _stream_ptr(device))
    _lib.check(rc, "peer_wait_outputs")
    _launched()
