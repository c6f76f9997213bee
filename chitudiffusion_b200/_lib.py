"""ctypes binding of libchitu_b200.so (the C ABI declared in include/chitu_b200.h).

There is no fallback: if the shared library is missing or a call fails, an
exception is raised.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# CHITU_B200_LIB points at another build of the same library (A/B measurements of kernel variants)
LIB_PATH = os.environ.get("CHITU_B200_LIB") or os.path.join(_PKG_DIR, "libchitu_b200.so")

OK, E_INVALID, E_UNSUPPORTED, E_CUDA = 0, -1, -2, -3
DTYPE_BF16, DTYPE_FP16, DTYPE_FP32 = 0, 1, 2

EXPORTS = (
    "chitu_b200_version",
    "chitu_b200_caps",
    "chitu_b200_last_error",
    "chitu_b200_attn_fwd",
    "chitu_b200_lse_combine",
    "chitu_b200_qk_norm_rope",
    "chitu_b200_strided_copy",
    "chitu_b200_qk_norm_rope_scatter",
    "chitu_b200_attn_fwd_scatter",
    "chitu_b200_peer_barrier",
    "chitu_b200_set_flag_wait_cycles",
    "chitu_b200_qk_norm_rope_batch_signal",
    "chitu_b200_attn_fwd_exchange",
    "chitu_b200_attn_fwd_exchange_push",
    "chitu_b200_qk_norm_rope_batch_stage",
    "chitu_b200_push_ctas",
    "chitu_b200_stamp",
    "chitu_b200_set_cluster_merge",
    "chitu_b200_attn_fwd_qpre",
    "chitu_b200_peer_wait_outputs",
    "chitu_b200_attn_splitkv_workspace_bytes",
    "chitu_b200_attn_fwd_splitkv",
    "chitu_b200_attn_fwd_splitkv_static",
    "chitu_b200_qk_norm_rope_batch",
    "chitu_b200_layernorm_modulate",
    "chitu_b200_gate_residual",
    "chitu_b200_cfg_combine",
    "chitu_b200_peer_copy_2d",
    "chitu_b200_scatter_rows",
    "chitu_b200_attn_q8_workspace_bytes",
    "chitu_b200_attn_fwd_q8",
)

_lib: Optional[ctypes.CDLL] = None

_i64p = ctypes.POINTER(ctypes.c_int64)
_vp = ctypes.c_void_p


class ChituB200Error(RuntimeError):
    pass


class NormRopeJob(ctypes.Structure):
    """Mirror of ``chitu_b200_norm_rope_job``."""

    _fields_ = [
        ("x", ctypes.c_void_p), ("x_row_stride", ctypes.c_int64), ("weight", ctypes.c_void_p),
        ("norm_mode", ctypes.c_int), ("rope_mode", ctypes.c_int), ("out", ctypes.c_void_p),
        ("out_ptrs", ctypes.POINTER(ctypes.c_void_p)), ("n_out_ptrs", ctypes.c_int), ("rstd_out", ctypes.c_void_p),
    ]


class PushDesc(ctypes.Structure):
    """Mirror of ``chitu_b200_push``."""

    _fields_ = [("stage", ctypes.c_void_p * 3), ("dest", ctypes.POINTER(ctypes.c_void_p) * 3),
                ("block_bytes", ctypes.c_int64)]


class PeerSyncDesc(ctypes.Structure):
    """Mirror of ``chitu_b200_peer_sync``."""

    _fields_ = [("blocks", ctypes.POINTER(ctypes.c_void_p)), ("rank", ctypes.c_int), ("world", ctypes.c_int)]


class QPre(ctypes.Structure):
    """Mirror of ``chitu_b200_q_pre``."""

    _fields_ = [
        ("norm_mode", ctypes.c_int), ("rope_mode", ctypes.c_int), ("round_mid", ctypes.c_int), ("w_dtype", ctypes.c_int),
        ("weight", ctypes.c_void_p), ("rstd", ctypes.c_void_p), ("eps", ctypes.c_float), ("rope_table", ctypes.c_void_p),
        ("table_rows", ctypes.c_int), ("gf", ctypes.c_int), ("gh", ctypes.c_int), ("gw", ctypes.c_int),
        ("n_t", ctypes.c_int), ("n_h", ctypes.c_int), ("pos_offset", ctypes.c_int64),
    ]


SYNC_INTS = 64


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ChituB200Error(
            f"{LIB_PATH} not found: build it with `python -m chitudiffusion_b200.build` "
            "(nvcc, sm_100a).  This package has no fallback path."
        )
    lib = ctypes.CDLL(LIB_PATH)
    lib.chitu_b200_version.restype = ctypes.c_int
    lib.chitu_b200_caps.restype = ctypes.c_uint
    lib.chitu_b200_last_error.restype = ctypes.c_char_p
    lib.chitu_b200_attn_fwd.restype = ctypes.c_int
    lib.chitu_b200_attn_fwd.argtypes = [
        _vp, _vp, _vp, _vp, _vp,
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        _i64p, _i64p, _i64p, ctypes.c_float, ctypes.c_int, _vp, _vp,
    ]
    lib.chitu_b200_lse_combine.restype = ctypes.c_int
    lib.chitu_b200_lse_combine.argtypes = [
        _vp, _vp, _vp, _vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        ctypes.c_int, ctypes.c_int, _vp, ctypes.c_int, _vp,
    ]
    lib.chitu_b200_qk_norm_rope.restype = ctypes.c_int
    lib.chitu_b200_qk_norm_rope.argtypes = [
        _vp, ctypes.c_int, ctypes.c_int64, _vp, ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_int,
        _vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_int64,
        _vp, ctypes.c_int, _i64p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        ctypes.c_int, _vp,
    ]
    lib.chitu_b200_strided_copy.restype = ctypes.c_int
    lib.chitu_b200_strided_copy.argtypes = [
        _vp, _vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, _i64p, _vp,
    ]
    _vpp = ctypes.POINTER(ctypes.c_void_p)
    lib.chitu_b200_qk_norm_rope_scatter.restype = ctypes.c_int
    lib.chitu_b200_qk_norm_rope_scatter.argtypes = [
        _vp, ctypes.c_int, ctypes.c_int64, _vp, ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_int,
        _vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_int64,
        _vpp, ctypes.c_int, ctypes.c_int, _i64p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        ctypes.c_int, ctypes.c_int, _vp,
    ]
    lib.chitu_b200_attn_fwd_scatter.restype = ctypes.c_int
    lib.chitu_b200_attn_fwd_scatter.argtypes = [
        _vp, _vp, _vp, _vpp, ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, _vp,
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        _i64p, _i64p, _i64p, ctypes.c_float, ctypes.c_int, ctypes.c_int, _vp, ctypes.c_int64, _vp, _vp,
    ]
    lib.chitu_b200_attn_splitkv_workspace_bytes.restype = ctypes.c_int64
    lib.chitu_b200_attn_splitkv_workspace_bytes.argtypes = [ctypes.c_int] * 5
    lib.chitu_b200_attn_fwd_splitkv.restype = ctypes.c_int
    lib.chitu_b200_attn_fwd_splitkv.argtypes = [
        _vp, _vp, _vp, _vp, _vp,
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        _i64p, _i64p, _i64p, ctypes.c_float, ctypes.c_int, ctypes.c_int, _vp, ctypes.c_int64, _vp, _vp,
    ]
    lib.chitu_b200_attn_fwd_splitkv_static.restype = ctypes.c_int
    lib.chitu_b200_attn_fwd_splitkv_static.argtypes = [
        _vp, _vp, _vp, _vp, _vp,
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        _i64p, _i64p, _i64p, ctypes.c_float, ctypes.c_int, ctypes.c_int, _vp, _vp,
    ]
    lib.chitu_b200_qk_norm_rope_batch.restype = ctypes.c_int
    lib.chitu_b200_qk_norm_rope_batch.argtypes = [
        ctypes.POINTER(NormRopeJob), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float, _vp, ctypes.c_int,
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_int64, ctypes.c_int,
        _i64p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, _vp,
    ]
    lib.chitu_b200_layernorm_modulate.restype = ctypes.c_int
    lib.chitu_b200_layernorm_modulate.argtypes = [_vp, ctypes.c_int, _vp, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                                  _vp, ctypes.c_int64, _vp, ctypes.c_int64, ctypes.c_int,
                                                  ctypes.c_float, _vp]
    lib.chitu_b200_gate_residual.restype = ctypes.c_int
    lib.chitu_b200_gate_residual.argtypes = [_vp, ctypes.c_int, _vp, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                             _vp, ctypes.c_int64, _vp]
    lib.chitu_b200_cfg_combine.restype = ctypes.c_int
    lib.chitu_b200_cfg_combine.argtypes = [_vp, _vp, _vp, ctypes.c_int, ctypes.c_int64, ctypes.c_int, ctypes.c_float,
                                           ctypes.c_int, _vp]
    lib.chitu_b200_peer_copy_2d.restype = ctypes.c_int
    lib.chitu_b200_peer_copy_2d.argtypes = [_vp, ctypes.c_int64, _vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, _vp]
    lib.chitu_b200_scatter_rows.restype = ctypes.c_int
    lib.chitu_b200_scatter_rows.argtypes = [_vp, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_int64,
                                            ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, _vp]
    lib.chitu_b200_attn_q8_workspace_bytes.restype = ctypes.c_int64
    lib.chitu_b200_attn_q8_workspace_bytes.argtypes = [ctypes.c_int] * 4
    lib.chitu_b200_attn_fwd_q8.restype = ctypes.c_int
    lib.chitu_b200_attn_fwd_q8.argtypes = [
        _vp, _vp, _vp, _vp, _vp,
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        _i64p, _i64p, _i64p, ctypes.c_float, ctypes.c_int, _vp, ctypes.c_int64, _vp, _vp,
    ]
    lib.chitu_b200_qk_norm_rope_batch_signal.restype = ctypes.c_int
    lib.chitu_b200_qk_norm_rope_batch_signal.argtypes = [
        ctypes.POINTER(NormRopeJob), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float, _vp, ctypes.c_int,
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_int64, ctypes.c_int,
        _i64p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        ctypes.POINTER(PeerSyncDesc), _vp,
    ]
    lib.chitu_b200_qk_norm_rope_batch_stage.restype = ctypes.c_int
    lib.chitu_b200_qk_norm_rope_batch_stage.argtypes = list(lib.chitu_b200_qk_norm_rope_batch_signal.argtypes)
    lib.chitu_b200_set_cluster_merge.restype = ctypes.c_int
    lib.chitu_b200_set_cluster_merge.argtypes = [ctypes.c_int]
    if os.environ.get("CHITU_B200_CLUSTER_MERGE", "1") == "0":
        lib.chitu_b200_set_cluster_merge(0)
    lib.chitu_b200_stamp.restype = ctypes.c_int
    lib.chitu_b200_stamp.argtypes = [_vp, _vp]
    lib.chitu_b200_push_ctas.restype = ctypes.c_int
    lib.chitu_b200_push_ctas.argtypes = [ctypes.c_int] * 4
    lib.chitu_b200_attn_fwd_exchange_push.restype = ctypes.c_int
    lib.chitu_b200_attn_fwd_exchange_push.argtypes = [
        _vp, _vp, _vp, _vpp, ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        _i64p, _i64p, _i64p, ctypes.c_float, ctypes.c_int, ctypes.c_int, _vp, ctypes.c_int64, ctypes.c_int,
        ctypes.POINTER(PushDesc), ctypes.POINTER(PeerSyncDesc), _vp, _vp,
    ]
    lib.chitu_b200_attn_fwd_exchange.restype = ctypes.c_int
    lib.chitu_b200_attn_fwd_exchange.argtypes = [
        _vp, _vp, _vp, _vpp, ctypes.c_int, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        _i64p, _i64p, _i64p, ctypes.c_float, ctypes.c_int, ctypes.c_int, _vp, ctypes.c_int64, ctypes.c_int,
        ctypes.c_int, _vpp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
        ctypes.POINTER(PeerSyncDesc), _vp, _vp,
    ]
    lib.chitu_b200_attn_fwd_qpre.restype = ctypes.c_int
    lib.chitu_b200_attn_fwd_qpre.argtypes = [
        _vp, _vp, _vp, _vp, _vp,
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
        _i64p, _i64p, _i64p, ctypes.c_float, ctypes.c_int, ctypes.POINTER(QPre), ctypes.c_int, _vp, ctypes.c_int64,
        _vp, _vp,
    ]
    lib.chitu_b200_peer_wait_outputs.restype = ctypes.c_int
    lib.chitu_b200_peer_wait_outputs.argtypes = [ctypes.POINTER(PeerSyncDesc), _vp, _vp]
    lib.chitu_b200_set_flag_wait_cycles.restype = ctypes.c_longlong
    lib.chitu_b200_set_flag_wait_cycles.argtypes = [ctypes.c_longlong]
    lib.chitu_b200_peer_barrier.restype = ctypes.c_int
    lib.chitu_b200_peer_barrier.argtypes = [_vpp, ctypes.c_int, ctypes.c_int, _vp, _vp]
    _lib = lib
    return lib


def push_desc(stage_ptrs: Sequence[int], dest_ptrs: Sequence[Sequence[int]], block_bytes: int):
    """``(descriptor, keep-alive)`` of ``chitu_b200_push``: staging areas of q, k, v and, per tensor, where this
    rank's block starts in every rank's gathered buffer."""
    arrs = [(ctypes.c_void_p * len(d))(*[int(x) for x in d]) for d in dest_ptrs]
    desc = PushDesc()
    for t in range(3):
        desc.stage[t] = int(stage_ptrs[t])
        desc.dest[t] = ctypes.cast(arrs[t], ctypes.POINTER(ctypes.c_void_p))
    desc.block_bytes = int(block_bytes)
    return desc, arrs


def peer_sync_desc(block_ptrs: Sequence[int], rank: int):
    """``(descriptor, keep-alive)`` for the sync blocks of a group (``block_ptrs[i]``: rank i's block as mapped here)."""
    arr = (ctypes.c_void_p * len(block_ptrs))(*[int(p) for p in block_ptrs])
    desc = PeerSyncDesc(ctypes.cast(arr, ctypes.POINTER(ctypes.c_void_p)), int(rank), len(block_ptrs))
    return desc, arr


def ptr_array(ptrs: Sequence[int]):
    return (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])


def i64_array(values: Sequence[int]):
    return (ctypes.c_int64 * len(values))(*[int(v) for v in values])


def check(rc: int, what: str) -> None:
    """Map a C-ABI return code to the reference's exception conventions."""
    if rc == OK:
        return
    msg = load().chitu_b200_last_error().decode("utf-8", "replace")
    if rc == E_UNSUPPORTED:
        raise NotImplementedError(f"{what}: {msg}")
    if rc == E_INVALID:
        raise ValueError(f"{what}: {msg}")
    raise ChituB200Error(f"{what}: {msg}")
