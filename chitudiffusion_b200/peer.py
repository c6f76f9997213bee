"""Ulysses sequence/head exchange over peer-mapped GPU memory (one node, NVLink).

Replaces, for the pure-Ulysses layout, the three all-to-all calls before the attention kernel and
the one after it (chitu_diffusion/modules/attention/diffusion_attn_backend.py:778-781,825-828)
together with their pack/unpack copies (chitu_diffusion/core/distributed/comm_group.py:350-384):

* one pre-attention launch stores q, k and v (norm + rotary + cast fused) straight into every rank's
  ``[B, U*s, H/U, D]`` buffer - rank r's rows land at ``[r*s, (r+1)*s)`` of each peer - and announces them
  with an arrival flag per source rank; in push mode only q goes out that way, k and v for the peers are
  staged locally and delivered by copy CTAs inside the attention launch;
* the attention kernel waits per source rank for the rows it is about to read, its own rows first, and its
  epilogue stores each output row into its owner's ``[B, s, H, D]`` buffer (head columns
  ``[r*H/U, (r+1)*H/U)``); its last CTA announces the outputs;
* a one-warp launch waits for every rank's output flag, after which this rank's output is complete and the
  exchange buffers may be reused.  No barrier launch.

Buffers come from ``torch.distributed._symmetric_memory`` (device memory mapped into every process
of the group); the data path is plain peer stores from this library's kernels - no NCCL call, no
TMA from or to peer memory.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import ops
from .comm import CommGroup


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class PeerUlysses:
    """Exchange buffers and per-layer schedule for one ``(B, s, H, D, dtype)`` problem shape.

    Per layer: ONE pre-attention launch stores this rank's q / k / v rows into every peer and announces
    them (arrival flags, ``csrc/peer_sync.cuh``); the attention kernel's copy warp waits per source rank
    for exactly the rows it is about to load - its own rows first - and its last CTA (or the key-split
    merge kernel's) announces the output rows; a one-warp kernel waits for every rank's output flag.
    Three launches per layer (four when the keys are split), no barrier launch, no NCCL call.

    The q / k / v buffers need no double buffering: a rank announces its outputs only when its whole
    attention grid has finished, and nobody scatters the next layer before having seen every rank's
    output flag.  The output buffer alternates between two slots, so the tensor handed back stays valid
    until the call after next (the reference hands back a fresh tensor; no copy is made here).
    """

    def __init__(self, group: CommGroup, B: int, s: int, H: int, D: int, dtype: torch.dtype, device: torch.device,
                 prefix_rows: int = 0):
        """``prefix_rows`` > 0: the replicated-text layout (Qwen-Image): the gathered tensors start with
        ``prefix_rows`` rows that every rank produces itself (it keeps its own head group of them), the
        exchanged rows follow, and the prefix rows of the result are stored to every rank (``txt_out``)."""
        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib

        U = group.group_size
        if H % U:
            raise ValueError(f"head dim {H} must be divisible by CP size {U}")
        if U > 8:
            raise NotImplementedError("peer exchange supports at most 8 GPUs")
        self.group, self.U, self.rank = group, U, group.rank_in_group
        self.B, self.s, self.H, self.D, self.hc = B, s, H, D, H // U
        self.dtype, self.device = dtype, device
        self.T = T = int(prefix_rows)
        es = torch.empty((), dtype=dtype).element_size()
        self.es = es
        tile = B * (T + U * s) * self.hc * D * es  # one of q / k / v in the gathered layout
        out_bytes = _align(B * s * H * D * es) + _align(B * T * H * D * es)  # image rows, then the text rows
        self._txt_out_off = _align(B * s * H * D * es)
        self.off_q = 0
        self.off_k = _align(tile)
        self.off_v = self.off_k + _align(tile)
        self.off_out = self.off_v + _align(tile)  # two output slots
        self.off_flags = self.off_out + 2 * out_bytes
        self._out_bytes = out_bytes
        total = self.off_flags + 4 * _lib.SYNC_INTS
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group.gpu_group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        torch.cuda.synchronize(device)
        dist.barrier(group=group.gpu_group)  # every sync block is zero before anyone signals

        def view(off, shape):
            n = 1
            for d in shape:
                n *= d
            return self.buf[off : off + n * es].view(dtype).view(shape)

        gathered = (B, T + U * s, self.hc, D)
        self.q, self.k, self.v = view(self.off_q, gathered), view(self.off_k, gathered), view(self.off_v, gathered)
        self.outs = [view(self.off_out + i * out_bytes, (B, s, H, D)) for i in range(2)]
        self.txt_outs = [view(self.off_out + i * out_bytes + self._txt_out_off, (B, T, H, D)) for i in range(2)]
        self.out = self.outs[0]
        self._out_slot = 0
        self.flag_ptrs = [p + self.off_flags for p in self.ptrs]
        self.sync = _lib.peer_sync_desc(self.flag_ptrs, self.rank)
        # element strides (b, s, -, h) of the gathered layout; this rank's rows start at prefix + rank * s
        self.gather_strides = ((T + U * s) * self.hc * D, self.hc * D, 0, D)
        self._row_bytes = self.hc * D * es
        self._row0 = (T + self.rank * s) * self._row_bytes
        # key-split scratch owned by this object: graphs captured over it keep a valid address
        self.n_splits = ops.auto_key_splits(B, T + U * s, T + U * s, self.hc)
        need = ops.splitkv_workspace_bytes(B, T + U * s, self.hc, D, self.n_splits)
        self.workspace = torch.zeros(max(need, 16), dtype=torch.uint8, device=device) if self.n_splits > 1 else None
        # Push mode: only the query rows are stored straight to the peers; key and value rows for the peers are
        # staged locally, and copy CTAs inside the attention launch - the first CTAs of its grid - deliver them
        # while the attention already runs (``chitu_b200_attn_fwd_exchange_push``).  One batch entry only: a
        # staged block is the contiguous image of this rank's rows in a peer's buffer.
        self.push = None
        self.trace = None  # optional callable(point): 0 before the first launch of a layer, 1 after the last
        #                    staging / scatter launch, 2 after the attention launch(es), 3 after the wait
        self._layer_open = False
        import os

        # CHITU_B200_PUSH: "0" never; "1" (default) for grids of at most four waves - beyond that the transfer
        # is a small share of the call and the direct stores are kept; "force" always
        mode = os.environ.get("CHITU_B200_PUSH", "1")
        n_push = ops.push_ctas(B, U * s, self.hc, self.n_splits) if (B == 1 and T == 0 and mode != "0") else 0
        small = -(-(U * s) // 256) * self.hc * B * self.n_splits <= 4 * ops.NUM_SMS
        if n_push > 0 and (small or mode == "force"):
            block = s * self._row_bytes
            self._stage = torch.empty(3 * U * block, dtype=torch.uint8, device=device)
            self._stage_ptrs = [self._stage.data_ptr() + t * U * block for t in range(3)]
            self._block_bytes = block
            dests = [[p + off + self._row0 for p in self.ptrs] for off in (self.off_q, self.off_k, self.off_v)]
            self.push = _lib.push_desc([0] + self._stage_ptrs[1:], dests, block)

    def dest_ptrs(self, which: str, row_offset: int = 0, direct: bool = False):
        """Per-destination base addresses for this rank's rows (from local row ``row_offset`` on) of q / k / v.
        In push mode (unless ``direct``) the peers' entries point into the local staging area."""
        off = {"q": self.off_q, "k": self.off_k, "v": self.off_v}[which]
        ptrs = [p + off + self._row0 + row_offset * self._row_bytes for p in self.ptrs]
        if self.push is not None and not direct and which != "q":  # query rows go straight to the peers
            t = ("q", "k", "v").index(which)
            for d in range(self.U):
                if d != self.rank:
                    ptrs[d] = self._stage_ptrs[t] + d * self._block_bytes + row_offset * self._row_bytes
        return ptrs

    def barrier(self) -> None:
        ops.peer_barrier(self.flag_ptrs, self.rank, self.U, self.device)

    def scatter_plain(self, x: torch.Tensor, which: str = "v") -> None:
        """``x [B, s, H*D]`` (or ``[B,s,H,D]``) 16-bit: copy each head group to its owner (no announcement)."""
        flat = x.reshape(self.B, self.s, self.H * self.D)
        ops.qk_norm_rope(flat, self.H, None, 0.0, norm_mode=2, rope_mode=0, rope_table=None,
                         out_ptrs=self.dest_ptrs(which, direct=True), out_strides=self.gather_strides,
                         heads_per_group=self.hc, out_dtype=self.dtype)

    def scatter_qkv(self, jobs, v: torch.Tensor, row_offset: int = 0, last: bool = True, **batch_args) -> None:
        """One launch: the q and k jobs of a pre-attention object plus the plain scatter of ``v``.

        The jobs cover local rows ``[row_offset, row_offset + rows)`` (a layer whose streams are projected
        separately - Flux's text and image streams - scatters them with one call each).  The call with
        ``last=True`` announces the rank's rows of this layer to its peers.
        """
        jobs = [dict(j) for j in jobs]
        batch_args.pop("out_dtype", None)  # the exchange buffers fix the store type
        if self.trace is not None and not self._layer_open:
            self.trace(0)
        self._layer_open = not last
        rows = jobs[0]["x"].shape[1]
        if v.dtype == jobs[0]["x"].dtype:
            jobs.append(dict(x=v.reshape(self.B, rows, self.H * self.D), norm_mode=2, rope_mode=0))
        else:  # a launch shares one input dtype
            flat = v.reshape(self.B, rows, self.H * self.D)
            ops.qk_norm_rope(flat, self.H, None, 0.0, norm_mode=2, rope_mode=0, rope_table=None,
                             out_ptrs=self.dest_ptrs("v", row_offset), out_strides=self.gather_strides,
                             heads_per_group=self.hc, out_dtype=self.dtype)
        for j, which in zip(jobs, ("q", "k", "v")):
            j["out_ptrs"] = self.dest_ptrs(which, row_offset)
        ops.qk_norm_rope_batch(jobs, out_strides=self.gather_strides, heads_per_group=self.hc, out_dtype=self.dtype,
                               sync=self.sync if last else None, stage_only=self.push is not None, **batch_args)
        if self.trace is not None and last:
            self.trace(1)

    def scatter_ready(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
        """q, k, v ``[B, s, H, D]`` that are already normalised and rotated: one launch of three plain jobs."""
        jobs = [dict(x=t.reshape(self.B, self.s, self.H * self.D), norm_mode=2, rope_mode=0,
                     out_ptrs=self.dest_ptrs(w)) for t, w in ((q, "q"), (k, "k"), (v, "v"))]
        ops.qk_norm_rope_batch(jobs, num_heads=self.H, eps=0.0, rope_table=None, out_strides=self.gather_strides,
                               heads_per_group=self.hc, out_dtype=self.dtype, sync=self.sync,
                               stage_only=self.push is not None)

    def scatter_prefix(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
        """Replicated rows ``[B, T, H, D]`` (every rank holds the same ones): this rank's head group of them goes
        to rows ``[0, T)`` of its OWN buffers; the other head groups are dropped.  No announcement (local rows)."""
        jobs = []
        for t, which in ((q, "q"), (k, "k"), (v, "v")):
            off = {"q": self.off_q, "k": self.off_k, "v": self.off_v}[which]
            ptrs = [0] * self.U
            ptrs[self.rank] = self.ptrs[self.rank] + off
            jobs.append(dict(x=t.reshape(self.B, self.T, self.H * self.D), norm_mode=2, rope_mode=0, out_ptrs=ptrs))
        ops.qk_norm_rope_batch(jobs, num_heads=self.H, eps=0.0, rope_table=None, out_strides=self.gather_strides,
                               heads_per_group=self.hc, out_dtype=self.dtype)

    def attention_full_txt(self, n_valid: int, softmax_scale: Optional[float] = None):
        """Attention over ``[text | gathered image rows]``; keys past ``n_valid`` image rows (the zero-padded tail of
        the last shard) are never attended.  Returns ``(text result [B, T, H, D] for all heads, this rank's image
        rows [B, s, H, D])``, both valid until the call after next."""
        self._out_slot ^= 1
        slot_off = self.off_out + self._out_slot * self._out_bytes
        Sk = self.T + min(int(n_valid), self.U * self.s)
        ops.attn_fwd_exchange(
            self.q, self.k[:, :Sk], self.v[:, :Sk], [p + slot_off for p in self.ptrs], rows_per_dest=self.s,
            dest_batch_stride=self.s * self.H * self.D, dest_row_stride=self.H * self.D,
            dest_head_offset=self.rank * self.hc * self.D, rows_per_src=self.s, sync=self.sync,
            softmax_scale=softmax_scale, n_splits=self.n_splits, workspace=self.workspace,
            prefix_rows=self.T, prefix_ptrs=[p + slot_off + self._txt_out_off for p in self.ptrs],
            prefix_batch_stride=self.T * self.H * self.D, prefix_row_stride=self.H * self.D,
            prefix_head_offset=self.rank * self.hc * self.D,
        )
        ops.peer_wait_outputs(self.sync, self.device)
        self.out = self.outs[self._out_slot]
        return self.txt_outs[self._out_slot], self.out

    def attention(self, softmax_scale: Optional[float] = None) -> torch.Tensor:
        """Attention over the gathered q/k/v as their rows arrive, output rows stored to their owners, then the
        wait for every rank's outputs.  Returns this rank's ``[B, s, H, D]`` result (valid until the call after next)."""
        self._out_slot ^= 1
        slot_off = self.off_out + self._out_slot * self._out_bytes
        ops.attn_fwd_exchange(
            self.q, self.k, self.v, [p + slot_off for p in self.ptrs], rows_per_dest=self.s,
            dest_batch_stride=self.s * self.H * self.D, dest_row_stride=self.H * self.D,
            dest_head_offset=self.rank * self.hc * self.D, rows_per_src=self.s, sync=self.sync,
            softmax_scale=softmax_scale, n_splits=self.n_splits, workspace=self.workspace, push=self.push,
        )
        if self.trace is not None:
            self.trace(2)
        ops.peer_wait_outputs(self.sync, self.device)
        if self.trace is not None:
            self.trace(3)
        self.out = self.outs[self._out_slot]
        return self.out


def _runs(indices):
    """Sorted indices grouped into runs of consecutive values: [(first, count), ...]."""
    runs = []
    for i in sorted(indices):
        if runs and runs[-1][0] + runs[-1][1] == i:
            runs[-1] = (runs[-1][0], runs[-1][1] + 1)
        else:
            runs.append((i, 1))
    return runs


class PeerRing:
    """Ring / Ulysses x ring / all-gather-KV exchange over peer-mapped memory for one problem shape.

    Every rank publishes its (post-Ulysses) K/V block in a buffer mapped into all ranks of the CP
    group.  Where the reference rotates K/V with send/recv pairs
    (chitu_diffusion/modules/attention/diffusion_attn_backend.py:783-835: send to ``(r-U) % P``,
    receive from ``(r+U) % P``), ring step ``t`` here PULLS the block of rank ``(r + t*U) % P`` - the
    block that rotation delivers at step ``t`` - into local memory with the copy engines on a side
    stream while the attention kernel works on block ``t-1``; partial results merge with the
    log-sum-exp combine kernel.  ``mode="agkv"`` (the AGCP branch, :581-597) pulls every block into one
    ``[B, P*s, H, D]`` buffer, owners walked upwards from this rank, in three stages whose pulls run under
    the previous stage's attention call; stage results merge by log-sum-exp and the result is handed back in
    the backend's dtype.  No NCCL call is on the data path, so the whole call can be captured in a CUDA graph.
    """

    def __init__(self, group: CommGroup, ulysses: int, B: int, s: int, H: int, D: int, dtype: torch.dtype,
                 device: torch.device, mode: str = "ring", merger_factory=None, direction: int = 1):
        import torch.distributed._symmetric_memory as symm_mem

        P = group.group_size
        U = 1 if mode == "agkv" else ulysses
        if P > 8:
            raise NotImplementedError("peer exchange supports at most 8 GPUs")
        if P % U or H % U:
            raise ValueError(f"CP size {P} and head count {H} must be divisible by the Ulysses degree {U}")
        self.group, self.P, self.U, self.R, self.rank = group, P, U, P // U, group.rank_in_group
        self.mode, self.B, self.s, self.H, self.D, self.hc = mode, B, s, H, D, H // U
        self.dtype, self.device, self.merger_factory = dtype, device, merger_factory
        self.direction = 1 if direction >= 0 else -1  # -1: blocks arrive in the order of a send-to-next ring
        es = torch.empty((), dtype=dtype).element_size()
        self.es = es
        self.block_bytes = B * U * s * self.hc * D * es  # one of q / k / v of a ring block
        out_es = 4 if self.R > 1 else es                 # merged ring results are fp32, like the reference's
        self.off_q, self.off_k = 0, _align(self.block_bytes)
        self.off_v = self.off_k + _align(self.block_bytes)
        self.off_out = self.off_v + _align(self.block_bytes)
        self.off_flags = self.off_out + _align(B * s * H * D * out_es)
        self.buf = symm_mem.empty(self.off_flags + 256, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group.gpu_group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        torch.cuda.synchronize(device)
        dist.barrier(group=group.gpu_group)

        def view(off, shape, dt):
            n = 1
            for d in shape:
                n *= d
            return self.buf[off : off + n * torch.empty((), dtype=dt).element_size()].view(dt).view(shape)

        block = (B, U * s, self.hc, D)
        self.q, self.k, self.v = (view(o, block, dtype) for o in (self.off_q, self.off_k, self.off_v))
        self.out = view(self.off_out, (B, s, H, D), torch.float32 if self.R > 1 else dtype)
        self.flag_ptrs = [p + self.off_flags for p in self.ptrs]
        self.members = [(self.rank // U) * U + i for i in range(U)]  # this rank's Ulysses group, CP-group indices
        self.gather_strides = (U * s * self.hc * D, self.hc * D, 0, D)
        self._row0 = (self.rank % U) * s * self.hc * D * es
        self.side = torch.cuda.Stream(device=device)
        if mode == "agkv":
            self.k_full = torch.empty((B, P * s, H, D), dtype=dtype, device=device)
            self.v_full = torch.empty_like(self.k_full)
        elif self.R > 1:
            self.k_fetch = [torch.empty(block, dtype=dtype, device=device) for _ in range(2)]
            self.v_fetch = [torch.empty(block, dtype=dtype, device=device) for _ in range(2)]

    def dest_ptrs(self, which: str):
        """Per-destination base addresses (the members of this rank's Ulysses group) for its rows of q / k / v."""
        off = {"q": self.off_q, "k": self.off_k, "v": self.off_v}[which]
        return [self.ptrs[m] + off + self._row0 for m in self.members]

    def barrier(self) -> None:
        ops.peer_barrier(self.flag_ptrs, self.rank, self.P, self.device)

    def scatter_plain(self, x: torch.Tensor, which: str) -> None:
        flat = x.reshape(self.B, self.s, self.H * self.D)
        ops.qk_norm_rope(flat, self.H, None, 0.0, norm_mode=2, rope_mode=0, rope_table=None,
                         out_ptrs=self.dest_ptrs(which), out_strides=self.gather_strides,
                         heads_per_group=self.hc, out_dtype=self.dtype)

    def _pull(self, owner: int, off: int, dst: torch.Tensor) -> None:
        ops.peer_copy_2d(dst.data_ptr(), self.block_bytes, self.ptrs[owner] + off, self.block_bytes,
                         self.block_bytes, 1, self.device)

    def _attention_agkv(self, q, softmax_scale, cur) -> torch.Tensor:
        """All-gather-KV with the gather pipelined against the attention.

        Every rank walks the owners upwards from itself, so at any time each owner serves one puller (all
        ranks pulling from rank 0 first, then rank 1, ... shared one GPU's outgoing link eight ways: 7 ms
        instead of 2 for a 14B layer on 8 GPUs).  The walk is cut into stages - own block, the next half of
        the peers, the rest; while the attention kernel works on the keys of one stage, the copy engines
        pull the next.  Stage results merge by log-sum-exp and the last merge writes the 16-bit result: the
        all-gather mode hands back the backend's own dtype.  Two ranks: one stage pulled up front, one call.
        """
        P, r = self.P, self.rank
        row = self.s * self.H * self.D * self.es

        def pull(owner):
            for off, full in ((self.off_k, self.k_full), (self.off_v, self.v_full)):
                ops.peer_copy_2d(full.data_ptr() + owner * row, P * row, self.ptrs[owner] + off, row, row, self.B,
                                 self.device)

        order = [(r + t) % P for t in range(P)]
        if P <= 2:
            for owner in order:
                pull(owner)
            result = ops.attn_fwd(q, self.k_full, self.v_full, softmax_scale=softmax_scale)[0]
            self.barrier()  # nobody still reads this rank's published block
            return result
        cut = 1 + (P - 1 + 1) // 2
        stages = [order[:1], order[1:cut], order[cut:]]
        pull(order[0])
        merger = self.merger_factory()
        result = torch.empty(q.shape, dtype=self.dtype, device=self.device)
        last_call = (len(stages) - 1, len(_runs(stages[-1])) - 1)
        for i, stage in enumerate(stages):
            if i + 1 < len(stages):
                self.side.wait_stream(cur)  # (the pulls of the stage after this one start now)
                with torch.cuda.stream(self.side):
                    for owner in stages[i + 1]:
                        pull(owner)
            for j, (first, count) in enumerate(_runs(stage)):
                rows = slice(first * self.s, (first + count) * self.s)
                block_out, block_lse = ops.attn_fwd(q, self.k_full[:, rows], self.v_full[:, rows],
                                                    softmax_scale=softmax_scale, return_lse=True)
                if (i, j) == last_call and hasattr(merger, "add_final"):
                    merger.add_final(block_out, block_lse, result)
                else:
                    merger.add(block_out, block_lse)
            if i + 1 < len(stages):
                cur.wait_stream(self.side)
        if not hasattr(merger, "add_final"):
            result.copy_(merger.result())
        self.barrier()  # nobody still reads this rank's published block
        return result

    def attention(self, softmax_scale: Optional[float] = None, q: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Barrier, pulls + attention (+ merge, + hand-back to the sequence owners), barrier.

        ``q`` is the local query tensor when the Ulysses degree is 1 (queries are then not exchanged).
        """
        if q is None:
            q = self.q
        self.barrier()  # every block is published
        cur = torch.cuda.current_stream(self.device)
        if self.mode == "agkv":
            return self._attention_agkv(q, softmax_scale, cur)
        merger = self.merger_factory()
        k_t, v_t = self.k, self.v
        for t in range(self.R):
            nxt = None
            if t + 1 < self.R:
                owner = (self.rank + self.direction * (t + 1) * self.U) % self.P
                kb, vb = self.k_fetch[(t + 1) & 1], self.v_fetch[(t + 1) & 1]
                self.side.wait_stream(cur)  # the attention call that last read these two buffers is enqueued
                with torch.cuda.stream(self.side):
                    self._pull(owner, self.off_k, kb)
                    self._pull(owner, self.off_v, vb)
                nxt = (kb, vb)
            block_out, block_lse = ops.attn_fwd(q, k_t, v_t, softmax_scale=softmax_scale, return_lse=True)
            merger.add(block_out, block_lse)
            if nxt is not None:
                cur.wait_stream(self.side)
                k_t, v_t = nxt
        merged = merger.result()  # fp32 [B, U*s, H/U, D]
        if self.U == 1:
            self.barrier()
            return merged
        col0 = (self.rank % self.U) * self.hc * self.D * 4
        ops.scatter_rows(merged, [self.ptrs[m] + self.off_out + col0 for m in self.members], self.s,
                         self.s * self.H * self.D * 4, self.H * self.D * 4)
        self.barrier()  # all head groups of this rank's rows have arrived; nobody still reads its block
        return self.out
