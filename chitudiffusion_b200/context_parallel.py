"""Context-parallel attention: Ulysses all-to-all, ring K/V rotation, all-gather-KV.

Mirrors the surface of ``DiffusionAttention_with_CP``
(chitu_diffusion/modules/attention/diffusion_attn_backend.py:449-1203): same
constructor, same ``__call__`` signature returning ``(out_local, None, None)``,
``uses_agcp()``, ``supports_fused_overlap()``, ``attention_fused()``,
``cp_attn_with_full_txt()`` and ``cp_attn_with_full_txt_fused()``, the ``attn``,
``ulysses_limit``, ``group``, ``cp_size`` and ``cp_backend`` attributes.

What differs is the schedule, not the result:

* the ring K/V exchange is posted on a side stream before the attention kernel
  of the current block is enqueued, into double-buffered receive tensors, so
  the NVLink transfer runs under the tensor-core work;
* partial results are merged by one fused kernel per step, in the Ulysses
  layout, and exchanged back ONCE after the last ring step (the reference
  exchanges and merges in fp32 after every step; the merge is element-wise per
  (token, head), so merging before the exchange gives the same numbers);
* all-gather-KV lands directly in the ``[B, P*s, H, D]`` buffer.
"""

from __future__ import annotations

import os
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from .comm import CommGroup, get_cp_group, get_up_group


class _KernelMerger:
    """Running (out, lse) accumulator backed by the fused LSE-combine kernel."""

    def __init__(self):
        self.out: Optional[torch.Tensor] = None
        self.lse: Optional[torch.Tensor] = None

    def add(self, block_out: torch.Tensor, block_lse: torch.Tensor) -> None:
        from . import ops

        first = self.out is None
        if first:
            self.out = torch.empty(block_out.shape, dtype=torch.float32, device=block_out.device)
            B, S, H, _ = block_out.shape
            self.lse = torch.empty((B, S, H, 1), dtype=torch.float32, device=block_out.device)
        ops.lse_combine(self.out, self.lse, block_out, block_lse, first=first)

    def add_final(self, block_out: torch.Tensor, block_lse: torch.Tensor, final_out: torch.Tensor) -> None:
        """The last block of a call: the merged rows are also written to ``final_out`` in its (16-bit) dtype."""
        from . import ops

        first = self.out is None
        if first:
            self.out = torch.empty(block_out.shape, dtype=torch.float32, device=block_out.device)
            B, S, H, _ = block_out.shape
            self.lse = torch.empty((B, S, H, 1), dtype=torch.float32, device=block_out.device)
        ops.lse_combine(self.out, self.lse, block_out, block_lse, first=first, final_out=final_out)

    def result(self) -> torch.Tensor:
        return self.out


class B200ContextParallel:
    """Drop-in for ``DiffusionAttention_with_CP`` built on the b200 backend and NCCL over NVLink."""

    def __init__(
        self,
        attn,
        ulysses_limit: int,
        ring_cudagraph: bool = False,
        cp_backend: str = "ucp",
        group: Optional[CommGroup] = None,
        up_group_lookup: Optional[Callable[[int], CommGroup]] = None,
        merger_factory: Optional[Callable[[], object]] = None,
    ):
        self.attn = attn
        self.ulysses_limit = ulysses_limit
        self.group = group if group is not None else get_cp_group()
        self.cp_size = self.group.group_size
        self.global_rank = dist.get_rank() if dist.is_initialized() else 0
        self.local_chunk_id = self.group.rank_in_group
        self.use_ring_cudagraph = bool(ring_cudagraph)
        self.cp_backend = self._validate_cp_backend(cp_backend)
        self._up_group_lookup = up_group_lookup or get_up_group
        self._merger_factory = merger_factory or _KernelMerger
        self._comm_stream: Optional[torch.cuda.Stream] = None
        self._graph_cache: dict = {}
        # pure-Ulysses exchange over peer-mapped memory instead of NCCL all-to-all (CUDA, one node,
        # at most 8 ranks); "nccl" keeps the collective form
        self.ulysses_exchange = os.environ.get("CHITU_B200_ULYSSES_EXCHANGE", "peer").strip().lower()
        self._peer_cache: dict = {}

    # ------------------------------------------------------------------ knobs
    @staticmethod
    def _validate_cp_backend(cp_backend: str) -> str:
        mode = str(cp_backend or "ucp").strip().lower()
        if mode not in {"agcp", "ucp"}:
            raise ValueError(f"Resolved CP backend must be one of agcp, ucp; got {cp_backend!r}.")
        return mode

    def uses_agcp(self) -> bool:
        return self.cp_backend == "agcp"

    def _split(self) -> Tuple[int, int]:
        """``(ulysses_size, ring_steps)`` as at diffusion_attn_backend.py:571-572."""
        u = self.cp_size if self.cp_size <= self.ulysses_limit else self.ulysses_limit
        return u, self.cp_size // u

    def supports_fused_overlap(self, *, use_varlen: bool = False, return_attn_probs: bool = False,
                               num_heads: Optional[int] = None) -> bool:
        u, r = self._split()
        return (
            self.cp_size > 1 and self.cp_size % u == 0 and not self.uses_agcp() and not use_varlen and r == 1
            and u > 1 and not return_attn_probs and torch.cuda.is_available()
            and (num_heads is None or num_heads % u == 0)
        )

    def _side_stream(self, device) -> Optional["torch.cuda.Stream"]:
        if device.type != "cuda":
            return None
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=device)
        return self._comm_stream

    # ------------------------------------------------------------------ main entry
    def __call__(
        self,
        q: torch.Tensor,
        k: torch.Tensor,
        v: torch.Tensor,
        cu_seqlens_q: Optional[torch.Tensor] = None,
        cu_seqlens_k: Optional[torch.Tensor] = None,
        max_seqlen_q: Optional[int] = None,
        max_seqlen_k: Optional[int] = None,
        dropout_p: float = 0,
        softmax_scale: Optional[float] = None,
        causal: bool = False,
        window_size: Tuple[int, int] = (-1, -1),
        deterministic: bool = False,
        return_attn_probs: bool = False,
    ):
        result = self._call(q, k, v, cu_seqlens_q, cu_seqlens_k, dropout_p, softmax_scale, causal, window_size,
                            deterministic)
        if q.is_cuda:
            from . import ops

            ops.poll_status(q.device)  # a barrier or kernel wait that timed out raises here, one call later at most
        return result

    def _call(self, q, k, v, cu_seqlens_q, cu_seqlens_k, dropout_p, softmax_scale, causal, window_size,
              deterministic):
        u, r = self._split()
        if r > 1 and getattr(self.attn, "impl", "") in {"sage", "sparge", "b200_q8"}:
            raise NotImplementedError(
                f"{self.attn.impl} context parallelism currently supports Ulysses only; "
                f"set infer.diffusion.up equal to cp_size ({self.cp_size})."
            )
        if cu_seqlens_q is not None or cu_seqlens_k is not None:
            raise NotImplementedError("b200 context parallelism does not support varlen attention.")
        kw = dict(dropout_p=dropout_p, softmax_scale=softmax_scale, causal=causal, window_size=window_size,
                  deterministic=deterministic)
        if self.uses_agcp():
            if self._peer_ok(q, k, kw):
                ring = self.peer_ring(q, "agkv")
                ring.scatter_plain(k, "k")
                ring.scatter_plain(v, "v")
                return ring.attention(kw["softmax_scale"], q=q), None, None
            k_full = self.group.all_gather_sequence(k)
            v_full = self.group.all_gather_sequence(v)
            out = self.attn(q, k_full, v_full, return_attn_probs=False, **kw)[0]
            return out, None, None
        if (self.use_ring_cudagraph and self.cp_size > 1 and q.is_cuda and not self.uses_agcp()
                and self._capturable(q, k, u, r, kw)):
            return self._cp_forward_graphed(q, k, v, u, r, kw), None, None
        return self._cp_forward(q, k, v, u, r, kw), None, None

    # ------------------------------------------------------------------ whole-call CUDA graph
    def _capturable(self, q, k, u: int, r: int, kw: dict) -> bool:
        """Only exchanges made of this library's own kernels over peer memory are captured.

        A captured NCCL send/recv ring (what the reference captures) did not complete in a 2-GPU run
        on B200 with torch 2.11 / NCCL 2.28, so layouts that still go through NCCL run eagerly even
        when ``ring_cudagraph`` is set.
        """
        return self._use_peer(q, k, u, r, kw) or self._use_peer_ring(q, k, u, r, kw)

    def _cp_forward_graphed(self, q, k, v, u: int, r: int, kw: dict) -> torch.Tensor:
        """Capture the whole exchange + attention + exchange-back once per problem and replay it.

        Mirror of ``_cp_forward_graphed`` (diffusion_attn_backend.py:1154-1203): the graph is keyed by
        shapes, dtype, ``causal`` and ``softmax_scale``; inputs are copied into static buffers, the
        static result is cloned out so that the next replay may overwrite it.  Everything inside is
        capturable: the kernels take their workspace from torch's allocator, device waits are bounded
        and report through the status word, and the peer barrier keeps its epoch on the device.
        """
        key = (tuple(q.shape), tuple(k.shape), tuple(v.shape), q.dtype, bool(kw["causal"]), kw["softmax_scale"])
        entry = self._graph_cache.get(key)
        if entry is None:
            sq, sk, sv = q.clone(), k.clone(), v.clone()
            cur = torch.cuda.current_stream(q.device)
            warm = torch.cuda.Stream(device=q.device)
            warm.wait_stream(cur)
            with torch.cuda.stream(warm):  # sets up communicators, peer buffers and the side stream
                for _ in range(3):
                    self._cp_forward(sq, sk, sv, u, r, kw)
            cur.wait_stream(warm)
            torch.cuda.synchronize(q.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_out = self._cp_forward(sq, sk, sv, u, r, kw)
            torch.cuda.synchronize(q.device)
            entry = dict(graph=graph, q=sq, k=sk, v=sv, out=static_out)
            self._graph_cache[key] = entry
        entry["q"].copy_(q)
        entry["k"].copy_(k)
        entry["v"].copy_(v)
        entry["graph"].replay()
        return entry["out"].clone()

    # ------------------------------------------------------------------ Ulysses x ring
    def _ring_peers(self, u: int) -> Tuple[int, int]:
        """(destination, source) inside the CP group: send to ``(r-U) % P``, receive from ``(r+U) % P``."""
        r = self.local_chunk_id
        return (r - u) % self.cp_size, (r + u) % self.cp_size

    def _post_ring_exchange(self, k, v, u, side):
        """Post the K/V rotation; returns ``(next_k, next_v, done)``, ``done()`` makes them usable."""
        dst, src = self._ring_peers(u)
        k, v = k.contiguous(), v.contiguous()
        nk, nv = torch.empty_like(k), torch.empty_like(v)
        g = self.group
        if side is not None:
            side.wait_stream(torch.cuda.current_stream(k.device))
            with torch.cuda.stream(side):
                g.p2p_isend(k, dst)
                g.p2p_irecv(None, None, src, out=nk)
                g.p2p_isend(v, dst)
                g.p2p_irecv(None, None, src, out=nv)
                g.p2p_commit()
                g.p2p_wait()
            for t in (k, v, nk, nv):
                t.record_stream(side)

            def done():
                torch.cuda.current_stream(k.device).wait_stream(side)
        else:
            g.p2p_isend(k, dst)
            g.p2p_irecv(None, None, src, out=nk)
            g.p2p_isend(v, dst)
            g.p2p_irecv(None, None, src, out=nv)
            g.p2p_commit()

            def done():
                g.p2p_wait()
        return nk, nv, done

    def peer_exchange(self, B: int, s: int, H: int, D: int, dtype: torch.dtype, device: torch.device,
                      prefix_rows: int = 0):
        """Cached peer-store exchange for one problem shape (collective on first use: every rank must call it)."""
        from .peer import PeerUlysses

        key = (B, s, H, D, dtype, str(device), prefix_rows)
        px = self._peer_cache.get(key)
        if px is None:
            u, _ = self._split()
            px = PeerUlysses(self._up_group_lookup(u), B, s, H, D, dtype, device, prefix_rows=prefix_rows)
            self._peer_cache[key] = px
        return px

    def peer_ring(self, q: torch.Tensor, mode: str):
        """Cached peer-memory ring / all-gather-KV exchange for one problem shape (collective on first use)."""
        from .peer import PeerRing

        B, s, H, D = q.shape
        key = (mode, B, s, H, D, q.dtype, str(q.device))
        ring = self._peer_cache.get(key)
        if ring is None:
            u, _ = self._split()
            ring = PeerRing(self.group, u, B, s, H, D, q.dtype, q.device, mode=mode,
                            merger_factory=self._merger_factory)
            self._peer_cache[key] = ring
        return ring

    def _peer_ok(self, q, k, kw: dict) -> bool:
        """The exchange may run over peer-mapped memory with this library's kernels (one node, <= 8 GPUs)."""
        return (
            self.ulysses_exchange == "peer" and 1 < self.cp_size <= 8 and q.is_cuda
            and getattr(self.attn, "impl", "") == "b200" and q.shape == k.shape
            and q.dtype in (torch.bfloat16, torch.float16) and not kw["causal"] and not kw["dropout_p"]
            and tuple(kw["window_size"]) == (-1, -1)
        )

    def _use_peer(self, q, k, u: int, r: int, kw: dict) -> bool:
        return r == 1 and u > 1 and q.shape[2] % u == 0 and self._peer_ok(q, k, kw)

    def _use_peer_ring(self, q, k, u: int, r: int, kw: dict) -> bool:
        return r > 1 and self.cp_size == u * r and q.shape[2] % u == 0 and self._peer_ok(q, k, kw)

    def _cp_forward(self, q, k, v, u: int, r: int, kw: dict) -> torch.Tensor:
        if self._use_peer(q, k, u, r, kw):
            B, s, H, D = q.shape
            px = self.peer_exchange(B, s, H, D, q.dtype, q.device)
            px.scatter_ready(q, k, v)
            # the result lives in one of the exchange object's two output slots: valid until the call
            # after next (the reference hands back a fresh tensor; a DiT block consumes it at once)
            return px.attention(kw["softmax_scale"])
        if self._use_peer_ring(q, k, u, r, kw):
            ring = self.peer_ring(q, "ring")
            if u > 1:
                ring.scatter_plain(q, "q")
            ring.scatter_plain(k, "k")
            ring.scatter_plain(v, "v")
            out = ring.attention(kw["softmax_scale"], q=None if u > 1 else q)
            return out.clone() if u > 1 else out
        up_group = self._up_group_lookup(u) if u > 1 else None
        if up_group is not None:
            q = up_group.all_to_all(q, 2, 1)
            k = up_group.all_to_all(k, 2, 1)
            v = up_group.all_to_all(v, 2, 1)
        if r == 1:
            out = self.attn(q, k, v, return_attn_probs=False, **kw)[0]
        else:
            side = self._side_stream(q.device)
            merger = self._merger_factory()
            for step in range(r):
                pending = None
                if step + 1 != r:
                    pending = self._post_ring_exchange(k, v, u, side)
                block_out, block_lse, _ = self.attn(q, k, v, return_attn_probs=True, **kw)
                merger.add(block_out, block_lse)
                if pending is not None:
                    k, v, done = pending
                    done()
            out = merger.result()  # fp32, like the reference's merged result
        if up_group is not None:
            out = up_group.all_to_all(out, 1, 2)
        return out

    # ------------------------------------------------------------------ projections in, attention out
    def attention_from_projections(self, jobs, v_proj: torch.Tensor, *, row_offset: int = 0, last: bool = True,
                                   softmax_scale: Optional[float] = None, **batch_args):
        """Pre-attention transform and context-parallel attention of one layer in one go.

        ``jobs`` are the q and k jobs of ``ops.qk_norm_rope_batch`` (projection output ``[B, rows, H*D]``,
        norm weight, norm / rotary modes), ``v_proj`` the value projection, ``batch_args`` the shared
        arguments (``num_heads``, ``eps``, ``rope_table``, ``grid``, ``axis_split``, ``pos_offset``, ``round_mid``:
        what ``WanPreAttention.batch_args`` / ``JointPreAttention.batch_args`` return).  On the
        pure-Ulysses peer path the transform's stores ARE the head/sequence exchange: RMSNorm, rotary and
        cast are written straight into the peers' buffers, the attention kernel picks the rows up as
        they arrive.  It is the fused form of what ``WanSelfAttention.forward`` does between the QKV
        projection and ``attn_func`` (chitu_diffusion/models/model_wan.py:152-156,194-203).  Other layouts
        run the transform locally and go through ``__call__``.

        A layer whose rows are projected in several pieces (Flux's text and image streams) calls this
        once per piece with ``row_offset`` and ``last=False`` on all but the final piece; only the final
        call returns the attention output ``[B, s, H, D]`` (``None`` before).
        """
        from . import ops

        pieces = getattr(self, "_pending_pieces", None) or []
        pieces.append((jobs, v_proj, row_offset, dict(batch_args)))
        self._pending_pieces = pieces
        if not last:
            return None
        self._pending_pieces = []
        x0 = jobs[0]["x"]
        B, _, C = x0.shape
        num_heads = int(batch_args["num_heads"])
        D = C // num_heads
        s_total = max(off + jb[0]["x"].shape[1] for jb, _, off, _ in pieces)
        dtype = batch_args.get("out_dtype", torch.bfloat16)
        u, r = self._split()
        kw = dict(dropout_p=0.0, softmax_scale=softmax_scale, causal=False, window_size=(-1, -1), deterministic=False)
        probe = torch.empty((B, 0, num_heads, D), dtype=dtype, device=x0.device)
        if (not self.uses_agcp() and r == 1 and u > 1 and num_heads % u == 0 and x0.is_cuda
                and self._peer_ok(probe, probe, kw)):
            px = self.peer_exchange(B, s_total, num_heads, D, dtype, x0.device)
            for i, (jb, vp, off, args) in enumerate(pieces):
                px.scatter_qkv(jb, vp, row_offset=off, last=(i + 1 == len(pieces)), **args)
            out = px.attention(softmax_scale)
            ops.poll_status(x0.device)
            return out
        from .pre_attention import transform_pieces

        q, k, v = transform_pieces(pieces, dtype)
        return self(q, k, v, softmax_scale=softmax_scale)[0]

    # ------------------------------------------------------------------ producer-callback form
    @torch.compiler.disable
    def attention_fused(self, *, produce_q, produce_k, produce_v, dropout_p: float = 0.0,
                        softmax_scale: Optional[float] = None, causal: bool = False,
                        window_size: Tuple[int, int] = (-1, -1), deterministic: bool = False,
                        return_attn_probs: bool = False, num_heads: Optional[int] = None):
        """Pure-Ulysses schedule with projection/exchange overlap.

        Same contract as diffusion_attn_backend.py:638-737: the three callables each return a
        contiguous ``[B,s,H,D]`` tensor; K's exchange runs on the side stream while V is produced,
        V's while Q is produced.
        """
        if not self.supports_fused_overlap(return_attn_probs=return_attn_probs, num_heads=num_heads):
            q, k, v = produce_q(), produce_k(), produce_v()
            return self(q, k, v, dropout_p=dropout_p, softmax_scale=softmax_scale, causal=causal,
                        window_size=window_size, deterministic=deterministic, return_attn_probs=return_attn_probs)
        u, _ = self._split()
        kw = dict(dropout_p=dropout_p, softmax_scale=softmax_scale, causal=causal, window_size=window_size,
                  deterministic=deterministic)
        k = produce_k()
        if self._use_peer(k, k, u, 1, kw):
            # peer-store exchange: the three tensors go out in one launch whose stores are the exchange;
            # there is no collective left to hide behind the projections, so the producers simply run
            v, q = produce_v(), produce_q()
            B, s, H, D = q.shape
            px = self.peer_exchange(B, s, H, D, q.dtype, q.device)
            px.scatter_ready(q, k, v)
            out = px.attention(softmax_scale)
            from . import ops

            ops.poll_status(q.device)
            return out, None, None
        up_group = self._up_group_lookup(u)
        side = self._side_stream(k.device)
        cur = torch.cuda.current_stream(k.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            k_x = up_group.all_to_all(k, 2, 1)
        k.record_stream(side)
        v = produce_v()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            v_x = up_group.all_to_all(v, 2, 1)
        v.record_stream(side)
        q = produce_q()
        q_x = up_group.all_to_all(q, 2, 1)
        cur.wait_stream(side)
        for t in (k_x, v_x):
            t.record_stream(cur)
        out = self.attn(q_x, k_x, v_x, return_attn_probs=False, **kw)[0]
        return up_group.all_to_all(out, 1, 2), None, None

    # ------------------------------------------------------------------ replicated text + sharded image
    @torch.compiler.disable
    def cp_attn_with_full_txt(self, txt_q, txt_k, txt_v, img_q, img_k, img_v, *, image_seq_len: Optional[int] = None,
                              dropout_p: float = 0.0, softmax_scale: Optional[float] = None, causal: bool = False,
                              window_size: Tuple[int, int] = (-1, -1), deterministic: bool = False):
        """Qwen-Image layout: text replicated on every rank, image tokens sharded.

        Same contract as diffusion_attn_backend.py:839-984; returns ``(text output for all heads,
        local image output)``.  ``image_seq_len`` is the unpadded image length: keys past it are
        dropped, never attended.
        """
        if causal:
            raise NotImplementedError("Qwen full-text CP attention only supports non-causal attention.")
        kw = dict(dropout_p=dropout_p, softmax_scale=softmax_scale, causal=False, window_size=window_size,
                  deterministic=deterministic)
        txt_len = txt_q.shape[1]
        if self.cp_size <= 1:
            out = self.attn(torch.cat([txt_q, img_q], 1), torch.cat([txt_k, img_k], 1), torch.cat([txt_v, img_v], 1),
                            return_attn_probs=False, **kw)[0]
            return out[:, :txt_len], out[:, txt_len:]
        if self.uses_agcp():
            n_img = int(image_seq_len if image_seq_len is not None else img_k.shape[1] * self.cp_size)
            k_img = self.group.all_gather_sequence(img_k)[:, :n_img]
            v_img = self.group.all_gather_sequence(img_v)[:, :n_img]
            out = self.attn(torch.cat([txt_q, img_q], 1), torch.cat([txt_k, k_img], 1), torch.cat([txt_v, v_img], 1),
                            return_attn_probs=False, **kw)[0]
            return out[:, :txt_len], out[:, txt_len:]

        u, r = self._split()
        if r > 1 and getattr(self.attn, "impl", "") in {"sage", "sparge", "torch_sdpa_math", "b200_q8"}:
            raise NotImplementedError(f"{self.attn.impl} cannot provide LSE for Qwen full-text ring attention.")
        if (self._use_peer(img_q, img_k, u, r, kw) and txt_q.dtype == img_q.dtype and txt_q.shape[1] % 8 == 0
                and txt_q.shape[0] == img_q.shape[0]):
            # Pure Ulysses over peer memory: every rank keeps its own head group of the (replicated) text rows
            # in front of the gathered image rows; the attention kernel reads the text rows at once and the
            # image rows as they arrive, never attends the zero-padded tail, returns each image row to its
            # owner and stores the text rows of its heads to every rank.  Four launches, no NCCL call.
            B, s, H, D = img_q.shape
            n_img = int(image_seq_len if image_seq_len is not None else s * self.cp_size)
            px = self.peer_exchange(B, s, H, D, img_q.dtype, img_q.device, prefix_rows=txt_len)
            px.scatter_prefix(txt_q, txt_k, txt_v)
            px.scatter_ready(img_q, img_k, img_v)
            txt_out, img_out = px.attention_full_txt(n_img, softmax_scale)
            from . import ops

            ops.poll_status(img_q.device)
            return txt_out, img_out
        up_group = None
        if u > 1:
            up_group = self._up_group_lookup(u)
            ur = up_group.rank_in_group
            txt_q, txt_k, txt_v = (torch.tensor_split(t, u, 2)[ur].contiguous() for t in (txt_q, txt_k, txt_v))
            img_q = up_group.all_to_all(img_q, 2, 1)
            img_k = up_group.all_to_all(img_k, 2, 1)
            img_v = up_group.all_to_all(img_v, 2, 1)
        n_img = int(image_seq_len if image_seq_len is not None else img_k.shape[1] * self.cp_size)
        local0 = img_q.shape[1] // u if u > 1 else img_q.shape[1]
        block_seq = img_k.shape[1]
        local_img_len = img_q.shape[1]
        q = torch.cat([txt_q, img_q], dim=1)
        side = self._side_stream(q.device)
        merger = self._merger_factory() if r > 1 else None
        out = None
        cur_k, cur_v = img_k, img_v
        ring_block = self.local_chunk_id // u
        for step in range(r):
            owner = (ring_block + step) % r
            valid = max(0, min(cur_k.shape[1], n_img - owner * block_seq))
            pending = None
            if step + 1 != r:
                pending = self._post_ring_exchange(cur_k, cur_v, u, side)
            if step == 0:
                bk = torch.cat([txt_k, cur_k[:, :valid]], dim=1)
                bv = torch.cat([txt_v, cur_v[:, :valid]], dim=1)
            else:
                bk, bv = cur_k[:, :valid], cur_v[:, :valid]
            if bk.shape[1] > 0:
                bo, bl, _ = self.attn(q, bk, bv, return_attn_probs=r > 1, **kw)
                if r == 1:
                    out = bo
                else:
                    merger.add(bo, bl)
            if pending is not None:
                cur_k, cur_v, done = pending
                done()
        if merger is not None:
            out = merger.result()
        if out is None:
            raise RuntimeError("Qwen full-text CP attention produced no output blocks.")
        txt_out = out[:, :txt_len]
        img_out = out[:, txt_len : txt_len + local_img_len]
        if up_group is not None:
            img_out = up_group.all_to_all(img_out.contiguous(), 1, 2)[:, :local0]
            txt_c = txt_out.contiguous()
            gathered = torch.empty((u * txt_c.shape[0],) + tuple(txt_c.shape[1:]), dtype=txt_c.dtype,
                                   device=txt_c.device)
            dist.all_gather_into_tensor(gathered, txt_c, group=up_group.gpu_group)
            gathered = gathered.view((u,) + tuple(txt_c.shape))
            txt_out = gathered.permute(1, 2, 0, 3, 4).reshape(txt_c.shape[0], txt_c.shape[1], -1, txt_c.shape[3])
        return txt_out, img_out

    @torch.compiler.disable
    def cp_attn_with_full_txt_fused(self, *, produce_txt_q, produce_txt_k, produce_txt_v, produce_img_q,
                                    produce_img_k, produce_img_v, image_seq_len: Optional[int] = None,
                                    dropout_p: float = 0.0, softmax_scale: Optional[float] = None,
                                    causal: bool = False, window_size: Tuple[int, int] = (-1, -1),
                                    deterministic: bool = False, num_heads: Optional[int] = None):
        """Producer-callback form of :meth:`cp_attn_with_full_txt` (diffusion_attn_backend.py:987-1065)."""
        return self.cp_attn_with_full_txt(
            produce_txt_q(), produce_txt_k(), produce_txt_v(), produce_img_q(), produce_img_k(), produce_img_v(),
            image_seq_len=image_seq_len, dropout_p=dropout_p, softmax_scale=softmax_scale, causal=causal,
            window_size=window_size, deterministic=deterministic,
        )


# The name models and adapters of the reference import.
DiffusionAttention_with_CP = B200ContextParallel
