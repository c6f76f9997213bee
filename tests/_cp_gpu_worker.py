"""Multi-GPU worker (launched by tests/test_gpu_cp.py under torchrun, one rank per GPU, NCCL).

Checks, against single-process fp32 attention from the CPU oracle on the same seeded tensors:
the NCCL context-parallel layouts (Ulysses, ring, Ulysses x ring, all-gather-KV) through
``B200ContextParallel`` with the b200 kernel, and the peer-store Ulysses exchange (``PeerUlysses``).
"""

import faulthandler
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from chitudiffusion_b200 import B200AttnBackend, comm, ops  # noqa: E402
from chitudiffusion_b200.context_parallel import B200ContextParallel  # noqa: E402
from chitudiffusion_b200.peer import PeerUlysses  # noqa: E402
from chitudiffusion_b200.pre_attention import WanPreAttention  # noqa: E402

REL = 2e-2


def rel_err(a, ref):
    return (a.float().cpu() - ref).abs().max().item() / ref.abs().max().item()


def main():
    # a rank that stops making progress dumps its stack and exits instead of waiting for the caller's timeout
    faulthandler.dump_traceback_later(240, exit=True)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    H, D, s = 8, 128, 200
    S = s * world
    gen = torch.Generator().manual_seed(7)
    q, k, v = ((torch.randn(1, S, H, D, generator=gen)).to(torch.bfloat16) for _ in range(3))
    full = oracle.sdpa_fp32(q, k, v)
    sl = slice(rank * s, (rank + 1) * s)
    ql, kl, vl = (t[:, sl].contiguous().to(dev) for t in (q, k, v))
    backend = B200AttnBackend("b200")
    results = {}
    layouts = [("ulysses_peer", world, "ucp"), ("ulysses_nccl", world, "ucp"), ("ring_peer", 1, "ucp"),
               ("ring_nccl", 1, "ucp"), ("agcp_peer", world, "agcp"), ("agcp_nccl", world, "agcp")]
    if world >= 4:
        layouts += [("usp_peer", world // 2, "ucp"), ("usp_nccl", world // 2, "ucp")]
    for name, up, cpb in layouts:
        comm.destroy_diffusion_parallel_groups()
        comm.initialize_diffusion_parallel_groups(1, world, up)
        wrapper = B200ContextParallel(backend, up, cp_backend=cpb)
        if name.endswith("_nccl"):
            wrapper.ulysses_exchange = "nccl"
        out = wrapper(ql, kl, vl)[0]
        if name.endswith("_peer"):  # second call reuses the exchange buffers
            assert wrapper._peer_cache, name
            out = wrapper(ql, kl, vl)[0]
        results[name] = rel_err(out, full[:, sl])
        print(f"rank {rank}: {name} done", flush=True)

    # whole-call CUDA graph (ring_cudagraph=True): capture once, replay on new inputs
    q2, k2, v2 = ((torch.randn(1, S, H, D, generator=gen)).to(torch.bfloat16) for _ in range(3))
    full2 = oracle.sdpa_fp32(q2, k2, v2)
    ql2, kl2, vl2 = (t[:, sl].contiguous().to(dev) for t in (q2, k2, v2))
    graphed = [("graph_ulysses", world), ("graph_ring", 1)] + ([("graph_usp", world // 2)] if world >= 4 else [])
    for name, up in graphed:
        comm.destroy_diffusion_parallel_groups()
        comm.initialize_diffusion_parallel_groups(1, world, up)
        wrapper = B200ContextParallel(backend, up, ring_cudagraph=True)
        first = wrapper(ql, kl, vl)[0]
        second = wrapper(ql2, kl2, vl2)[0]  # replay of the captured graph
        assert len(wrapper._graph_cache) == 1
        results[name] = max(rel_err(first, full[:, sl]), rel_err(second, full2[:, sl]))
        print(f"rank {rank}: {name} done", flush=True)

    # stand-alone graphed ring (send-to-next order, GQA keys / values) and the image-CP core
    from chitudiffusion_b200.graphed_ring import B200GraphedRingAttention
    from chitudiffusion_b200.image_cp import B200ImageContextParallel

    comm.destroy_diffusion_parallel_groups()
    comm.initialize_diffusion_parallel_groups(1, world, world)
    kg, vg = ((torch.randn(1, S, H // 2, D, generator=gen)).to(torch.bfloat16) for _ in range(2))
    full_gqa = oracle.sdpa_fp32(q, kg.repeat_interleave(2, dim=2), vg.repeat_interleave(2, dim=2))
    ring = B200GraphedRingAttention(comm.get_cp_group(), use_cuda_graph=True)
    o1 = ring(ql, kg[:, sl].contiguous().to(dev), vg[:, sl].contiguous().to(dev))
    o2 = ring(ql, kl, vl)
    o3 = ring(ql, kl, vl)  # replay
    assert o1.dtype == torch.bfloat16 and len(ring._graph_cache) == 1  # GQA keys are broadcast before the graph key is formed
    results["graphed_ring"] = max(rel_err(o1, full_gqa[:, sl]), rel_err(o2, full[:, sl]), rel_err(o3, full[:, sl]))
    print(f"rank {rank}: graphed_ring done", flush=True)
    txt = [(torch.randn(1, 24, H, D, generator=gen)).to(torch.bfloat16) for _ in range(3)]
    full_it = oracle.sdpa_fp32(torch.cat([txt[0], q], 1), torch.cat([txt[1], k], 1), torch.cat([txt[2], v], 1))
    for mode in ("ulysses", "ring", "agkv"):
        core = B200ImageContextParallel(backend, mode=mode)
        core.enable(comm.get_cp_group())
        t_out, i_out = core.attention(*(t.to(dev) for t in txt), ql, kl, vl)
        results[f"imagecp_{mode}"] = max(rel_err(t_out, full_it[:, :24]), rel_err(i_out, full_it[:, 24:][:, sl]))
    print(f"rank {rank}: imagecp done", flush=True)
    # replicated text + sharded image with a zero-padded tail (the Qwen-Image layout), Ulysses over peer memory:
    # text rows kept locally, image rows exchanged, padded keys never attended, text result stored to every rank
    n_img = S - 5
    iq, ik, iv = (t[:, :n_img] for t in (q, k, v))
    full_pad = oracle.sdpa_fp32(torch.cat([txt[0], iq], 1), torch.cat([txt[1], ik], 1), torch.cat([txt[2], iv], 1))
    shards = [oracle.split_sequence_padding(t, world, 1)[rank].contiguous().to(dev) for t in (iq, ik, iv)]
    ls = shards[0].shape[1]
    wrapper = B200ContextParallel(backend, world, cp_backend="ucp")
    for rep in range(2):
        t_out, i_out = wrapper.cp_attn_with_full_txt(*(t.to(dev) for t in txt), *shards, image_seq_len=n_img)
    assert any(getattr(px, "T", 0) == 24 for px in wrapper._peer_cache.values()), "peer path not taken"
    valid = max(0, min(ls, n_img - rank * ls))
    results["fulltxt_peer"] = max(rel_err(t_out, full_pad[:, :24]),
                                  rel_err(i_out[:, :valid], full_pad[:, 24 + rank * ls: 24 + rank * ls + valid]))
    # the same with the keys of every query block split over two CTAs (the merging CTA also stores the text rows
    # to every rank)
    os.environ["CHITU_B200_KEY_SPLITS"] = "2"
    wrapper2 = B200ContextParallel(backend, world, cp_backend="ucp")
    for rep in range(2):
        t_out, i_out = wrapper2.cp_attn_with_full_txt(*(t.to(dev) for t in txt), *shards, image_seq_len=n_img)
    os.environ.pop("CHITU_B200_KEY_SPLITS")
    assert any(getattr(px, "T", 0) == 24 and px.n_splits == 2 for px in wrapper2._peer_cache.values())
    results["fulltxt_peer_split"] = max(rel_err(t_out, full_pad[:, :24]),
                                        rel_err(i_out[:, :valid], full_pad[:, 24 + rank * ls: 24 + rank * ls + valid]))
    print(f"rank {rank}: fulltxt_peer done", flush=True)

    # ring attention that keeps the state of every source block: all fresh, then the odd source offsets reused
    from chitudiffusion_b200.cached_ring import CachedRingAttention
    comm.destroy_diffusion_parallel_groups()
    comm.initialize_diffusion_parallel_groups(1, world, 1)
    cached = CachedRingAttention(backend, comm.get_cp_group())
    results["cached_ring_fresh"] = rel_err(cached(ql, kl, vl), full[:, sl])
    results["cached_ring_reuse"] = rel_err(cached(ql, kl, vl, plan=[True] + [t % 2 == 0 for t in range(1, world)]),
                                           full[:, sl])
    assert cached.stats["reused_blocks"] == world // 2
    print(f"rank {rank}: cached_ring done", flush=True)
    # peer-store exchange: norm + rotary pre-pass scattered to the owners, attention scattered back
    comm.destroy_diffusion_parallel_groups()
    comm.initialize_diffusion_parallel_groups(1, world, world)
    grid = (2, 10, S // 20)
    C = H * D
    xq, xk, xv = ((torch.randn(1, S, C, generator=gen) * 0.5).to(torch.bfloat16) for _ in range(3))
    wq, wk = (1.0 + 0.05 * torch.randn(C, generator=gen) for _ in range(2))
    freqs = oracle.wan_rope_table(D)
    rq, rk, rv = oracle.wan_self_attention_pre(xq, xk, xv, wq, wk, H, [list(grid)], freqs)
    ref2 = oracle.sdpa_fp32(rq, rk, rv)
    px = PeerUlysses(comm.get_up_group(world), 1, s, H, D, torch.bfloat16, dev)
    pre = WanPreAttention(H, D, cp_size=world, cp_rank=rank, device=dev)
    place = dict(out_strides=px.gather_strides, heads_per_group=px.hc)
    for rep in range(3):  # buffers and barriers are reused call after call
        lq, lk, lv = (t[:, sl].contiguous().to(dev) for t in (xq, xk, xv))
        if rep == 0:  # transform locally, then one launch of three plain scatters that announces the rows
            tq, tk, tv = pre(lq, lk, lv, wq.to(dev), wk.to(dev), grid)
            px.scatter_ready(tq, tk, tv)
        else:  # norm + rotary + scatter of q, k and v in one launch
            px.scatter_qkv(pre.jobs(lq, lk, wq.to(dev), wk.to(dev)), lv, **pre.batch_args(s, grid))
        out = px.attention()
        results[f"peer{rep}"] = rel_err(out, ref2[:, sl])
    # this small grid leaves SMs idle, so the object above delivered its rows with copy CTAs inside the attention
    # launch; the same layer with that mode switched off: stores straight to the peers, one flag per rank
    assert px.push is not None, "push mode was expected for this shape"
    os.environ["CHITU_B200_PUSH"] = "0"
    px_direct = PeerUlysses(comm.get_up_group(world), 1, s, H, D, torch.bfloat16, dev)
    os.environ.pop("CHITU_B200_PUSH")
    assert px_direct.push is None
    for rep in range(2):
        px_direct.scatter_qkv(pre.jobs(lq, lk, wq.to(dev), wk.to(dev)), lv, **pre.batch_args(s, grid))
        results[f"direct{rep}"] = rel_err(px_direct.attention(), ref2[:, sl])
    # both modes again with the keys of every query block split over two CTAs (the CTA that finishes last
    # merges the ranges, stores the rows to their owners and takes part in the announcement)
    os.environ["CHITU_B200_KEY_SPLITS"] = "2"
    px_split = PeerUlysses(comm.get_up_group(world), 1, s, H, D, torch.bfloat16, dev)
    os.environ["CHITU_B200_PUSH"] = "0"
    px_split_direct = PeerUlysses(comm.get_up_group(world), 1, s, H, D, torch.bfloat16, dev)
    os.environ.pop("CHITU_B200_PUSH")
    os.environ.pop("CHITU_B200_KEY_SPLITS")
    assert px_split.n_splits == 2 and px_split.push is not None and px_split_direct.push is None
    for name, obj in (("split_push", px_split), ("split_direct", px_split_direct)):
        for rep in range(2):
            obj.scatter_qkv(pre.jobs(lq, lk, wq.to(dev), wk.to(dev)), lv, **pre.batch_args(s, grid))
            results[f"{name}{rep}"] = rel_err(obj.attention(), ref2[:, sl])
    # a grid of more CTAs than the GPU has SMs: the copy CTAs are the first of the launch, so the attention CTAs
    # of the first wave find their peers' rows arriving; checked against the direct exchange and against one GPU
    hc = H // world
    s_big = 256 * (ops.NUM_SMS // hc + 2) // world
    gen_big = torch.Generator(device=dev).manual_seed(100 + rank)
    bq, bk, bv = ((torch.randn(1, s_big, H, D, generator=gen_big, device=dev) * 0.7).to(torch.bfloat16) for _ in range(3))
    os.environ["CHITU_B200_PUSH"] = "force"
    px_waves = PeerUlysses(comm.get_up_group(world), 1, s_big, H, D, torch.bfloat16, dev)
    os.environ["CHITU_B200_PUSH"] = "0"
    px_waves_direct = PeerUlysses(comm.get_up_group(world), 1, s_big, H, D, torch.bfloat16, dev)
    os.environ.pop("CHITU_B200_PUSH")
    assert px_waves.push is not None and px_waves_direct.push is None
    assert -(-(world * s_big) // 256) * hc * px_waves.n_splits > ops.NUM_SMS
    outs_big = []
    for obj in (px_waves, px_waves_direct):
        for rep in range(2):
            obj.scatter_ready(bq, bk, bv)
            got = obj.attention().clone()
        outs_big.append(got)
    gathered = []
    for t in (bq, bk, bv):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        gathered.append(torch.cat(parts, 1))
    single = backend(gathered[0][:, rank * s_big:(rank + 1) * s_big], gathered[1], gathered[2])[0]
    results["waves_push_vs_direct"] = rel_err(outs_big[0], outs_big[1].float().cpu())
    results["waves_push_vs_single"] = rel_err(outs_big[0], single.float().cpu())
    # the same through the wrapper's projections-in entry, whole and in two row pieces (as Flux's two streams arrive)
    wrapper = B200ContextParallel(backend, world, cp_backend="ucp")
    lq, lk, lv = (t[:, sl].contiguous().to(dev) for t in (xq, xk, xv))
    out = wrapper.attention_from_projections(pre.jobs(lq, lk, wq.to(dev), wk.to(dev)), lv, **pre.batch_args(s, grid))
    results["from_proj"] = rel_err(out, ref2[:, sl])
    h = s // 2
    args = pre.batch_args(s, grid)
    first = wrapper.attention_from_projections(pre.jobs(lq[:, :h], lk[:, :h], wq.to(dev), wk.to(dev)), lv[:, :h],
                                               row_offset=0, last=False, **args)
    assert first is None
    args2 = dict(args, pos_offset=args["pos_offset"] + h)
    out = wrapper.attention_from_projections(pre.jobs(lq[:, h:], lk[:, h:], wq.to(dev), wk.to(dev)), lv[:, h:],
                                             row_offset=h, last=True, **args2)
    results["from_proj_pieces"] = rel_err(out, ref2[:, sl])
    out = wrapper.attention_fused(produce_q=lambda: tq, produce_k=lambda: tk, produce_v=lambda: tv, num_heads=H)[0]
    results["attention_fused"] = rel_err(out, ref2[:, sl])
    torch.cuda.synchronize()
    ops.check_status(dev)
    ok = all(e <= REL for e in results.values())
    print(f"rank {rank}: " + " ".join(f"{n}={e:.2e}" for n, e in results.items()), flush=True)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
