"""Worker for the multi-process context-parallel tests (launched by tests/test_cp_gloo.py).

Each rank builds the same seeded global problem, shards it the way the runtime does, runs the
context-parallel wrapper over gloo with an oracle-backed attention callable (the CUDA backend is
not needed to check rank maps, chunk order, valid-length handling and merge order), and compares
its local result with single-process attention over the full sequence.
"""

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from chitudiffusion_b200 import comm  # noqa: E402
from chitudiffusion_b200.context_parallel import B200ContextParallel  # noqa: E402


class OracleBackend:
    """Duck-typed backend: ``impl`` attribute + ``(q,k,v,...) -> (out, lse, None)``."""

    impl = "torch_sdpa"

    def __call__(self, q, k, v, *_, softmax_scale=None, return_attn_probs=False, **__):
        out, lse = oracle.sdpa_fp32(q, k, v, softmax_scale, return_lse=True)
        return out.to(q.dtype), (lse if return_attn_probs else None), None


class OracleMerger:
    def __init__(self):
        self.out, self.lse = None, None

    def add(self, block_out, block_lse):
        self.out, self.lse = oracle.update_out_and_lse(self.out, self.lse, block_out, block_lse)

    def result(self):
        return self.out


def main():
    cfg_size, up, cp_backend, modes = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4].split(",")
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cp_size = world // cfg_size
    comm.initialize_diffusion_parallel_groups(cfg_size, cp_size, up)
    group = comm.get_cp_group()
    assert group.rank_list == oracle.cp_rank_lists(world, cfg_size)[rank // cp_size if cfg_size == 2 else 0]
    assert comm.get_cfg_group().rank_list in oracle.cfg_rank_lists(world, cfg_size)
    r = group.rank_in_group
    all_ok = True
    for mode in modes:
        wrapper = B200ContextParallel(OracleBackend(), up, cp_backend=cp_backend, merger_factory=OracleMerger)
        # each CP group (cond / uncond under CFG parallelism) works on its own seeded problem
        gen = torch.Generator().manual_seed(100 + group.rank_list[0])
        B, H, D = (2 if mode == "batch2" else 1), 8, 16
        s = 6
        ok = True
        if mode in ("plain", "batch2"):
            S = s * cp_size
            q, k, v = (torch.randn(B, S, H, D, generator=gen) for _ in range(3))
            full = oracle.sdpa_fp32(q, k, v)
            sl = slice(r * s, (r + 1) * s)
            out, lse, probs = wrapper(q[:, sl].contiguous(), k[:, sl].contiguous(), v[:, sl].contiguous())
            assert lse is None and probs is None
            err = (out.float() - full[:, sl]).abs().max().item()
            ok = err < 2e-6 and tuple(out.shape) == (B, s, H, D)
            # the single-process layout simulator agrees too
            sim = (oracle.simulate_agcp if cp_backend == "agcp" else
                   (lambda a, b, c: oracle.simulate_ucp(a, b, c, up)))(
                [q[:, i * s:(i + 1) * s] for i in range(cp_size)], [k[:, i * s:(i + 1) * s] for i in range(cp_size)],
                [v[:, i * s:(i + 1) * s] for i in range(cp_size)])
            err2 = (out.float() - sim[r].float()).abs().max().item()
            ok = ok and err2 < 2e-6
            print(f"rank {rank} mode {mode} err {err:.2e} sim {err2:.2e}", flush=True)
        elif mode == "fulltxt":
            n_img = s * cp_size - 3  # not divisible: zero-padded tail that must never be attended
            txt_len = 5
            tq, tk, tv = (torch.randn(1, txt_len, H, D, generator=gen) for _ in range(3))
            iq, ik, iv = (torch.randn(1, n_img, H, D, generator=gen) for _ in range(3))
            full = oracle.sdpa_fp32(torch.cat([tq, iq], 1), torch.cat([tk, ik], 1), torch.cat([tv, iv], 1))
            shards = [oracle.split_sequence_padding(t, cp_size, 1) for t in (iq, ik, iv)]
            t_out, i_out = wrapper.cp_attn_with_full_txt(tq, tk, tv, shards[0][r], shards[1][r], shards[2][r],
                                                         image_seq_len=n_img)
            ls = shards[0][r].shape[1]  # padded shard length
            assert tuple(t_out.shape) == (1, txt_len, H, D) and tuple(i_out.shape) == (1, ls, H, D)
            err_t = (t_out.float() - full[:, :txt_len]).abs().max().item()
            valid = max(0, min(ls, n_img - r * ls))
            err_i = (i_out[:, :valid].float() - full[:, txt_len + r * ls: txt_len + r * ls + valid]).abs().max().item()
            ok = err_t < 2e-6 and err_i < 2e-6
            print(f"rank {rank} fulltxt err_txt {err_t:.2e} err_img {err_i:.2e}", flush=True)
        elif mode.startswith("imagecp_"):
            from chitudiffusion_b200.image_cp import B200ImageContextParallel
            txt_len = 5
            tq, tk, tv = (torch.randn(1, txt_len, H, D, generator=gen) for _ in range(3))
            iq, ik, iv = (torch.randn(1, s * cp_size, H, D, generator=gen) for _ in range(3))
            full = oracle.sdpa_fp32(torch.cat([tq, iq], 1), torch.cat([tk, ik], 1), torch.cat([tv, iv], 1))
            core = B200ImageContextParallel(wrapper, mode=mode.split("_", 1)[1], ulysses_size=up,
                                            merger_factory=wrapper._merger_factory)
            assert core.attn_backend is wrapper.attn and not core.enabled
            core.enable(wrapper.group)
            sl = slice(r * s, (r + 1) * s)
            t_out, i_out = core.attention(tq, tk, tv, iq[:, sl], ik[:, sl], iv[:, sl])
            packed = core._attention_from_packed(torch.cat([iq[:, sl], tq], 1), torch.cat([ik[:, sl], tk], 1),
                                                 torch.cat([iv[:, sl], tv], 1), s)
            err_t = (t_out.float() - full[:, :txt_len]).abs().max().item()
            err_i = (i_out.float() - full[:, txt_len + r * s: txt_len + (r + 1) * s]).abs().max().item()
            ok = (err_t < 2e-6 and err_i < 2e-6 and torch.equal(packed[0], t_out) and torch.equal(packed[1], i_out)
                  and core.stats()["calls"] == 2)
            print(f"rank {rank} {mode} err_txt {err_t:.2e} err_img {err_i:.2e}", flush=True)
            # producer-callback entries take the same path
            fused = core.attention_fused(produce_img_q=lambda: iq[:, sl], produce_img_k=lambda: ik[:, sl],
                                         produce_img_v=lambda: iv[:, sl], produce_txt_q=lambda: tq,
                                         produce_txt_k=lambda: tk, produce_txt_v=lambda: tv, num_heads=H)
            fused2 = core.cp_attn_with_full_txt_fused(
                produce_txt_q=lambda: tq, produce_txt_k=lambda: tk, produce_txt_v=lambda: tv,
                produce_img_q=lambda: iq[:, sl], produce_img_k=lambda: ik[:, sl], produce_img_v=lambda: iv[:, sl],
                num_heads=H, image_seq_len=s * cp_size)
            fused3 = core.attention_fused_packed(
                img_len=s, produce_q=lambda: torch.cat([iq[:, sl], tq], 1), produce_k=lambda: torch.cat([ik[:, sl], tk], 1),
                produce_v=lambda: torch.cat([iv[:, sl], tv], 1), num_heads=H)
            for got in (fused, fused2, fused3):
                ok = ok and torch.equal(got[0], t_out) and torch.equal(got[1], i_out)
            if mode == "imagecp_agkv":
                from chitudiffusion_b200.image_cp import dequantize_fp8, quantize_fp8_per_head

                def local_view(tk_, tv_, ik_, iv_):  # fp32 attention of this rank's queries against given keys
                    o = oracle.sdpa_fp32(torch.cat([iq[:, sl], tq], 1), torch.cat([ik_, tk_], 1), torch.cat([iv_, tv_], 1))
                    return o[:, s:], o[:, :s]

                # FP8 transfer: the other ranks' shards arrive quantised per head, the local one stays exact
                os.environ["CHITU_CP_FP8_KV"] = "1"
                core8 = B200ImageContextParallel(wrapper, mode="agkv")
                os.environ.pop("CHITU_CP_FP8_KV")
                core8.enable(wrapper.group)

                def through_fp8(x):
                    parts = []
                    for j in range(cp_size):
                        piece = x[:, j * s:(j + 1) * s]
                        parts.append(piece if j == r else dequantize_fp8(*quantize_fp8_per_head(piece), x.dtype))
                    return torch.cat(parts, 1)

                want_t, want_i = local_view(tk, tv, through_fp8(ik), through_fp8(iv))
                got_t, got_i = core8.attention(tq, tk, tv, iq[:, sl], ik[:, sl], iv[:, sl])
                e8 = max((got_t - want_t).abs().max().item(), (got_i - want_i).abs().max().item())
                coarse = (got_i.float() - full[:, txt_len + r * s: txt_len + (r + 1) * s]).abs().max().item()
                ok = ok and e8 < 2e-6 and 0 < coarse < 0.2
                # cross-step cache: fresh on steps 0 and 2, stale on step 1 (remote shards of step 0, local shard new)
                os.environ.update(CHITU_CP_KV_CACHE="1", CHITU_CP_KV_CACHE_WARMUP="1", CHITU_CP_KV_CACHE_INTERVAL="2",
                                  CHITU_CP_KV_CACHE_TAIL="1")
                corec = B200ImageContextParallel(wrapper, mode="agkv")
                for name in ("CHITU_CP_KV_CACHE", "CHITU_CP_KV_CACHE_WARMUP", "CHITU_CP_KV_CACHE_INTERVAL",
                             "CHITU_CP_KV_CACHE_TAIL"):
                    os.environ.pop(name)
                corec.enable(wrapper.group)
                ik1, iv1 = ik + 0.3 * torch.randn(ik.shape, generator=gen), iv + 0.3 * torch.randn(iv.shape, generator=gen)
                errs = []
                for step, (kk, vv) in enumerate(((ik, iv), (ik1, iv1), (ik1, iv1), (ik1, iv1), (ik1, iv1))):
                    corec.begin_forward(step, 5, "cond")
                    got_t, got_i = corec.attention(tq, tk, tv, iq[:, sl], kk[:, sl], vv[:, sl])
                    if step == 1:  # stale: the other ranks' keys are those of step 0
                        mix_k, mix_v = ik.clone(), iv.clone()
                        mix_k[:, sl], mix_v[:, sl] = ik1[:, sl], iv1[:, sl]
                        want_t, want_i = local_view(tk, tv, mix_k, mix_v)
                    else:
                        want_t, want_i = local_view(tk, tv, kk, vv)
                    errs.append(max((got_t - want_t).abs().max().item(), (got_i - want_i).abs().max().item()))
                fresh = [corec._kvcache_is_fresh() for corec._cur_step in range(5)]
                ok = ok and max(errs) < 2e-6 and fresh == [True, False, True, False, True]
                print(f"rank {rank} {mode} fp8 {e8:.2e} (vs exact {coarse:.2e}) cache {max(errs):.2e}", flush=True)
        elif mode == "cached_ring":
            from chitudiffusion_b200.cached_ring import CachedRingAttention
            ring = CachedRingAttention(OracleBackend(), group, layer_id=3, merger_factory=OracleMerger)
            P = cp_size
            qs, ks, vs = [[torch.randn(1, s * P, H, D, generator=gen) for _ in range(2)] for _ in range(3)]
            sl = slice(r * s, (r + 1) * s)

            def expect(versions):  # versions[t]: which step's (q, k, v) the state of source offset t was computed with
                out = lse = None
                for t in range(P):
                    ver = versions[t]
                    src = slice(((r + t) % P) * s, ((r + t) % P + 1) * s)
                    o, l = oracle.sdpa_fp32(qs[ver][:, sl], ks[ver][:, src], vs[ver][:, src], return_lse=True)
                    out, lse = oracle.update_out_and_lse(out, lse, o, l)
                return out

            got0 = ring(qs[0][:, sl], ks[0][:, sl], vs[0][:, sl])  # step 0: everything fresh = exact attention
            full0 = oracle.sdpa_fp32(qs[0][:, sl], ks[0], vs[0])
            plan = [True] + [t % 2 == 0 for t in range(1, P)]  # odd offsets reuse their state of step 0
            got1 = ring(qs[1][:, sl], ks[1][:, sl], vs[1][:, sl], plan=plan)
            want1 = expect([1 if plan[t] else 0 for t in range(P)])
            got2 = ring(qs[1][:, sl], ks[1][:, sl], vs[1][:, sl], plan=[True] * P)  # all fresh again
            full1 = oracle.sdpa_fp32(qs[1][:, sl], ks[1], vs[1])
            errs = [(got0 - full0).abs().max().item(), (got1 - want1).abs().max().item(), (got2 - full1).abs().max().item()]
            refused = False
            try:
                ring(qs[1][:, sl], ks[1][:, sl], vs[1][:, sl], plan=plan, tag="uncond")  # nothing kept under this tag
            except RuntimeError:
                refused = True
            ok = max(errs) < 2e-6 and refused and ring.stats["reused_blocks"] == sum(1 for x in plan if not x)
            print(f"rank {rank} cached_ring errs {errs}", flush=True)
        elif mode == "dispatch":
            from chitudiffusion_b200.dispatch import CfgDispatcher, ContextParallelDispatcher, SequencePadder
            disp = ContextParallelDispatcher()
            tokens = torch.randn(2, s * cp_size - 1, 12, generator=gen)  # not divisible: padded tail
            ref_parts = oracle.split_sequence_padding(tokens, cp_size, 1)
            local = disp.dispatch(tokens, name="hidden_states")
            ids = torch.arange(s * cp_size * 3).view(s * cp_size, 3)
            ok = torch.equal(local, ref_parts[r]) and torch.equal(disp.dispatch_id_sequence(ids, "ids"),
                                                                  ids[r * s:(r + 1) * s])
            back = disp.gather(local * 2.0, name="hidden_states")
            ok = ok and torch.equal(back, tokens * 2.0)
            ok = ok and torch.equal(SequencePadder.remove_sequence_padding_and_concat(ref_parts, 1, "hidden_states"), tokens)
            if cfg_size == 2:
                def host_combine(cond, uncond, scale, rescale):  # stands in for the CUDA kernel on gloo ranks
                    out = uncond + scale * (cond - uncond)
                    if rescale:
                        out = out * (torch.norm(cond, dim=-1, keepdim=True) / torch.norm(out, dim=-1, keepdim=True))
                    return out

                cfg = CfgDispatcher(combine=host_combine)
                branch = cfg.group.rank_in_group
                gen2 = torch.Generator().manual_seed(7 + r)  # both branches of one CP rank share the generator
                preds = [torch.randn(1, 9, 16, generator=gen2) for _ in range(2)]
                cond, uncond = cfg.all_gather_cfg_noise_preds(preds[branch])
                ok = ok and torch.equal(cond, preds[0]) and torch.equal(uncond, preds[1])
                guided = cfg.guided_noise_pred(preds[branch], 4.0, rescale=True)
                comb = preds[1] + 4.0 * (preds[0] - preds[1])
                want = comb * (torch.norm(preds[0], dim=-1, keepdim=True) / torch.norm(comb, dim=-1, keepdim=True))
                ok = ok and torch.allclose(guided, want, atol=1e-6)
            print(f"rank {rank} dispatch ok={ok}", flush=True)
        elif mode.startswith("golden:"):
            # replay of a fixture that the reference's own DiffusionAttention_with_CP produced on gloo ranks
            # (tests/golden/make_golden_cp.py): same values, same dtype, same shape on every rank
            case = torch.load(os.path.join(ROOT, "tests", "golden", "cp_layouts_golden.pt"))[mode.split(":", 1)[1]]
            assert case["ranks"] == world and case["up"] == up and case["cp_backend"] == cp_backend
            inp, want = case["inputs"], case["per_rank"][r]
            if case["kind"] == "plain":
                n = inp["q"].shape[1] // cp_size
                sl = slice(r * n, (r + 1) * n)
                got = {"out": wrapper(inp["q"][:, sl].contiguous(), inp["k"][:, sl].contiguous(),
                                      inp["v"][:, sl].contiguous())[0]}
            else:
                sh = [oracle.split_sequence_padding(inp[key], cp_size, 1)[r].contiguous()
                      for key in ("img_q", "img_k", "img_v")]
                t_out, i_out = wrapper.cp_attn_with_full_txt(inp["txt_q"], inp["txt_k"], inp["txt_v"], *sh,
                                                             image_seq_len=inp["img_q"].shape[1])
                got = {"txt_out": t_out, "img_out": i_out}
                # rows of the zero-padded tail are computed from padding and carry no meaning: compare valid rows
                ls = sh[0].shape[1]
                valid = max(0, min(ls, inp["img_q"].shape[1] - r * ls))
                got["img_out"], want = got["img_out"][:, :valid], dict(want, img_out=want["img_out"][:, :valid])
                assert tuple(i_out.shape) == tuple(case["per_rank"][r]["img_out"].shape)
            for key, ref in want.items():
                same_meta = got[key].dtype == ref.dtype and tuple(got[key].shape) == tuple(ref.shape)
                tol = 2e-6 if ref.dtype == torch.float32 else 2 ** -7  # 16-bit: one rounding step of the backend's cast
                err = (got[key].float() - ref.float()).abs().max().item() if ref.numel() else 0.0
                ok = ok and same_meta and err <= tol * max(1.0, ref.float().abs().max().item() if ref.numel() else 1.0)
                print(f"rank {rank} {mode} {key} dtype {got[key].dtype} err {err:.2e} ok={ok}", flush=True)
        elif mode.startswith("imgolden:"):
            # replay of a fixture that the reference's own ImageContextParallelAttention produced on gloo ranks
            # (tests/golden/make_golden_imagecp.py), its environment switches included
            from chitudiffusion_b200.image_cp import B200ImageContextParallel
            sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
            from make_golden_imagecp import CASES as IMG_CASES, S_LOCAL

            name = mode.split(":", 1)[1]
            case = torch.load(os.path.join(ROOT, "tests", "golden", "imagecp_golden.pt"))[name]
            assert case["ranks"] == world
            env = IMG_CASES[name][3]
            os.environ.update(env)
            core = B200ImageContextParallel(wrapper, mode=case["mode"], ulysses_size=case["ulysses_size"],
                                            merger_factory=wrapper._merger_factory)
            for key in env:
                os.environ.pop(key)
            core.enable(wrapper.group)
            inp = case["inputs"]
            sl = slice(r * S_LOCAL, (r + 1) * S_LOCAL)
            worst = 0.0
            for step in range(case["steps"]):
                if case["steps"] > 1:
                    core.begin_forward(step, case["steps"], "cond")
                t_out, i_out = core.attention(inp["txt_q"], inp["txt_k"], inp["txt_v"], inp["img_q"][:, sl].contiguous(),
                                              inp["img_k"][step][:, sl].contiguous(), inp["img_v"][step][:, sl].contiguous())
                want = case["per_rank"][r][step]
                for got, ref in ((t_out, want["txt_out"]), (i_out, want["img_out"])):
                    ok = ok and got.dtype == ref.dtype and tuple(got.shape) == tuple(ref.shape)
                    worst = max(worst, (got.float() - ref.float()).abs().max().item())
            ok = ok and worst < 2e-6
            print(f"rank {rank} {mode} worst {worst:.2e} ok={ok}", flush=True)
        elif mode == "qwen":
            # the Qwen-Image processor mirror over the replicated-text layout: image tokens sharded with a zero-padded
            # tail, rotary rows taken at this rank's image offset (zero past the end), text replicated
            from chitudiffusion_b200.pre_attention import table_from_complex
            from chitudiffusion_b200.qwen import B200QwenAttnProcessor, QwenDoubleBlock, QwenJointAttention

            class HostProcessor(B200QwenAttnProcessor):
                """Same control flow; the per-stream kernel launch is replaced by the oracle's arithmetic on host tensors."""

                def _stream(self, x, proj_q, proj_k, proj_v, norm_q, norm_k, heads, table, outs=None, row_offset=0):
                    Bx, Sx, _ = x.shape
                    q = oracle.per_head_rms_norm(proj_q(x).view(Bx, Sx, heads, -1), norm_q.weight)
                    k = oracle.per_head_rms_norm(proj_k(x).view(Bx, Sx, heads, -1), norm_k.weight)
                    v = proj_v(x).view(Bx, Sx, heads, -1)
                    if table is not None:
                        cos, sin = table[..., 0].double(), table[..., 1].double()
                        q, k = oracle.apply_rope_interleaved(q, cos, sin), oracle.apply_rope_interleaved(k, cos, sin)
                    return q, k, v

            Cq, Hq = 64, 4
            n_img, n_txt = s * cp_size - 3, 5
            pq = {}
            for name, shape in QwenDoubleBlock.param_shapes(Cq, Hq).items():
                if name.startswith("attn."):
                    pq[name] = (1.0 + 0.1 * torch.randn(shape, generator=gen)) if "norm" in name else \
                        0.2 * torch.randn(shape, generator=gen)
            hi = torch.randn(1, n_img, Cq, generator=gen)
            ht = torch.randn(1, n_txt, Cq, generator=gen)
            half = Cq // Hq // 2
            rotary = (torch.polar(torch.ones(n_img, half, dtype=torch.float64), torch.randn(n_img, half, generator=gen).double()),
                      torch.polar(torch.ones(n_txt, half, dtype=torch.float64), torch.randn(n_txt, half, generator=gen).double()))
            ref_img, ref_txt = oracle.qwen_attention(hi, ht, pq, Hq, rotary)
            shard = oracle.split_sequence_padding(hi, cp_size, 1)[r]
            ls = shard.shape[1]
            proc = HostProcessor(wrapper)
            assert proc.base_attn_backend is wrapper.attn
            info = {"image_offset": r * ls, "image_seq_len": n_img}
            img_o, txt_o = proc(QwenJointAttention(pq, Hq), shard, ht, None, None, rotary, info)
            valid = max(0, min(ls, n_img - r * ls))
            err_i = (img_o[:, :valid] - ref_img[:, r * ls:r * ls + valid]).abs().max().item() if valid else 0.0
            err_t = (txt_o - ref_txt).abs().max().item()
            ok = err_i < 1e-4 and err_t < 1e-4 and tuple(img_o.shape) == (1, ls, Cq)
            # the table handed to the image stream: this rank's rows, zeros past the true image length
            tab = proc._table(rotary[0], torch.device("cpu"), r * ls, ls)
            full = table_from_complex(rotary[0])
            ok = ok and torch.equal(tab[:valid], full[r * ls:r * ls + valid]) and not tab[valid:].any()
            print(f"rank {rank} qwen err_img {err_i:.2e} err_txt {err_t:.2e} ok={ok}", flush=True)
        elif mode == "fused":
            S = s * cp_size
            q, k, v = (torch.randn(B, S, H, D, generator=gen) for _ in range(3))
            full = oracle.sdpa_fp32(q, k, v)
            sl = slice(r * s, (r + 1) * s)
            out = wrapper.attention_fused(produce_q=lambda: q[:, sl].contiguous(), produce_k=lambda: k[:, sl].contiguous(),
                                          produce_v=lambda: v[:, sl].contiguous(), num_heads=H)[0]
            err = (out.float() - full[:, sl]).abs().max().item()
            ok = err < 2e-6
        all_ok = all_ok and ok

    flag = torch.tensor([1 if all_ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
