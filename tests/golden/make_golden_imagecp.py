"""Golden vectors for the replicated-text / sharded-image attention core, made by EXECUTING the reference's own class.

Run where the reference tree is mounted (CHITU_REFERENCE_ROOT points at it):

    CHITU_REFERENCE_ROOT=<tree> python tests/golden/make_golden_imagecp.py

Every case launches CPU (gloo) ranks; each rank imports the reference's ``ImageContextParallelAttention``
(chitu_diffusion/modules/attention/image_cp_attention.py) unchanged, wraps the same fp32 attention callable as
``make_golden_cp.py``, enables it on the context-parallel group, and calls ``attention`` on its shard of a seeded
problem - under the reference's own environment switches where the case names one (FP8 transfer of the gathered
K/V; the cross-step K/V cache driven through ``begin_forward`` over five steps).  Rank 0 writes
``tests/golden/imagecp_golden.pt``; ``tests/test_cp_gloo.py`` replays the cases through this repository's mirror.
The comm-layer patches are those of ``make_golden_cp.py`` (plain barrier, host receive buffers, list all-to-all
emulated on gloo); none touches the arithmetic, the schedule or the cache policy.
"""

from __future__ import annotations

import os
import subprocess
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, "..", ".."))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

OUT_PATH = os.path.join(HERE, "imagecp_golden.pt")
TXT_LEN, S_LOCAL, H, D = 5, 6, 8, 16

# name: (ranks, mode, ulysses_size, environment of the reference's switches, steps)
CASES = {
    "agkv2": (2, "agkv", 1, {}, 1),
    "ulysses2": (2, "ulysses", 1, {}, 1),
    "ring2": (2, "ring", 1, {}, 1),
    "unified4_u2": (4, "unified", 2, {}, 1),
    "agkv2_fp8": (2, "agkv", 1, {"CHITU_CP_FP8_KV": "1"}, 1),
    "agkv2_cache": (2, "agkv", 1, {"CHITU_CP_KV_CACHE": "1", "CHITU_CP_KV_CACHE_WARMUP": "1",
                                   "CHITU_CP_KV_CACHE_INTERVAL": "2", "CHITU_CP_KV_CACHE_TAIL": "1"}, 5),
}


def case_inputs(name):
    """Seeded inputs of a case: text Q/K/V, image Q, and one image K/V pair per step (the same from step 1 on)."""
    ranks, _mode, _u, _env, steps = CASES[name]
    gen = torch.Generator().manual_seed(sum(map(ord, "imagecp:" + name)))
    n_img = S_LOCAL * ranks
    d = {key: torch.randn(1, TXT_LEN, H, D, generator=gen) for key in ("txt_q", "txt_k", "txt_v")}
    d["img_q"] = torch.randn(1, n_img, H, D, generator=gen)
    k0, v0 = torch.randn(1, n_img, H, D, generator=gen), torch.randn(1, n_img, H, D, generator=gen)
    k1, v1 = k0 + 0.3 * torch.randn(k0.shape, generator=gen), v0 + 0.3 * torch.randn(v0.shape, generator=gen)
    d["img_k"] = [k0] + [k1] * (steps - 1)
    d["img_v"] = [v0] + [v1] * (steps - 1)
    return d


def _worker(name: str, out_file: str) -> None:
    import importlib

    import torch.distributed as dist

    from make_golden_cp import _Fp32Backend
    from oracle import ref_import

    ns = ref_import.load()
    ranks, mode, usize, _env, steps = CASES[name]
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    ns.comm_group.CommGroup.barrier = lambda self: dist.barrier(group=self.gpu_group)

    def list_all_to_all(output_list, input_list, group=None, async_op=False):
        send = torch.stack([t.contiguous() for t in input_list])
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        for dst, src in zip(output_list, recv.unbind(0)):
            dst.copy_(src)

    dist.all_to_all = list_all_to_all
    try:
        from chitu_diffusion.observability.timer import Timer

        Timer.disable()
    except Exception:
        pass
    ps = ns.parallel_state
    ps.initialize_diffusion_parallel_groups(1, ranks, max(usize, 1))
    groups = [ps.get_cp_group()]
    for size in (usize, ranks):
        try:
            groups.append(ps.get_up_group(size))
        except Exception:
            pass
    for g in groups:
        g.device = torch.device("cpu")
    mod = importlib.import_module("chitu_diffusion.modules.attention.image_cp_attention")
    core = mod.ImageContextParallelAttention(_Fp32Backend(), mode=mode, profile=False, use_cudagraph=False,
                                             ulysses_size=usize)
    core.enable(ps.get_cp_group())
    inp = case_inputs(name)
    r = ps.get_cp_group().rank_in_group
    sl = slice(r * S_LOCAL, (r + 1) * S_LOCAL)
    outs = []
    for step in range(steps):
        if steps > 1:
            core.begin_forward(step, steps, "cond")
        t_out, i_out = core.attention(inp["txt_q"], inp["txt_k"], inp["txt_v"], inp["img_q"][:, sl].contiguous(),
                                      inp["img_k"][step][:, sl].contiguous(), inp["img_v"][step][:, sl].contiguous())
        outs.append({"txt_out": t_out.detach().clone(), "img_out": i_out.detach().clone()})
    gathered = [None] * ranks
    dist.gather_object(outs, gathered if rank == 0 else None, dst=0)
    if rank == 0:
        torch.save({"inputs": inp, "ranks": ranks, "mode": mode, "ulysses_size": usize, "steps": steps,
                    "per_rank": gathered}, out_file)
    dist.destroy_process_group()


def main() -> None:
    if len(sys.argv) == 4 and sys.argv[1] == "--worker":
        _worker(sys.argv[2], sys.argv[3])
        return
    from oracle import ref_import

    if not ref_import.available():
        raise SystemExit("set CHITU_REFERENCE_ROOT to the mounted ChituDiffusion tree")
    golden = {}
    port = 29790
    with tempfile.TemporaryDirectory() as tmp:
        for name, case in CASES.items():
            port += 1
            out_file = os.path.join(tmp, name + ".pt")
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={case[0]}",
                   "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__), "--worker",
                   name, out_file]
            env = dict(os.environ, OMP_NUM_THREADS="1", PYTHONDONTWRITEBYTECODE="1", **case[3])
            proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
            if proc.returncode != 0:
                raise SystemExit(f"case {name} failed:\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}")
            golden[name] = torch.load(out_file)
            first = golden[name]["per_rank"][0][0]
            print(f"{name}: {case[0]} ranks, {case[4]} step(s), outputs "
                  f"{ {k_: (tuple(v_.shape), str(v_.dtype)) for k_, v_ in first.items()} }", flush=True)
    torch.save(golden, OUT_PATH)
    print("wrote", OUT_PATH, os.path.getsize(OUT_PATH), "bytes")


if __name__ == "__main__":
    main()
