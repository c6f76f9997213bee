"""Golden vectors for the context-parallel layouts, made by EXECUTING the reference's own wrapper.

Run where the reference tree is mounted (CHITU_REFERENCE_ROOT points at it):

    CHITU_REFERENCE_ROOT=<tree> python tests/golden/make_golden_cp.py

For every case below the script launches CPU (gloo) ranks with ``torch.distributed.run``; each rank
imports the reference's ``DiffusionAttention_with_CP``, ``CommGroup`` and
``initialize_diffusion_parallel_groups`` unchanged, wraps a plain fp32 attention callable that
returns ``(out, lse[B,H,S], None)``, runs the layout on its shard of a seeded problem and sends its
result to rank 0.  Rank 0 writes ``tests/golden/cp_layouts_golden.pt``: per case the full inputs and
every rank's output (values, dtype, shape).  ``tests/test_cp_gloo.py`` replays the cases through this
repository's wrapper.

Three run-time patches make the reference's comm layer usable on gloo ranks; none touches the
arithmetic or the schedule:

* ``CommGroup.barrier`` passes ``device_ids`` (CUDA only) - replaced by a plain barrier;
* ``CommGroup.device`` is ``cuda:<local_rank>`` - set to ``cpu`` after construction, so that the
  ring's receive buffers are host tensors;
* gloo has no list ``all_to_all`` (the 3-d LSE exchange of Ulysses x ring takes that form) - emulated
  with a stack and ``all_to_all_single``.

The reference's ``Timer`` is switched off (it would synchronise a CUDA device).
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

OUT_PATH = os.path.join(HERE, "cp_layouts_golden.pt")

# name: (ranks, ulysses limit, cp_backend, kind, B, tokens per rank, H, D)
CASES = {
    "ulysses2": (2, 2, "ucp", "plain", 1, 6, 8, 16),
    "ring2": (2, 1, "ucp", "plain", 1, 6, 8, 16),
    "agcp2": (2, 2, "agcp", "plain", 1, 6, 8, 16),
    "ulysses4": (4, 4, "ucp", "plain", 1, 5, 8, 16),
    "ring4": (4, 1, "ucp", "plain", 1, 5, 8, 16),
    "usp_u2r2": (4, 2, "ucp", "plain", 1, 6, 8, 16),
    "usp_u2r2_batch2": (4, 2, "ucp", "plain", 2, 6, 8, 16),
    "agcp4": (4, 4, "agcp", "plain", 1, 5, 8, 16),
    # 16-bit inputs (names ending in _bf16): pins the result dtype - the backend's own for Ulysses and
    # all-gather-KV, fp32 wherever ring partials were merged
    "ulysses2_bf16": (2, 2, "ucp", "plain", 1, 6, 8, 16),
    "ring2_bf16": (2, 1, "ucp", "plain", 1, 6, 8, 16),
    "usp_u2r2_bf16": (4, 2, "ucp", "plain", 1, 6, 8, 16),
    "agcp2_bf16": (2, 2, "agcp", "plain", 1, 6, 8, 16),
    # replicated text + sharded image, image length not divisible by the ranks (zero-padded tail)
    "fulltxt_agcp2": (2, 2, "agcp", "fulltxt", 1, 6, 8, 16),
    "fulltxt_ulysses2": (2, 2, "ucp", "fulltxt", 1, 6, 8, 16),
    "fulltxt_usp_u2r2": (4, 2, "ucp", "fulltxt", 1, 6, 8, 16),
    "fulltxt_ring4": (4, 1, "ucp", "fulltxt", 1, 6, 8, 16),
}
TXT_LEN = 5
PAD = 3  # image tokens short of a multiple of the rank count in the fulltxt cases


def case_inputs(name):
    """Seeded full-sequence inputs of a case (the same on every rank and in the replaying test)."""
    ranks, _up, _backend, kind, B, s, H, D = CASES[name]
    gen = torch.Generator().manual_seed(sum(map(ord, name)))
    dtype = torch.bfloat16 if name.endswith("_bf16") else torch.float32
    if kind == "plain":
        S = s * ranks
        return dict(q=torch.randn(B, S, H, D, generator=gen).to(dtype), k=torch.randn(B, S, H, D, generator=gen).to(dtype),
                    v=torch.randn(B, S, H, D, generator=gen).to(dtype))
    n_img = s * ranks - PAD
    d = {}
    for key, n in (("txt_q", TXT_LEN), ("txt_k", TXT_LEN), ("txt_v", TXT_LEN), ("img_q", n_img), ("img_k", n_img),
                   ("img_v", n_img)):
        d[key] = torch.randn(B, n, H, D, generator=gen)
    return d


class _Fp32Backend:
    """``impl`` + ``(q, k, v, ...) -> (out of q's dtype, lse[B,H,S] fp32 | None, None)``, fp32 arithmetic on the host."""

    impl = "torch_sdpa"

    def __call__(self, q, k, v, *args, softmax_scale=None, return_attn_probs=False, **kwargs):
        import oracle

        out, lse = oracle.sdpa_fp32(q, k, v, softmax_scale, return_lse=True)
        return out.to(q.dtype), (lse if return_attn_probs else None), None


def _worker(name: str, out_file: str) -> None:
    import torch.distributed as dist

    from oracle import ref_import

    ns = ref_import.load()
    ranks, up, cp_backend, kind, B, s, H, D = CASES[name]
    dist.init_process_group("gloo")
    rank = dist.get_rank()

    cg = ns.comm_group
    cg.CommGroup.barrier = lambda self: dist.barrier(group=self.gpu_group)
    real_list_a2a = dist.all_to_all

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
    ps.initialize_diffusion_parallel_groups(1, ranks, up)
    groups = [ps.get_cp_group()]
    for size in (min(up, ranks), min(up, ranks) // 2):
        try:
            groups.append(ps.get_up_group(size))
        except ValueError:
            pass
    for g in groups:
        g.device = torch.device("cpu")

    wrapper = ns.DiffusionAttention_with_CP(_Fp32Backend(), up, ring_cudagraph=False, cp_backend=cp_backend)
    inp = case_inputs(name)
    r = ps.get_cp_group().rank_in_group
    if kind == "plain":
        sl = slice(r * s, (r + 1) * s)
        out = wrapper(inp["q"][:, sl].contiguous(), inp["k"][:, sl].contiguous(), inp["v"][:, sl].contiguous())
        assert out[1] is None and out[2] is None
        mine = {"out": out[0]}
    else:
        shards = {key: ns.SequencePadder.split_sequence_padding(inp[key], ranks, 1, name=key)[r].contiguous()
                  for key in ("img_q", "img_k", "img_v")}
        txt_out, img_out = wrapper.cp_attn_with_full_txt(
            inp["txt_q"], inp["txt_k"], inp["txt_v"], shards["img_q"], shards["img_k"], shards["img_v"],
            image_seq_len=inp["img_q"].shape[1])
        mine = {"txt_out": txt_out, "img_out": img_out}
    gathered = [None] * ranks
    dist.gather_object({k_: (v_.detach().clone(), str(v_.dtype), tuple(v_.shape)) for k_, v_ in mine.items()},
                       gathered if rank == 0 else None, dst=0)
    if rank == 0:
        torch.save({"inputs": inp, "ranks": ranks, "up": up, "cp_backend": cp_backend, "kind": kind,
                    "per_rank": [{k_: v_[0] for k_, v_ in g.items()} for g in gathered],
                    "dtypes": [{k_: v_[1] for k_, v_ in g.items()} for g in gathered]}, out_file)
    dist.all_to_all = real_list_a2a
    dist.destroy_process_group()


def dispatcher_golden(root: str) -> dict:
    """Outputs of the reference's ``ContextParallelDispatcher`` methods for every rank of a 2- and a 4-rank group.

    The class lives in ``chitu_diffusion/runtime/generator.py``, whose module imports the whole runtime
    (adapters, samplers, real ``diffusers``).  Only the class statement is executed here: it is cut out
    of the file's syntax tree and run with the names it needs - ``torch``, the reference's own
    ``SequencePadder`` and a stand-in ``get_cp_group`` that reports the rank being emulated.  The
    methods are pure tensor slicing, so no process group is needed.
    """
    import ast
    import importlib
    import types

    path = os.path.join(root, "chitu_diffusion", "runtime", "generator.py")
    with open(path) as f:
        tree = ast.parse(f.read(), filename=path)
    node = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == "ContextParallelDispatcher")
    putils = importlib.import_module("chitu_diffusion.runtime.parallel_utils")
    fake = types.SimpleNamespace(group_size=1, global_rank=0, local_rank=0, rank_in_group=0, gpu_group=None)
    scope = {"torch": torch, "dist": torch.distributed, "SequencePadder": putils.SequencePadder,
             "get_cp_group": lambda: fake, "DiffusionBackend": None}
    exec(compile(ast.Module(body=[node], type_ignores=[]), path, "exec"), scope)
    cls = scope["ContextParallelDispatcher"]
    gen = torch.Generator().manual_seed(4242)
    n_txt, n_img, half = 5, 13, 8  # neither part divisible by the rank counts
    rotary = (torch.randn(n_txt + n_img, half, generator=gen), torch.randn(n_txt + n_img, half, generator=gen))
    tokens = torch.randn(2, n_img, 6, generator=gen)
    ids = torch.arange(n_img * 3).view(n_img, 3)
    out = {"rotary": rotary, "tokens": tokens, "ids": ids, "n_txt": n_txt, "n_img": n_img, "per_size": {}}
    for size in (2, 4):
        rows = []
        for r in range(size):
            fake.group_size, fake.rank_in_group, fake.global_rank = size, r, r
            d = cls()
            d._last_text_seq_len, d._last_image_seq_len = n_txt, n_img
            rows.append({"rotary": d.dispatch_flux_rotary_emb(rotary, text_seq_len=n_txt),
                         "tokens": d.dispatch(tokens, name="hidden_states"),
                         "ids": d.dispatch_id_sequence(ids, name="img_ids")})
        out["per_size"][size] = rows
    return out


def main() -> None:
    if len(sys.argv) == 4 and sys.argv[1] == "--worker":
        _worker(sys.argv[2], sys.argv[3])
        return
    from oracle import ref_import

    if not ref_import.available():
        raise SystemExit("set CHITU_REFERENCE_ROOT to the mounted ChituDiffusion tree")
    golden = {}
    port = 29730
    with tempfile.TemporaryDirectory() as tmp:
        for name, case in CASES.items():
            port += 1
            out_file = os.path.join(tmp, name + ".pt")
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={case[0]}",
                   "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__), "--worker",
                   name, out_file]
            env = dict(os.environ, OMP_NUM_THREADS="1", PYTHONDONTWRITEBYTECODE="1")
            proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
            if proc.returncode != 0:
                raise SystemExit(f"case {name} failed:\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}")
            golden[name] = torch.load(out_file)
            shapes = {k_: tuple(v_.shape) for k_, v_ in golden[name]["per_rank"][0].items()}
            print(f"{name}: {case[0]} ranks, outputs {shapes}, dtypes {golden[name]['dtypes'][0]}", flush=True)
    ref_import.install_stubs()
    golden["dispatcher"] = dispatcher_golden(ref_import.DEFAULT_ROOT)
    print("dispatcher: rotary shards", [tuple(t.shape) for t in golden["dispatcher"]["per_size"][4][3]["rotary"]])
    torch.save(golden, OUT_PATH)
    print("wrote", OUT_PATH, os.path.getsize(OUT_PATH), "bytes")


if __name__ == "__main__":
    main()
