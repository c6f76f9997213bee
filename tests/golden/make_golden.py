"""Generate golden input/output vectors by EXECUTING the reference's own code.

Run where the reference tree is mounted:

    python tests/golden/make_golden.py

Writes ``tests/golden/hotpath_golden.pt`` (a dict of small CPU tensors).  The
reference has no recorded vectors for this path, so these fixtures - produced by
its torch-SDPA backend, ``WanRMSNorm``, ``rope_apply``, ``rope_apply_with_cp``,
``update_out_and_lse``, ``WanSelfAttention.forward`` and ``SequencePadder`` on
seeded inputs - are what pins the CPU oracle.  ``make_golden_cp.py`` adds the
multi-rank layouts.
"""

from __future__ import annotations

import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))

from oracle import ref_import  # noqa: E402


def wan_freqs(ns, d):
    return torch.cat(
        [
            ns.rope_params(1024, d - 4 * (d // 6)),
            ns.rope_params(1024, 2 * (d // 6)),
            ns.rope_params(1024, 2 * (d // 6)),
        ],
        dim=1,
    )


def main():
    ns = ref_import.load()
    torch.set_num_threads(4)
    g = {}

    # 1. attention core through the reference backend callable (fp32, CPU)
    gen = torch.Generator().manual_seed(1234)
    backend = ns.DiffusionAttnBackend("torch_sdpa")
    for name, (B, Sq, Sk, H, D, scale) in {
        "sdpa_square": (1, 24, 24, 2, 128, None),
        "sdpa_ragged": (2, 13, 37, 2, 128, None),
        "sdpa_scale": (1, 8, 66, 1, 128, 0.05),
        "sdpa_d64": (1, 17, 33, 2, 64, None),
    }.items():
        q = torch.randn(B, Sq, H, D, generator=gen)
        k = torch.randn(B, Sk, H, D, generator=gen)
        v = torch.randn(B, Sk, H, D, generator=gen)
        out = backend(q, k, v, softmax_scale=scale)[0]
        g[name] = dict(q=q, k=k, v=v, scale=scale, out=out)

    # 2. LSE merge: chain of three partials through update_out_and_lse
    outs = [torch.randn(1, 20, 2, 16, generator=gen) for _ in range(3)]
    lses = [torch.randn(1, 2, 20, generator=gen) * 3 for _ in range(3)]
    o, l = None, None
    for bo, bl in zip(outs, lses):
        o, l = ns.update_out_and_lse(o, l, bo, bl)
    g["lse_merge"] = dict(outs=outs, lses=lses, out=o, lse=l)
    # bf16 partials
    outs16 = [t.to(torch.bfloat16) for t in outs]
    o, l = None, None
    for bo, bl in zip(outs16, lses):
        o, l = ns.update_out_and_lse(o, l, bo, bl)
    g["lse_merge_bf16"] = dict(outs=outs16, lses=lses, out=o, lse=l)

    # 3. Wan RMSNorm over the full channel dim
    norm = ns.WanRMSNorm(96, eps=1e-6)
    with torch.no_grad():
        norm.weight.copy_(1.0 + 0.1 * torch.randn(96, generator=gen))
        for name, dt in (("wan_norm_fp32", torch.float32), ("wan_norm_bf16", torch.bfloat16)):
            x = (torch.randn(2, 11, 96, generator=gen) * 1.7).to(dt)
            g[name] = dict(x=x, weight=norm.weight.detach().clone(), eps=1e-6, out=norm(x))

    # 4. Wan 3-axis RoPE (grid smaller than the sequence -> pass-through tail)
    freqs = wan_freqs(ns, 128)
    x = torch.randn(2, 26, 1, 128, generator=gen)
    grid = torch.tensor([[2, 3, 4], [1, 5, 5]])
    g["wan_rope"] = dict(x=x, grid=grid, out=ns.rope_apply(x, grid, freqs))
    xb = x.to(torch.bfloat16)
    g["wan_rope_bf16"] = dict(x=xb, grid=grid, out=ns.rope_apply(xb, grid, freqs))

    # 5. rank-local RoPE under context parallelism (3 ranks, padded tail)
    grid1 = torch.tensor([[2, 3, 4]])  # 24 tokens, padded to 27 = 3 * 9
    xs = [torch.randn(1, 9, 1, 128, generator=gen) for _ in range(3)]
    g["wan_rope_cp"] = dict(
        xs=xs, grid=grid1, cp_size=3, outs=[ns.rope_apply_with_cp(xs[r], grid1, freqs, 3, r) for r in range(3)]
    )

    # 6. whole Wan self-attention layer, random-init N(0, 0.02^2) weights
    dim, heads = 64, 2
    layer = ns.WanSelfAttention(backend, None, dim, heads, (-1, -1), True, 1e-6)
    with torch.no_grad():
        for lin in (layer.q, layer.k, layer.v, layer.o):
            lin.weight.copy_(0.02 * torch.randn(dim, dim, generator=gen))
            lin.bias.zero_()
        xl = torch.randn(1, 24, dim, generator=gen)
        gl = torch.tensor([[2, 3, 4]])
        y = layer(xl, torch.tensor([24]), gl, wan_freqs(ns, dim // heads))
        qp, kp, vp = layer.q(xl), layer.k(xl), layer.v(xl)
    g["wan_layer"] = dict(
        x=xl, grid=gl, heads=heads,
        wq=layer.q.weight.detach().clone(), wk=layer.k.weight.detach().clone(),
        wv=layer.v.weight.detach().clone(), wo=layer.o.weight.detach().clone(),
        q_proj=qp, k_proj=kp, v_proj=vp, out=y,
    )

    # 7. zero-pad split used when tokens do not divide the CP size
    t = torch.randn(1, 13, 4, generator=gen)
    parts = ns.SequencePadder.split_sequence_padding(t, 4, 1, name="golden")
    g["pad_split"] = dict(x=t, parts=[p.clone() for p in parts], n=4, dim=1)

    path = os.path.join(HERE, "hotpath_golden.pt")
    torch.save(g, path)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
