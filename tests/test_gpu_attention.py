"""GPU parity of the attention kernel, called through the backend callable and the C ABI, against the CPU oracle.

Tolerance (bf16 inputs, fp32 oracle on the same bf16-rounded inputs):
max-abs <= 2e-2 * max|ref|, cosine >= 0.9999, LSE max-abs <= 1e-3.
"""

import math

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

REL_MAX_ABS = 2e-2
MIN_COSINE = 0.9999
LSE_ABS = 1e-3


@pytest.fixture(scope="module")
def backend():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from chitudiffusion_b200 import B200AttnBackend

    return B200AttnBackend("b200")


def _check(out, ref, lse=None, ref_lse=None):
    out = out.float().cpu()
    assert out.shape == ref.shape
    assert torch.isfinite(out).all()
    err = (out - ref).abs().max().item()
    assert err <= REL_MAX_ABS * ref.abs().max().item(), f"max-abs {err}"
    cos = torch.nn.functional.cosine_similarity(out.flatten(), ref.flatten(), dim=0).item()
    assert cos >= MIN_COSINE, f"cosine {cos}"
    if lse is not None:
        assert lse.dtype == torch.float32 and lse.shape == ref_lse.shape
        assert (lse.cpu() - ref_lse).abs().max().item() <= LSE_ABS


def _rand(shape, dtype, gen, scale=1.0):
    return (torch.randn(shape, generator=gen) * scale).to(dtype)


@pytest.mark.parametrize("S", [1, 63, 64, 65, 127, 128, 129, 255, 256, 257, 300, 1000])
def test_square_sizes(backend, S):
    gen = torch.Generator().manual_seed(S)
    q, k, v = (_rand((1, S, 3, 128), torch.bfloat16, gen) for _ in range(3))
    ref, ref_lse = oracle.sdpa_fp32(q, k, v, return_lse=True)
    out, lse, probs = backend(q.cuda(), k.cuda(), v.cuda(), return_attn_probs=True)
    assert probs is None and out.is_contiguous() and out.dtype == torch.bfloat16
    _check(out, ref, lse, ref_lse)
    out2, lse2, _ = backend(q.cuda(), k.cuda(), v.cuda())
    assert lse2 is None and torch.equal(out2, out)


@pytest.mark.parametrize("Sq,Sk,B,H", [(128, 640, 1, 1), (300, 333, 2, 2), (130, 7, 1, 5), (7, 1300, 2, 1), (975, 7800, 1, 2)])
def test_ragged_cross_shapes(backend, Sq, Sk, B, H):
    gen = torch.Generator().manual_seed(Sq * 7 + Sk)
    q = _rand((B, Sq, H, 128), torch.bfloat16, gen)
    k = _rand((B, Sk, H, 128), torch.bfloat16, gen)
    v = _rand((B, Sk, H, 128), torch.bfloat16, gen)
    ref, ref_lse = oracle.sdpa_fp32(q, k, v, return_lse=True)
    out, lse, _ = backend(q.cuda(), k.cuda(), v.cuda(), return_attn_probs=True)
    _check(out, ref, lse, ref_lse)


def test_golden_vectors_from_reference_backend(backend, golden):
    """fp32 fixtures produced by the reference's torch-SDPA backend, replayed in bf16."""
    for name in ("sdpa_square", "sdpa_ragged", "sdpa_scale"):
        c = golden[name]
        q, k, v = (c[n].to(torch.bfloat16) for n in ("q", "k", "v"))
        out = backend(q.cuda(), k.cuda(), v.cuda(), softmax_scale=c["scale"])[0]
        # bf16 rounding of the inputs is part of the error here
        err = (out.float().cpu() - c["out"]).abs().max().item()
        assert err <= 3e-2 * c["out"].abs().max().item(), (name, err)
        _check(out, oracle.sdpa_fp32(q, k, v, c["scale"]))


def test_large_logits_force_rescaling(backend):
    gen = torch.Generator().manual_seed(11)
    q = _rand((1, 512, 2, 128), torch.bfloat16, gen, 3.0)
    k = _rand((1, 2048, 2, 128), torch.bfloat16, gen, 3.0)
    # ascending key magnitude makes the running maximum grow tile after tile
    k = k * torch.linspace(0.2, 1.0, 2048).view(1, -1, 1, 1).to(torch.bfloat16)
    v = _rand((1, 2048, 2, 128), torch.bfloat16, gen)
    ref, ref_lse = oracle.sdpa_fp32(q, k, v, return_lse=True)
    out, lse, _ = backend(q.cuda(), k.cuda(), v.cuda(), return_attn_probs=True)
    _check(out, ref, lse, ref_lse)


def test_strided_views_like_flux_processor(backend):
    """The Flux processor hands over [B,S,H,D] views of [B,H,S,D] memory."""
    gen = torch.Generator().manual_seed(12)
    qh, kh, vh = (_rand((1, 4, 384, 128), torch.bfloat16, gen) for _ in range(3))
    q, k, v = (t.cuda().transpose(1, 2) for t in (qh, kh, vh))
    assert not q.is_contiguous()
    out = backend(q, k, v, causal=False)[0]
    _check(out, oracle.sdpa_fp32(qh.transpose(1, 2), kh.transpose(1, 2), vh.transpose(1, 2)))
    assert out.is_contiguous()
    # head slices of a wider tensor need no repack either
    wide = _rand((1, 200, 8, 128), torch.bfloat16, gen)
    sl = wide.cuda()[:, :, 2:5]
    out = backend(sl, sl, sl)[0]
    _check(out, oracle.sdpa_fp32(wide[:, :, 2:5], wide[:, :, 2:5], wide[:, :, 2:5]))


def test_fp16_and_keyword_call(backend):
    gen = torch.Generator().manual_seed(13)
    q, k, v = (_rand((2, 200, 2, 128), torch.float16, gen) for _ in range(3))
    out = backend(q=q.cuda(), k=k.cuda(), v=v.cuda(), window_size=(-1, -1))[0]
    assert out.dtype == torch.float16
    _check(out, oracle.sdpa_fp32(q, k, v))


def test_inputs_not_mutated_and_padding_rows_untouched(backend):
    gen = torch.Generator().manual_seed(14)
    q, k, v = (_rand((1, 130, 1, 128), torch.bfloat16, gen).cuda() for _ in range(3))
    q0, k0, v0 = q.clone(), k.clone(), v.clone()
    from chitudiffusion_b200 import ops

    big = torch.full((1, 140, 1, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.attn_fwd(q, k, v, out=big[:, :130])
    assert torch.equal(q, q0) and torch.equal(k, k0) and torch.equal(v, v0)
    assert (big[:, 130:] == 7.0).all()  # rows past Sq are never written


def test_wan_1p3b_layer_shape_config1(backend):
    """B=1, H=12, D=128, S=7800 (5x30x52 grid), pre-ops by the oracle, kernel vs fp32 oracle."""
    gen = torch.Generator().manual_seed(0)
    S, H, D = 7800, 12, 128
    C = H * D
    x = torch.randn(1, S, C, generator=gen)
    wq, wk, wv = (0.02 * torch.randn(C, C, generator=gen) for _ in range(3))
    freqs = oracle.wan_rope_table(D)
    ones = torch.ones(C)
    q, k, v = oracle.wan_self_attention_pre(x @ wq.t(), x @ wk.t(), x @ wv.t(), ones, ones, H, [[5, 30, 52]], freqs)
    ref, ref_lse = oracle.sdpa_fp32(q, k, v, return_lse=True)
    out, lse, _ = backend(q.cuda(), k.cuda(), v.cuda(), return_attn_probs=True)
    _check(out, ref, lse, ref_lse)


def test_unsupported_features_raise_like_the_reference(backend):
    q = torch.zeros(1, 8, 1, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NotImplementedError):
        backend(q, q, q, causal=True)
    with pytest.raises(NotImplementedError):
        backend(q, q, q, dropout_p=0.1)
    with pytest.raises(NotImplementedError):
        backend(q, q, q, window_size=(3, 3))
    with pytest.raises(NotImplementedError):
        backend(q.view(8, 1, 128), q.view(8, 1, 128), q.view(8, 1, 128), torch.tensor([0, 8]), torch.tensor([0, 8]), 8, 8)
    with pytest.raises(NotImplementedError):
        backend(q.float(), q.float(), q.float())
    q64 = torch.zeros(1, 8, 1, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NotImplementedError):
        backend(q64, q64, q64)
    with pytest.raises(RuntimeError):
        backend(q.cpu(), q.cpu(), q.cpu())


def test_linearity_in_v_at_full_size(backend):
    """Size-independent property at the Flux shape: attention is linear in V."""
    gen = torch.Generator().manual_seed(15)
    S, H = 4608, 24
    q, k, v1, v2 = (_rand((1, S, H, 128), torch.bfloat16, gen).cuda() for _ in range(4))
    o1 = backend(q, k, v1)[0].float()
    o2 = backend(q, k, v2)[0].float()
    o12 = backend(q, k, (v1.float() + v2.float()).to(torch.bfloat16))[0].float()
    assert (o12 - (o1 + o2)).abs().max().item() <= 2e-2 * o12.abs().max().item() + 2e-3
    # rows of P sum to one: V = const gives that const back
    ones = torch.ones_like(v1)
    oc, lse, _ = backend(q, k, ones, return_attn_probs=True)
    assert (oc.float() - 1.0).abs().max().item() <= 1e-2
    assert torch.isfinite(lse).all() and lse.min().item() > math.log(S) - 40


@pytest.mark.parametrize("Sq,Sk,H,n_splits", [(200, 1000, 2, 3), (130, 4608, 3, 8), (64, 333, 1, 16), (256, 256, 1, 2),
                                               (700, 1900, 3, 2)])
def test_key_split_matches_oracle(backend, Sq, Sk, H, n_splits):
    """Keys split over several CTAs, merged inside the launch (the path small grids take) against the oracle:
    through scratch memory by the CTA that finishes last, and - two ranges - through the shared memory of a
    thread-block cluster as well."""
    from chitudiffusion_b200 import ops

    gen = torch.Generator().manual_seed(Sq + Sk)
    q = _rand((2, Sq, H, 128), torch.bfloat16, gen)
    k = _rand((2, Sk, H, 128), torch.bfloat16, gen)
    v = _rand((2, Sk, H, 128), torch.bfloat16, gen)
    ref, ref_lse = oracle.sdpa_fp32(q, k, v, return_lse=True)
    out, lse = ops.attn_fwd(q.cuda(), k.cuda(), v.cuda(), return_lse=True, n_splits=n_splits)
    _check(out, ref, lse, ref_lse)
    one, _ = ops.attn_fwd(q.cuda(), k.cuda(), v.cuda(), n_splits=1)
    assert (out.float() - one.float()).abs().max().item() <= 1e-2 * ref.abs().max().item()
    if n_splits == 2:  # the launch above merged through the cluster; now the scratch form of the same split
        assert ops.set_cluster_merge(False) is True
        try:
            out2, lse2 = ops.attn_fwd(q.cuda(), k.cuda(), v.cuda(), return_lse=True, n_splits=2)
        finally:
            ops.set_cluster_merge(True)
        _check(out2, ref, lse2, ref_lse)
        assert (out2.float() - out.float()).abs().max().item() <= 1e-2 * ref.abs().max().item()
    auto, _ = ops.attn_fwd(q.cuda(), k.cuda(), v.cuda())  # the heuristic picks a split for this small grid
    _check(auto, ref)
    assert ops.auto_key_splits(2, Sq, Sk, H) >= 1 and ops.auto_key_splits(1, 4608, 4608, 24) == 1


def test_attention_state_composes(backend):
    """Key partitions folded into states in two different groupings give the full attention."""
    from chitudiffusion_b200.state import AttentionState

    gen = torch.Generator().manual_seed(31)
    q, k, v = (_rand((1, 300, 2, 128), torch.bfloat16, gen) for _ in range(3))
    ref, ref_lse = oracle.sdpa_fp32(q, k, v, return_lse=True)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    parts = [slice(0, 100), slice(100, 228), slice(228, 300)]
    blocks = [backend(qc, kc[:, p], vc[:, p], return_attn_probs=True)[:2] for p in parts]
    chain = AttentionState()
    assert chain.is_empty()
    for bo, bl in blocks:
        chain.update(bo, bl)
    left, right = AttentionState(), AttentionState()
    left.update(*blocks[0])
    right.update(*blocks[1])
    right.update(*blocks[2])
    tree = AttentionState.merge(AttentionState.merge(AttentionState(), left), right)
    for st in (chain, tree):
        assert st.out.dtype == torch.float32 and tuple(st.lse.shape) == (1, 300, 2, 1)
        assert (st.out.cpu() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
        assert (st.lse.cpu().squeeze(-1).transpose(1, 2) - ref_lse).abs().max().item() <= 2e-3
    shifted = chain.corrected(torch.ones_like(chain.out), torch.zeros_like(chain.lse))
    assert torch.allclose(shifted.out, chain.out + 1.0) and AttentionState().corrected(chain.out, chain.lse).is_empty()


@pytest.mark.parametrize("Sq,Sk,H", [(256, 75600, 1), (256, 32760, 2), (4608, 4608, 2)])
def test_long_key_and_full_size_shapes_against_oracle(backend, Sq, Sk, H):
    """The Wan 720p / 480p key lengths (591 and 256 key tiles: every ring slot and barrier phase wraps
    hundreds of times) on a query block, and the full Flux sequence on two of its heads, against the
    fp32 oracle - output and log-sum-exp."""
    gen = torch.Generator().manual_seed(Sk + H)
    q = _rand((1, Sq, H, 128), torch.bfloat16, gen)
    k = _rand((1, Sk, H, 128), torch.bfloat16, gen)
    v = _rand((1, Sk, H, 128), torch.bfloat16, gen)
    ref, ref_lse = oracle.sdpa_fp32(q, k, v, return_lse=True)
    out, lse, _ = backend(q.cuda(), k.cuda(), v.cuda(), return_attn_probs=True)
    _check(out, ref, lse, ref_lse)
    if Sq != Sk:
        # the same problem without the key split the small grid would pick by itself
        from chitudiffusion_b200 import ops

        one, lse1 = ops.attn_fwd(q.cuda(), k.cuda(), v.cuda(), return_lse=True, n_splits=1)
        _check(one, ref, lse1, ref_lse)


def test_key_split_scratch_survives_regrow_under_a_graph(backend):
    """A captured graph keeps the address of the key-split scratch it was captured with.  A later,
    larger eager call makes the shared scratch grow; the superseded buffer must stay alive (and not be
    handed to anyone else), so replaying the old graph still gives the right answer."""
    from chitudiffusion_b200 import ops

    gen = torch.Generator().manual_seed(5)
    q, k, v = (_rand((1, 130, 2, 128), torch.bfloat16, gen) for _ in range(3))
    ref = oracle.sdpa_fp32(q, k, v)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ops.attn_fwd(qc, kc, vc, n_splits=2)  # warm-up on the capture stream: its scratch exists
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out, _ = ops.attn_fwd(qc, kc, vc, n_splits=2)
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    _check(out, ref)
    with torch.cuda.stream(stream):
        big = [_rand((2, 700, 4, 128), torch.bfloat16, gen).cuda() for _ in range(3)]
        ops.attn_fwd(*big, n_splits=8)  # needs far more scratch on the same (device, stream): regrow
        churn = [torch.full((1 << 20,), 7.0, device="cuda") for _ in range(8)]  # allocator churn over freed blocks
    torch.cuda.synchronize()
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    _check(out, ref)
    del churn


def test_two_devices_in_one_process(backend):
    """The opt-in to large dynamic shared memory is per device: a process that drives two GPUs must be
    able to launch on both."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs in one process")
    gen = torch.Generator().manual_seed(77)
    q, k, v = (_rand((1, 200, 2, 128), torch.bfloat16, gen) for _ in range(3))
    ref = oracle.sdpa_fp32(q, k, v)
    for dev in ("cuda:0", "cuda:1"):
        out = backend(q.to(dev), k.to(dev), v.to(dev))[0]
        torch.cuda.synchronize(dev)
        _check(out, ref)


def test_query_transform_inside_the_kernel_equals_the_pre_pass(backend):
    """q normalised / rotated / rounded in shared memory by the attention kernel gives bit-for-bit the result of
    running the pre-pass kernel on q first: per-head norm + per-token rotary table (Flux / Qwen form), and
    full-width norm (factor from a statistics-only job) + three-axis rotary (Wan form)."""
    from chitudiffusion_b200 import ops, pre_attention

    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(91)
    H, D = 3, 128
    C = H * D
    # Flux form: ragged length, strided views of a fused qkv projection, learned per-head weights
    S = 333
    qkv = _rand((2, S, 3 * C), torch.bfloat16, gen, 0.7).to(dev)
    ids = torch.stack([torch.zeros(S, dtype=torch.long), torch.arange(S) // 19, torch.arange(S) % 19], 1)
    table = pre_attention.axis_rope_table(ids, (16, 56, 56)).to(dev)
    wq = (1.0 + 0.1 * torch.randn(D, generator=gen)).to(dev)
    wk = (1.0 + 0.1 * torch.randn(D, generator=gen)).to(dev)
    pre = pre_attention.JointPreAttention(H, D, table)
    jobs = pre.jobs(qkv[..., :C], qkv[..., C:2 * C], wq, wk)
    backend.q_in_kernel = True
    fused = backend.attention_from_projections(jobs, qkv[..., 2 * C:], **pre.batch_args())
    q, k, v = pre(qkv[..., :C], qkv[..., C:2 * C], qkv[..., 2 * C:], wq, wk)
    plain = backend(q, k, v)[0]
    assert torch.equal(fused, plain)
    ref = oracle.sdpa_fp32(q.cpu(), k.cpu(), v.cpu())
    _check(fused, ref)
    # Wan form: full-width statistics, grid rotary, fp32 weights with the intermediate rounding of the reference
    grid = (3, 10, 13)
    S = grid[0] * grid[1] * grid[2] + 5  # five padding tokens past the grid pass through unrotated
    qkv = _rand((1, S, 3 * C), torch.bfloat16, gen, 0.7).to(dev)
    nq = (1.0 + 0.1 * torch.randn(C, generator=gen)).to(dev)
    nk = (1.0 + 0.1 * torch.randn(C, generator=gen)).to(dev)
    wan = pre_attention.WanPreAttention(H, D, device=dev)
    fused = backend.attention_from_projections(wan.jobs(qkv[..., :C], qkv[..., C:2 * C], nq, nk), qkv[..., 2 * C:],
                                               **wan.batch_args(S, grid))
    q, k, v = wan(qkv[..., :C], qkv[..., C:2 * C], qkv[..., 2 * C:], nq, nk, grid)
    plain = backend(q, k, v)[0]
    assert torch.equal(fused, plain)
    backend.q_in_kernel = False
    default = backend.attention_from_projections(wan.jobs(qkv[..., :C], qkv[..., C:2 * C], nq, nk), qkv[..., 2 * C:],
                                                 **wan.batch_args(S, grid))
    assert torch.equal(default, plain)
    ops.check_status(dev)
