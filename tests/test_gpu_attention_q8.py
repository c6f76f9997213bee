"""GPU checks of the quantised attention variant (per-block INT8 QK^T, E4M3 PV).

Two references: the CPU emulation of the same recipe in the same tiling (`oracle.attention_q8`; tight
tolerance - differences come only from the approximate exp2 and accumulation order, which can flip an
E4M3 rounding here and there) and the fp32 oracle (loose tolerance: cosine >= 0.998, relative L1 <=
5e-2, the accuracy class of 8-bit attention).  The reference's own quantised backend is a
third-party wheel that cannot be installed here, so parity with it is unpinned.
"""

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from chitudiffusion_b200 import B200AttnBackend

    return B200AttnBackend("b200_q8")


def _metrics(out, ref):
    out, ref = out.float().cpu(), ref.float()
    cos = torch.nn.functional.cosine_similarity(out.flatten(), ref.flatten(), dim=0).item()
    rel_l1 = ((out - ref).abs().sum() / ref.abs().sum()).item()
    max_rel = ((out - ref).abs().max() / ref.abs().max()).item()
    return cos, rel_l1, max_rel


@pytest.mark.parametrize("B,Sq,Sk,H", [(1, 128, 128, 1), (1, 300, 333, 2), (2, 130, 700, 3), (1, 1000, 64, 1),
                                        (1, 7145, 7145, 2)])
def test_q8_matches_emulation_and_fp32(backend, B, Sq, Sk, H):
    gen = torch.Generator().manual_seed(Sq * 3 + Sk)
    q = torch.randn(B, Sq, H, 128, generator=gen).to(torch.bfloat16)
    k = (torch.randn(B, Sk, H, 128, generator=gen) + 0.3).to(torch.bfloat16)  # non-zero channel means
    v = torch.randn(B, Sk, H, 128, generator=gen).to(torch.bfloat16)
    out, lse, _ = backend(q.cuda(), k.cuda(), v.cuda(), return_attn_probs=True)
    assert backend.impl == "b200_q8" and out.dtype == torch.bfloat16 and torch.isfinite(out.float()).all()
    emu, emu_lse = oracle.attention_q8(q, k, v, return_lse=True)
    cos, rel_l1, max_rel = _metrics(out, emu)
    assert cos >= 0.9995 and rel_l1 <= 1.5e-2 and max_rel <= 5e-2, ("vs emulation", cos, rel_l1, max_rel)
    assert (lse.cpu() - emu_lse).abs().max().item() <= 5e-3
    ref, ref_lse = oracle.sdpa_fp32(q, k, v, return_lse=True)
    cos, rel_l1, max_rel = _metrics(out, ref)
    assert cos >= 0.998 and rel_l1 <= 5e-2, ("vs fp32", cos, rel_l1, max_rel)
    assert (lse.cpu() - ref_lse).abs().max().item() <= 5e-2


def test_q8_zero_keys_and_scale_argument(backend):
    gen = torch.Generator().manual_seed(5)
    q = torch.randn(1, 200, 1, 128, generator=gen).to(torch.bfloat16)
    v = torch.randn(1, 150, 1, 128, generator=gen).to(torch.bfloat16)
    k0 = torch.zeros(1, 150, 1, 128, dtype=torch.bfloat16)
    out = backend(q.cuda(), k0.cuda(), v.cuda())[0]  # uniform attention: the mean of v, padding keys excluded
    assert (out.float().cpu() - v.float().mean(dim=1, keepdim=True)).abs().max().item() <= 3e-2
    k = torch.randn(1, 150, 1, 128, generator=gen).to(torch.bfloat16)
    out = backend(q.cuda(), k.cuda(), v.cuda(), softmax_scale=0.03)[0]
    cos, rel_l1, _ = _metrics(out, oracle.sdpa_fp32(q, k, v, 0.03))
    assert cos >= 0.998 and rel_l1 <= 5e-2


def test_q8_refused_for_ring_like_the_reference():
    from chitudiffusion_b200.context_parallel import B200ContextParallel

    class FakeGroup:
        group_size, rank_in_group = 4, 0

    class Q8:
        impl = "b200_q8"

    wrapper = B200ContextParallel(Q8(), 2, group=FakeGroup())
    with pytest.raises(NotImplementedError):
        wrapper(torch.zeros(1, 8, 4, 128), torch.zeros(1, 8, 4, 128), torch.zeros(1, 8, 4, 128))
