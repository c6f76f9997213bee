"""``ContextParallelDispatcher`` against the outputs of the reference's own class (no process group needed:
the dispatch methods are pure slicing; the emulated rank comes from a stand-in group object)."""

import os
import types

import pytest
import torch

from chitudiffusion_b200.dispatch import ContextParallelDispatcher

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "cp_layouts_golden.pt")


@pytest.mark.parametrize("size", [2, 4])
def test_dispatch_matches_reference_class(size):
    g = torch.load(GOLDEN)["dispatcher"]
    for r, want in enumerate(g["per_size"][size]):
        group = types.SimpleNamespace(group_size=size, rank_in_group=r, global_rank=r, local_rank=r)
        d = ContextParallelDispatcher(group=group)
        d._last_text_seq_len, d._last_image_seq_len = g["n_txt"], g["n_img"]
        got = d.dispatch_flux_rotary_emb(g["rotary"], text_seq_len=g["n_txt"])
        assert isinstance(got, tuple) and len(got) == 2
        for a, b in zip(got, want["rotary"]):
            assert torch.equal(a, b)
        assert torch.equal(d.dispatch(g["tokens"], name="hidden_states"), want["tokens"])
        assert torch.equal(d.dispatch_id_sequence(g["ids"], name="img_ids"), want["ids"])
    # pass-through forms
    assert d.dispatch_flux_rotary_emb(None, 3) is None
    t = torch.ones(2)
    assert d.dispatch_flux_rotary_emb(t, 3) is t


def test_wrapped_model_compute_modes():
    """Replicated mode splits and gathers around the call; local-latent mode leaves the tokens alone and
    refuses a precomputed joint rotary pair."""
    group = types.SimpleNamespace(group_size=1, rank_in_group=0, global_rank=0, local_rank=0)
    d = ContextParallelDispatcher(group=group)
    seen = {}

    def model_compute(tokens, **kw):
        seen.update(kw, tokens=tokens)
        return tokens * 2

    fn = d.wrap_model_compute(model_compute)
    x = torch.randn(1, 7, 4)
    enc = torch.randn(1, 3, 4)
    out = fn(x, encoder_hidden_states=enc, seq_lens=torch.tensor([99]), img_ids=torch.zeros(7, 3))
    assert torch.equal(out, x * 2) and int(seen["seq_lens"][0]) == 7 and d._last_image_seq_len == 7
    d.local_latent_mode = True
    out = fn(x, encoder_hidden_states=enc)
    assert torch.equal(out, x * 2) and d._last_image_seq_len == 7
    with pytest.raises(NotImplementedError):
        fn(x, encoder_hidden_states=enc, image_rotary_emb=(torch.zeros(10, 2), torch.zeros(10, 2)))
