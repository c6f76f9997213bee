"""install() against the reference tree, where it is mounted (skipped elsewhere)."""

import pytest

from oracle import ref_import


@pytest.mark.skipif(not ref_import.available(), reason="reference tree not mounted")
def test_install_registers_b200_with_the_reference():
    ref_import.install_stubs()
    from chitudiffusion_b200 import B200AttnBackend, install
    from chitudiffusion_b200.context_parallel import B200ContextParallel

    assert install.install()
    assert install.install()  # idempotent
    from chitu_diffusion.modules.attention import diffusion_attn_backend as ref

    backend = ref.DiffusionAttnBackend("b200")
    assert isinstance(backend, B200AttnBackend) and backend.impl == "b200"
    stock = ref.DiffusionAttnBackend("torch_sdpa")
    assert type(stock).__name__ == "DiffusionAttnBackend" and stock.impl == "torch_sdpa"
    assert ref.DiffusionAttention_with_CP is B200ContextParallel


def test_make_backend_single_rank():
    from chitudiffusion_b200 import B200AttnBackend, install

    assert isinstance(install.make_backend("b200"), B200AttnBackend)
