"""CPU oracle for the DiT attention hot path.  TEST INFRASTRUCTURE ONLY.

Everything in this package is a plain-PyTorch, CPU, fp32/fp64 restatement of
the arithmetic that ChituDiffusion performs on the context-parallel attention
path.  It exists so that the CUDA kernels can be checked against known-good
answers; it is never imported by the product package ``chitudiffusion_b200``.
Only the test-suite, the smoke entry and the CPU-baseline leg of the benchmark
may import it.

Pinning: the reference tree has no golden vectors for this path, so these
functions are pinned by *executing the reference's own Python code* on seeded
inputs (``tests/golden/make_golden.py``) and committing the results as small
fixtures that ``tests/test_oracle_golden.py`` replays.  The per-head RMSNorm and
axis-RoPE used by the Flux/Qwen callers live in the un-vendored third-party
package ``diffusers`` (pinned 0.36.0 by the reference's requirements.txt) and
are restated from their published definition: parity for those two functions is
unpinned.
"""

from .reference_math import (  # noqa: F401
    sdpa_fp32,
    sdpa_reference_call,
    wan_rms_norm,
    wan_rope_params,
    wan_rope_table,
    wan_rope_apply,
    wan_rope_apply_with_cp,
    wan_self_attention_pre,
    per_head_rms_norm,
    axis_rope_table,
    apply_rope_interleaved,
    update_out_and_lse,
    merge_partials,
    split_sequence_padding,
)
from .layouts import (  # noqa: F401
    ulysses_scatter_heads,
    ulysses_gather_heads,
    simulate_ucp,
    simulate_agcp,
    simulate_full_txt,
    cp_rank_lists,
    cfg_rank_lists,
    up_rank_lists,
)
from .quantised import attention_q8  # noqa: F401,E402
from .dit_block import layer_norm_fp32, wan_block  # noqa: F401,E402
from .flux_block import flux_double_block, flux_single_block  # noqa: F401,E402
from .qwen_block import qwen_attention, qwen_double_block, qwen_streams, slice_rotary_freqs, apply_rotary_complex  # noqa: F401,E402
