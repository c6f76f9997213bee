"""Register the b200 backend with an importable ChituDiffusion tree.

The reference has no plugin registry: the backend name is checked against a hard-coded
allow-list (chitu_diffusion/core/config_loader.py:117-141), resolved by
``DiffusionAttnBackend.__init__`` (modules/attention/diffusion_attn_backend.py:61-83) and the
wrapper class is named at chitu_diffusion/parallel/dit.py:9-19.  ``install()`` patches those three
places at import time so that ``infer.attn_type: b200`` selects ``B200AttnBackend`` and context
parallelism wraps it with ``B200ContextParallel``; nothing in the reference tree is modified on
disk.  Call it before ``chitu_init``.
"""

from __future__ import annotations

import importlib
from typing import Optional

from .attention import _ALIASES, B200AttnBackend
from .context_parallel import B200ContextParallel


def install(strict: bool = True) -> bool:
    """Patch ``chitu_diffusion`` in this process; returns False if it is not importable (and not ``strict``)."""
    try:
        backend_mod = importlib.import_module("chitu_diffusion.modules.attention.diffusion_attn_backend")
    except ImportError:
        if strict:
            raise
        return False

    ref_cls = backend_mod.DiffusionAttnBackend
    if getattr(ref_cls, "_b200_installed", False):
        return True
    ref_new = ref_cls.__new__

    def _new(cls, attn_type: str = "torch_sdpa", *args, **kwargs):
        # ``DiffusionAttnBackend('b200')`` hands back the b200 backend object itself
        if cls is ref_cls and str(attn_type or "").strip().lower() in _ALIASES:
            return B200AttnBackend(attn_type)
        return ref_new(cls) if ref_new is object.__new__ else ref_new(cls, attn_type, *args, **kwargs)

    ref_cls.__new__ = staticmethod(_new)
    ref_cls._b200_installed = True

    # the CP wrapper name the runtime and the model processors import
    backend_mod.DiffusionAttention_with_CP = B200ContextParallel
    for name in ("chitu_diffusion.parallel.dit",):
        try:
            mod = importlib.import_module(name)
            mod.DiffusionAttention_with_CP = B200ContextParallel
        except ImportError:
            pass

    # allow-list of infer.attn_type values: a local set inside validate_config
    # (core/config_loader.py:117-141), so the validator itself is wrapped
    try:
        cfg = importlib.import_module("chitu_diffusion.core.config_loader")
        original = cfg.validate_config

        def validate_config(config):
            name = str(config.infer.attn_type)
            if name.strip().lower() not in _ALIASES:
                return original(config)
            config.infer.attn_type = "torch_sdpa"
            try:
                return original(config)
            finally:
                config.infer.attn_type = name

        cfg.validate_config = validate_config
    except (ImportError, AttributeError):
        pass
    return True


def make_backend(attn_type: str = "b200", cp_size: int = 1, up: int = 1, cp_backend: str = "ucp",
                 ring_cudagraph: bool = False):
    """What ``DiffusionBackend._init_attention_backend`` builds (runtime/backend.py:589-614), without the runtime."""
    attn = B200AttnBackend(attn_type)
    if cp_size <= 1:
        return attn
    return B200ContextParallel(attn, up, ring_cudagraph=ring_cudagraph, cp_backend=cp_backend)
