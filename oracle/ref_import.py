"""Import the reference's own Python code for the hot path, where it is mounted.

TEST INFRASTRUCTURE ONLY - never imported by the product package.

The reference project depends on packages that carry no arithmetic for this
path and that are absent here (``netifaces``, ``omegaconf``, ``diffusers``).
This module registers empty stand-ins for them so that the reference's
attention backend, LSE merge, comm group and Wan pre-attention modules import
unchanged.  Nothing is copied: the reference files are executed from where
they lie.  Used only to generate and cross-check golden fixtures; the GPU box
has no reference tree and never calls this.
"""

from __future__ import annotations

import importlib
import importlib.util
import os
import sys
import types

# where the ChituDiffusion tree is mounted: taken from the environment only
DEFAULT_ROOT = os.environ.get("CHITU_REFERENCE_ROOT", "")


def available(root: str = DEFAULT_ROOT) -> bool:
    return bool(root) and os.path.isdir(os.path.join(root, "chitu_diffusion"))


def _stub(name: str, **attrs) -> types.ModuleType:
    mod = sys.modules.get(name)
    if mod is None:
        mod = types.ModuleType(name)
        sys.modules[name] = mod
    for key, val in attrs.items():
        setattr(mod, key, val)
    return mod


def install_stubs(root: str = DEFAULT_ROOT) -> None:
    import torch

    sys.dont_write_bytecode = True  # the reference tree is read-only
    if root not in sys.path:
        sys.path.insert(0, root)
    try:
        import netifaces  # noqa: F401
    except ImportError:
        _stub("netifaces")
    try:
        import omegaconf  # noqa: F401
    except ImportError:

        class _Cfg(dict):
            pass

        class _OmegaConf:
            @staticmethod
            def create(obj=None):
                return obj

        _stub("omegaconf", OmegaConf=_OmegaConf, DictConfig=_Cfg, ListConfig=list, MISSING="???")
    for optional in ("imageio", "torchvision"):
        try:
            importlib.import_module(optional)
        except Exception:
            _stub(optional)
    try:
        import diffusers  # noqa: F401
    except ImportError:

        class ConfigMixin:
            pass

        class ModelMixin(torch.nn.Module):
            pass

        def register_to_config(fn):
            return fn

        pkg = _stub("diffusers")
        pkg.__path__ = []  # mark as package
        _stub("diffusers.configuration_utils", ConfigMixin=ConfigMixin, register_to_config=register_to_config)
        models = _stub("diffusers.models")
        models.__path__ = []
        _stub("diffusers.models.modeling_utils", ModelMixin=ModelMixin)


def load(root: str = DEFAULT_ROOT):
    """Return a namespace with the reference symbols used to pin the oracle."""
    if not available(root):
        raise RuntimeError(f"reference tree not found at {root}")
    install_stubs(root)
    ns = types.SimpleNamespace()
    backend = importlib.import_module("chitu_diffusion.modules.attention.diffusion_attn_backend")
    putils = importlib.import_module("chitu_diffusion.runtime.parallel_utils")
    ns.DiffusionAttnBackend = backend.DiffusionAttnBackend
    ns.DiffusionAttention_with_CP = backend.DiffusionAttention_with_CP
    ns.backend_module = backend
    ns.update_out_and_lse = putils.update_out_and_lse
    ns.SequencePadder = putils.SequencePadder
    ns.comm_group = importlib.import_module("chitu_diffusion.core.distributed.comm_group")
    ns.parallel_state = importlib.import_module("chitu_diffusion.core.distributed.parallel_state")

    # model_wan.py: its package __init__ pulls in the Flux models (real diffusers
    # needed), so seed a bare package object and load the one file by path.
    pkg_name = "chitu_diffusion.models"
    if pkg_name not in sys.modules:
        pkg = types.ModuleType(pkg_name)
        pkg.__path__ = [os.path.join(root, "chitu_diffusion", "models")]
        sys.modules[pkg_name] = pkg
    path = os.path.join(root, "chitu_diffusion", "models", "model_wan.py")
    spec = importlib.util.spec_from_file_location("chitu_diffusion.models.model_wan", path)
    wan = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = wan
    spec.loader.exec_module(wan)
    ns.model_wan = wan
    ns.WanRMSNorm = wan.WanRMSNorm
    ns.WanSelfAttention = wan.WanSelfAttention
    ns.rope_params = wan.rope_params
    ns.rope_apply = wan.rope_apply
    try:
        wan_utils = importlib.import_module("chitu_diffusion.modules.utils.wan")
        ns.rope_apply_with_cp = wan_utils.rope_apply_with_cp
    except Exception:
        ns.rope_apply_with_cp = None
    return ns
