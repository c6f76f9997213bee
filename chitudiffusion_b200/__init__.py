"""B200-native attention hot path for ChituDiffusion-style DiT inference.

Public surface (mirrors the reference's attention-backend and parallel API):

* ``B200AttnBackend``            - per-rank backend callable (``infer.attn_type: b200``)
* ``ops``                        - operator-level calls into libchitu_b200.so
"""

from .attention import B200AttnBackend, BACKEND_NAME  # noqa: F401
from . import ops  # noqa: F401

__all__ = ["B200AttnBackend", "BACKEND_NAME", "ops"]
