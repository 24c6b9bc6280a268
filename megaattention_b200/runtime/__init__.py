"""Run-time resource contract of the fused prefill path (mirror of the reference's
``src/mega_attention/runtime/__init__.py:1-3``), plus the per-layer serving wrapper the
reference only sketches in its design notes."""
from .workspace import FusedFaOprojArWorkspace
from .prefill_layer import FusedPrefillLayer

from .residual_rmsnorm import residual_rmsnorm
from .rope import rope_qk_

__all__ = ["FusedFaOprojArWorkspace", "FusedPrefillLayer", "residual_rmsnorm", "rope_qk_"]
