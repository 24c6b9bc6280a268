"""Run-time resource contract of the fused prefill path (mirror of the reference's
``src/mega_attention/runtime/__init__.py:1-3``)."""
from .workspace import FusedFaOprojArWorkspace

__all__ = ["FusedFaOprojArWorkspace"]
