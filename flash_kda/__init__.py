"""Drop-in module name of the reference operator.

``flash-linear-attention`` enables its FlashKDA backend when ``import flash_kda`` succeeds
(fla/ops/kda/backends/flashkda.py) and then calls ``flash_kda.fwd(...)``; this shim makes the
B200 implementation answer under that name with the reference's signature
(flash_kda/__init__.py:5 in the reference project).
"""
from flashkda_b200 import fwd, get_workspace_size  # noqa: F401

__all__ = ["fwd", "get_workspace_size"]
