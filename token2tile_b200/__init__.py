"""token2tile_b200: the Token2Tile sparse attention operator, written for B200 (sm_100a).

Mirrors the package entry of the reference (token2tile/__init__.py:7-9): callers
locate the operator through `operator_dir()` and import `deploy_step` from it, or
import `MaskedStepDeploy` from this package directly.
"""
from pathlib import Path

__version__ = "0.1.0"


def operator_dir() -> str:
    """Directory of the attention operator (deploy_step.py and the CUDA sources)."""
    return str(Path(__file__).resolve().parent)


def __getattr__(name):
    if name in ("MaskedStepDeploy", "online_u"):
        from . import deploy_step
        return getattr(deploy_step, name)
    raise AttributeError(name)
