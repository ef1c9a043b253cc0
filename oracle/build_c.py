"""Compiles the oracle's C helper (oracle/chain_dot.c) into oracle/_build/libt2t_chain.so.

    python oracle/build_c.py

Test infrastructure only.  The PyTorch loop in t2t_oracle.chain_dot is the
definition; the C twin gives the same bits at the speed the 480p / 720p parity
tests need.  Without a C compiler the oracle falls back to the loop.
"""
from __future__ import annotations

import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "chain_dot.c"
OUT = HERE / "_build" / "libt2t_chain.so"


def build(force: bool = False):
    """Returns the library path, or None when no C compiler is available."""
    if OUT.exists() and not force and OUT.stat().st_mtime >= SRC.stat().st_mtime:
        return OUT
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        return None
    OUT.parent.mkdir(exist_ok=True)
    cmd = [cc, "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC", str(SRC), "-o", str(OUT)]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
