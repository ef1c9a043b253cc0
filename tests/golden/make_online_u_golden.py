"""Generates tests/golden/online_u.pt from the reference's own `online_u`
(token2tile/operator/deploy_step.py:122-149) executed on the CPU.

Run in a container that has the reference checkout:

    python tests/golden/make_online_u_golden.py [REFERENCE_CHECKOUT]

The fixture stores the seeds, not the inputs: the test regenerates q and k with
the same generator calls.
"""
import importlib.util
import os
import sys
from pathlib import Path

import torch

CASES = [dict(H=2, N=512, D=128, r=32, seed=11, corr=0.0),
         dict(H=1, N=2048, D=128, r=32, seed=12, corr=0.7)]


def make_inputs(case):
    g = torch.Generator().manual_seed(case["seed"])
    H, N, D = case["H"], case["N"], case["D"]
    scale = torch.linspace(2.0, 0.05, D)
    k = torch.randn(H, N, D, generator=g) * scale
    q = case["corr"] * k + (1.0 - case["corr"]) * torch.randn(H, N, D, generator=g) * scale.flip(0)
    return q, k


def main():
    here = Path(__file__).resolve()
    root = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("T2T_REFERENCE_DIR") or here.parents[3] / "reference")
    ref = root / "token2tile" / "operator"
    sys.path.insert(0, str(ref))
    spec = importlib.util.spec_from_file_location("ref_deploy_step", ref / "deploy_step.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = []
    for case in CASES:
        q, k = make_inputs(case)
        Uq, Uk = mod.online_u(q, k, case["r"])
        out.append(dict(case=case, Uq=Uq, Uk=Uk))
    torch.save(out, Path(__file__).resolve().parent / "online_u.pt")
    print("wrote", len(out), "cases")


if __name__ == "__main__":
    main()
