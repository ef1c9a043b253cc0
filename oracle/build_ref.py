"""Builds oracle/_ref/libt2t_ref.so: the reference's own kmeans_maintain and
select_union CUDA sources, compiled where they lie in the reference checkout
with the reference's flags (deploy_step.py:46-47, 95-97) except for the target
architecture (sm_100a instead of sm_90a), plus the thin C wrapper ref_wrap.cu.

    python oracle/build_ref.py [REFERENCE_CHECKOUT]

The output is a checker used by tests/test_gpu_ref_pin.py to pin the CPU oracle
against the reference's real kernels.  The reference's tile_attn sources are
not built: they use wgmma, which does not exist on sm_100a.
"""
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"


def main():
    # the reference checkout: argument, else T2T_REFERENCE_DIR, else a "reference" directory beside this repository
    ref = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("T2T_REFERENCE_DIR") or HERE.parent.parent / "reference")
    kern = ref / "token2tile" / "operator" / "kernels"
    kmm, sel = kern / "kmeans_maintain" / "src", kern / "select_union" / "src"
    if not (kmm / "kernels.cu").exists():
        print(f"reference sources not found under {ref}; keeping any prebuilt {OUT}")
        return 0
    OUT.mkdir(exist_ok=True)
    flags = ["-O3", "--use_fast_math", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
             "-gencode=arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
             "-DANGR=6", "-DAMINB=2", "-DAW_NTILE=256"]
    cmd = ["nvcc", "-shared", *flags, f"-I{kmm}", f"-I{sel}", str(HERE / "ref_wrap.cu"), str(kmm / "kernels.cu"),
           str(sel / "kernel.cu"), "-o", str(OUT / "libt2t_ref.so")]
    subprocess.run(cmd, check=True)
    print(OUT / "libt2t_ref.so")
    return 0


if __name__ == "__main__":
    sys.exit(main())
