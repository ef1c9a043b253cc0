"""ctypes binding of libt2t_b200.so (the C ABI declared in include/t2t_b200.h).

There is no fallback: if the shared library has not been built the import of
the operator fails with instructions, and every call checks its return code.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libt2t_b200.so"
_lib = None

ERRORS = {1: "bad argument", 2: "CUDA launch failed", 3: "workspace too small",
          4: "shape exceeds the fixed capacity of a no-allocation entry point"}
STATUS = {0: "ok", 1: "a bounded device wait timed out", 2: "task plan exceeded its bounds"}

_P, _I, _S, _F, _L = C.c_void_p, C.c_int, C.c_size_t, C.c_float, C.c_longlong

SIGNATURES = {
    "t2t_version": (_I, []),
    "t2t_project": (_I, [_P, _P, _P, _I, _I, _P, _P]),
    "t2t_lowrank_fit_ws_bytes": (_S, [_I, _I]),
    "t2t_lowrank_fit": (_I, [_P, _P, _P, _P, _I, _I, _P, _S, _P, _P, _P]),
    "t2t_assign_ws_bytes": (_S, [_I, _I]),
    "t2t_assign": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _P, _S, _P, _P]),
    "t2t_assign_exact": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "t2t_centroid_update_ws_bytes": (_S, [_I, _I, _I]),
    "t2t_centroid_update": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _P, _S, _P]),
    "t2t_kmeans_maintain_ws_bytes": (_S, [_I, _I, _I, _I]),
    "t2t_kmeans_maintain": (_I, [_P] * 18 + [_F, _I, _I, _I, _I, _I, _P, _S, _P, _P]),
    "t2t_vstats_gather_ws_bytes": (_S, [_I, _I]),
    "t2t_vstats_gather": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _S, _P]),
    "t2t_vstats_gather_static_max_hc": (_S, []),
    "t2t_vstats_gather_static": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "t2t_gather_rows": (_I, [_P, _P, _P, _I, _I, _P]),
    "t2t_score_select_union_ws_bytes": (_S, [_I, _I]),
    "t2t_score_select_union": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _S, _P, _P]),
    "t2t_score_select_union_exact": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "t2t_tile_attn_plan_ints": (_S, [_I, _I, _I]),
    "t2t_tile_attn_ws_bytes": (_S, [_I, _I]),
    "t2t_tile_attn": (_I, [_P] * 15 + [_I, _I, _I, _I, _P, _S, _P, _P]),
    "t2t_tile_attn_plan": (_I, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "t2t_tile_attn_exact": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _S, _P, _P]),
    "t2t_tile_attn_merge": (_I, [_P] * 10 + [_I, _I, _I, _P, _S, _P, _P]),
    "t2t_tile_attn_plan_info": (_I, [_P, _I, _I, _I, _P, _P]),
    "t2t_project_strided": (_I, [_P, _L, _L, _P, _P, _I, _I, _P, _P]),
    "t2t_lowrank_fit_strided": (_I, [_P, _P, _L, _L, _P, _P, _I, _I, _P, _S, _P, _P, _P]),
    "t2t_gather_rows_strided": (_I, [_P, _L, _L, _P, _P, _I, _I, _P]),
    "t2t_kmeans_maintain_strided": (_I, [_P, _P, _P, _L, _L] + [_P] * 15 + [_F, _I, _I, _I, _I, _I, _P, _S, _P, _P]),
    "t2t_vstats_gather_strided": (_I, [_P, _L, _L, _P, _P, _P, _P, _P, _I, _I, _I, _P, _S, _P]),
    "t2t_tile_attn_exact_strided": (_I, [_P, _L, _L, _P, _P, _P, _P, _P, _I, _I, _I, _P, _S, _P, _P]),
    "t2t_tile_attn_merge_strided": (_I, [_P] * 10 + [_L, _L, _I, _I, _I, _P, _S, _P, _P]),
    "t2t_umma_selftest": (_I, [_P, _P, _P, _P, _P, _P, _P]),
    "t2t_gather4_selftest": (_I, [_P, _I, _P, _P, _P, _P]),
    "t2t_wait_timeout_selftest": (_I, [_P, _P, _P]),
}


def lib_path() -> Path:
    return _LIB_PATH


def load():
    """Loads the shared library once and sets the argument types."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH.name} is not built; run `python -m token2tile_b200.build` "
                "(needs nvcc with sm_100a support). There is no CPU or PyTorch fallback.")
        lib = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed: {ERRORS.get(code, code)}")


def ptr(t) -> int:
    """Device pointer of a tensor (None -> NULL)."""
    return 0 if t is None else t.data_ptr()
