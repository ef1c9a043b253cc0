"""The C ABI without a GPU: the library loads, exports every declared symbol,
and rejects bad arguments before touching the device."""
import re
from pathlib import Path

from token2tile_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "t2t_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(t2t_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    names = declared_symbols()
    assert len(names) >= 19
    for n in names:
        assert hasattr(lib, n), n
    assert set(_lib.SIGNATURES) == set(names)
    assert lib.t2t_version() >= 100


def test_workspace_sizes_are_pure_host_functions(lib):
    assert lib.t2t_kmeans_maintain_ws_bytes(40, 75600, 512, 2048) > 40 * 75600 * 4
    assert lib.t2t_vstats_gather_ws_bytes(40, 2048) >= 40 * 2048 * 128 * 4
    assert lib.t2t_tile_attn_ws_bytes(2, 4096) >= 2 * 4096 * (256 + 4)
    ints = lib.t2t_tile_attn_plan_ints(40, 75600, 512)
    assert ints >= 40 * 2049 + 4 * 40 * (512 + 75600 // 256) + 40 * 512
    assert lib.t2t_centroid_update_ws_bytes(2, 4096, 2048) > 0


def test_null_and_bad_arguments_are_rejected(lib):
    assert lib.t2t_project(0, 0, 0, 1, 1, 0, 0) == 1
    assert lib.t2t_assign(0, 0, 0, 2, 4096, 32, -1, 0, 0, 0, 0, 0) == 1
    assert lib.t2t_assign_exact(0, 0, 0, 2, 4096, 32, -1, 0, 0) == 1
    assert lib.t2t_gather_rows(0, 0, 0, 2, 4096, 0) == 1
    assert lib.t2t_score_select_union(0, 0, 0, 0, 0, 0, 0, 0, 2, 4096, 32, 0, 0, 0, 0, 0) == 1
    assert lib.t2t_score_select_union_exact(0, 0, 0, 0, 0, 0, 0, 0, 2, 4096, 32, 0, 0) == 1
    assert lib.t2t_vstats_gather(0, 0, 0, 0, 0, 0, 2, 4096, 2048, 0, 0, 0) == 1
    assert lib.t2t_tile_attn_plan(0, 0, 0, 0, 2, 4096, 32, 0) == 1
    assert lib.t2t_umma_selftest(0, 0, 0, 0, 0, 0, 0) == 1
    assert lib.t2t_gather4_selftest(0, 0, 0, 0, 0, 0) == 1
    assert lib.t2t_wait_timeout_selftest(0, 0, 0) == 1


def test_operator_dir_points_at_the_sources():
    import token2tile_b200
    d = Path(token2tile_b200.operator_dir())
    assert (d / "deploy_step.py").exists() and (d / "csrc" / "tile_attn.cu").exists()
