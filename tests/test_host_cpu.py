"""Host-side logic of the operator and the multi-GPU plumbing, on the CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from token2tile_b200 import parallel
from token2tile_b200.synth import GRIDS, grid_tokens, locality_mixture


def _bare_operator(mask_refresh, cfg_reuse=False):
    from token2tile_b200.deploy_step import MaskedStepDeploy
    op = MaskedStepDeploy.__new__(MaskedStepDeploy)
    op.mask_refresh = mask_refresh
    op.cfg_reuse = cfg_reuse
    op._cfg_on = cfg_reuse or mask_refresh > 1
    op._cfg_hold, op._cfg_parity, op._cfg_key, op._cfg_step = {}, None, 0, 0
    op._struct = {"name": "shared"}
    op._new_structure = lambda: {"name": "fresh"}
    return op


def _run_schedule(op, calls):
    out = []
    for parity, key, step in calls:
        if parity is not None:
            op.set_cfg_call(parity, key=key, step=step)
        snap, target, publish = op._pick()
        if snap is None:
            target["step"] = op._cfg_step
            if publish:
                op._cfg_hold[op._cfg_key] = target
        out.append("reuse" if snap is not None else "rebuild")
    return out


def test_rebuild_reuse_schedule_matches_the_reference_rule():
    op = _bare_operator(mask_refresh=4)
    calls = [(p, 0, s) for s in range(9) for p in (0, 1)]
    got = _run_schedule(op, calls)
    want = []
    held = None
    for p, _, s in calls:
        age = None if held is None else s - held
        reuse = held is not None and age >= 0 and not (p == 0 and age >= 4)
        want.append("reuse" if reuse else "rebuild")
        if not reuse:
            held = s
    assert got == want
    assert got[:2] == ["rebuild", "reuse"] and got[8] == "rebuild" and got.count("rebuild") == 3


def test_unannotated_calls_always_rebuild_and_do_not_consume_annotations():
    op = _bare_operator(mask_refresh=4)
    assert _run_schedule(op, [(None, 0, 0), (None, 0, 0)]) == ["rebuild", "rebuild"]
    assert _run_schedule(op, [(0, 3, 0), (None, 0, 0), (1, 3, 0)]) == ["rebuild", "rebuild", "reuse"]


def test_unannotated_rebuild_is_stored_under_the_last_annotation_like_the_reference():
    """With snapshots switched on the reference stores every rebuild, also the one of a call without
    set_cfg_call, under the key and step of the last annotation (deploy_step.py:420-440); a later
    annotated branch-1 call of that key then reuses it."""
    op = _bare_operator(mask_refresh=4)
    assert _run_schedule(op, [(None, 0, 0)]) == ["rebuild"]
    assert list(op._cfg_hold) == [0] and op._cfg_hold[0]["name"] == "fresh" and op._cfg_hold[0]["step"] == 0
    assert _run_schedule(op, [(1, 0, 0)]) == ["reuse"]
    first = op._cfg_hold[0]
    assert _run_schedule(op, [(None, 0, 0)]) == ["rebuild"]
    assert op._cfg_hold[0] is not first              # tensors of its own, the old snapshot is left alone
    # snapshots off: nothing is stored and the shared structure is used
    off = _bare_operator(mask_refresh=1)
    assert _run_schedule(off, [(None, 0, 0), (0, 0, 0), (1, 0, 0)]) == ["rebuild"] * 3
    assert off._cfg_hold == {}


def test_step_counter_going_backwards_and_reset_force_a_rebuild():
    op = _bare_operator(mask_refresh=4)
    assert _run_schedule(op, [(0, 1, 10), (1, 1, 10), (1, 1, 2)]) == ["rebuild", "reuse", "rebuild"]
    op.reset_cfg_reuse()
    assert _run_schedule(op, [(1, 1, 2)]) == ["rebuild"]


def test_layers_keep_separate_snapshots_and_recycle_their_tensors():
    op = _bare_operator(mask_refresh=2)
    _run_schedule(op, [(0, "a", 0), (0, "b", 0)])
    a0, b0 = op._cfg_hold["a"], op._cfg_hold["b"]
    assert a0 is not b0
    _run_schedule(op, [(0, "a", 2)])
    assert op._cfg_hold["a"] is a0 and a0["step"] == 2 and b0["step"] == 0


def test_cfg_reuse_with_refresh_one_rebuilds_every_branch_zero_call():
    op = _bare_operator(mask_refresh=1, cfg_reuse=True)
    got = _run_schedule(op, [(0, 0, 0), (1, 0, 0), (0, 0, 1), (1, 0, 1)])
    assert got == ["rebuild", "reuse", "rebuild", "reuse"]


def test_head_ranges_tile_the_heads():
    for H, world in ((40, 1), (40, 2), (40, 4), (40, 8), (12, 5)):
        spans = [parallel.head_range(r, world, H) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == H
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1
    assert [parallel.head_range(r, 8, 40) for r in (0, 7)] == [(0, 5), (35, 40)]


def test_synthetic_heads_are_independent_of_the_sharding():
    grid = (2, 8, 8)
    full = locality_mixture(4, grid)
    part = locality_mixture(2, grid, heads=[2, 3])
    for a, b in zip(full, part):
        assert torch.equal(a[2:], b)
    assert grid_tokens(GRIDS["720p"]) == 75600 and grid_tokens(GRIDS["480p"]) == 32760


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ulysses_worker(rank, world, port, q, N, H, D):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        full = torch.randn(N, H, D, generator=g)
        n = N // world
        mine = full[rank * n:(rank + 1) * n].contiguous()
        heads = parallel.seq_to_head(mine)
        lo, hi = parallel.head_range(rank, world, H)
        ok = torch.equal(heads, full[:, lo:hi])
        # head-parallel "attention": anything that only mixes tokens inside a head
        back = parallel.head_to_seq((heads * 2.0).contiguous())
        ok = ok and torch.equal(back, mine * 2.0)
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_ulysses_all_to_all_round_trip_on_gloo(world):
    from conftest import run_gloo_ranks
    res = sorted(run_gloo_ranks(_ulysses_worker, world, args=(24, 4, 8)))
    assert res == [(r, True) for r in range(world)]
