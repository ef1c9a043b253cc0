"""The operator at the 480p and 720p layer shapes (one head of each), against the CPU oracle.

These are the sizes at which the kernels' fast paths actually run: the window
search and the re-queue of the selection, the near-tie re-check of the
assignment, unions of many 128-key tiles, query clusters above and below one
tensor-core tile, several attention tasks per query cluster.  Every stage is
teacher-forced: the oracle recomputes it from the device's own inputs to that
stage, so integer outputs (labels, counts, permutations, scoring centroids,
union bitmaps, row counts, executed pairs) must match bit for bit; the bf16
output is compared with the oracle's exact attention + residual merge within
max-abs 2e-2 / mean-abs 2e-3 (the tolerance of the operator's contract).
"""
import pytest
import torch

from oracle import t2t_oracle as O

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
DEV = "cuda"
MAX_ABS, MEAN_ABS = 2e-2, 2e-3

# grid, query clusters, head of the 40-head layer, budgets (the first one also gets a reuse call)
CASES = [
    ("480p", 256, 3, (0.015, 0.05)),
    ("720p", 512, 17, (0.015, 0.0125, 0.05)),
]


def _bits(t):
    return t.view(torch.int16) if t.dtype == BF else t


def _close(got, want, what):
    err = (got - want).abs()
    assert err.max() < MAX_ABS and err.mean() < MEAN_ABS, (what, float(err.max()), float(err.mean()))


@pytest.mark.parametrize("grid,CQ,head,budgets", CASES, ids=[c[0] for c in CASES])
def test_layer_shape_against_the_oracle(grid, CQ, head, budgets):
    from token2tile_b200 import MaskedStepDeploy
    from token2tile_b200.synth import GRIDS, grid_tokens, locality_mixture
    N = grid_tokens(GRIDS[grid])
    q, k, v = locality_mixture(1, GRIDS[grid], heads=[head])
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)

    first = MaskedStepDeploy(1, N, CQ, s_frac=budgets[0], mask_refresh=4)
    state0 = first.init_state(qd, kd, warm_iters=2, seed=0)
    before = {n: t.cpu().clone() for n, t in state0.items()}

    km = cks = QU = None
    unions = None
    for bi, frac in enumerate(budgets):
        op = first if bi == 0 else MaskedStepDeploy(1, N, CQ, s_frac=frac)
        state = {n: t.to(DEV).clone() for n, t in before.items()}
        if bi == 0:
            op.set_cfg_call(0, key=0, step=0)
        out = op.step(qd, kd, vd, state).float().cpu()
        torch.cuda.synchronize()
        assert op.device_status() == 0 and op.last_rebuilt is True
        S = op.last_structure
        if km is None:
            # clustering does not depend on the budget: checked once, from the device's own projections
            QU, KU = op.QU.cpu(), op.KU.cpu()
            want_QU = O.project(q, before["Uq"], BF).float()
            assert (QU.float() - want_QU).abs().max() <= want_QU.abs().max() * 2.0 ** -7
            km = O.kmeans_maintain(QU, KU, v, before["cq"], before["ck"], 0, BF)
            cks = (km["ck2"] * op.scale).to(BF)
            unions = O.select_union_budgets(QU, cks, km["kcounts"], km["qlab"], CQ,
                                            [max(1, int(f * N)) for f in budgets])
            assert torch.equal(op._kmm_ck2.cpu(), km["ck2"])
            assert torch.equal(_bits(state["cq"].cpu()), _bits(km["cq2"]))
            assert torch.equal(_bits(state["ck"].cpu()), _bits(km["ck2"].to(BF)))
            assert torch.equal(_bits(op._kmm_sumv.cpu()), _bits(km["sumv"]))
            assert torch.equal(op._kmm_lam.cpu(), km["lam"])
        else:
            assert torch.equal(_bits(op.QU.cpu()), _bits(QU))       # same kernels, same inputs, same bits
        for mine, theirs in (("qlab", "qlab"), ("klab", "klab"), ("qperm", "qperm"), ("kperm", "kperm"),
                             ("tile_sizes", "qcounts"), ("counts", "kcounts")):
            assert torch.equal(S[mine].cpu(), km[theirs]), (mine, frac)
        assert torch.equal(_bits(S["cks"].cpu()), _bits(cks))
        unip, rowcnt = unions[bi]
        assert op.ns == max(1, int(frac * N))
        assert torch.equal(op.rowcnt.cpu(), rowcnt), frac
        assert torch.equal(S["unip"].cpu(), unip), frac
        kv_len = O.kv_lengths(unip, km["qcounts"], km["kcounts"])
        _, pairs = op.plan_info()
        assert pairs == int((km["qcounts"].long() * kv_len.long()).sum()), frac

        o, lse = O.exact_attention(q, k, v, km["qlab"], km["klab"], unip, op.scale)
        want = O.residual_merge(o, lse, QU, cks, km["sumv"], km["lam"], km["kcounts"], unip, km["qlab"], 1.0)
        _close(out, want, f"{grid} budget {frac}")

        if bi == 0:
            # the other CFG branch of the same step reuses the structure with its own q and v
            g = torch.Generator().manual_seed(5)
            q2 = (q.float() + 0.05 * torch.randn(q.shape, generator=g)).to(BF)
            v2 = torch.randn(v.shape, generator=g).to(BF)
            op.set_cfg_call(1, key=0, step=0)
            out2 = op.step(q2.to(DEV), kd, v2.to(DEV), state).float().cpu()
            torch.cuda.synchronize()
            assert op.device_status() == 0 and op.last_rebuilt is False
            QU2 = op.QU.cpu()
            _, sumv2, lam2, _ = O.vstats(v2, km["kperm"], km["kcounts"], BF)
            assert torch.equal(_bits(op._kmm_sumv.cpu()), _bits(sumv2)) and torch.equal(op._kmm_lam.cpu(), lam2)
            o2, lse2 = O.exact_attention(q2, k, v2, km["qlab"], km["klab"], unip, op.scale)
            want2 = O.residual_merge(o2, lse2, QU2, cks, sumv2, lam2, km["kcounts"], unip, km["qlab"], 1.0)
            _close(out2, want2, f"{grid} reuse call")
