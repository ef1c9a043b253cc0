"""The operator as a caller uses it (MaskedStepDeploy), against the CPU oracle."""
import math

import pytest
import torch

from oracle import t2t_oracle as O

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
DEV = "cuda"


def _bits(t):
    return t.view(torch.int16) if t.dtype == BF else t


def _check_structure(op, c, state_before, ns, pin_tail=0):
    """Teacher-forced stage check: the oracle recomputes every stage from the
    device's own inputs to that stage."""
    S = op.last_structure
    QU, KU = op.QU.cpu(), op.KU.cpu()
    want_QU = O.project(c["q"], state_before["Uq"], BF).float()
    assert (QU.float() - want_QU).abs().max() <= want_QU.abs().max() * 2.0 ** -7
    km = O.kmeans_maintain(QU, KU, c["v"], state_before["cq"], state_before["ck"], pin_tail, BF)
    for mine, theirs in (("qlab", "qlab"), ("klab", "klab"), ("qperm", "qperm"), ("kperm", "kperm"),
                         ("tile_sizes", "qcounts"), ("counts", "kcounts")):
        assert torch.equal(S[mine].cpu(), km[theirs]), mine
    assert torch.equal(op._kmm_ck2.cpu(), km["ck2"])
    cks = (km["ck2"] * op.scale).to(BF)
    assert torch.equal(_bits(S["cks"].cpu()), _bits(cks))
    unip, rowcnt = O.select_union(QU, cks, km["kcounts"], km["qlab"], op.CQ, ns, pin_tail)
    assert torch.equal(op.rowcnt.cpu(), rowcnt)
    assert torch.equal(S["unip"].cpu(), unip)
    return km, cks, unip


def test_operator_rebuild_then_reuse(small_case):
    from token2tile_b200 import MaskedStepDeploy
    c = small_case
    H, N, CQ = c["H"], c["N"], c["CQ"]
    op = MaskedStepDeploy(H, N, CQ, s_frac=0.05, mask_refresh=4)
    q, k, v = (c[n].to(DEV) for n in "qkv")
    state = {n: t.to(DEV) for n, t in c["state"].items()}
    before = {n: t.clone() for n, t in c["state"].items()}

    op.set_cfg_call(0, key=0, step=0)
    out = op.step(q, k, v, state).cpu().float()
    torch.cuda.synchronize()
    assert op.device_status() == 0 and op.last_rebuilt is True
    km, cks, unip = _check_structure(op, c, before, op.ns)
    assert torch.equal(_bits(state["cq"].cpu()), _bits(km["cq2"]))
    assert torch.equal(_bits(state["ck"].cpu()), _bits(km["ck2"].to(BF)))

    QU = op.QU.cpu()
    o, lse = O.exact_attention(c["q"], c["k"], c["v"], km["qlab"], km["klab"], unip, op.scale)
    want = O.residual_merge(o, lse, QU, cks, km["sumv"], km["lam"], km["kcounts"], unip, km["qlab"], 1.0)
    err = (out - want).abs()
    assert err.max() < 2e-2 and err.mean() < 2e-3, (err.max(), err.mean())
    dense = O.dense_attention(c["q"], c["k"], c["v"], op.scale)
    rel = ((out - dense).norm() / dense.norm()).item()
    assert rel < 0.05, rel

    # parity-1 call of the same step reuses the structure with new values
    g = torch.Generator().manual_seed(5)
    q2 = (c["q"].float() + 0.05 * torch.randn(c["q"].shape, generator=g)).to(BF)
    v2 = torch.randn(c["v"].shape, generator=g).to(BF)
    op.set_cfg_call(1, key=0, step=0)
    out2 = op.step(q2.to(DEV), k, v2.to(DEV), state).cpu().float()
    torch.cuda.synchronize()
    assert op.device_status() == 0 and op.last_rebuilt is False
    QU2 = op.QU.cpu()
    _, sumv2, lam2, _ = O.vstats(v2, km["kperm"], km["kcounts"], BF)
    o2, lse2 = O.exact_attention(q2, c["k"], v2, km["qlab"], km["klab"], unip, op.scale)
    want2 = O.residual_merge(o2, lse2, QU2, cks, sumv2, lam2, km["kcounts"], unip, km["qlab"], 1.0)
    err2 = (out2 - want2).abs()
    assert err2.max() < 2e-2 and err2.mean() < 2e-3, (err2.max(), err2.mean())

    # step 4, parity 0: refresh is due
    op.set_cfg_call(0, key=0, step=4)
    op.step(q, k, v, state)
    assert op.last_rebuilt is True
    op.set_cfg_call(0, key=0, step=5)
    op.step(q, k, v, state)
    assert op.last_rebuilt is False
    torch.cuda.synchronize()
    assert op.device_status() == 0


def test_operator_is_deterministic(small_case):
    from token2tile_b200 import MaskedStepDeploy
    c = small_case
    op = MaskedStepDeploy(c["H"], c["N"], c["CQ"], s_frac=0.05)
    q, k, v = (c[n].to(DEV) for n in "qkv")
    outs = []
    for _ in range(2):
        state = {n: t.to(DEV) for n, t in c["state"].items()}
        outs.append(op.step(q, k, v, state).clone())
    torch.cuda.synchronize()
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))


def test_caller_owned_output_tensor(small_case):
    """step(..., out=t) writes the same bits into t and leaves the previous result alone."""
    from token2tile_b200 import MaskedStepDeploy
    c = small_case
    op = MaskedStepDeploy(c["H"], c["N"], c["CQ"], s_frac=0.05)
    q, k, v = (c[n].to(DEV) for n in "qkv")
    state = {n: t.to(DEV) for n, t in c["state"].items()}
    ref = op.step(q, k, v, state).clone()
    mine = torch.full_like(ref, 7.0)
    state = {n: t.to(DEV) for n, t in c["state"].items()}
    got = op.step(q, k, v, state, out=mine)
    torch.cuda.synchronize()
    assert got is mine and torch.equal(mine.view(torch.int16), ref.view(torch.int16))
    with pytest.raises(ValueError):
        op.step(q, k, v, state, out=mine.float())
    with pytest.raises(ValueError):
        op.step(q, k, v, state, out=mine[:, :-1])


def test_views_of_token_major_tensors_are_read_and_written_in_place(small_case):
    """q, k, v and the output as [H, N, 128] views of tensors stored [N, H, 128] (what a serving host holds):
    same bits as with contiguous tensors, for a rebuild call, a reuse call and init_state."""
    from token2tile_b200 import MaskedStepDeploy
    c = small_case
    H, N, CQ = c["H"], c["N"], c["CQ"]
    q, k, v = (c[n].to(DEV) for n in "qkv")
    token_major = lambda t: t.transpose(0, 1).contiguous().transpose(0, 1)      # [H, N, D] view of [N, H, D] storage
    qs, ks, vs = token_major(q), token_major(k), token_major(v)
    assert not qs.is_contiguous() and qs.stride() == (128, H * 128, 1)
    results = []
    for tensors, strided_out in (((q, k, v), False), ((qs, ks, vs), True)):
        op = MaskedStepDeploy(H, N, CQ, s_frac=0.05, mask_refresh=4)
        state = op.init_state(tensors[0], tensors[1], warm_iters=2, seed=3)
        out = torch.zeros(N, H, 128, dtype=BF, device=DEV).transpose(0, 1) if strided_out else None
        op.set_cfg_call(0, key=0, step=0)
        first = op.step(*tensors, state, out=out).clone()
        op.set_cfg_call(1, key=0, step=0)
        second = op.step(*tensors, state, out=out).clone()
        torch.cuda.synchronize()
        assert op.device_status() == 0 and op.last_rebuilt is False
        results.append((state, first.contiguous(), second.contiguous()))
    (st_a, a1, a2), (st_b, b1, b2) = results
    for name in ("Uq", "Uk", "ck", "cq"):
        assert torch.equal(st_a[name].view(torch.int16), st_b[name].view(torch.int16)), name
    assert torch.equal(a1.view(torch.int16), b1.view(torch.int16))
    assert torch.equal(a2.view(torch.int16), b2.view(torch.int16))
    with pytest.raises(ValueError):
        op.step(qs[:, :, :].float(), ks, vs, state)
    with pytest.raises(ValueError):                                      # rows that are not contiguous
        bad = torch.zeros(H, N, 256, dtype=BF, device=DEV)[:, :, ::2]
        op.step(bad, ks, vs, state)


def test_init_state_projection_fit(small_case):
    from token2tile_b200 import MaskedStepDeploy
    c = small_case
    op = MaskedStepDeploy(c["H"], c["N"], c["CQ"], s_frac=0.05)
    q, k = c["q"].to(DEV), c["k"].to(DEV)
    st = op.init_state(q, k, warm_iters=2, seed=0)
    assert st["Uq"].shape == (c["H"], 128, 32) and st["ck"].shape == (c["H"], 2048, 32)
    assert st["cq"].shape == (c["H"], c["CQ"], 32)
    Uq, Uk = O.online_u(c["q"].float(), c["k"].float(), 32)
    want = torch.bmm(Uq.to(BF).float(), Uk.to(BF).float().transpose(1, 2))
    got = torch.bmm(st["Uq"].cpu().float(), st["Uk"].cpu().float().transpose(1, 2))
    assert (got - want).abs().max() <= 0.02 * want.abs().max()
    # the warm iterations, redone by the oracle from the device's projections
    KU = torch.empty(c["H"], c["N"], 32, dtype=BF, device=DEV)
    QU = torch.empty_like(KU)
    s = torch.cuda.current_stream().cuda_stream
    op._project(k, st["Uk"], KU, s)
    op._project(q, st["Uq"], QU, s)
    torch.cuda.synchronize()
    KU, QU = KU.cpu(), QU.cpu()
    g = torch.Generator(device="cpu").manual_seed(0)
    ck = KU[:, O.sample_rows(c["N"], 2048, g), :].contiguous()
    cq = QU[:, O.sample_rows(c["N"], c["CQ"], g), :].contiguous()
    for _ in range(2):
        ck, _ = O.fixed_point_mean(KU, O.assign(KU, ck), ck, BF)
        cq, _ = O.fixed_point_mean(QU, O.assign(QU, cq), cq, BF)
    assert torch.equal(_bits(st["ck"].cpu()), _bits(ck))
    assert torch.equal(_bits(st["cq"].cpu()), _bits(cq))


def test_argument_errors(small_case):
    from token2tile_b200 import MaskedStepDeploy
    with pytest.raises(ValueError):
        MaskedStepDeploy(2, 4096, 32, C=1024)
    with pytest.raises(ValueError):
        MaskedStepDeploy(2, 4096, 32, D=64)
    c = small_case
    op = MaskedStepDeploy(c["H"], c["N"], c["CQ"])
    q = c["q"].to(DEV)
    with pytest.raises(ValueError):
        op.step(q.float(), q, q, {})
    bad = q.clone()
    bad[0, 0, 0] = float("nan")
    with pytest.raises(RuntimeError):
        op.init_state(bad, q)


def test_head_sharding_is_bitwise_neutral(small_case):
    """Heads never interact: running each head in its own operator (what a rank
    of a head-parallel layout does) gives the bits of the joint run."""
    from token2tile_b200 import MaskedStepDeploy
    c = small_case
    H, N, CQ = c["H"], c["N"], c["CQ"]
    q, k, v = (c[n].to(DEV) for n in "qkv")
    joint = MaskedStepDeploy(H, N, CQ, s_frac=0.05)
    out = joint.step(q, k, v, {n: t.to(DEV) for n, t in c["state"].items()}).clone()
    torch.cuda.synchronize()
    for h in range(H):
        part = MaskedStepDeploy(1, N, CQ, s_frac=0.05)
        st = {n: t[h:h + 1].contiguous().to(DEV) for n, t in c["state"].items()}
        o = part.step(q[h:h + 1].contiguous(), k[h:h + 1].contiguous(), v[h:h + 1].contiguous(), st)
        torch.cuda.synchronize()
        assert part.device_status() == 0
        assert torch.equal(o.view(torch.int16), out[h:h + 1].view(torch.int16))
        assert torch.equal(part.last_structure["unip"], joint.last_structure["unip"][h:h + 1])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_devices_give_the_same_bits(small_case):
    from token2tile_b200 import MaskedStepDeploy
    c = small_case
    outs = []
    for dev in ("cuda:0", "cuda:1"):
        with torch.cuda.device(dev):
            op = MaskedStepDeploy(c["H"], c["N"], c["CQ"], s_frac=0.05, device=dev)
            o = op.step(*(c[n].to(dev) for n in "qkv"), {n: t.to(dev) for n, t in c["state"].items()})
            torch.cuda.synchronize(dev)
            outs.append(o.cpu())
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))


@pytest.mark.parametrize("CQ", [4, 7])
def test_operator_with_few_large_query_clusters(small_case, CQ):
    """Query clusters of ~600-1000 rows: several full 256-row attention tasks plus
    a remainder per cluster (both attention kernels), an odd cluster count."""
    from token2tile_b200 import MaskedStepDeploy
    c = dict(small_case, CQ=CQ)
    H, N = c["H"], c["N"]
    op = MaskedStepDeploy(H, N, CQ, s_frac=0.03)
    q, k, v = (c[n].to(DEV) for n in "qkv")
    state = op.init_state(q, k, warm_iters=2, seed=1)
    before = {n: t.cpu().clone() for n, t in state.items()}
    out = op.step(q, k, v, state).cpu().float()
    torch.cuda.synchronize()
    assert op.device_status() == 0
    km, cks, unip = _check_structure(op, c, before, op.ns)
    sizes = km["qcounts"]
    assert int(sizes.max()) > 256                    # at least one cluster is split into several tasks
    tasks, pairs = op.plan_info()
    want_tasks = int(((sizes + 255) // 256).sum())
    assert tasks == want_tasks
    o, lse = O.exact_attention(c["q"], c["k"], c["v"], km["qlab"], km["klab"], unip, op.scale)
    want = O.residual_merge(o, lse, op.QU.cpu(), cks, km["sumv"], km["lam"], km["kcounts"], unip, km["qlab"], 1.0)
    err = (out - want).abs()
    assert err.max() < 2e-2 and err.mean() < 2e-3, (err.max(), err.mean())


def test_module_level_helpers_of_the_reference_module(small_case):
    """fast_assign / fused_update_vstats / fast_gather, the names the reference's
    hosts reach through the operator module, against the oracle."""
    import token2tile_b200.deploy_step as D
    c = small_case
    QU = O.project(c["q"], c["state"]["Uq"], BF)
    cq = c["state"]["cq"]
    lab = D.fast_assign(QU.to(DEV), cq.to(DEV))
    assert torch.equal(lab.cpu(), O.assign(QU, cq, 0))
    newc, counts, mean_v = D.fused_update_vstats(QU.to(DEV), lab, cq.to(DEV), None)
    want_c, want_counts = O.fixed_point_mean(QU, lab.cpu(), cq, BF)
    assert mean_v is None and torch.equal(counts.cpu(), want_counts)
    assert torch.equal(newc.cpu().view(torch.int16), want_c.view(torch.int16))
    g = torch.Generator().manual_seed(4)
    p = torch.stack([torch.randperm(c["N"], generator=g) for _ in range(c["H"])])
    got = D.fast_gather(c["k"].to(DEV), p.to(DEV))
    assert torch.equal(got.cpu().view(torch.int16),
                       torch.gather(c["k"], 1, p[..., None].expand(-1, -1, 128)).view(torch.int16))
    with pytest.raises(NotImplementedError):
        D.fused_update_vstats(QU.to(DEV), lab, cq.to(DEV), c["v"].to(DEV))
