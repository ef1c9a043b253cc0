"""The CPU oracle against the reference's golden vectors and against
independent brute-force restatements of its integer rules."""
import math
import random
from pathlib import Path

import pytest
import torch

from oracle import t2t_oracle as O

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_online_u_matches_reference_golden():
    import importlib.util
    spec = importlib.util.spec_from_file_location("mk", GOLDEN / "make_online_u_golden.py")
    mk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mk)
    for item in torch.load(GOLDEN / "online_u.pt"):
        q, k = mk.make_inputs(item["case"])
        Uq, Uk = O.online_u(q, k, item["case"]["r"])
        want = torch.bmm(item["Uq"], item["Uk"].transpose(1, 2))
        got = torch.bmm(Uq, Uk.transpose(1, 2))
        assert (got - want).abs().max() <= 1e-4 * want.abs().max()
        # the logit approximation it is fitted for
        s_want = torch.bmm(torch.bmm(q, item["Uq"]), torch.bmm(k, item["Uk"]).transpose(1, 2))
        s_got = torch.bmm(torch.bmm(q, Uq), torch.bmm(k, Uk).transpose(1, 2))
        assert (s_got - s_want).norm() <= 1e-4 * s_want.norm()


def test_online_u_rejects_non_finite():
    q = torch.randn(1, 64, 128)
    q[0, 3, 5] = float("inf")
    with pytest.raises(RuntimeError):
        O.online_u(q, torch.randn(1, 64, 128))


def test_key_transform_is_monotone_with_signed_zero():
    # -1e-9 rounds to the fp16 value -0, which must order below +0
    vals = torch.tensor([-65504.0, -3.5, -1.0, -6e-8, -1e-9, 0.0, 6e-8, 0.33, 1.0, 1.001, 7.0, 65504.0])
    QU = torch.zeros(len(vals), 32)
    QU[:, 0] = 1.0
    cks = torch.zeros(1, 32)
    cks[0, 0] = 1.0
    keys = torch.cat([O.score_keys(v * QU[:1], cks) for v in vals]).flatten().tolist()
    assert keys == sorted(keys) and len(set(keys)) == len(keys)


def _brute_select(keys, sizes, ns):
    order = sorted(range(len(keys)), key=lambda c: (-keys[c], c))
    sel, run, rc = set(), 0, None
    for c in order:
        if run < ns:
            sel.add(c)
            if run + sizes[c] >= ns and rc is None:
                rc = run + sizes[c]
        run += sizes[c]
    return sel, rc if rc is not None else run


@pytest.mark.parametrize("seed", range(6))
def test_select_rows_against_brute_force(seed):
    rnd = random.Random(seed)
    C = 64
    keys = [rnd.randint(-4, 4) for _ in range(C)]                 # heavy ties
    sizes = [rnd.choice([0, 0, 1, 2, 5, 9]) for _ in range(C)]    # empty clusters
    total = sum(sizes)
    for ns in (1, 2, 7, max(1, total // 2), total):
        sel, rc = O.select_rows(torch.tensor([keys], dtype=torch.int16), torch.tensor(sizes, dtype=torch.int32), ns)
        want_sel, want_rc = _brute_select(keys, sizes, ns)
        assert set(sel[0].nonzero().flatten().tolist()) == want_sel
        assert int(rc[0]) == want_rc


def test_bitmap_layout_is_lsb_first():
    sel = torch.zeros(2, 2048, dtype=torch.bool)
    sel[0, 0] = sel[0, 31] = sel[0, 32] = sel[1, 2047] = True
    w = O.pack_bits(sel)
    assert w.shape == (2, 64)
    assert int(w[0, 0]) == ((1 | (1 << 31)) ^ 0x80000000) - 0x80000000 and int(w[0, 1]) == 1
    assert int(w[1, 63]) == -(1 << 31)
    assert torch.equal(O.unpack_bits(w, 2048), sel)
    assert torch.equal(w.view(torch.uint8).reshape(2, 256)[0, :5], torch.tensor([1, 0, 0, 128, 1], dtype=torch.uint8))


def test_stable_group_keeps_row_order():
    g = torch.Generator().manual_seed(1)
    lab = torch.randint(0, 17, (2, 500), generator=g).to(torch.int32)
    counts, perm = O.stable_group(lab, 20)
    for h in range(2):
        pos = 0
        for c in range(20):
            rows = [i for i in range(500) if int(lab[h, i]) == c]
            assert int(counts[h, c]) == len(rows)
            assert perm[h, pos:pos + len(rows)].tolist() == rows
            pos += len(rows)


def test_fixed_point_mean_is_exact_integer_arithmetic():
    from fractions import Fraction
    g = torch.Generator().manual_seed(2)
    x = torch.randn(1, 300, 32, generator=g).to(torch.bfloat16)
    lab = torch.randint(0, 6, (1, 300), generator=g).to(torch.int32)
    lab[lab == 4] = 3                                               # cluster 4 empty
    old = torch.randn(1, 6, 32, generator=g).to(torch.bfloat16)
    newc, counts = O.fixed_point_mean(x, lab, old, torch.bfloat16)
    assert int(counts[0, 4]) == 0 and torch.equal(newc[0, 4], old[0, 4])
    for c in (0, 3, 5):
        rows = (lab[0] == c).nonzero().flatten().tolist()
        for d in (0, 17, 31):
            s = sum(round(Fraction(float(x[0, r, d])) * 32768) for r in rows)
            want = torch.tensor(float(s), dtype=torch.float32) / (32768.0 * torch.tensor(float(len(rows))))
            assert newc[0, c, d] == want.to(torch.bfloat16)


def test_assign_breaks_ties_towards_the_lowest_index_and_pins_the_tail():
    x = torch.tensor([[[1.0] + [0.0] * 31, [0.0, 1.0] + [0.0] * 30]]).to(torch.bfloat16)
    cen = torch.zeros(1, 4, 32)
    cen[0, 1, 0] = cen[0, 2, 0] = 1.0
    cen[0, 3, 1] = 1.0
    lab = O.assign(x, cen.to(torch.bfloat16))
    assert lab.tolist() == [[1, 3]]
    assert O.assign(x, cen.to(torch.bfloat16), pin_tail=1).tolist() == [[1, 3]]
    assert O.assign(x.flip(1), cen.to(torch.bfloat16), pin_tail=1).tolist() == [[3, 3]]


def _tiny_problem(H=1, N=512, C=2048, CQ=4, seed=3):
    g = torch.Generator().manual_seed(seed)
    bf = torch.bfloat16
    q, k, v = (torch.randn(H, N, 128, generator=g).to(bf) for _ in range(3))
    QU = torch.randn(H, N, 32, generator=g).to(bf)
    cks = (0.3 * torch.randn(H, C, 32, generator=g)).to(bf)
    klab = torch.randint(0, C, (H, N), generator=g).to(torch.int32)
    qlab = torch.randint(0, CQ, (H, N), generator=g).to(torch.int32)
    kcounts, kperm = O.stable_group(klab, C)
    _, sumv, lam, _ = O.vstats(v, kperm, kcounts, bf)
    return dict(q=q, k=k, v=v, QU=QU, cks=cks, klab=klab, qlab=qlab, kcounts=kcounts, sumv=sumv, lam=lam, CQ=CQ)


def test_full_union_is_dense_attention_and_residual_vanishes():
    p = _tiny_problem()
    scale = 1.0 / math.sqrt(128.0)
    full = torch.full((1, p["CQ"], 64), -1, dtype=torch.int32)
    o, lse = O.exact_attention(p["q"], p["k"], p["v"], p["qlab"], p["klab"], full, scale)
    out = O.residual_merge(o, lse, p["QU"], p["cks"], p["sumv"], p["lam"], p["kcounts"], full, p["qlab"], 1.0)
    dense = O.dense_attention(p["q"], p["k"], p["v"], scale)
    assert torch.allclose(out, dense, atol=1e-5)


def test_empty_union_is_the_pure_centroid_residual():
    p = _tiny_problem()
    none = torch.zeros(1, p["CQ"], 64, dtype=torch.int32)
    o, lse = O.exact_attention(p["q"], p["k"], p["v"], p["qlab"], p["klab"], none, 0.1)
    assert float(o.abs().max()) == 0.0 and bool(torch.isinf(lse).all())
    out = O.residual_merge(o, lse, p["QU"], p["cks"], p["sumv"], p["lam"], p["kcounts"], none, p["qlab"], 1.0)
    g = O.chain_dot(p["QU"][0].float(), p["cks"][0].float()).half().float()
    w = torch.exp(g - g.max(dim=1, keepdim=True).values)
    want = (w @ (p["sumv"][0].float() * p["lam"][0])) / (w * p["kcounts"][0].float()).sum(1, keepdim=True)
    assert torch.allclose(out[0], want, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("tailw", [1.0, 0.5])
def test_partial_union_is_one_softmax_over_union_keys_and_unselected_centroids(tailw):
    """The two-stage form (exact part with its log-sum-exp, then the merge with the centroid residual) against
    the single formula it implements, evaluated query by query in float64: every key of the query cluster's
    union enters with its true logit and its value, every key cluster outside the union enters once with the
    fp16-rounded centroid logit, weight n_c in the denominator and lam * sumv_c in the numerator, both scaled
    by tailw (tile_attn/src/kernel.cu:1248-1449)."""
    p = _tiny_problem(N=256, seed=11)
    scale = 1.0 / math.sqrt(128.0)
    g = torch.Generator().manual_seed(5)
    sel = torch.rand(1, p["CQ"], 2048, generator=g) < 0.3        # a third of the key clusters per query cluster
    unip = O.pack_bits(sel)
    o, lse = O.exact_attention(p["q"], p["k"], p["v"], p["qlab"], p["klab"], unip, scale)
    got = O.residual_merge(o, lse, p["QU"], p["cks"], p["sumv"], p["lam"], p["kcounts"], unip, p["qlab"], tailw)
    gl = O.chain_dot(p["QU"][0].float(), p["cks"][0].float()).half().double()      # [N, C] centroid logits
    q, k, v = (p[n][0].double() for n in ("q", "k", "v"))
    klab, qlab = p["klab"][0].long(), p["qlab"][0].long()
    nc, sumv, lam = p["kcounts"][0].double(), p["sumv"][0].double(), float(p["lam"][0])
    for i in range(0, 256, 7):
        inside = sel[0, qlab[i]]                                  # [C] clusters of this query's union
        keys = inside[klab].nonzero()[:, 0]
        s = (k[keys] @ q[i]) * scale
        gi = gl[i][~inside]
        m = max(float(s.max()) if keys.numel() else -math.inf, float(gi.max()))
        es, eg = torch.exp(s - m), torch.exp(gi - m)
        num = es @ v[keys] + tailw * lam * (eg @ sumv[~inside])
        den = es.sum() + tailw * (eg * nc[~inside]).sum()
        assert torch.allclose(got[0, i].double(), num / den, atol=2e-5, rtol=1e-4), i


def test_reuse_schedule_follows_the_reference_rule():
    """Rebuild iff no snapshot, the step counter went backwards, or branch 0 with
    step - snapshot_step >= mask_refresh (deploy_step.py:297-309)."""
    op = O.OracleOperator(1, 4096, 32, mask_refresh=4)
    held = None
    trace = []
    for step in list(range(10)) + [2, 3]:
        for parity in (0, 1):
            op.set_cfg_call(parity, key=7, step=step)
            age = None if held is None else step - held
            want_reuse = held is not None and age >= 0 and not (parity == 0 and (age < 0 or age >= 4))
            snap = op._pick_snapshot()
            assert (snap is not None) == want_reuse
            if snap is None:
                op._cfg_hold[7] = {"step": step}
                held = step
            trace.append(snap is None)
    assert trace[:10] == [True, False, False, False, False, False, False, False, True, False]
    assert op._pick_snapshot() is None      # an unannotated call always rebuilds


def test_c_twin_of_the_ordered_chain_gives_the_same_bits():
    """oracle/chain_dot.c against the PyTorch loop that defines the chain."""
    if O._chain_lib() is None:
        pytest.skip("no C compiler: the oracle runs the PyTorch loop")
    g = torch.Generator().manual_seed(31)
    x = torch.randn(777, 32, generator=g).to(torch.bfloat16).float()
    c = (torch.randn(301, 32, generator=g) * 3).to(torch.bfloat16).float()
    init = torch.randn(301, generator=g)
    assert torch.equal(O.chain_dot(x, c, init), O.chain_dot_loop(x, c, init))
    assert torch.equal(O.chain_dot(x, c), O.chain_dot_loop(x, c))
    # arbitrary fp32 inputs too: products and sums are rounded separately in both
    xf, cf = torch.randn(50, 32, generator=g), torch.randn(40, 32, generator=g)
    assert torch.equal(O.chain_dot(xf, cf), O.chain_dot_loop(xf, cf))
