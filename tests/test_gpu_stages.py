"""Stage-wise parity of the CUDA kernels against the CPU oracle, through the C ABI.

Every stage is fed the same inputs as the oracle; integer outputs (labels,
counts, permutations, bitmaps, row counts) and order-defined sums must match
bit for bit, tensor-core products within a stated tolerance.
"""
import math

import pytest
import torch

from oracle import t2t_oracle as O

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
DEV = "cuda"


def _st():
    return torch.cuda.current_stream().cuda_stream


def _ok(code):
    assert code == 0, f"C ABI returned {code}"


def test_gather4_selftest(lib):
    """Four-row TMA gathers fill a 128-byte-swizzled tile exactly as the manual
    16-byte copies of the other kernels do."""
    g = torch.Generator().manual_seed(11)
    rows = 1000
    src = torch.randn(rows, 128, generator=g).to(BF)
    gidx = torch.randint(0, rows, (128,), generator=g, dtype=torch.int32)
    gidx[5] = gidx[4]                      # repeated rows are allowed
    gidx[127] = rows - 1
    out = torch.zeros(32768, dtype=torch.uint8, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    srcd, gd = src.to(DEV), gidx.to(DEV)
    _ok(lib.t2t_gather4_selftest(srcd.data_ptr(), rows, gd.data_ptr(), out.data_ptr(), status.data_ptr(), _st()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    got = out.cpu().view(torch.int16).view(2, 128, 8, 8)          # [block][row][stored chunk][8 values]
    want = src[gidx.long()].view(torch.int16).view(128, 2, 8, 8).permute(1, 0, 2, 3)   # [block][row][chunk][8]
    r = torch.arange(128)[:, None]
    c = torch.arange(8)[None, :]
    stored = (c ^ (r & 7)).long()                                   # chunk c of row r lives at chunk c ^ (r & 7)
    unsw = torch.gather(got, 2, stored[None, :, :, None].expand(2, 128, 8, 8))
    assert torch.equal(unsw, want)


def test_bounded_wait_gives_up_cleanly(lib):
    """A wait that can never complete ends by its spin limit, raises the abort
    flag for the other warps, reports through the status word, and the context
    stays usable."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((2,), -1, dtype=torch.int32, device=DEV)
    _ok(lib.t2t_wait_timeout_selftest(status.data_ptr(), out.data_ptr(), _st()))
    torch.cuda.synchronize()
    assert int(status.item()) == 1 and out.tolist() == [0, 0]
    assert float((torch.ones(4, device=DEV) * 2).sum()) == 8.0      # the device still works


def test_umma_selftest(lib):
    g = torch.Generator().manual_seed(7)
    A = (torch.randn(128, 128, generator=g) * 0.5).to(BF)
    B = (torch.randn(128, 128, generator=g) * 0.5).to(BF)
    V = torch.randn(128, 128, generator=g).to(BF)
    S = torch.zeros(128, 128, device=DEV)
    Oo = torch.zeros(128, 128, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    Ad, Bd, Vd = A.to(DEV), B.to(DEV), V.to(DEV)
    _ok(lib.t2t_umma_selftest(Ad.data_ptr(), Bd.data_ptr(), Vd.data_ptr(), S.data_ptr(), Oo.data_ptr(),
                              status.data_ptr(), _st()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    S_ref = A.float() @ B.float().T
    assert torch.allclose(S.cpu(), S_ref, atol=1e-3, rtol=1e-4), (S.cpu() - S_ref).abs().max()
    # accumulation error of the tensor core against the real sum, relative to sum |a||b|: the assignment
    # and selection kernels assume it is below 2^-16
    S64 = A.double() @ B.double().T
    mag = A.double().abs() @ B.double().abs().T
    kappa = float(((S.cpu().double() - S64).abs() / mag).max())
    print(f"tensor-core accumulation error: {kappa:.3e} of sum|a||b| (2^{math.log2(kappa):.1f})")
    assert kappa < 2.0 ** -18
    P = (S.cpu() * 0.0625).to(BF).float()
    O_ref = P @ V.float()
    assert torch.allclose(Oo.cpu(), O_ref, atol=2e-3, rtol=1e-4), (Oo.cpu() - O_ref).abs().max()


def test_project(lib, small_case):
    c = small_case
    x, U = c["q"].to(DEV), c["state"]["Uq"].to(DEV)
    out = torch.empty(c["H"], c["N"], 32, dtype=BF, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    _ok(lib.t2t_project(x.data_ptr(), U.data_ptr(), out.data_ptr(), c["H"], c["N"], status.data_ptr(), _st()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    exact = torch.bmm(c["q"].float(), c["state"]["Uq"].float())
    got = out.cpu().float()
    # one bf16 rounding of an fp32-accumulated product: at most one ulp from the exact value's rounding
    tol = exact.abs() * 2.0 ** -7 + 1e-3
    assert bool(((got - exact).abs() <= tol).all())
    assert (got == exact.to(BF).float()).float().mean() > 0.98


def _assign(lib, x, cen, pin_begin=-1, pin_label=0):
    """Tensor-core assignment; also checks it against the all-exact kernel."""
    H, N, _ = x.shape
    lab = torch.empty(H, N, dtype=torch.int32, device=DEV)
    lab_exact = torch.empty_like(lab)
    ws = torch.empty(lib.t2t_assign_ws_bytes(H, N), dtype=torch.uint8, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    _ok(lib.t2t_assign(x.data_ptr(), cen.data_ptr(), lab.data_ptr(), H, N, cen.shape[1], pin_begin, pin_label,
                       ws.data_ptr(), ws.numel(), status.data_ptr(), _st()))
    _ok(lib.t2t_assign_exact(x.data_ptr(), cen.data_ptr(), lab_exact.data_ptr(), H, N, cen.shape[1], pin_begin,
                             pin_label, _st()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(lab, lab_exact)
    _assign.requeued = int(ws[:4].view(torch.int32).item())
    return lab


def test_assign_tensor_core_path_equals_exact_path_at_scale(lib):
    """480p-sized random problem: the tensor-core labels must equal the all-exact
    labels, with only a small share of rows sent to the exact re-evaluation."""
    from token2tile_b200.synth import GRIDS, locality_mixture
    H, N = 4, 32760
    q, k, _ = locality_mixture(H, GRIDS["480p"])
    g = torch.Generator().manual_seed(5)
    U = (torch.randn(H, 128, 32, generator=g) * 0.1).to(BF)
    x = torch.bmm(k.float(), U.float()).to(BF).to(DEV)
    for Cn in (2048, 256):
        idx = torch.randperm(N, generator=g)[:Cn].sort().values
        cen = x[:, idx.to(DEV), :].contiguous()
        _assign(lib, x, cen)
        assert _assign.requeued < 0.05 * H * N, _assign.requeued


def test_assign_bit_exact(lib, small_case):
    c = small_case
    QU = O.project(c["q"], c["state"]["Uq"], BF)
    KU = O.project(c["k"], c["state"]["Uk"], BF)
    for x, cen, pin in ((QU, c["state"]["cq"], 0), (KU, c["state"]["ck"], 0), (KU, c["state"]["ck"], 100)):
        want = O.assign(x, cen, pin)
        got = _assign(lib, x.to(DEV), cen.to(DEV), c["N"] - pin if pin else -1, cen.shape[1] - 1)
        assert torch.equal(got.cpu(), want)


def test_assign_ties_go_to_lowest_index(lib):
    H, N, Cn = 1, 2048, 64
    g = torch.Generator().manual_seed(3)
    x = torch.randint(-3, 4, (H, N, 32), generator=g).to(BF)
    cen = torch.randint(-2, 3, (H, Cn, 32), generator=g).to(BF)
    cen[:, 10] = cen[:, 3]                      # duplicated centroids tie everywhere
    cen[:, 40] = cen[:, 3]
    want = O.assign(x, cen)
    got = _assign(lib, x.to(DEV), cen.to(DEV))
    assert torch.equal(got.cpu(), want)
    assert not bool(((want == 10) | (want == 40)).any())


def test_centroid_update_bit_exact(lib, small_case):
    c = small_case
    H, N = c["H"], c["N"]
    KU = O.project(c["k"], c["state"]["Uk"], BF)
    old = c["state"]["ck"]
    lab = O.assign(KU, old)
    lab[:, :] = torch.where(lab == 5, torch.full_like(lab, 6), lab)      # cluster 5 empty: keeps its centroid
    want_c, want_n = O.fixed_point_mean(KU, lab, old, BF)
    ws = torch.empty(lib.t2t_centroid_update_ws_bytes(H, N, 2048), dtype=torch.uint8, device=DEV)
    newc = torch.empty(H, 2048, 32, dtype=BF, device=DEV)
    counts = torch.empty(H, 2048, dtype=torch.int32, device=DEV)
    KUd, labd, oldd = KU.to(DEV), lab.to(DEV), old.to(DEV)      # keep the device copies alive
    _ok(lib.t2t_centroid_update(KUd.data_ptr(), labd.data_ptr(), oldd.data_ptr(),
                                newc.data_ptr(), counts.data_ptr(), H, N, 2048, ws.data_ptr(), ws.numel(), _st()))
    torch.cuda.synchronize()
    assert torch.equal(counts.cpu(), want_n)
    assert torch.equal(newc.cpu().view(torch.int16), want_c.view(torch.int16))


def _kmm(lib, QU, KU, V, cq0, ck0, CQ, pin_tail=0):
    H, N, _ = QU.shape
    C = 2048
    i32 = torch.int32
    e = lambda *s, dtype: torch.empty(*s, dtype=dtype, device=DEV)
    out = dict(qlab=e(H, N, dtype=i32), cq2=e(H, CQ, 32, dtype=BF), klab=e(H, N, dtype=i32),
               ck2=e(H, C, 32, dtype=torch.float32), ck16=e(H, C, 32, dtype=BF), cks16=e(H, C, 32, dtype=BF),
               qcounts=e(H, CQ, dtype=i32), qperm=e(H, N, dtype=i32), kcounts=e(H, C, dtype=i32),
               kperm=e(H, N, dtype=i32), V_sorted=e(H, N, 128, dtype=BF), sumv=e(H, C, 128, dtype=BF),
               lam=e(H, dtype=torch.float32))
    ws = torch.empty(lib.t2t_kmeans_maintain_ws_bytes(H, N, CQ, C), dtype=torch.uint8, device=DEV)
    dev = [t.to(DEV) for t in (QU, KU, V, cq0, ck0)]
    order = ["qlab", "cq2", "klab", "ck2", "ck16", "cks16", "qcounts", "qperm", "kcounts", "kperm", "V_sorted",
             "sumv", "lam"]
    _ok(lib.t2t_kmeans_maintain(*[t.data_ptr() for t in dev], *[out[k].data_ptr() for k in order],
                                1.0 / math.sqrt(128.0), H, N, CQ, C, pin_tail, ws.data_ptr(), ws.numel(), 0, _st()))
    torch.cuda.synchronize()
    return {k: t.cpu() for k, t in out.items()}


@pytest.mark.parametrize("pin_tail", [0, 77])
def test_kmeans_maintain_bit_exact(lib, small_case, pin_tail):
    c = small_case
    QU = O.project(c["q"], c["state"]["Uq"], BF)
    KU = O.project(c["k"], c["state"]["Uk"], BF)
    want = O.kmeans_maintain(QU, KU, c["v"], c["state"]["cq"], c["state"]["ck"], pin_tail, BF)
    got = _kmm(lib, QU, KU, c["v"], c["state"]["cq"], c["state"]["ck"], c["CQ"], pin_tail)
    for name in ("qlab", "klab", "qcounts", "kcounts", "qperm", "kperm"):
        assert torch.equal(got[name], want[name]), name
    assert torch.equal(got["cq2"].view(torch.int16), want["cq2"].view(torch.int16))
    assert torch.equal(got["ck2"], want["ck2"])
    assert torch.equal(got["ck16"].view(torch.int16), want["ck2"].to(BF).view(torch.int16))
    scale = 1.0 / math.sqrt(128.0)
    assert torch.equal(got["cks16"].view(torch.int16), (want["ck2"] * scale).to(BF).view(torch.int16))
    assert torch.equal(got["V_sorted"].view(torch.int16), want["V_sorted"].view(torch.int16))
    assert torch.equal(got["lam"], want["lam"])
    assert torch.equal(got["sumv"].view(torch.int16), want["sumv"].view(torch.int16))


def test_vstats_gather_and_gather_rows(lib, small_case):
    c = small_case
    H, N = c["H"], c["N"]
    KU = O.project(c["k"], c["state"]["Uk"], BF)
    klab = O.assign(KU, c["state"]["ck"])
    kcounts, kperm = O.stable_group(klab, 2048)
    v2 = (c["v"].float() * 1.5 + 0.25).to(BF)
    want_vs, want_sumv, want_lam, _ = O.vstats(v2, kperm, kcounts, BF)
    vs = torch.empty(H, N, 128, dtype=BF, device=DEV)
    sumv = torch.empty(H, 2048, 128, dtype=BF, device=DEV)
    lam = torch.empty(H, dtype=torch.float32, device=DEV)
    ws = torch.empty(lib.t2t_vstats_gather_ws_bytes(H, 2048), dtype=torch.uint8, device=DEV)
    v2d, kpermd, kcountsd, kd = v2.to(DEV), kperm.to(DEV), kcounts.to(DEV), c["k"].to(DEV)
    _ok(lib.t2t_vstats_gather(v2d.data_ptr(), kpermd.data_ptr(), kcountsd.data_ptr(),
                              vs.data_ptr(), sumv.data_ptr(), lam.data_ptr(), H, N, 2048, ws.data_ptr(),
                              ws.numel(), _st()))
    torch.cuda.synchronize()
    assert torch.equal(vs.cpu().view(torch.int16), want_vs.view(torch.int16))
    assert torch.equal(sumv.cpu().view(torch.int16), want_sumv.view(torch.int16))
    assert torch.equal(lam.cpu(), want_lam)
    kp = torch.empty(H, N, 128, dtype=BF, device=DEV)
    _ok(lib.t2t_gather_rows(kd.data_ptr(), kpermd.data_ptr(), kp.data_ptr(), H, N, _st()))
    torch.cuda.synchronize()
    want_kp = torch.gather(c["k"], 1, kperm.long()[..., None].expand(H, N, 128))
    assert torch.equal(kp.cpu().view(torch.int16), want_kp.view(torch.int16))


def _select(lib, QU, cks, kcounts, qperm, qcounts, ns, pin_tail=0):
    H, N, _ = QU.shape
    CQ = qcounts.shape[1]
    unip = torch.empty(H, CQ, 64, dtype=torch.int32, device=DEV)
    rowcnt = torch.full((H, N), -7, dtype=torch.int32, device=DEV)
    unip_x, rowcnt_x = torch.empty_like(unip), torch.empty_like(rowcnt)
    ns_t = torch.tensor(ns, dtype=torch.int32, device=DEV)
    ws = torch.empty(lib.t2t_score_select_union_ws_bytes(H, N), dtype=torch.uint8, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    dev = [t.to(DEV) for t in (QU, cks, kcounts, qperm, qcounts)]
    _ok(lib.t2t_score_select_union(*[t.data_ptr() for t in dev], ns_t.data_ptr(), unip.data_ptr(),
                                   rowcnt.data_ptr(), H, N, CQ, pin_tail, ws.data_ptr(), ws.numel(),
                                   status.data_ptr(), _st()))
    _ok(lib.t2t_score_select_union_exact(*[t.data_ptr() for t in dev], ns_t.data_ptr(), unip_x.data_ptr(),
                                         rowcnt_x.data_ptr(), H, N, CQ, pin_tail, _st()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # the tensor-core path and the all-exact path must agree bit for bit
    assert torch.equal(rowcnt, rowcnt_x)
    assert torch.equal(unip, unip_x)
    q = ws.view(torch.int32)[: H * (2 * N + 1)].view(H, 2 * N + 1)[:, 0]      # per head: count, then the queue
    _select.requeued = int(q.sum().item())
    return unip.cpu(), rowcnt.cpu()


def test_select_tensor_core_path_equals_exact_path_at_scale(lib):
    """480p-sized problem through real clustering: both selection paths must agree
    and only a small share of rows may need the exact re-evaluation."""
    from token2tile_b200.synth import GRIDS, locality_mixture
    H, N, CQ = 2, 32760, 256
    q, k, v = locality_mixture(H, GRIDS["480p"])
    g = torch.Generator().manual_seed(9)
    Uq = (torch.randn(H, 128, 32, generator=g) * 0.1).to(BF)
    QU = torch.bmm(q.float(), Uq.float()).to(BF)
    KU = torch.bmm(k.float(), Uq.float()).to(BF)
    ck0 = KU[:, torch.randperm(N, generator=g)[:2048].sort().values].contiguous()
    cq0 = QU[:, torch.randperm(N, generator=g)[:CQ].sort().values].contiguous()
    km = _kmm(lib, QU, KU, v, cq0, ck0, CQ)
    for ns in (491, 1638, 5):
        _select(lib, QU, km["cks16"], km["kcounts"], km["qperm"], km["qcounts"], ns)
        assert _select.requeued < 0.02 * H * N, (ns, _select.requeued)


@pytest.mark.parametrize("ns,pin_tail", [(204, 0), (1, 0), (4096, 0), (61, 33)])
def test_select_union_bit_exact(lib, small_case, ns, pin_tail):
    c = small_case
    QU = O.project(c["q"], c["state"]["Uq"], BF)
    KU = O.project(c["k"], c["state"]["Uk"], BF)
    km = O.kmeans_maintain(QU, KU, c["v"], c["state"]["cq"], c["state"]["ck"], pin_tail, BF)
    cks = (km["ck2"] * (1.0 / math.sqrt(128.0))).to(BF)
    want_u, want_rc = O.select_union(QU, cks, km["kcounts"], km["qlab"], c["CQ"], ns, pin_tail)
    got_u, got_rc = _select(lib, QU, cks, km["kcounts"], km["qperm"], km["qcounts"], ns, pin_tail)
    assert torch.equal(got_rc, want_rc)
    assert torch.equal(got_u, want_u)


def test_select_union_ties_and_empty_clusters(lib):
    """Small-integer scores tie massively; a third of the key clusters are empty,
    and one query cluster has no rows."""
    H, N, CQ, C = 1, 4096, 16, 2048
    g = torch.Generator().manual_seed(11)
    QU = torch.randint(-2, 3, (H, N, 32), generator=g).to(BF)
    cks = (torch.randint(-2, 3, (H, C, 32), generator=g).float() * 0.125).to(BF)
    klab = torch.randint(0, C, (H, N), generator=g).to(torch.int32)
    klab = torch.where(klab % 3 == 0, klab + 1, klab).clamp_max(C - 1)
    kcounts, _ = O.stable_group(klab, C)
    qlab = torch.randint(0, CQ - 1, (H, N), generator=g).to(torch.int32)      # cluster CQ-1 stays empty
    qcounts, qperm = O.stable_group(qlab, CQ)
    for ns in (40, 300):
        want_u, want_rc = O.select_union(QU, cks, kcounts, qlab, CQ, ns)
        got_u, got_rc = _select(lib, QU, cks, kcounts, qperm, qcounts, ns)
        assert torch.equal(got_rc, want_rc)
        assert torch.equal(got_u, want_u)
    assert int(got_u[0, CQ - 1].abs().sum()) == 0


def _tile_attn(lib, q, k, v, QU, km, cks, unip, tailw=1.0):
    H, N, _ = q.shape
    CQ = km["qcounts"].shape[1]
    kp = torch.gather(k, 1, km["kperm"].long()[..., None].expand(H, N, 128)).contiguous()
    plan = torch.zeros(lib.t2t_tile_attn_plan_ints(H, N, CQ), dtype=torch.int32, device=DEV)
    ws = torch.empty(lib.t2t_tile_attn_ws_bytes(H, N), dtype=torch.uint8, device=DEV)
    out = torch.zeros(H, N, 128, dtype=BF, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    tw = torch.tensor(float(tailw), dtype=torch.float32, device=DEV)
    host = [q, kp, km["V_sorted"], km["qcounts"], km["kcounts"], unip, QU, cks, km["sumv"], km["lam"], km["qlab"],
            km["qperm"]]
    dev = [t.to(DEV).contiguous() for t in host]
    _ok(lib.t2t_tile_attn(*[t.data_ptr() for t in dev], tw.data_ptr(), out.data_ptr(), plan.data_ptr(), 1, H, N,
                          CQ, ws.data_ptr(), ws.numel(), status.data_ptr(), _st()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    info = torch.zeros(4, dtype=torch.int32, device=DEV)
    _ok(lib.t2t_tile_attn_plan_info(plan.data_ptr(), H, N, CQ, info.data_ptr(), _st()))
    i = info.cpu().tolist()
    lse = ws[((H * N * 256 + 255) // 256) * 256:].view(torch.float32)[: H * N].view(H, N).cpu()
    attn_o = ws[: H * N * 256].view(BF).view(H, N, 128).cpu()
    return out.cpu(), dict(tasks=i[0], pairs=(i[1] & 0xFFFFFFFF) | ((i[2] & 0xFFFFFFFF) << 32), lse=lse,
                           attn_o=attn_o)


def _structure(c, ns, pin_tail=0):
    QU = O.project(c["q"], c["state"]["Uq"], BF)
    KU = O.project(c["k"], c["state"]["Uk"], BF)
    km = O.kmeans_maintain(QU, KU, c["v"], c["state"]["cq"], c["state"]["ck"], pin_tail, BF)
    cks = (km["ck2"] * (1.0 / math.sqrt(128.0))).to(BF)
    unip, _ = O.select_union(QU, cks, km["kcounts"], km["qlab"], c["CQ"], ns, pin_tail)
    return QU, km, cks, unip


@pytest.mark.parametrize("ns", [204, 20])
def test_tile_attn_matches_oracle(lib, small_case, ns):
    c = small_case
    scale = 1.0 / math.sqrt(128.0)
    QU, km, cks, unip = _structure(c, ns)
    o, lse = O.exact_attention(c["q"], c["k"], c["v"], km["qlab"], km["klab"], unip, scale)
    want = O.residual_merge(o, lse, QU, cks, km["sumv"], km["lam"], km["kcounts"], unip, km["qlab"], 1.0)
    got, info = _tile_attn(lib, c["q"], c["k"], c["v"], QU, km, cks, unip)
    # exact part, in sorted row order on the device
    perm = km["qperm"].long()
    o_sorted = torch.gather(o, 1, perm[..., None].expand_as(o))
    lse_sorted = torch.gather(lse, 1, perm)
    fin = torch.isfinite(lse_sorted)
    assert torch.equal(fin, torch.isfinite(info["lse"]))
    assert (info["lse"][fin] - lse_sorted[fin]).abs().max() < 2e-2
    assert (info["attn_o"].float() - o_sorted).abs().max() < 2e-2
    err = (got.float() - want).abs()
    assert err.max() < 2e-2, err.max()
    assert err.mean() < 2e-3, err.mean()
    kv = O.kv_lengths(unip, km["qcounts"], km["kcounts"])
    assert info["pairs"] == int((kv.long() * km["qcounts"].long()).sum())


def test_tile_attn_full_union_equals_dense(lib, small_case):
    """With every key cluster selected the operator is dense attention."""
    c = small_case
    QU, km, cks, unip = _structure(c, 204)
    full = torch.full_like(unip, -1)
    got, info = _tile_attn(lib, c["q"], c["k"], c["v"], QU, km, cks, full)
    want = O.dense_attention(c["q"], c["k"], c["v"], 1.0 / math.sqrt(128.0))
    err = (got.float() - want).abs()
    assert err.max() < 2e-2 and err.mean() < 2e-3
    assert info["pairs"] == c["H"] * c["N"] * c["N"]


def test_tile_attn_empty_union_is_pure_residual(lib, small_case):
    c = small_case
    QU, km, cks, unip = _structure(c, 204)
    none = torch.zeros_like(unip)
    got, info = _tile_attn(lib, c["q"], c["k"], c["v"], QU, km, cks, none)
    o = torch.zeros(c["H"], c["N"], 128)
    lse = torch.full((c["H"], c["N"]), -math.inf)
    want = O.residual_merge(o, lse, QU, cks, km["sumv"], km["lam"], km["kcounts"], none, km["qlab"], 1.0)
    err = (got.float() - want).abs()
    assert err.max() < 2e-2 and err.mean() < 2e-3
    assert info["pairs"] == 0
