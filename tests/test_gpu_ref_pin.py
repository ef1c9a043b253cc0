"""Pins the CPU oracle against the reference's own CUDA kernels.

oracle/_ref/libt2t_ref.so holds the reference's kmeans_maintain and
select_union sources compiled unmodified for sm_100a (oracle/build_ref.py).
They take float16, so the oracle runs in its float16 mode here.  Integer rules
(stable grouping, fixed-point query means, selection, bitmap layout, row
counts) must agree exactly; nearest-centroid labels may differ only where two
distances are within tensor-core rounding of each other, and every later stage
is then compared with the reference's labels fed to the oracle.
"""
import ctypes as C
import math
from pathlib import Path

import pytest
import torch

from oracle import t2t_oracle as O

pytestmark = pytest.mark.gpu
REF = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libt2t_ref.so"
F16 = torch.float16
DEV = "cuda"
P, I, S = C.c_void_p, C.c_int, C.c_size_t


@pytest.fixture(scope="module")
def ref():
    if not REF.exists():
        pytest.skip("oracle/_ref/libt2t_ref.so not built (needs the reference checkout at build time)")
    lib = C.CDLL(str(REF))
    lib.ref_kmm_ws_bytes.restype, lib.ref_kmm_ws_bytes.argtypes = S, [I, I, I, I]
    lib.ref_kmm_run.restype, lib.ref_kmm_run.argtypes = I, [P] * 16 + [I, I, I, I, I, P, P]
    lib.ref_select_packed.restype, lib.ref_select_packed.argtypes = I, [P] * 9 + [I, I, I, P]
    return lib


@pytest.fixture(scope="module")
def case16(small_case):
    """The small locality-mixture case in float16 with an oracle state."""
    c = small_case
    q, k, v = c["q"].to(F16), c["k"].to(F16), c["v"].to(F16)
    st = O.init_state(q, k, c["CQ"], 2048, 32, 2, 0, F16)
    QU = O.project(q, st["Uq"], F16)
    KU = O.project(k, st["Uk"], F16)
    return dict(H=c["H"], N=c["N"], CQ=c["CQ"], v=v, QU=QU, KU=KU, cq0=st["cq"], ck0=st["ck"])


def _ref_kmm(ref, c, pin_tail):
    H, N, CQ, CK = c["H"], c["N"], c["CQ"], 2048
    i32 = torch.int32
    e = lambda *s, dtype: torch.empty(*s, dtype=dtype, device=DEV)
    out = dict(qlab=e(H, N, dtype=i32), cq2=e(H, CQ, 32, dtype=F16), klab=e(H, N, dtype=i32),
               ck2=e(H, CK, 32, dtype=torch.float32), qcounts=e(H, CQ, dtype=i32), qperm=e(H, N, dtype=i32),
               kcounts=e(H, CK, dtype=i32), kperm=e(H, N, dtype=i32), V_sorted=e(H, N, 128, dtype=F16),
               sumv=e(H, CK, 128, dtype=F16), lam=e(H, dtype=torch.float32))
    ws = torch.zeros(ref.ref_kmm_ws_bytes(H, N, CQ, CK), dtype=torch.uint8, device=DEV)
    ins = [c[n].to(DEV).contiguous() for n in ("QU", "KU", "v", "cq0", "ck0")]
    order = ["qlab", "cq2", "klab", "ck2", "qcounts", "qperm", "kcounts", "kperm", "V_sorted", "sumv", "lam"]
    rc = ref.ref_kmm_run(*[t.data_ptr() for t in ins], *[out[n].data_ptr() for n in order], H, N, CQ, CK,
                         pin_tail, ws.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0
    return {n: t.cpu() for n, t in out.items()}


@pytest.mark.parametrize("pin_tail", [0, 50])
def test_oracle_clustering_matches_reference_kernels(ref, case16, pin_tail):
    c = case16
    H, N = c["H"], c["N"]
    r = _ref_kmm(ref, c, pin_tail)
    want = O.kmeans_maintain(c["QU"], c["KU"], c["v"], c["cq0"], c["ck0"], pin_tail, F16)

    # key labels: one pass from ck0; any disagreement must be a near-tie of the two distances
    diff = (r["klab"] != want["klab"])
    assert diff.float().mean() < 2e-3, float(diff.float().mean())
    for h in range(H):
        rows = diff[h].nonzero().flatten()
        if rows.numel():
            cen = c["ck0"][h].float()
            d = O.chain_dot(c["KU"][h, rows].float(), -2.0 * cen, O.centroid_norms(cen))
            da = d.gather(1, r["klab"][h, rows].long()[:, None])
            db = d.gather(1, want["klab"][h, rows].long()[:, None])
            assert float(((da - db).abs() / db.abs().clamp_min(1.0)).max()) < 1e-4
    # Query labels come out of two passes.  The reference keeps the centroids between the passes (cq1) inside
    # its workspace, so its second pass cannot be replayed from its own cq1; instead every disagreement must be
    # a near-tie under the oracle's cq1.  A first-pass near-tie that goes the other way moves two centroids by
    # about one row in a few hundred, i.e. by a few float16 ulps (2^-11 relative), and a distance is linear in
    # the centroid: the two candidate distances of a disagreeing row may differ by that much, not by more.
    qd = (r["qlab"] != want["qlab"])
    qdiff = float(qd.float().mean())
    worst = 0.0
    for h in range(H):
        rows = qd[h].nonzero().flatten()
        if rows.numel():
            cen = want["cq1"][h].float()
            d = O.chain_dot(c["QU"][h, rows].float(), -2.0 * cen, O.centroid_norms(cen))
            da = d.gather(1, r["qlab"][h, rows].long()[:, None])
            db = d.gather(1, want["qlab"][h, rows].long()[:, None])
            worst = max(worst, float(((da - db).abs() / db.abs().clamp_min(1.0)).max()))
    print(f"query labels: {qdiff:.2e} of the rows differ, largest relative distance gap {worst:.2e}")
    assert qdiff < 2e-3 and worst < 2e-2, (qdiff, worst)      # measured on a B200: no row differs on this case

    # everything downstream, with the reference's labels fed to the oracle
    kcounts, kperm = O.stable_group(r["klab"], 2048)
    assert torch.equal(r["kcounts"], kcounts) and torch.equal(r["kperm"], kperm)
    qcounts, qperm = O.stable_group(r["qlab"], c["CQ"])
    assert torch.equal(r["qcounts"], qcounts) and torch.equal(r["qperm"], qperm)
    ck2 = O.key_means_f32(c["KU"], kperm, kcounts, c["ck0"])
    assert torch.allclose(r["ck2"], ck2, rtol=3e-7, atol=1e-9)          # the reference divides with fast-math
    cq2, _ = O.fixed_point_mean(c["QU"], r["qlab"], c["cq0"], F16)
    live = (qcounts > 0)[..., None].expand_as(cq2)
    ulp = (r["cq2"].view(torch.int16).int() - cq2.view(torch.int16).int()).abs()
    assert int(ulp[live].max()) <= 1 and float((ulp[live] > 0).float().mean()) < 1e-2
    v_sorted, sumv, lam, _ = O.vstats(c["v"], kperm, kcounts, F16)
    assert torch.equal(r["V_sorted"].view(torch.int16), v_sorted.view(torch.int16))
    assert torch.equal(r["lam"], lam)
    assert torch.equal(r["sumv"].view(torch.int16), sumv.view(torch.int16))
    if pin_tail:
        assert bool((r["klab"][:, N - pin_tail:] == 2047).all())


@pytest.mark.parametrize("ns", [204, 17, 1])
def test_oracle_selection_matches_reference_kernel(ref, case16, ns):
    c = case16
    H, N, CQ = c["H"], c["N"], c["CQ"]
    km = O.kmeans_maintain(c["QU"], c["KU"], c["v"], c["cq0"], c["ck0"], 0, F16)
    cks = (km["ck2"] * (1.0 / math.sqrt(128.0))).to(F16)
    gl = torch.stack([O.chain_dot(c["QU"][h].float(), cks[h].float()).to(F16) for h in range(H)])
    if ns == 17:      # force exact ties and empty key clusters through the same kernel
        gl = (gl.float() * 2.0).round().clamp(-6, 6).mul(0.5).to(F16)
    want_u, want_rc = O.select_union(None, None, km["kcounts"], km["qlab"], CQ, ns, gl16=gl)
    unip = torch.zeros(H, CQ, 64, dtype=torch.int32, device=DEV)
    rowcnt = torch.zeros(H, N, dtype=torch.int32, device=DEV)
    partial = torch.zeros(H, CQ, 6 * 128, dtype=torch.int16, device=DEV)
    off = torch.zeros(H, CQ, dtype=torch.int32, device=DEV)
    ns_t = torch.tensor(ns, dtype=torch.int32, device=DEV)
    ins = [t.to(DEV).contiguous() for t in (gl, km["kcounts"], km["qperm"], km["qcounts"])]
    rc = ref.ref_select_packed(*[t.data_ptr() for t in ins], ns_t.data_ptr(), partial.data_ptr(), unip.data_ptr(),
                               rowcnt.data_ptr(), off.data_ptr(), H, N, CQ,
                               torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0
    assert torch.equal(rowcnt.cpu(), want_rc)
    assert torch.equal(unip.cpu(), want_u)
