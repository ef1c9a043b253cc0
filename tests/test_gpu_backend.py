"""The SGLang backend mirror driving the real operator on a GPU: dense prefix,
sparse steps with CFG branch reuse, fast state initialisation, and the packed
[context | video] document path with pinned context keys."""
import math
from types import SimpleNamespace

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
DEV = "cuda"
SCALE = 1.0 / math.sqrt(128)


def _dense(q, k, v):
    """q [R, H, D] over k, v [T, H, D] -> [R, H, D] float32."""
    out = torch.nn.functional.scaled_dot_product_attention(q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1),
                                                           scale=SCALE)
    return out.transpose(0, 1).float()


@pytest.fixture()
def backend():
    from token2tile_b200 import t2t_attn as B
    B.clear_runtimes()
    B.set_backend_config({})
    B.set_forward_context(None)
    B.set_ulysses_world_size(1)
    yield B
    B.clear_runtimes()
    B.set_backend_config({})
    B.set_forward_context(None)


def _wan_inputs(H=12):
    from token2tile_b200.synth import GRIDS, locality_mixture
    q, k, v = locality_mixture(H, GRIDS["cpu"])
    # host layout: [1, N, H, D]
    return tuple(t.transpose(0, 1).unsqueeze(0).contiguous().to(DEV) for t in (q, k, v))


def cache_state_uq(impl):
    """Query projection of the packed path's last head chunk (the implementation keeps one state per chunk)."""
    return impl._h3_states[max(impl._h3_states)]["Uq"].cpu()


def _meta(B, cache, step, **kw):
    return B.T2TAttentionMetadataBuilder().build(
        step, 50, cache, profile_name="manual", ns_base=204, dense_prefix_steps=1, cq=32, ck=2048,
        step_profile=(1.0, 1.0, 1.0, 1.0), layer_profile=(1.0,) * 6, cfg_mult=(1.0, 1.0), **kw)


def test_wan_path_matches_a_direct_operator_call(backend):
    B = backend
    from token2tile_b200 import MaskedStepDeploy
    q, k, v = _wan_inputs()
    impl = B.T2TAttentionImpl(12, 128, False, SCALE, prefix="blocks.3.attn1")
    cache = B.T2TRequestCache()
    dense = _dense(q[0], k[0], v[0])
    out = impl.forward(q, k, v, _meta(B, cache, 0))
    assert (out[0].float() - dense).abs().max() < 2e-2                    # prefix step
    assert not B._RUNTIMES

    out0 = impl.forward(q, k, v, _meta(B, cache, 1)).clone()
    runtime, = B._RUNTIMES.values()
    dep = runtime.deploy
    assert dep.last_rebuilt is True and int(dep.ns_t) == 204
    out1 = impl.forward(q, k, v, _meta(B, cache, 1)).clone()
    assert dep.last_rebuilt is False                                       # branch 1 reuses branch 0's structure
    torch.cuda.synchronize()
    assert dep.device_status() == 0
    for o in (out0, out1):
        assert o.shape == q.shape and o.dtype == BF
        rel = ((o[0].float() - dense).norm() / dense.norm()).item()
        assert rel < 0.05, rel

    # the same call made directly on a fresh operator gives the same bits
    op = MaskedStepDeploy(12, 4096, 32, s_frac=204 / 4096, mask_refresh=4, cfg_reuse=True)
    qh, kh, vh = (t[0].transpose(0, 1).contiguous() for t in (q, k, v))
    state = op.init_state(qh, kh, warm_iters=4, seed=3 * 2 + 0)
    op.set_cfg_call(0, 3, 1)
    direct = op.step(qh, kh, vh, state).transpose(0, 1)
    torch.cuda.synchronize()
    assert torch.equal(direct.contiguous().view(torch.int16), out0[0].view(torch.int16))
    # steps 2..4 reuse, step 5 rebuilds (mask_refresh = 4)
    rebuilt = []
    for step in (2, 3, 4, 5):
        impl.forward(q, k, v, _meta(B, cache, step))
        rebuilt.append(dep.last_rebuilt)
        impl.forward(q, k, v, _meta(B, cache, step))
    assert rebuilt == [False, False, False, True]
    torch.cuda.synchronize()
    assert dep.device_status() == 0


def test_fast_init_state(backend):
    B = backend
    B.set_backend_config({"t2t_fast_init": True})
    q, k, v = _wan_inputs()
    impl = B.T2TAttentionImpl(12, 128, False, SCALE, prefix="blocks.0.attn1")
    cache = B.T2TRequestCache()
    out = impl.forward(q, k, v, _meta(B, cache, 1))
    torch.cuda.synchronize()
    runtime, = B._RUNTIMES.values()
    assert runtime.deploy.device_status() == 0
    state = cache.states[(0, 0)]
    assert state["Uq"].shape == (12, 128, 32) and state["ck"].shape == (12, 2048, 32)
    assert all(bool(torch.isfinite(t.float()).all()) for t in state.values())
    dense = _dense(q[0], k[0], v[0])
    rel = ((out[0].float() - dense).norm() / dense.norm()).item()
    assert rel < 0.05, rel


def test_fast_init_state_against_the_oracle(backend):
    """`t2t_fast_init` end to end: the projections against the oracle's fit (as products Uq Uk^T), and the
    first centroids bit for bit against the oracle's Lloyd rounds replayed from the device's own projected rows
    and the same row draws (a device generator with the same seed repeats its draws)."""
    B = backend
    from oracle import t2t_oracle as O
    from token2tile_b200 import MaskedStepDeploy
    from token2tile_b200.synth import GRIDS, locality_mixture
    H, N, CQ, warm, seed = 3, 4096, 32, 2, 5
    q, k, _ = locality_mixture(H, GRIDS["cpu"])
    qd, kd = q.to(DEV), k.to(DEV)
    op = MaskedStepDeploy(H, N, CQ, s_frac=0.05)
    st = B.make_fast_init_state(op)(qd, kd, warm_iters=warm, seed=seed)
    torch.cuda.synchronize()
    assert op.device_status() == 0
    oq, ok = O.online_u(q.float(), k.float(), 32)
    want = oq.to(BF).double() @ ok.to(BF).double().transpose(1, 2)
    got = st["Uq"].cpu().double() @ st["Uk"].cpu().double().transpose(1, 2)
    assert (got - want).abs().max() <= 0.02 * want.abs().max()
    KU, QU = torch.empty_like(op.KU), torch.empty_like(op.QU)
    stream = torch.cuda.current_stream().cuda_stream
    op._project(kd, st["Uk"], KU, stream)
    op._project(qd, st["Uq"], QU, stream)
    gen = torch.Generator(device=DEV).manual_seed(seed)
    rows_k = torch.randperm(N, generator=gen, device=DEV)[:2048].sort().values.cpu()
    rows_q = torch.randperm(N, generator=gen, device=DEV)[:CQ].sort().values.cpu()
    torch.cuda.synchronize()
    KU, QU = KU.cpu(), QU.cpu()
    ck, cq = KU[:, rows_k, :].contiguous(), QU[:, rows_q, :].contiguous()
    for _ in range(warm):
        ck, _ = O.fixed_point_mean(KU, O.assign(KU, ck), ck, BF)
        cq, _ = O.fixed_point_mean(QU, O.assign(QU, cq), cq, BF)
    assert torch.equal(st["ck"].cpu().view(torch.int16), ck.view(torch.int16))
    assert torch.equal(st["cq"].cpu().view(torch.int16), cq.view(torch.int16))


def test_packed_document_path(backend):
    B = backend
    from token2tile_b200.synth import locality_mixture
    H, video, context, pad = 56, 3072, 1024, 64
    used = video + context
    qv, kv, vv = locality_mixture(H, (3, 32, 32))
    g = torch.Generator().manual_seed(9)
    rows = lambda n: torch.randn(H, n, 128, generator=g).to(BF)
    # packed order: [context | video | pad], tensors [T, H, D]
    pack = lambda ctx, vid: torch.cat((ctx, vid, torch.zeros(H, pad, 128, dtype=BF)), dim=1).transpose(0, 1) \
        .contiguous().to(DEV)
    q, k, v = pack(rows(context), qv), pack(rows(context), kv), pack(rows(context), vv)
    B.set_backend_config({"t2t_h3_video_tokens": video, "t2t_h3_s_frac": 0.05, "t2t_cq": 32,
                          "t2t_dense_prefix_steps": 2})
    B.set_forward_context(SimpleNamespace(current_timestep=2))
    impl = B.T2TAttentionImpl(H, 128, False, SCALE, prefix="blocks.0.attn1")
    cu = torch.tensor([0, used], dtype=torch.int32, device=DEV)
    out = impl.forward_varlen(q, k, v, cu_seqlens=cu, max_seqlen=used, cu_seqlens_host=(0, used))
    torch.cuda.synchronize()
    runtime, = B._H3_RUNTIMES.values()
    dep = runtime.deploy
    assert dep.device_status() == 0 and (dep.H, dep.N, dep.pin_tail) == (28, used, context)
    S = dep.last_structure
    # the context keys (the operator's last rows) form the reserved last key cluster ...
    assert bool((S["klab"][:, video:] == 2047).all()) and bool((S["klab"][:, :video] != 2047).all())
    # ... which every non-empty query cluster's union contains
    has = (S["unip"][:, :, 63] >> 31) & 1
    assert bool((has[S["tile_sizes"] > 0] == 1).all())
    dense = _dense(q[:used], k[:used], v[:used])
    assert (out[:context].float() - dense[:context]).abs().max() < 2e-2     # context rows are dense
    rel = ((out[context:used].float() - dense[context:]).norm() / dense[context:].norm()).item()
    assert rel < 0.08, rel
    assert bool((out[used:] == 0).all())

    # The operator's last call (heads 28..55) against the oracle.  Its rows are [video | context] for keys and
    # values and [video | the first `context` video queries again] for the queries; the stages that follow the
    # clustering are replayed from the device's own labels and projections: selection with the pinned context
    # cluster bit for bit, exact attention + residual merge within the operator's tolerance.
    from oracle import t2t_oracle as O
    hs = slice(28, 56)
    tok = lambda t, rows: t[rows, hs].transpose(0, 1).cpu()                      # [28, rows, 128]
    vid, ctx = slice(context, used), slice(0, context)
    q_op = torch.cat((tok(q, vid), tok(q, vid)[:, :context]), dim=1)
    k_op = torch.cat((tok(k, vid), tok(k, ctx)), dim=1)
    v_op = torch.cat((tok(v, vid), tok(v, ctx)), dim=1)
    QU, cks, counts = dep.QU.cpu(), S["cks"].cpu(), S["counts"].cpu()
    qlab, klab = S["qlab"].cpu(), S["klab"].cpu()
    kcounts, kperm = O.stable_group(klab, 2048)
    assert torch.equal(counts, kcounts) and torch.equal(S["kperm"].cpu(), kperm)
    want_QU = O.project(q_op, cache_state_uq(impl), BF).float()
    assert (QU.float() - want_QU).abs().max() <= want_QU.abs().max() * 2.0 ** -7
    unip, rowcnt = O.select_union(QU, cks, counts, qlab, dep.CQ, int(dep.ns_t.item()), pin_tail=context)
    assert torch.equal(S["unip"].cpu(), unip) and torch.equal(dep.rowcnt.cpu(), rowcnt)
    _, sumv, lam, _ = O.vstats(v_op, kperm, kcounts, BF)
    assert torch.equal(dep._kmm_sumv.cpu().view(torch.int16), sumv.view(torch.int16))
    o, lse = O.exact_attention(q_op, k_op, v_op, qlab, klab, unip, SCALE)
    want = O.residual_merge(o, lse, QU, cks, sumv, lam, counts, unip, qlab, 1.0)
    err = (dep.tile_attn_out.float().cpu() - want).abs()
    assert err.max() < 2e-2 and err.mean() < 2e-3, (float(err.max()), float(err.mean()))
