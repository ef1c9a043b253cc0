"""Host logic of the SGLang backend mirror (token2tile_b200/t2t_attn.py) on the
CPU: budget schedule, profile resolution, budget tables, request cache and CFG
branch bookkeeping, dense prefix, state sanitising, packed-document path.  A
recording stand-in replaces the operator (which needs a GPU); its `step`
returns dense attention so outputs can be checked too."""
import json
import math
from types import SimpleNamespace

import pytest
import torch

from token2tile_b200 import t2t_attn as B

SCALE = 1.0 / math.sqrt(128)


class FakeDeploy:
    """Records what the backend asks of the operator."""
    instances = []

    def __init__(self, H, N, CQ, *, C=2048, D=128, r=32, s_frac=0.05, mask_refresh=1, cfg_reuse=False, pin_tail=0,
                 device="cpu", **kw):
        self.H, self.N, self.CQ, self.C, self.D, self.r = H, N, CQ, C, D, r
        self.s_frac, self.mask_refresh, self.cfg_reuse, self.pin_tail = s_frac, mask_refresh, cfg_reuse, pin_tail
        self.ns_t = torch.tensor(max(1, int(s_frac * N)), dtype=torch.int32)
        self.s_main = self.s_side = None
        self.calls, self.inits, self.resets = [], [], 0
        self.poison = False
        FakeDeploy.instances.append(self)

    def init_state(self, q, k, *, warm_iters=4, seed=0):
        self.inits.append(dict(warm_iters=warm_iters, seed=seed, shape=tuple(q.shape)))
        return {"Uq": torch.zeros(self.H, 128, 32), "Uk": torch.zeros(self.H, 128, 32),
                "ck": torch.ones(self.H, 8, 32), "cq": torch.ones(self.H, 4, 32)}

    def set_cfg_call(self, parity, key=0, step=0):
        self._next = (parity, key, step)

    def reset_cfg_reuse(self):
        self.resets += 1

    def check_status(self, wait=True):
        self.status_checks = getattr(self, "status_checks", 0) + 1

    def step(self, q, k, v, state):
        assert q.dtype == torch.bfloat16 and q.is_contiguous() and q.shape == (self.H, self.N, 128)
        self.calls.append(dict(cfg=self._next, ns=int(self.ns_t)))
        state["ck"] = state["ck"] * 2
        if self.poison:
            state["ck"][:, 0] = float("nan")
            state["cq"][:, 1] = 0
        return torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float()).to(q.dtype)


@pytest.fixture(autouse=True)
def fake_operator(monkeypatch):
    FakeDeploy.instances = []
    B.clear_runtimes()
    B.set_backend_config({})
    B.set_forward_context(None)
    B.set_ulysses_world_size(1)
    monkeypatch.setattr(B, "_load_operator", lambda tag: SimpleNamespace(MaskedStepDeploy=FakeDeploy))
    yield
    B.clear_runtimes()
    B.set_backend_config({})
    B.set_forward_context(None)
    B.set_ulysses_world_size(1)


def manual_meta(cache, step, *, total=50, ns_base=40, prefix=2, cq=4, ck=8, cfg_mult=(1.0, 0.5), **kw):
    return B.T2TAttentionMetadataBuilder().build(
        step, total, cache, profile_name="manual", ns_base=ns_base, dense_prefix_steps=prefix, cq=cq, ck=ck,
        step_profile=B.DEFAULT_STEP_PROFILE, layer_profile=B.DEFAULT_LAYER_PROFILE, cfg_mult=cfg_mult, **kw)


def qkv(n=64, h=12, seed=0):
    g = torch.Generator().manual_seed(seed)
    return tuple(torch.randn(1, n, h, 128, generator=g).to(torch.bfloat16) for _ in range(3))


# -- schedule -----------------------------------------------------------------
def test_step_windows():
    assert [B.step_window(s) for s in (0, 20, 21, 30, 31, 40, 41, 49)] == [0, 0, 1, 1, 2, 2, 3, 3]


def test_layer_groups_and_budget_map():
    p = B.BUILTIN_PROFILES["wan21_t2v_14b_n75600_t50"]
    assert B.profile_num_layers(p) == 40
    groups = [min(i * 6 // 40, 5) for i in range(40)]
    assert [B.layer_factor(i, p) for i in range(40)] == [p.layer_profile[g] for g in groups]
    with pytest.raises(ValueError):
        B.layer_factor(40, p)
    m = B.budget_map(p, p.seq_len)
    assert len(m) == 4 * 40 * 2
    assert m[(0, 0, 0)] == int(round(2424 * 1.574482 * 1.189098))
    assert m[(2, 39, 1)] == int(round(2424 * 0.555188 * 0.537588))
    assert all(1 <= v <= p.seq_len for v in m.values())
    assert B.budget(10, 1e9, 1.0, 1.0, 500) == 500 and B.budget(10, 1e-9, 1.0, 1.0, 500) == 1


def test_per_layer_profile_is_used_directly():
    layers = tuple(1.0 + 0.01 * i for i in range(30))
    p = B.T2TProfile("manual", 12, 4096, 50, 100, 0, 32, 2048, B.DEFAULT_STEP_PROFILE, layers)
    B.validate_profile(p)
    assert B.layer_factor(7, p) == layers[7]


def test_profile_resolution_rules():
    cache = B.T2TRequestCache()
    build = B.T2TAttentionMetadataBuilder().build
    auto = build(0, 50, cache)
    assert B.resolve_profile(auto, 75600, 40).name == "wan21_t2v_14b_n75600_t50"
    assert B.resolve_profile(auto, 32760, 12).name == "wan21_t2v_n32760_t50"
    with pytest.raises(ValueError, match="No built-in"):
        B.resolve_profile(auto, 1000, 40)
    with pytest.raises(ValueError, match="Unknown"):
        B.resolve_profile(build(0, 50, cache, profile_name="nope"), 75600, 40)
    with pytest.raises(ValueError, match="expects"):
        B.resolve_profile(build(0, 50, cache, profile_name="wan21_t2v_n32760_t50"), 75600, 40)
    with pytest.raises(ValueError, match="require t2t_profile='manual'"):
        B.resolve_profile(build(0, 50, cache, ns_base=5), 75600, 40)
    with pytest.raises(ValueError, match="requires ns_base"):
        B.resolve_profile(build(0, 50, cache, profile_name="manual", ns_base=5), 75600, 40)
    with pytest.raises(ValueError, match="ns_base"):
        B.resolve_profile(manual_meta(cache, 0, ns_base=10 ** 9), 64, 12)
    with pytest.raises(ValueError, match="head count"):
        B.resolve_profile(manual_meta(cache, 0), 64, 7)


def test_ns_table_loader(tmp_path):
    good = {"schema": "t2t_ns_table_v1", "heads": 12, "seq_len": 64, "ns": [[3] * 30, [4] * 30, [5] * 30, [6] * 30]}
    path = tmp_path / "t.json"
    path.write_text(json.dumps(good))
    rows, digest, header = B.load_ns_table(str(path), expected_layers=30, max_ns=64)
    assert rows[2][7] == 5 and len(digest) == 64 and header["heads"] == 12
    for bad in ({**good, "schema": "v0"}, {**good, "ns": good["ns"][:3]}, {**good, "ns": [[0] * 30] * 4},
                {**good, "ns": [[65] * 30] * 4}, {**good, "ns": [[3] * 29] * 4}):
        path.write_text(json.dumps(bad))
        with pytest.raises(ValueError):
            B.load_ns_table(str(path), expected_layers=30, max_ns=64)


# -- backend descriptor ---------------------------------------------------------
def test_backend_descriptor_and_constructor_checks():
    be = B.T2TAttentionBackend
    assert be.accept_output_buffer is True and be.get_supported_head_sizes() == [128]
    assert be.get_impl_cls() is B.T2TAttentionImpl and be.get_metadata_cls() is B.T2TAttentionMetadata
    assert be.get_builder_cls() is B.T2TAttentionMetadataBuilder and be.get_enum().name == "T2T_ATTN"
    ok = dict(num_heads=12, head_size=128, causal=False, softmax_scale=SCALE, prefix="blocks.3.attn1.attn")
    assert B.T2TAttentionImpl(**ok).layer_idx == 3
    assert B.T2TAttentionImpl(**{**ok, "prefix": "model.transformer_blocks.17.attn"}).layer_idx == 17
    assert B.T2TAttentionImpl(**{**ok, "prefix": "a.5.b.c"}).layer_idx == 5
    for change in (dict(causal=True), dict(head_size=64), dict(num_kv_heads=4), dict(softmax_scale=0.1),
                   dict(prefix="x.y")):
        with pytest.raises(ValueError):
            B.T2TAttentionImpl(**{**ok, **change})
    assert B.T2TAttentionImpl(**{**ok, "num_kv_heads": 12}).num_heads == 12


# -- request lifecycle ----------------------------------------------------------
def make_impl(layer=0, heads=12):
    return B.T2TAttentionImpl(heads, 128, False, SCALE, prefix=f"blocks.{layer}.attn")


def test_dense_prefix_then_sparse_with_parity_and_budgets():
    impl = make_impl(layer=5)
    cache = B.T2TRequestCache()
    q, k, v = qkv()
    want = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2).float(), k.transpose(1, 2).float(), v.transpose(1, 2).float()).transpose(1, 2)
    out = impl.forward(q, k, v, manual_meta(cache, 1))
    assert not FakeDeploy.instances and (out.float() - want).abs().max() < 2e-2      # prefix step: dense
    for step in (2, 3):
        for branch in range(2):
            out = impl.forward(q, k, v, manual_meta(cache, step, mask_refresh=4))
            assert out.shape == q.shape and out.dtype == q.dtype
            assert (out.float() - want).abs().max() < 2e-2
    dep, = FakeDeploy.instances
    assert (dep.H, dep.N, dep.CQ, dep.C, dep.mask_refresh, dep.cfg_reuse) == (12, 64, 4, 8, 4, True)
    assert dep.s_frac == 40 / 64 and dep.resets == 1
    assert [c["cfg"] for c in dep.calls] == [(0, 5, 2), (1, 5, 2), (0, 5, 3), (1, 5, 3)]
    lf = B.DEFAULT_LAYER_PROFILE[5 * 6 // 30]
    b0 = min(64, int(round(40 * B.DEFAULT_STEP_PROFILE[0] * lf)))
    b1 = min(64, max(1, int(round(40 * B.DEFAULT_STEP_PROFILE[0] * lf * 0.5))))
    assert [c["ns"] for c in dep.calls] == [b0, b1, b0, b1]
    # one state per (layer, branch), seeded 2*layer + branch, created once
    assert [i["seed"] for i in dep.inits] == [10, 11] and set(cache.states) == {(5, 0), (5, 1)}
    assert cache.call_counts == {(2, 5): 2, (3, 5): 2} and cache.initialized_runtime
    with pytest.raises(RuntimeError, match="more than two"):
        impl.forward(q, k, v, manual_meta(cache, 3, mask_refresh=4))


def test_budget_follows_window_and_table(tmp_path):
    impl = make_impl(layer=0)
    q, k, v = qkv(n=512)
    cache = B.T2TRequestCache()
    for step in (12, 25, 35, 45):
        impl.forward(q, k, v, manual_meta(cache, step, ns_base=100, cfg_mult=(1.0, 1.0)))
    dep, = FakeDeploy.instances
    want = [int(round(100 * s * B.DEFAULT_LAYER_PROFILE[0])) for s in B.DEFAULT_STEP_PROFILE]
    assert [c["ns"] for c in dep.calls] == want
    # an exact table replaces the product for both branches
    table = {"schema": "t2t_ns_table_v1", "heads": 12, "seq_len": 512,
             "ns": [[w * 100 + layer + 1 for layer in range(30)] for w in range(4)]}
    path = tmp_path / "ns.json"
    path.write_text(json.dumps(table))
    cache2 = B.T2TRequestCache()
    meta = lambda s: manual_meta(cache2, s, ns_base=100, cfg_mult=(1.0, 0.25), ns_table=str(path))
    impl.forward(q, k, v, meta(35))
    impl.forward(q, k, v, meta(35))
    dep2 = FakeDeploy.instances[-1]
    assert dep2 is not dep and [c["ns"] for c in dep2.calls] == [201, 201]
    table["heads"] = 40
    path.write_text(json.dumps(table))
    with pytest.raises(ValueError, match="geometry mismatch"):
        impl.forward(q, k, v, manual_meta(B.T2TRequestCache(), 35, ns_table=str(path)))


def test_new_request_resets_snapshots_and_runtime_is_shared():
    a, b = make_impl(layer=0), make_impl(layer=1)
    q, k, v = qkv()
    c1, c2 = B.T2TRequestCache(), B.T2TRequestCache()
    a.forward(q, k, v, manual_meta(c1, 5))
    b.forward(q, k, v, manual_meta(c1, 5))
    dep, = FakeDeploy.instances          # both layers share one operator instance
    assert dep.resets == 1
    a.forward(q, k, v, manual_meta(c2, 5))
    assert dep.resets == 2 and len(FakeDeploy.instances) == 1
    assert dep.status_checks == 2                # the device status word is examined at every request boundary
    # a request may not change geometry or settings half-way
    with pytest.raises(RuntimeError, match="geometry changed"):
        a.forward(q, k, v, manual_meta(c2, 6, mask_refresh=2))


def test_geometry_checks():
    impl = make_impl()
    q, k, v = qkv()
    cache = B.T2TRequestCache()
    with pytest.raises(ValueError, match="rank-4"):
        impl.forward(q[0], k[0], v[0], manual_meta(cache, 5))
    with pytest.raises(ValueError, match="equal self-attention"):
        impl.forward(q, k[:, :32], v[:, :32], manual_meta(cache, 5))
    with pytest.raises(ValueError, match="one request"):
        impl.forward(q.repeat(2, 1, 1, 1), k.repeat(2, 1, 1, 1), v.repeat(2, 1, 1, 1), manual_meta(cache, 5))
    with pytest.raises(ValueError, match="cluster count exceeds"):
        impl.forward(q, k, v, manual_meta(cache, 5, ck=128))
    B.set_ulysses_world_size(4)
    with pytest.raises(ValueError, match="geometry changed after"):
        impl.forward(q, k, v, manual_meta(cache, 5))
    q3, k3, v3 = (t[:, :, :3].contiguous() for t in (q, k, v))
    out = impl.forward(q3, k3, v3, manual_meta(cache, 5))       # 12 heads / 4 ranks = 3 local heads
    assert out.shape == q3.shape and FakeDeploy.instances[-1].H == 3


def test_sanitize_keeps_previous_centroid():
    impl = make_impl()
    q, k, v = qkv()
    cache = B.T2TRequestCache()
    impl.forward(q, k, v, manual_meta(cache, 5))
    dep, = FakeDeploy.instances
    state = cache.states[(0, 0)]
    assert torch.equal(state["ck"], torch.full((12, 8, 32), 2.0))
    dep.poison = True
    impl.forward(q, k, v, manual_meta(cache, 6))
    state = cache.states[(0, 0)]
    assert torch.isfinite(state["ck"]).all()
    assert torch.equal(state["ck"][:, 0], torch.full((12, 32), 2.0))      # NaN row: previous value kept
    assert torch.equal(state["ck"][:, 1], torch.full((12, 32), 4.0))
    assert torch.equal(state["cq"][:, 1], torch.ones(12, 32))             # all-zero row: previous value kept


# -- packed [context | video | pad] documents -------------------------------------
def packed(total=96, heads=56, seed=1):
    g = torch.Generator().manual_seed(seed)
    return tuple(torch.randn(total, heads, 128, generator=g).to(torch.bfloat16) for _ in range(3))


def dense_rows(q, k, v):
    return torch.nn.functional.scaled_dot_product_attention(
        q.transpose(0, 1).float(), k.transpose(0, 1).float(), v.transpose(0, 1).float()).transpose(0, 1)


def test_varlen_stays_dense_outside_the_main_document():
    q, k, v = packed(total=40, heads=12)
    cu = torch.tensor([0, 40], dtype=torch.int32)
    out = make_impl(heads=12).forward_varlen(q, k, v, cu_seqlens=cu, max_seqlen=40)       # other head count
    assert not FakeDeploy.instances and (out.float() - dense_rows(q, k, v)).abs().max() < 2e-2
    q, k, v = packed(total=40)
    impl = make_impl(heads=56)
    B.set_backend_config({"t2t_h3_video_tokens": 24})
    B.set_forward_context(SimpleNamespace(current_timestep=3))                           # prefix step
    impl.forward_varlen(q, k, v, cu_seqlens=cu, max_seqlen=40, cu_seqlens_host=(0, 40))
    B.set_backend_config({})                                                             # no layout, no constant
    B.set_forward_context(SimpleNamespace(current_timestep=20))
    impl.forward_varlen(q, k, v, cu_seqlens=cu, max_seqlen=40)
    assert not FakeDeploy.instances


def test_varlen_sparse_path_layout_chunks_and_budget():
    total, used, video = 96, 80, 56
    context = used - video
    q, k, v = packed(total)
    B.set_backend_config({"t2t_h3_video_tokens": video, "t2t_h3_s_frac": 0.25, "t2t_cq": 4, "t2t_ck": 8,
                          "t2t_mask_refresh": 2})
    impl = make_impl(layer=9, heads=56)
    cu = torch.tensor([0, used], dtype=torch.int32)
    B.set_forward_context(SimpleNamespace(current_timestep=12))
    out = impl.forward_varlen(q, k, v, cu_seqlens=cu, max_seqlen=used)
    dep, = FakeDeploy.instances
    assert (dep.H, dep.N, dep.CQ, dep.C, dep.pin_tail, dep.mask_refresh) == (28, used, 4, 8, context, 2)
    # two chunks of 28 heads: snapshot key (layer, chunk), branch 0, seeds 8*layer + chunk
    assert [c["cfg"] for c in dep.calls] == [(0, (9, 0), 12), (0, (9, 1), 12)]
    assert [i["seed"] for i in dep.inits] == [72, 73]
    ns = B.budget(int(0.25 * used), B.DEFAULT_STEP_PROFILE[0], B.DEFAULT_LAYER_PROFILE[9 * 6 // 50], 1.0, used)
    assert [c["ns"] for c in dep.calls] == [ns, ns]
    # the stand-in operator is dense over [video | context] keys, so every used row equals dense attention
    want = dense_rows(q[:used], k[:used], v[:used])
    assert (out[:used].float() - want).abs().max() < 3e-2
    assert (out[used:] == 0).all() and out.dtype == q.dtype and out.shape == q.shape
    # second sparse step: states are kept, nothing is re-initialised
    B.set_forward_context(SimpleNamespace(current_timestep=13))
    impl.forward_varlen(q, k, v, cu_seqlens=cu, max_seqlen=used)
    assert len(dep.inits) == 2 and len(dep.calls) == 4
    # the first sparse step of the next request drops them (and keeps them with t2t_persist_state)
    B.set_forward_context(SimpleNamespace(current_timestep=12))
    impl.forward_varlen(q, k, v, cu_seqlens=cu, max_seqlen=used)
    assert len(dep.inits) == 4
    B.set_backend_config({"t2t_h3_video_tokens": video, "t2t_h3_s_frac": 0.25, "t2t_cq": 4, "t2t_ck": 8,
                          "t2t_mask_refresh": 2, "t2t_persist_state": True})
    impl.forward_varlen(q, k, v, cu_seqlens=cu, max_seqlen=used)
    assert len(dep.inits) == 4


def test_varlen_reset_only_from_layer_zero_and_ulysses_chunks():
    used, video = 80, 56
    B.set_backend_config({"t2t_h3_video_tokens": video, "t2t_cq": 4, "t2t_ck": 8})
    B.set_forward_context(SimpleNamespace(current_timestep=12))
    B.set_ulysses_world_size(8)
    q, k, v = packed(used, heads=7)
    cu = torch.tensor([0, used], dtype=torch.int32)
    l0, l1 = make_impl(layer=0, heads=56), make_impl(layer=1, heads=56)
    l1.forward_varlen(q, k, v, cu_seqlens=cu, max_seqlen=used)
    dep, = FakeDeploy.instances
    assert dep.H == 7 and dep.resets == 0        # 56 / 8 ranks: one chunk of 7 heads
    l0.forward_varlen(q, k, v, cu_seqlens=cu, max_seqlen=used)
    assert dep.resets == 1
    with pytest.raises(ValueError, match="sharding mismatch"):
        l0.forward_varlen(*packed(used, heads=5), cu_seqlens=cu, max_seqlen=used)
    with pytest.raises(ValueError, match="used length"):
        l0.forward_varlen(q, k, v, cu_seqlens=cu, max_seqlen=used + 1)
    B.set_backend_config({"t2t_h3_video_tokens": 30, "t2t_cq": 4, "t2t_ck": 8})
    with pytest.raises(ValueError, match="video >= context"):
        l0.forward_varlen(q, k, v, cu_seqlens=cu, max_seqlen=used)


def test_video_tokens_from_published_layout_and_condition_rows():
    used = 80
    layout = {"video": 56, "video_start": 24, "video_stop": 80}
    B.set_forward_context(SimpleNamespace(current_timestep=12, minimax_h3_layout=layout))
    cpu = torch.device("cpu")
    assert B._h3_split(used, "dense", cpu) == (56, None)
    assert B._h3_split(81, "dense", cpu) == (0, None)                    # not the main document
    layout2 = {"video": 56, "video_start": 10, "video_stop": 80}
    B.set_forward_context(SimpleNamespace(current_timestep=12, minimax_h3_layout=layout2))
    assert B._h3_split(used, "dense", cpu) == (0, None)                  # video is not the contiguous tail
    # condition frames precede the audio rows: only the generated tail is sparse
    layout3 = {"video": 56, "video_tail": 48, "video_start": 4, "video_stop": 80}
    B.set_forward_context(SimpleNamespace(current_timestep=12, minimax_h3_layout=layout3))
    assert B._h3_split(used, "dense", cpu) == (48, None)
    video, (vid, ctx) = B._h3_split(used, "sparse", cpu)
    assert video == 56 and vid.tolist() == list(range(4, 12)) + list(range(32, 80))
    assert ctx.tolist() == list(range(0, 4)) + list(range(12, 32))
    B.set_backend_config({"t2t_h3_cond_mode": "sparse", "t2t_cq": 4, "t2t_ck": 8})
    q, k, v = packed(used)
    out = make_impl(layer=0, heads=56).forward_varlen(q, k, v, cu_seqlens=torch.tensor([0, used]), max_seqlen=used)
    assert FakeDeploy.instances[-1].pin_tail == 24
    assert (out.float() - dense_rows(q, k, v)).abs().max() < 3e-2
    assert B.h3_auto_cq(75600) == 592 and B.h3_auto_cq(4096) == 64
