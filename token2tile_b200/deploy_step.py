"""Token2Tile attention operator for B200: one sparse attention call of one layer.

Host-side mirror of the reference operator module
(token2tile/operator/deploy_step.py): same class, constructor arguments,
methods, attributes and rebuild / reuse rules, over the sm_100a kernels of
libt2t_b200.so.  `MaskedStepDeploy.step(q, k, v, state)` runs, for q, k, v of
shape [H, N, 128] (bfloat16):

  1. projection   Q -> Q Uq, K -> K Uk into the rank-32 space      t2t_project
  2. clustering   warm-started k-means of keys (2048 clusters) and
                  queries (CQ clusters), stable grouping, cluster-
                  major V and per-cluster value sums                t2t_kmeans_maintain
  3. scoring +    every query against every key centroid, budgeted
     selection    prefix of whole clusters, union per query cluster t2t_score_select_union
  4. attention    exact attention of every query cluster over its
                  union + centroid residual, one softmax            t2t_tile_attn

PyTorch supplies device memory and streams; every stage above, and the
projection fit of `init_state`, is a hand-written CUDA kernel.  There is no
CPU path: the module refuses to load without the compiled library.
"""
from __future__ import annotations

import math

import torch

try:
    from . import _lib
except ImportError:      # imported as a top-level module from operator_dir(), the way the reference's hosts do
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from token2tile_b200 import _lib
check, ptr = _lib.check, _lib.ptr

BF16 = torch.bfloat16


# ---------------------------------------------------------------------------
# low-rank space
# ---------------------------------------------------------------------------

def lowrank_fit(q, k, r=32, *, check_finite=True):
    """Runs the projection-fit kernels (t2t_lowrank_fit) on q, k [H, N, 128] and
    returns fp32 Uq, Uk [H, 128, r].

    The second moments Mq = Q^T Q / N, Mk = K^T K / N come from the tensor cores
    (bfloat16 inputs, fp32 slabs summed in fp64 in a fixed order); their
    symmetric roots and the singular triplets of Mq^(1/2) Mk^(1/2) come from an
    fp64 Jacobi kernel, one CTA per matrix, batched over heads.  Inputs of
    another dtype are rounded to bfloat16 first: the operator's own tensors are
    bfloat16, so nothing is lost on its path.

    check_finite=True reads one flag per head back (a host synchronisation) and
    raises RuntimeError for non-finite inputs, like the reference
    (deploy_step.py:127-132); check_finite=False returns without synchronising
    and leaves the projections of such a head at zero."""
    if r != 32:
        raise ValueError("the kernels require r=32")
    if q.dim() != 3 or q.shape[2] != 128 or k.shape != q.shape or not q.is_cuda or k.device != q.device:
        raise ValueError(f"lowrank_fit: expected CUDA tensors [H, N, 128] of one shape, got {tuple(q.shape)} "
                         f"and {tuple(k.shape)}")
    lib = _lib.load()
    qb = q if q.dtype == BF16 else q.to(BF16)
    kb = k if k.dtype == BF16 else k.to(BF16)
    try:                                    # views of [N, H, 128] tensors are read in place
        lay = rows_layout(qb)
        if rows_layout(kb) != lay:
            raise ValueError("q and k are laid out differently")
    except ValueError:
        qb, kb = qb.contiguous(), kb.contiguous()
        lay = rows_layout(qb)
    H, N, D = qb.shape
    dev = qb.device
    Uq = torch.zeros(H, D, r, device=dev, dtype=torch.float32)
    Uk = torch.zeros(H, D, r, device=dev, dtype=torch.float32)
    flags = torch.zeros(2 * H + 1, device=dev, dtype=torch.int32)       # [2 H] non-finite, [1] wait status
    ws = torch.empty(int(lib.t2t_lowrank_fit_ws_bytes(H, N)), device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        check(lib.t2t_lowrank_fit_strided(ptr(qb), ptr(kb), lay[0], lay[1], ptr(Uq), ptr(Uk), H, N, ptr(ws), ws.numel(),
                                          ptr(flags), ptr(flags) + 8 * H,
                                          _stream_ptr(torch.cuda.current_stream(dev))), "t2t_lowrank_fit")
    if check_finite:
        f = flags.cpu()
        if int(f[2 * H]) != 0:
            raise RuntimeError("lowrank_fit: a bounded device wait timed out")
        for name, part in (("q", f[:H]), ("k", f[H:2 * H])):
            if bool(part.any()):
                raise RuntimeError(f"online_u: non-finite {name} input in heads {part.nonzero()[:, 0].tolist()}, "
                                   f"shape {tuple(q.shape)}")
    return Uq, Uk


def online_u(qf, kf, r=32):
    """Matched rank-r projections Uq, Uk [H, 128, r] (fp32) that minimise
    ||Q K^T - (Q Uq)(K Uk)^T||_F; same contract as the reference's function of
    this name (deploy_step.py:122-149).  With the second moments Mq, Mk and the
    singular value decomposition Mq^(1/2) Mk^(1/2) = U S V^T (eigenvalues of
    the moments clamped at 1e-8),

        Uq = Mq^(-1/2) U_r S_r^(1/2),    Uk = Mk^(-1/2) V_r S_r^(1/2).

    The columns are defined up to a common sign (and a rotation inside equal
    singular values): compare Uq Uk^T, not the factors.  Runs on the GPU only
    (see `lowrank_fit`); raises RuntimeError for non-finite inputs."""
    return lowrank_fit(qf, kf, r, check_finite=True)


def _stream_ptr(stream) -> int:
    return stream.cuda_stream


def rows_layout(t):
    """(row stride, head stride) in elements of a bfloat16 tensor indexed [head, row, 128] whose 128
    elements of a row are contiguous: (128, N * 128) for a contiguous [H, N, 128] tensor, (H * 128, 128) for
    the [H, N, 128] view of a tensor stored [N, H, 128].  The kernels take both; strides must be whole rows
    (multiples of 128 elements) and the storage 16-byte aligned."""
    if t.dim() != 3 or t.shape[2] != 128 or t.dtype != BF16 or t.stride(2) != 1:
        raise ValueError(f"expected a bfloat16 [H, n, 128] tensor with contiguous rows, got {t.dtype} "
                         f"{tuple(t.shape)} strides {tuple(t.stride())}")
    head, row = t.stride(0), t.stride(1)
    if t.shape[0] == 1:
        head = max(head, 128)            # the stride of a singleton dimension is arbitrary
    if row % 128 or head % 128 or row <= 0 or head <= 0 or t.data_ptr() % 16:
        raise ValueError(f"row and head strides must be positive multiples of 128 elements, got {tuple(t.stride())}")
    return row, head


# ---------------------------------------------------------------------------
# module-level helpers of the reference operator module
# ---------------------------------------------------------------------------
# The reference's deploy_step imports fast_assign, fast_gather and
# fused_update_vstats into its namespace (deploy_step.py:40-42) and its hosts call
# them through the module (integrations/sglang/backend/t2t_attn.py:275-278).  The
# same names here run the library's kernels on the current stream.

def _cur_stream(t):
    return _stream_ptr(torch.cuda.current_stream(t.device))


def _check_rows(name, t, inner):
    if t.dtype != BF16 or t.dim() != 3 or t.shape[2] != inner or not t.is_contiguous() or not t.is_cuda:
        raise ValueError(f"{name}: expected a contiguous CUDA bfloat16 [H, n, {inner}] tensor, got "
                         f"{t.dtype} {tuple(t.shape)}")


def fast_assign(x, centroids, out=None, **_tuning):
    """Nearest centroid of every row, lowest index on ties (fast_assign.py:79-106).
    x [H, N, 32], centroids [H, C, 32] bfloat16 -> labels [H, N] int32.  Tuning
    keywords of the reference are accepted and ignored.  Distances are the
    exact fp32 chains of the operator (the reference truncates the low 11 bits
    of the distance in its packed key)."""
    _check_rows("fast_assign x", x, 32)
    _check_rows("fast_assign centroids", centroids, 32)
    H, N, _ = x.shape
    if centroids.shape[0] != H:
        raise ValueError("fast_assign: head counts differ")
    lib = _lib.load()
    if out is None:
        out = torch.empty(H, N, device=x.device, dtype=torch.int32)
    ws = torch.empty(int(lib.t2t_assign_ws_bytes(H, N)), device=x.device, dtype=torch.uint8)
    status = torch.zeros(1, device=x.device, dtype=torch.int32)
    with torch.cuda.device(x.device):
        check(lib.t2t_assign(ptr(x), ptr(centroids), ptr(out), H, N, centroids.shape[1], -1, 0, ptr(ws), ws.numel(),
                             ptr(status), _cur_stream(x)), "t2t_assign")
    return out


def fast_gather(x, perm, out=None, **_tuning):
    """o[h, i] = x[h, perm[h, i]] for x [H, N, 128] bfloat16 (fast_permute.py:54-56)."""
    _check_rows("fast_gather x", x, 128)
    H, N, _ = x.shape
    perm_i = perm.to(torch.int32).contiguous()
    if out is None:
        out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(_lib.load().t2t_gather_rows(ptr(x), ptr(perm_i), ptr(out), H, N, _cur_stream(x)), "t2t_gather_rows")
    return out


def fused_update_vstats(ku, labels, old_centroids, v=None, **_tuning):
    """Cluster means of ku under `labels`; an empty cluster keeps its old centroid
    (fused_update_vstats.py:72-115).  Returns (new_centroids [H, C, 32] bfloat16,
    counts [H, C] int32, None).  The means are the deterministic fixed-point ones
    (the reference accumulates with fp32 atomics).  Only v=None is supported: the
    operator computes value statistics inside t2t_kmeans_maintain."""
    if v is not None:
        raise NotImplementedError("fused_update_vstats: value statistics are part of t2t_kmeans_maintain here")
    _check_rows("fused_update_vstats ku", ku, 32)
    _check_rows("fused_update_vstats old_centroids", old_centroids, 32)
    H, N, _ = ku.shape
    Cn = old_centroids.shape[1]
    lib = _lib.load()
    lab = labels.to(torch.int32).contiguous()
    newc = torch.empty_like(old_centroids)
    counts = torch.empty(H, Cn, device=ku.device, dtype=torch.int32)
    ws = torch.empty(int(lib.t2t_centroid_update_ws_bytes(H, N, Cn)), device=ku.device, dtype=torch.uint8)
    with torch.cuda.device(ku.device):
        check(lib.t2t_centroid_update(ptr(ku), ptr(lab), ptr(old_centroids), ptr(newc), ptr(counts), H, N, Cn,
                                      ptr(ws), ws.numel(), _cur_stream(ku)), "t2t_centroid_update")
    return newc, counts, None


class MaskedStepDeploy:
    """Persistent buffers and kernels for one (H, N, C_Q) attention shape
    (deploy_step.py:152-242).

    s_frac: per-query token budget as a fraction of N; `ns_t` holds the token
        count on the device and may be overwritten between calls.
    mask_refresh: rebuild the structure every this many annotated steps.
    cfg_reuse: reuse the structure across CFG branches even when
        mask_refresh is 1.
    pin_tail: the last pin_tail keys form one reserved key cluster that every
        query executes exactly.
    split_cap: accepted for interface compatibility; selection here works per
        query row, so there is nothing to split."""

    def __init__(self, H, N, CQ, *, C=2048, D=128, r=32, s_frac=0.05, tailw=1.0, device="cuda",
                 mask_refresh=1, cfg_reuse=False, pin_tail=0, split_cap="auto"):
        if C != 2048 or D != 128:
            raise ValueError("the kernels require C=2048 and D=128")
        if r != 32:
            raise ValueError("the kernels require r=32")
        if N < max(C, CQ):
            raise ValueError("N must be at least max(C, CQ)")
        self.lib = _lib.load()
        self.H, self.N, self.CQ, self.C, self.D, self.r = H, N, CQ, C, D, r
        self.ns = max(1, int(s_frac * N))
        self.tailw = tailw
        self.dev = dev = torch.device(device)
        self.scale = 1.0 / math.sqrt(D)
        self.pin_tail = int(pin_tail)
        self.split_cap = 0

        f32, i32 = torch.float32, torch.int32
        e = lambda *shape, dtype: torch.empty(*shape, device=dev, dtype=dtype)
        # persistent buffers, allocated once
        self.QU = e(H, N, r, dtype=BF16)
        self.KU = e(H, N, r, dtype=BF16)
        self.rowcnt = e(H, N, dtype=i32)
        self.kp = e(H, N, D, dtype=BF16)
        self.vp = e(H, N, D, dtype=BF16)
        self.tile_attn_out = e(H, N, D, dtype=BF16)
        self._kmm_cq2 = e(H, CQ, r, dtype=BF16)
        self._kmm_ck2 = e(H, C, r, dtype=f32)
        self._kmm_sumv = e(H, C, D, dtype=BF16)
        self._kmm_lam = e(H, dtype=f32)
        self.tailw_t = torch.tensor(float(tailw), device=dev, dtype=f32)
        self.ns_t = torch.tensor(self.ns, device=dev, dtype=i32)
        self.status = torch.zeros(1, device=dev, dtype=i32)
        # host copy of the status word, refreshed asynchronously after every step() (see check_status)
        self._status_host = torch.zeros(1, dtype=i32).pin_memory() if dev.type == "cuda" else torch.zeros(1, dtype=i32)
        self._status_event = None
        L = self.lib
        self._tile_attn_plan_ints = int(L.t2t_tile_attn_plan_ints(H, N, CQ))
        ws = max(int(L.t2t_kmeans_maintain_ws_bytes(H, N, CQ, C)),
                 int(L.t2t_vstats_gather_ws_bytes(H, C)),
                 int(L.t2t_centroid_update_ws_bytes(H, N, C)), int(L.t2t_assign_ws_bytes(H, N)),
                 int(L.t2t_score_select_union_ws_bytes(H, N)))
        self._ws = e(ws, dtype=torch.uint8)
        self._attn_ws = e(int(L.t2t_tile_attn_ws_bytes(H, N)), dtype=torch.uint8)
        self._struct = self._new_structure()      # structure of unannotated calls

        # Structure reuse (deploy_step.py:210-221).  A full call (branch 0 and
        # snapshot age >= mask_refresh) rebuilds the structure and stores it per
        # key (layer); every other annotated call reuses the stored snapshot.
        self.cfg_reuse = bool(cfg_reuse)
        self.mask_refresh = max(1, int(mask_refresh))
        self._cfg_on = self.cfg_reuse or self.mask_refresh > 1
        self._cfg_hold = {}
        self._cfg_parity = None
        self._cfg_key = 0
        self._cfg_step = 0

        self.s_main = torch.cuda.Stream(device=dev)
        self.s_side = torch.cuda.Stream(device=dev)
        self.last_rebuilt = None
        self.last_structure = None
        # optional per-stage CUDA-event timing of step(), recorded on s_main
        self.profile = False
        self._marks = []

    def _new_structure(self):
        """Tensors that describe one structure (labels, groupings, centroids,
        union, task plan); a snapshot owns one such set."""
        H, N, CQ, C, r, dev = self.H, self.N, self.CQ, self.C, self.r, self.dev
        i32 = torch.int32
        e = lambda *shape, dtype: torch.empty(*shape, device=dev, dtype=dtype)
        return {
            "qlab": e(H, N, dtype=i32), "klab": e(H, N, dtype=i32),
            "qperm": e(H, N, dtype=i32), "kperm": e(H, N, dtype=i32),
            "tile_sizes": e(H, CQ, dtype=i32), "counts": e(H, C, dtype=i32),
            "cks": e(H, C, r, dtype=BF16), "unip": e(H, CQ, C // 32, dtype=i32),
            "tile_attn_plan": e(self._tile_attn_plan_ints, dtype=i32),
            "Uq": None, "step": 0,
        }

    def _check_qkv(self, *tensors):
        """q, k, v (and a caller's output tensor): bfloat16 [H, N, 128] on the operator's device, contiguous or
        a view with whole-row strides (the [H, N, 128] view of a [N, H, 128] tensor: see rows_layout)."""
        for t in tensors:
            if t.dtype != BF16 or tuple(t.shape) != (self.H, self.N, self.D) or t.device != self.QU.device:
                raise ValueError(
                    f"expected bfloat16 [{self.H}, {self.N}, {self.D}] on {self.QU.device}, got "
                    f"{t.dtype} {tuple(t.shape)} on {t.device}")
            rows_layout(t)

    # -- stage timing ------------------------------------------------------------
    def _mark(self, name):
        if self.profile:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(self.s_main)
            self._marks.append((name, ev))

    def stage_times(self):
        """Milliseconds per stage of the last step() when `profile` was set
        (synchronises).  Stage names: project, kmeans, select, gather_k, vstats,
        plan, attn_exact, residual_merge."""
        torch.cuda.synchronize(self.dev)
        out = {}
        for (_, e0), (name, e1) in zip(self._marks[:-1], self._marks[1:]):
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
        return out

    # -- kernel wrappers -------------------------------------------------------
    def _project(self, x, U, out, st):
        row, head = rows_layout(x)
        check(self.lib.t2t_project_strided(ptr(x), row, head, ptr(U), ptr(out), self.H, self.N, ptr(self.status), st),
              "t2t_project")

    def _assign(self, x, cen, labels, st):
        check(self.lib.t2t_assign(ptr(x), ptr(cen), ptr(labels), self.H, self.N, cen.shape[1], -1, 0,
                                  ptr(self._ws), self._ws.numel(), ptr(self.status), st), "t2t_assign")

    def _centroid_update(self, x, labels, old, st):
        newc = torch.empty_like(old)
        counts = torch.empty(self.H, old.shape[1], device=self.dev, dtype=torch.int32)
        check(self.lib.t2t_centroid_update(ptr(x), ptr(labels), ptr(old), ptr(newc), ptr(counts), self.H, self.N,
                                           old.shape[1], ptr(self._ws), self._ws.numel(), st), "t2t_centroid_update")
        return newc, counts

    # -- state init ------------------------------------------------------------
    def warm_start(self, q, k, Uq, Uk, rows_k, rows_q, warm_iters):
        """Common tail of the state initialisers: rounds the fitted projections to
        bfloat16, projects q and k, takes the rows `rows_k` / `rows_q` (sorted row
        indices on the device) of the projected keys / queries as first centroids
        and runs `warm_iters` Lloyd rounds on each side with the operator's exact
        assignment and deterministic fixed-point mean.  Queues work on the current
        stream of the operator's device; does not synchronise."""
        with torch.cuda.device(self.dev):
            st = _stream_ptr(torch.cuda.current_stream(self.dev))
            state = {"Uq": Uq.to(BF16).contiguous(), "Uk": Uk.to(BF16).contiguous()}
            labels = torch.empty(self.H, self.N, device=self.dev, dtype=torch.int32)
            for side, x, proj, rows in (("ck", k, state["Uk"], rows_k), ("cq", q, state["Uq"], rows_q)):
                low = torch.empty_like(self.KU)
                self._project(x, proj, low, st)
                cen = low[:, rows, :].contiguous()
                for _ in range(warm_iters):
                    self._assign(low, cen, labels, st)
                    cen, _ = self._centroid_update(low, labels, cen, st)
                state[side] = cen.contiguous()
        return state

    def init_state(self, q, k, *, warm_iters=4, seed=0):
        """Projections and first centroids of one layer (deploy_step.py:245-266):
        the projection fit (`online_u`, raising on non-finite input), C key rows
        and CQ query rows drawn by a seeded CPU generator as first centroids, and
        `warm_iters` Lloyd rounds per side.  The projections stay for the whole
        request; the centroids warm-start every rebuild.  Ends with a host
        synchronisation, like the reference."""
        self._check_qkv(q, k)
        Uq, Uk = online_u(q, k, self.r)
        gen = torch.Generator(device="cpu").manual_seed(seed)
        rows_k = torch.randperm(self.N, generator=gen)[: self.C].sort().values.to(self.dev)
        rows_q = torch.randperm(self.N, generator=gen)[: self.CQ].sort().values.to(self.dev)
        state = self.warm_start(q, k, Uq, Uk, rows_k, rows_q, warm_iters)
        torch.cuda.synchronize(self.dev)
        return state

    def set_cfg_call(self, parity, key=0, step=0):
        """Annotate the next step() call (deploy_step.py:268-277): parity is the
        CFG branch (0 = the branch allowed to rebuild), key the snapshot slot
        (one per layer), step the denoising step.  A branch-0 call rebuilds when
        step - snapshot_step >= mask_refresh."""
        self._cfg_parity = int(parity)
        self._cfg_key = key
        self._cfg_step = int(step)

    def reset_cfg_reuse(self):
        """Drop all snapshots and any pending annotation (deploy_step.py:279-283)."""
        self._cfg_hold.clear()
        self._cfg_parity = None

    def _pick(self):
        """Decides between a rebuild and a reuse call (deploy_step.py:297-316, 420-440).
        Returns (snapshot, structure, publish): the snapshot to reuse (None for a
        rebuild), the set of structure tensors a rebuild writes into, and whether
        the rebuilt structure becomes the stored snapshot of the current key.

        An annotated call (set_cfg_call) looks its key up: the stored snapshot is
        reused unless this is branch 0 and the snapshot is mask_refresh steps
        old, or the step counter ran backwards (a new request).  Its rebuild
        recycles the tensors of the snapshot it replaces.  An unannotated call
        always rebuilds; with snapshots switched on the result is still stored,
        under the key and step of the last annotation, in tensors of its own -
        as the reference does, so a later annotated call of that key can reuse it."""
        parity, self._cfg_parity = self._cfg_parity, None      # an annotation is good for one call
        if not self._cfg_on:
            return None, self._struct, False
        if parity is None:
            return None, self._new_structure(), True
        stored = self._cfg_hold.get(self._cfg_key)
        if stored is not None:
            age = self._cfg_step - stored["step"]
            stale = age >= self.mask_refresh
            if age >= 0 and not (parity == 0 and stale):
                return stored, self._struct, False
            return None, stored, True
        return None, self._new_structure(), True

    # -- the attention call ------------------------------------------------------
    def step(self, q, k, v, state, out=None):
        """q, k, v: [H, N, 128] bfloat16, original row order; contiguous, or views with whole-row
        strides (the [H, N, 128] view of a tensor stored [N, H, 128], which a serving host holds,
        is read in place: no transposing copy).  state:
        dict(Uq, Uk, ck, cq); ck / cq are replaced by the centroids that
        warm-start the next call.  Returns out [H, N, 128] bfloat16: the tensor
        passed as `out` (same shape, dtype, device, contiguous), else a buffer
        owned by the operator and overwritten by the next call.  A caller that
        still reads the previous result while the next call runs (a copy to the
        host in flight, say) alternates two `out` tensors."""
        self._check_qkv(q, k, v)
        self.check_status(wait=False)
        if out is None:
            out = self.tile_attn_out
        else:
            try:
                self._check_qkv(out)
            except ValueError as exc:
                raise ValueError("out must be a bfloat16 tensor [H, N, 128] on the operator's device, contiguous or "
                                 f"with whole-row strides ({exc})") from None
        q_lay, k_lay, v_lay, o_lay = rows_layout(q), rows_layout(k), rows_layout(v), rows_layout(out)
        caller = torch.cuda.current_stream(self.dev)
        if caller != self.s_main:
            self.s_main.wait_stream(caller)
        H, N, C, CQ = self.H, self.N, self.C, self.CQ
        L = self.lib
        snap, S, publish = self._pick()
        st = _stream_ptr(self.s_main)
        self._marks = []
        with torch.cuda.stream(self.s_main):
            self._mark("start")
            if snap is None:
                self._project(q, state["Uq"], self.QU, st)
                self._project(k, state["Uk"], self.KU, st)
                self._mark("project")
                ck16 = torch.empty(H, C, self.r, device=self.dev, dtype=BF16)
                check(L.t2t_kmeans_maintain_strided(
                    ptr(self.QU), ptr(self.KU), ptr(v), v_lay[0], v_lay[1], ptr(state["cq"]), ptr(state["ck"]),
                    ptr(S["qlab"]), ptr(self._kmm_cq2), ptr(S["klab"]), ptr(self._kmm_ck2), ptr(ck16),
                    ptr(S["cks"]), ptr(S["tile_sizes"]), ptr(S["qperm"]), ptr(S["counts"]), ptr(S["kperm"]),
                    ptr(self.vp), ptr(self._kmm_sumv), ptr(self._kmm_lam), self.scale, H, N, CQ, C,
                    self.pin_tail, ptr(self._ws), self._ws.numel(), ptr(self.status), st), "t2t_kmeans_maintain")
                # fresh tensors, so the next call's inputs never alias kernel outputs
                state["ck"] = ck16
                state["cq"] = self._kmm_cq2.clone()
                self._mark("kmeans")
                # the key gather only needs kperm: it runs on the side stream, under the selection
                # (one is bound by HBM, the other by integer arithmetic)
                self.s_side.wait_stream(self.s_main)
                check(L.t2t_gather_rows_strided(ptr(k), k_lay[0], k_lay[1], ptr(S["kperm"]), ptr(self.kp), H, N,
                                                _stream_ptr(self.s_side)), "t2t_gather_rows")
                check(L.t2t_score_select_union(
                    ptr(self.QU), ptr(S["cks"]), ptr(S["counts"]), ptr(S["qperm"]), ptr(S["tile_sizes"]),
                    ptr(self.ns_t), ptr(S["unip"]), ptr(self.rowcnt), H, N, CQ, self.pin_tail, ptr(self._ws),
                    self._ws.numel(), ptr(self.status), st), "t2t_score_select_union")
                self._mark("select")
                S["Uq"] = state["Uq"]
                S["step"] = self._cfg_step
                if publish:
                    self._cfg_hold[self._cfg_key] = S
                self.s_main.wait_stream(self.s_side)      # kp is ready
                self._mark("gather_k")
                check(L.t2t_tile_attn_plan(ptr(S["tile_sizes"]), ptr(S["counts"]), ptr(S["unip"]),
                                           ptr(S["tile_attn_plan"]), H, N, CQ, st), "t2t_tile_attn_plan")
                self._mark("plan")
            else:
                S = snap
                # a reuse call projects its queries with the snapshot's Uq so that
                # QU and the stored centroids share a basis
                self._project(q, S["Uq"], self.QU, st)
                self._mark("project")
                check(L.t2t_gather_rows_strided(ptr(k), k_lay[0], k_lay[1], ptr(S["kperm"]), ptr(self.kp), H, N, st),
                      "t2t_gather_rows")
                self._mark("gather_k")
                check(L.t2t_vstats_gather_strided(ptr(v), v_lay[0], v_lay[1], ptr(S["kperm"]), ptr(S["counts"]), ptr(self.vp),
                                          ptr(self._kmm_sumv), ptr(self._kmm_lam), H, N, C, ptr(self._ws),
                                          self._ws.numel(), st), "t2t_vstats_gather")
                self._mark("vstats")
            # the plan belongs to the structure: a reuse call only resets its task cursor
            check(L.t2t_tile_attn_exact_strided(
                ptr(q), q_lay[0], q_lay[1], ptr(self.kp), ptr(self.vp), ptr(S["unip"]), ptr(S["qperm"]),
                ptr(S["tile_attn_plan"]),
                H, N, CQ, ptr(self._attn_ws), self._attn_ws.numel(), ptr(self.status), st), "t2t_tile_attn_exact")
            self._mark("attn_exact")
            check(L.t2t_tile_attn_merge_strided(
                ptr(self.QU), ptr(S["cks"]), ptr(self._kmm_sumv), ptr(S["counts"]), ptr(S["unip"]),
                ptr(S["qlab"]), ptr(S["qperm"]), ptr(self._kmm_lam), ptr(self.tailw_t), ptr(out), o_lay[0], o_lay[1],
                H, N, CQ, ptr(self._attn_ws), self._attn_ws.numel(), ptr(self.status), st), "t2t_tile_attn_merge")
            self._mark("residual_merge")
            # the status word travels to pinned host memory behind the kernels; nobody waits for it here
            self._status_host.copy_(self.status, non_blocking=True)
            if self._status_event is None:
                self._status_event = torch.cuda.Event()
            self._status_event.record(self.s_main)
        self.last_rebuilt = snap is None
        self.last_structure = S
        # order the caller's stream after ours instead of a host sync
        cur = torch.cuda.current_stream(self.dev)
        cur.wait_stream(self.s_main)
        cur.wait_stream(self.s_side)
        return out

    # -- diagnostics -------------------------------------------------------------
    def check_status(self, wait=True):
        """Raises RuntimeError if a kernel of an earlier step() reported that one of its
        bounded waits gave up or that a task plan exceeded its bounds (the output of that
        call is then unusable).  step() copies the device status word to pinned host
        memory behind its kernels; with wait=False (what step() itself does on entry) only
        a copy that has already arrived is looked at, so the hot path never synchronises;
        with wait=True (request boundaries) the last copy is waited for."""
        ev = self._status_event
        if ev is None:
            return
        if wait:
            ev.synchronize()
        elif not ev.query():
            return
        code = int(self._status_host[0])
        if code != 0:
            self._status_host.zero_()
            with torch.cuda.device(self.dev):
                self.status.zero_()
            raise RuntimeError(f"Token2Tile kernels reported status {code}: {_lib.STATUS.get(code, 'unknown')}; "
                               "the result of the affected call is not valid")

    def device_status(self) -> int:
        """Status word of the bounded device waits (synchronises)."""
        return int(self.status.item())

    def plan_info(self):
        """(tasks, executed query-key pairs) of the structure used last (synchronises)."""
        info = torch.zeros(4, device=self.dev, dtype=torch.int32)
        with torch.cuda.device(self.dev):
            st = _stream_ptr(torch.cuda.current_stream(self.dev))
            check(self.lib.t2t_tile_attn_plan_info(ptr(self.last_structure["tile_attn_plan"]), self.H, self.N,
                                                   self.CQ, ptr(info), st), "t2t_tile_attn_plan_info")
        a = info.cpu().tolist()
        return a[0], (a[1] & 0xFFFFFFFF) | ((a[2] & 0xFFFFFFFF) << 32)
