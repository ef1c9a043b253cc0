"""CPU oracle for the Token2Tile sparse attention operator.

TEST INFRASTRUCTURE ONLY.  This file restates, on the CPU and in plain PyTorch,
the arithmetic of the reference operator so that the CUDA path can be checked
against it.  Nothing in the shipped package imports it; only the tests, the
smoke check and the CPU-baseline leg of the benchmark do.

Parity status: the reference repository holds no tests, golden vectors or
fixtures for this path, so the oracle is pinned in two other ways:
  * `online_u` is checked against the reference's own `online_u`
    (token2tile/operator/deploy_step.py:122-149) executed on the CPU; the
    vectors live in tests/golden/ with the script that produced them;
  * clustering, grouping, value statistics and selection are checked on a
    B200 against the reference's own kmeans_maintain and select_union CUDA
    sources compiled unmodified (oracle/build_ref.py -> oracle/_ref/).
The exact tile attention and the residual merge of the reference use `wgmma`
and cannot be built for sm_100a; for those two stages parity is UNPINNED and
the oracle follows the reference's formulas (cited per function) and is
checked through its dense-attention limits.

Every function works per call on tensors shaped like the operator's
([H, N, ...]).  `dt` is the 16-bit storage type: torch.bfloat16 for the
product, torch.float16 when the oracle is compared with the reference kernels.

Arithmetic conventions that make integer results reproducible bit for bit:
  * a dot product over the rank-32 space is the fp32 chain
    acc <- fl32(acc + x_k * c_k), k = 0..31 in order; products of two 16-bit
    values are exact in fp32, so this equals a chain of fused multiply-adds;
  * centroid norms are the same chain over c_k * c_k starting from 0;
  * ties are broken towards the lowest cluster index.
"""
from __future__ import annotations

import math

import torch

F32 = torch.float32
QSCALE = 32768.0          # fixed-point scale of the query-side sums (kernels.cu:538)
ROW_CHUNK = 4096          # rows per block in the chained dot products
# When True, rank-32 dot products use one sgemm instead of the ordered chain.
# Only the timed CPU-baseline leg of the benchmark sets it: same mathematics at
# the speed a CPU implementation would have, but no longer bit-reproducible.
FAST_DOT = False


# ---------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------

def round16(x: torch.Tensor, dt: torch.dtype) -> torch.Tensor:
    """Round to the 16-bit storage type and return as fp32."""
    return x.to(dt).to(F32)


_CHAIN_LIB = False          # False: not looked for yet; None: unavailable


def _chain_lib():
    """The C twin of the chain (oracle/chain_dot.c), built on first use when a C
    compiler is present; None otherwise."""
    global _CHAIN_LIB
    if _CHAIN_LIB is False:
        _CHAIN_LIB = None
        try:
            import ctypes
            import importlib.util
            from pathlib import Path
            spec = importlib.util.spec_from_file_location("_t2t_oracle_build_c", Path(__file__).with_name("build_c.py"))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            path = mod.build()
            if path is not None:
                lib = ctypes.CDLL(str(path))
                lib.t2t_chain_dot.restype = ctypes.c_int
                lib.t2t_chain_dot.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_long, ctypes.c_long, ctypes.c_int]
                _CHAIN_LIB = lib
        except Exception:       # no compiler, read-only tree, ...: the PyTorch loop below is the definition anyway
            _CHAIN_LIB = None
    return _CHAIN_LIB


def chain_dot_loop(x: torch.Tensor, c: torch.Tensor, init: torch.Tensor | None = None) -> torch.Tensor:
    """The definition of the chain, as a PyTorch loop over k."""
    n, r = x.shape
    m = c.shape[0]
    acc = torch.zeros(n, m, dtype=F32) if init is None else init[None, :].expand(n, m).clone()
    for k in range(r):
        acc += x[:, k:k + 1] * c[None, :, k]
    return acc


def chain_dot(x: torch.Tensor, c: torch.Tensor, init: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 chain  acc <- acc + x[:, k] * c[:, k]  for k in order.

    x [n, r] fp32 (16-bit values), c [m, r] fp32 (16-bit values),
    init [m] fp32 or None (0).  Returns [n, m] fp32.  Uses the C twin of the
    loop when it could be built (same bits, all host threads)."""
    n, r = x.shape
    m = c.shape[0]
    if FAST_DOT:
        return x @ c.T if init is None else torch.addmm(init[None, :].expand(n, m), x, c.T)
    lib = _chain_lib()
    if lib is None or x.device.type != "cpu":
        return chain_dot_loop(x, c, init)
    xc, cc = x.to(F32).contiguous(), c.to(F32).contiguous()
    ic = None if init is None else init.to(F32).contiguous()
    out = torch.empty(n, m, dtype=F32)
    rc = lib.t2t_chain_dot(xc.data_ptr(), cc.data_ptr(), 0 if ic is None else ic.data_ptr(), out.data_ptr(), n, m, r)
    if rc != 0:
        raise RuntimeError(f"t2t_chain_dot failed: {rc}")
    return out


def centroid_norms(c: torch.Tensor) -> torch.Tensor:
    """||c||^2 in fp32, summed in index order (kernels.cu:85-94)."""
    s = torch.zeros(c.shape[:-1], dtype=F32)
    for k in range(c.shape[-1]):
        s = s + c[..., k] * c[..., k]
    return s


# ---------------------------------------------------------------------------
# A.1  projection fit
# ---------------------------------------------------------------------------

def online_u(qf: torch.Tensor, kf: torch.Tensor, r: int = 32):
    """Matched rank-r projections (deploy_step.py:122-149), fp64 per head.

    Mq = Q^T Q / N, Mk = K^T K / N; symmetric square roots and inverse roots
    from eigendecompositions with eigenvalues clamped at 1e-8; SVD of
    Rq^T Rk = U S V^T; Uq = Rq^-T U_r sqrt(S_r), Uk = Rk^-1 V_r sqrt(S_r)."""
    for name, t in (("q", qf), ("k", kf)):
        if not bool(torch.isfinite(t).all()):
            raise RuntimeError(f"online_u: non-finite {name} input")
    Uqs, Uks = [], []
    for h in range(qf.shape[0]):
        q, k = qf[h].double(), kf[h].double()
        Mq = (q.T @ q) / q.shape[0]
        Mk = (k.T @ k) / k.shape[0]
        eq, Vq = torch.linalg.eigh(Mq)
        ek, Vk = torch.linalg.eigh(Mk)
        eq = eq.clamp_min(1e-8)
        ek = ek.clamp_min(1e-8)
        Rq = Vq @ torch.diag(eq.sqrt()) @ Vq.T
        Rk = Vk @ torch.diag(ek.sqrt()) @ Vk.T
        Rqi = Vq @ torch.diag(eq.rsqrt()) @ Vq.T
        Rki = Vk @ torch.diag(ek.rsqrt()) @ Vk.T
        U, S, Vh = torch.linalg.svd(Rq.T @ Rk)
        sr = S[:r].sqrt()
        Uqs.append((Rqi.T @ U[:, :r] * sr).float())
        Uks.append((Rki @ Vh[:r].T * sr).float())
    return torch.stack(Uqs), torch.stack(Uks)


# ---------------------------------------------------------------------------
# A.2  projection
# ---------------------------------------------------------------------------

def project(x16: torch.Tensor, U16: torch.Tensor, dt: torch.dtype) -> torch.Tensor:
    """QU = round16(x . U) with fp32 accumulation (deploy_step.py:321-324).

    The accumulation order of the GEMM is not part of the contract; this stage
    is compared by tolerance."""
    return torch.bmm(x16.to(F32), U16.to(F32)).to(dt)


# ---------------------------------------------------------------------------
# A.3  clustering
# ---------------------------------------------------------------------------

def assign(x16: torch.Tensor, cen16: torch.Tensor, pin_tail: int = 0) -> torch.Tensor:
    """label(i) = argmin_c (||c||^2 - 2 x_i.c), ties -> lowest c
    (kernels.cu:102-257).  The distance is the fp32 chain started at ||c||^2
    over the products x_k * (-2 c_k).  Rows >= N - pin_tail are forced to the
    last cluster (kernels.cu:250-252)."""
    H, N, r = x16.shape
    C = cen16.shape[1]
    labels = torch.empty(H, N, dtype=torch.int32)
    for h in range(H):
        c = cen16[h].to(F32)
        cn = centroid_norms(c)
        m2c = -2.0 * c
        x = x16[h].to(F32)
        for s in range(0, N, ROW_CHUNK):
            d = chain_dot(x[s:s + ROW_CHUNK], m2c, cn)
            mn = d.min(dim=1, keepdim=True).values
            labels[h, s:s + ROW_CHUNK] = (d == mn).to(torch.uint8).argmax(dim=1).to(torch.int32)
    if pin_tail > 0:
        labels[:, N - pin_tail:] = C - 1
    return labels


def stable_group(labels: torch.Tensor, C: int):
    """Stable counting sort of rows by label (kernels.cu:266-371):
    counts [H, C] and perm [H, N] with perm[base(c) + rank] = row, rows
    ascending inside a cluster."""
    H, N = labels.shape
    counts = torch.zeros(H, C, dtype=torch.int32)
    perm = torch.empty(H, N, dtype=torch.int32)
    for h in range(H):
        lab = labels[h].to(torch.int64)
        counts[h] = torch.bincount(lab, minlength=C).to(torch.int32)
        perm[h] = torch.sort(lab, stable=True).indices.to(torch.int32)
    return counts, perm


def fixed_point_mean(x16: torch.Tensor, labels: torch.Tensor, old16: torch.Tensor,
                     dt: torch.dtype):
    """Cluster means from exact integer sums (kernels.cu:540-616):
    s = sum_i rint(x_i * 2^15) as integers, mean = round16(float(s) /
    (2^15 * float(n))); an empty cluster keeps its previous centroid.
    Returns (centroids [H, C, r] in dt, counts [H, C] int32)."""
    H, N, r = x16.shape
    C = old16.shape[1]
    xi = torch.round(x16.to(F32) * QSCALE).to(torch.int64)      # round half to even, like cvt.rni
    lab = labels.to(torch.int64)
    sums = torch.zeros(H, C, r, dtype=torch.int64).scatter_add_(
        1, lab[..., None].expand(H, N, r), xi)
    counts = torch.zeros(H, C, dtype=torch.int64).scatter_add_(1, lab, torch.ones_like(lab))
    den = (QSCALE * counts.to(F32))[..., None]
    mean = sums.to(F32) / den.clamp_min(1.0)
    out = torch.where((counts > 0)[..., None], mean.to(dt), old16)
    return out.contiguous(), counts.to(torch.int32)


def sequential_cluster_sums(x: torch.Tensor, perm: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    """Per-cluster fp32 sums accumulated one row at a time in grouped order
    (kernels.cu:394-424): ((x_0 + x_1) + x_2) + ...   x [H, N, d] fp32."""
    H, N, d = x.shape
    C = counts.shape[1]
    out = torch.zeros(H, C, d, dtype=F32)
    for h in range(H):
        cnt = counts[h].to(torch.int64)
        base = torch.cumsum(cnt, 0) - cnt
        acc = torch.zeros(C, d, dtype=F32)
        p = perm[h].to(torch.int64)
        for j in range(int(cnt.max().item()) if C else 0):
            live = cnt > j
            rows = p[(base + j).clamp_max(N - 1)]
            acc = torch.where(live[:, None], acc + x[h, rows], acc)
        out[h] = acc
    return out


def key_means_f32(KU16: torch.Tensor, kperm, kcounts, old16) -> torch.Tensor:
    """ck2 = sum of the cluster's KU rows / n in fp32, or the old centroid for
    an empty cluster (kernels.cu:635-647)."""
    ksum = sequential_cluster_sums(KU16.to(F32), kperm, kcounts)
    n = kcounts.to(F32)[..., None]
    return torch.where(kcounts[..., None] > 0, ksum / n.clamp_min(1.0), old16.to(F32))


def vstats(v16: torch.Tensor, kperm: torch.Tensor, kcounts: torch.Tensor, dt: torch.dtype):
    """Cluster-major V, fp32 value sums, lam = max(1, max|sum| / 32768) and
    sumv = round16(sum * (1 / lam)) (kernels.cu:481-531, 649-692)."""
    H, N, D = v16.shape
    idx = kperm.to(torch.int64)[..., None].expand(H, N, D)
    v_sorted = torch.gather(v16, 1, idx)
    vsum = sequential_cluster_sums(v16.to(F32), kperm, kcounts)
    lam = torch.clamp(vsum.abs().amax(dim=(1, 2)) / 32768.0, min=1.0)
    inv = (1.0 / lam)[:, None, None]
    sumv = (vsum * inv).to(dt)
    return v_sorted, sumv, lam, vsum


def kmeans_maintain(QU16, KU16, V16, cq0, ck0, pin_tail: int, dt: torch.dtype) -> dict:
    """One structure rebuild (kernels.cu:787-876): queries take two Lloyd
    passes from cq0, keys one pass from ck0."""
    CQ, C = cq0.shape[1], ck0.shape[1]
    qlab1 = assign(QU16, cq0)
    cq1, _ = fixed_point_mean(QU16, qlab1, cq0, dt)
    qlab = assign(QU16, cq1)
    cq2, qcounts = fixed_point_mean(QU16, qlab, cq1, dt)
    _, qperm = stable_group(qlab, CQ)
    klab = assign(KU16, ck0, pin_tail)
    kcounts, kperm = stable_group(klab, C)
    ck2 = key_means_f32(KU16, kperm, kcounts, ck0)
    v_sorted, sumv, lam, vsum = vstats(V16, kperm, kcounts, dt)
    return dict(qlab=qlab, cq2=cq2, qcounts=qcounts, qperm=qperm, klab=klab, ck2=ck2,
                kcounts=kcounts, kperm=kperm, V_sorted=v_sorted, sumv=sumv, lam=lam,
                vsum=vsum, qlab1=qlab1, cq1=cq1)


# ---------------------------------------------------------------------------
# A.4  scoring and selection
# ---------------------------------------------------------------------------

def score_keys(QU16: torch.Tensor, cks16: torch.Tensor) -> torch.Tensor:
    """Signed 16-bit selection keys of g = round_fp16(QU_i . cks_c)
    (deploy_step.py:394; key transform select_union/src/kernel.cu:56-74,160:
    the fp16 bit pattern with its low 15 bits flipped when the sign bit is set,
    read as a signed 16-bit integer).  One head: QU16 [n, r], cks16 [C, r]."""
    return keys_from_fp16(chain_dot(QU16.to(F32), cks16.to(F32)).to(torch.float16))


def keys_from_fp16(g: torch.Tensor) -> torch.Tensor:
    """Order-preserving signed 16-bit key of an fp16 score (kernel.cu:56-74, 160)."""
    u = g.view(torch.int16).to(torch.int32) & 0xFFFF
    u = u ^ (((u >> 15) & 1) * 0x7FFF)
    return ((u ^ 0x8000) - 0x8000).to(torch.int16)


def select_rows(keys: torch.Tensor, sizes: torch.Tensor, ns: int):
    """Per query: clusters ordered by (key descending, index ascending); a
    cluster is selected iff the total size of the clusters strictly before it
    is < ns (select_union/src/kernel.cu:288-392).  rowcnt is the inclusive
    total at the crossing.  keys [n, C] int16, sizes [C] int32.
    Returns (sel [n, C] bool, rowcnt [n] int32)."""
    order = torch.sort(-keys.to(torch.int32), dim=1, stable=True).indices
    return select_rows_sorted(order, sizes, ns)


def pack_bits(sel: torch.Tensor) -> torch.Tensor:
    """[.., C] bool -> [.., C/32] int32, bit b of word w <=> cluster 32 w + b
    (select_union/src/kernel.cu:469-487)."""
    C = sel.shape[-1]
    b = sel.reshape(*sel.shape[:-1], C // 32, 32).to(torch.int64)
    w = (b << torch.arange(32, dtype=torch.int64)).sum(-1)
    return ((w ^ 0x80000000) - 0x80000000).to(torch.int32)


def unpack_bits(words: torch.Tensor, C: int) -> torch.Tensor:
    w = words.to(torch.int64) & 0xFFFFFFFF
    return ((w[..., None] >> torch.arange(32, dtype=torch.int64)) & 1).bool().reshape(*words.shape[:-1], C)


def select_rows_sorted(order: torch.Tensor, sizes: torch.Tensor, ns: int):
    """select_rows for a precomputed order (clusters by key descending, index
    ascending): the selection rule only needs the sizes along that order."""
    n, C = order.shape
    sz = sizes.to(torch.int64)[order]
    incl = torch.cumsum(sz, dim=1)
    excl = incl - sz
    sel = torch.zeros(n, C, dtype=torch.bool).scatter_(1, order, excl < ns)
    cross = (incl >= ns).to(torch.uint8).argmax(dim=1)          # first position reaching ns
    reached = incl[:, -1] >= ns
    rowcnt = torch.where(reached, incl.gather(1, cross[:, None])[:, 0], incl[:, -1])
    return sel, rowcnt.to(torch.int32)


def select_union_budgets(QU16, cks16, kcounts, qlab, CQ: int, ns_list, pin_tail: int = 0,
                         row_chunk: int = 2048, gl16=None):
    """select_union for several budgets at once: the keys and their order do
    not depend on the budget, so they are computed once per block of rows.
    Returns one (unip, rowcnt) pair per entry of ns_list."""
    H, N = qlab.shape
    C = kcounts.shape[1]
    hits = [torch.zeros(H, CQ, C, dtype=torch.int32) for _ in ns_list]
    rowcnt = [torch.empty(H, N, dtype=torch.int32) for _ in ns_list]
    for h in range(H):
        lab = qlab[h].to(torch.int64)
        for s in range(0, N, row_chunk):
            keys = (score_keys(QU16[h, s:s + row_chunk], cks16[h]) if gl16 is None
                    else keys_from_fp16(gl16[h, s:s + row_chunk]))
            order = torch.sort(-keys.to(torch.int32), dim=1, stable=True).indices
            for b, ns in enumerate(ns_list):
                sel, rc = select_rows_sorted(order, kcounts[h], ns)
                rowcnt[b][h, s:s + row_chunk] = rc
                hits[b][h].index_add_(0, lab[s:s + row_chunk], sel.to(torch.int32))
    out = []
    for b in range(len(ns_list)):
        union = hits[b] > 0
        if pin_tail > 0:
            union[:, :, C - 1] = True
        out.append((pack_bits(union), rowcnt[b]))
    return out


def select_union(QU16, cks16, kcounts, qlab, CQ: int, ns: int, pin_tail: int = 0,
                 row_chunk: int = 2048, gl16=None):
    """Union bitmap unip [H, CQ, C/32] int32 and rowcnt [H, N] int32.
    U_t = OR of the selections of the queries labelled t; pin_tail > 0 also
    sets cluster C-1 everywhere (deploy_step.py:444-448).  With gl16 (an fp16
    score matrix [H, N, C], the reference's `gl`) the scores are taken from it
    instead of being recomputed."""
    return select_union_budgets(QU16, cks16, kcounts, qlab, CQ, [ns], pin_tail, row_chunk, gl16)[0]


def kv_lengths(unip, qcounts, kcounts) -> torch.Tensor:
    """Tokens in each query cluster's union; 0 for an empty query cluster
    (tile_attn/src/kernel.cu:259-275)."""
    C = kcounts.shape[1]
    u = unpack_bits(unip, C)
    tot = (u.to(torch.int64) * kcounts.to(torch.int64)[:, None, :]).sum(-1)
    return torch.where(qcounts > 0, tot, torch.zeros_like(tot)).to(torch.int32)


# ---------------------------------------------------------------------------
# A.5  exact part,  A.6  residual and merge
# ---------------------------------------------------------------------------

def exact_attention(q16, k16, v16, qlab, klab, unip, scale: float):
    """For every query i of query cluster t: softmax attention over the tokens
    whose key cluster is in U_t (tile_attn/src/kernel.cu:820-1096).
    Returns o [H, N, D] fp32 (normalised, original order) and lse [H, N]
    (natural log of sum exp(s); -inf for an empty union, where o = 0)."""
    H, N, D = q16.shape
    C = unip.shape[2] * 32
    CQ = unip.shape[1]
    o = torch.zeros(H, N, D, dtype=F32)
    lse = torch.full((H, N), -math.inf, dtype=F32)
    for h in range(H):
        u = unpack_bits(unip[h], C)
        kl = klab[h].to(torch.int64)
        ql = qlab[h].to(torch.int64)
        kf, vf, qf = k16[h].to(F32), v16[h].to(F32), q16[h].to(F32)
        for t in range(CQ):
            rows = (ql == t).nonzero()[:, 0]
            if rows.numel() == 0:
                continue
            cols = u[t][kl].nonzero()[:, 0]
            if cols.numel() == 0:
                continue
            s = (qf[rows] @ kf[cols].T) * scale
            m = s.max(dim=1, keepdim=True).values
            p = torch.exp(s - m)
            l = p.sum(dim=1, keepdim=True)
            o[h, rows] = (p @ vf[cols]) / l
            lse[h, rows] = (m + torch.log(l))[:, 0]
    return o, lse


def residual_merge(o, lse, QU16, cks16, sumv16, lam, kcounts, unip, qlab, tailw: float):
    """out_i = (L_i o_i + tw T_i) / max(L_i + tw phi_i, tiny) with
    phi_i = sum_{c not in U_t} n_c e^{g_ic}, T_i = lam sum_{c not in U_t}
    e^{g_ic} sumv_c and g rounded to fp16 (tile_attn/src/kernel.cu:1248-1449);
    the residual is dropped when phi_i <= 1e-6 L_i."""
    H, N, D = o.shape
    C = cks16.shape[1]
    out = torch.empty(H, N, D, dtype=F32)
    for h in range(H):
        u = unpack_bits(unip[h], C)
        ql = qlab[h].to(torch.int64)
        cksf, sv, nc = cks16[h].to(F32), sumv16[h].to(F32), kcounts[h].to(F32)
        for s in range(0, N, ROW_CHUNK):
            e = min(N, s + ROW_CHUNK)
            g = chain_dot(QU16[h, s:e].to(F32), cksf).to(torch.float16).to(F32)
            g = torch.where(u[ql[s:e]], torch.full_like(g, -math.inf), g)
            m = g.max(dim=1, keepdim=True).values
            m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
            p = torch.exp(g - m)
            phi = (p * nc[None, :]).sum(dim=1, keepdim=True)
            T = (p @ sv) * lam[h]
            le = lse[h, s:e, None]
            M = torch.maximum(le, m)
            ex = torch.exp(le - M)                  # exact-part weight, 0 for an empty union
            st = torch.exp(m - M)
            ph = st * phi
            bad = ph <= 1.0e-6 * ex
            den = torch.clamp(ex + ph * tailw, min=1.0e-12)
            merged = (ex * o[h, s:e] + (st * tailw) * T) / den
            out[h, s:e] = torch.where(bad, o[h, s:e], merged)
    return out


def dense_attention(q16, k16, v16, scale: float) -> torch.Tensor:
    """Plain softmax attention in fp32, for the limit checks."""
    s = torch.matmul(q16.to(F32), k16.to(F32).transpose(-1, -2)) * scale
    return torch.matmul(torch.softmax(s, dim=-1), v16.to(F32))


# ---------------------------------------------------------------------------
# operator with the reference's call interface, on the CPU
# ---------------------------------------------------------------------------

def sample_rows(N: int, count: int, gen: torch.Generator) -> torch.Tensor:
    """Sorted row indices of the initial centroids (deploy_step.py:254-258)."""
    return torch.randperm(N, generator=gen)[:count].sort().values


def init_state(q16, k16, CQ: int, C: int, r: int, warm_iters: int, seed: int, dt: torch.dtype):
    """Projections and initial centroids (deploy_step.py:245-266).  The warm
    Lloyd iterations use the exact assignment rule and the fixed-point mean,
    the deterministic variant the reference's serving backend substitutes
    (integrations/sglang/backend/t2t_attn.py:242-281)."""
    N = q16.shape[1]
    Uq, Uk = online_u(q16.float(), k16.float(), r)
    Uq, Uk = Uq.to(dt).contiguous(), Uk.to(dt).contiguous()
    KU = project(k16, Uk, dt)
    QU = project(q16, Uq, dt)
    g = torch.Generator(device="cpu").manual_seed(seed)
    ck = KU[:, sample_rows(N, C, g), :].contiguous()
    cq = QU[:, sample_rows(N, CQ, g), :].contiguous()
    for _ in range(warm_iters):
        ck, _ = fixed_point_mean(KU, assign(KU, ck), ck, dt)
        cq, _ = fixed_point_mean(QU, assign(QU, cq), cq, dt)
    return {"Uq": Uq, "Uk": Uk, "ck": ck, "cq": cq}


class OracleOperator:
    """CPU twin of MaskedStepDeploy (deploy_step.py:152-477): same constructor
    arguments, `init_state`, `set_cfg_call`, `reset_cfg_reuse`, `step`, and the
    same rebuild / reuse decision.  `last` keeps every intermediate tensor of
    the most recent call for stage-wise comparison."""

    def __init__(self, H, N, CQ, *, C=2048, D=128, r=32, s_frac=0.05, tailw=1.0,
                 mask_refresh=1, cfg_reuse=False, pin_tail=0, dtype=torch.bfloat16):
        if C != 2048 or D != 128:
            raise ValueError("the kernels require C=2048 and D=128")
        self.H, self.N, self.CQ, self.C, self.D, self.r = H, N, CQ, C, D, r
        self.ns = max(1, int(s_frac * N))
        self.tailw = float(tailw)
        self.scale = 1.0 / math.sqrt(D)
        self.pin_tail = int(pin_tail)
        self.dt = dtype
        self.cfg_reuse = bool(cfg_reuse)
        self.mask_refresh = max(1, int(mask_refresh))
        self._cfg_on = self.cfg_reuse or self.mask_refresh > 1
        self._cfg_hold = {}
        self._cfg_parity = None
        self._cfg_key = 0
        self._cfg_step = 0
        self.last = {}

    def init_state(self, q, k, *, warm_iters=4, seed=0):
        return init_state(q, k, self.CQ, self.C, self.r, warm_iters, seed, self.dt)

    def set_cfg_call(self, parity, key=0, step=0):
        self._cfg_parity, self._cfg_key, self._cfg_step = int(parity), key, int(step)

    def reset_cfg_reuse(self):
        self._cfg_hold.clear()
        self._cfg_parity = None

    def _pick_snapshot(self):
        """Rebuild / reuse decision (deploy_step.py:297-309)."""
        snap = None
        parity = self._cfg_parity
        self._cfg_parity = None
        if self._cfg_on and parity is not None:
            held = self._cfg_hold.get(self._cfg_key)
            age = None if held is None else self._cfg_step - held["step"]
            refresh_due = age is None or age < 0 or age >= self.mask_refresh
            if held is not None and age >= 0 and not (parity == 0 and refresh_due):
                snap = held
        return snap

    def step(self, q, k, v, state):
        dt = self.dt
        snap = self._pick_snapshot()
        L = {}
        if snap is None:
            QU = project(q, state["Uq"], dt)
            KU = project(k, state["Uk"], dt)
            km = kmeans_maintain(QU, KU, v, state["cq"], state["ck"], self.pin_tail, dt)
            state["ck"] = km["ck2"].to(dt).contiguous()
            state["cq"] = km["cq2"].clone()
            cks = (km["ck2"] * self.scale).to(dt).contiguous()
            unip, rowcnt = select_union(QU, cks, km["kcounts"], km["qlab"], self.CQ, self.ns,
                                        self.pin_tail)
            struct = dict(qlab=km["qlab"], qperm=km["qperm"], tile_sizes=km["qcounts"],
                          klab=km["klab"], kperm=km["kperm"], counts=km["kcounts"], cks=cks,
                          Uq=state["Uq"], unip=unip, step=self._cfg_step)
            if self._cfg_on:
                self._cfg_hold[self._cfg_key] = struct
            sumv, lam = km["sumv"], km["lam"]
            L.update(km, KU=KU, rowcnt=rowcnt)
        else:
            struct = snap
            QU = project(q, snap["Uq"], dt)
            _, sumv, lam, _ = vstats(v, snap["kperm"], snap["counts"], dt)
        o, lse = exact_attention(q, k, v, struct["qlab"], struct["klab"], struct["unip"], self.scale)
        out = residual_merge(o, lse, QU, struct["cks"], sumv, lam, struct["counts"],
                             struct["unip"], struct["qlab"], self.tailw)
        L.update(QU=QU, cks=struct["cks"], unip=struct["unip"], sumv=sumv, lam=lam,
                 attn_o=o, attn_lse=lse, out=out, rebuilt=snap is None,
                 kv_len=kv_lengths(struct["unip"], struct["tile_sizes"], struct["counts"]))
        self.last = L
        return out.to(dt)
