"""The projection-fit kernels (t2t_lowrank_fit: tensor-core second moments, fp64
Jacobi factorisations) against the reference's own `online_u` run on the CPU
(tests/golden/online_u.pt) and against the oracle.

The factors are defined up to a common sign per component (and a rotation
inside equal singular values), so the products Uq Uk^T are compared."""
import importlib.util
from pathlib import Path

import pytest
import torch

from oracle import t2t_oracle as O

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
DEV = "cuda"
GOLDEN = Path(__file__).resolve().parent / "golden"


def _product(Uq, Uk):
    return Uq.double().cpu() @ Uk.double().cpu().transpose(1, 2)


def _golden_inputs():
    spec = importlib.util.spec_from_file_location("mk", GOLDEN / "make_online_u_golden.py")
    mk = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mk)
    return mk


def test_fit_matches_the_reference_golden_vectors():
    """The golden inputs are fp32; the kernels take them rounded to bfloat16 (a relative
    perturbation of 2^-9 per element), which bounds the agreement."""
    from token2tile_b200.deploy_step import online_u
    mk = _golden_inputs()
    for item in torch.load(GOLDEN / "online_u.pt"):
        q, k = mk.make_inputs(item["case"])
        Uq, Uk = online_u(q.to(DEV), k.to(DEV), item["case"]["r"])
        want = _product(item["Uq"], item["Uk"])
        got = _product(Uq, Uk)
        assert (got - want).abs().max() <= 2e-2 * want.abs().max(), item["case"]
        # and tightly against the oracle given the very same bfloat16 values
        qb, kb = q.to(BF).float(), k.to(BF).float()
        oq, ok = O.online_u(qb, kb, item["case"]["r"])
        want_b = _product(oq, ok)
        assert (got - want_b).abs().max() <= 1e-4 * want_b.abs().max(), item["case"]


@pytest.mark.parametrize("N", [4096, 20001])
def test_fit_matches_the_oracle_on_bfloat16_inputs(N):
    """N = 20,001: three slabs of the Gram kernel and a ragged last tile."""
    from token2tile_b200.deploy_step import online_u
    from token2tile_b200.t2t_attn import fast_online_u
    g = torch.Generator().manual_seed(21)
    H = 3
    k = (torch.randn(H, N, 128, generator=g) * torch.linspace(2.0, 0.05, 128)).to(BF)
    q = (0.6 * k.float() + 0.4 * torch.randn(H, N, 128, generator=g) * torch.linspace(0.05, 2.0, 128)).to(BF)
    Uq, Uk = online_u(q.to(DEV), k.to(DEV), 32)
    assert Uq.dtype == torch.float32 and Uq.shape == (H, 128, 32)
    oq, ok = O.online_u(q.float(), k.float(), 32)
    want, got = _product(oq, ok), _product(Uq, Uk)
    assert (got - want).abs().max() <= 1e-4 * want.abs().max()
    # the logit approximation the projections exist for
    err = ((q.double() @ got) @ k.double().transpose(1, 2) - (q.double() @ want) @ k.double().transpose(1, 2))[:, :256, :256]
    assert err.abs().max() <= 1e-3 * (q.double() @ k.double().transpose(1, 2))[:, :256, :256].abs().max()
    fq, fk = fast_online_u(q.to(DEV), k.to(DEV), 32)       # same kernels, no finiteness read-back
    torch.cuda.synchronize()
    assert torch.equal(fq, Uq) and torch.equal(fk, Uk)


def test_fit_of_rank_deficient_inputs():
    """Queries confined to a 20-dimensional subspace: 108 clamped eigenvalues on the query side and
    fewer than 32 non-zero singular values."""
    from token2tile_b200.deploy_step import online_u
    g = torch.Generator().manual_seed(22)
    basis = torch.linalg.qr(torch.randn(128, 20, generator=g)).Q
    q = ((torch.randn(2, 3000, 20, generator=g) @ basis.T)).to(BF)
    k = torch.randn(2, 3000, 128, generator=g).to(BF)
    Uq, Uk = online_u(q.to(DEV), k.to(DEV), 32)
    assert bool(torch.isfinite(Uq).all()) and bool(torch.isfinite(Uk).all())
    logits = q.double() @ k.double().transpose(1, 2)
    approx = (q.double() @ _product(Uq, Uk)) @ k.double().transpose(1, 2)
    oq, ok = O.online_u(q.float(), k.float(), 32)
    approx_o = (q.double() @ _product(oq, ok)) @ k.double().transpose(1, 2)
    # rank 20 < 32: the fit reproduces the logits, as the oracle's does
    assert (approx - logits).abs().max() <= 1e-2 * logits.abs().max()
    assert (approx - approx_o).abs().max() <= 1e-2 * logits.abs().max()


def test_fit_rejects_non_finite_inputs():
    from token2tile_b200.deploy_step import online_u
    from token2tile_b200.t2t_attn import fast_online_u
    g = torch.Generator().manual_seed(23)
    q = torch.randn(2, 1024, 128, generator=g).to(BF).to(DEV)
    k = q.clone()
    k[1, 7, 3] = float("inf")
    with pytest.raises(RuntimeError, match="non-finite k input in heads \\[1\\]"):
        online_u(q, k, 32)
    fq, fk = fast_online_u(q, k, 32)          # no exception: the bad head's projections stay zero
    torch.cuda.synchronize()
    assert bool((fq[1] == 0).all()) and bool((fk[1] == 0).all()) and bool(fq[0].abs().sum() > 0)
    with pytest.raises(ValueError):
        online_u(q, k, 16)
