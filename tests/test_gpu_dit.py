"""The transformer-step harness on a GPU with the real attention backend: a small model
(2 blocks, 12 heads of 128, 4,096 tokens) against the same model whose self-attention
is the CPU oracle operator, and - where two GPUs are present - a two-rank Ulysses run
over NCCL against the single-GPU run."""
import math
import os

import pytest
import torch

from oracle import t2t_oracle as O
from token2tile_b200.dit_step import DiTShape, DiTStep

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
# 12 heads: the smallest head count the backend knows a layer count for
TINY = DiTShape(blocks=2, dim=1536, heads=12, head_dim=128, ffn=2048, text_len=8, text_dim=64, freq_dim=32)
N, CQ, NS = 4096, 32, 204


def _inputs():
    """A residual stream with the locality structure of video latents (blocks of 16 tokens share a centre)."""
    g = torch.Generator().manual_seed(2)
    centres = torch.randn(256, TINY.dim, generator=g)
    x = centres[torch.arange(N) // 16] + 0.3 * torch.randn(N, TINY.dim, generator=g)
    return x.to(BF), torch.randn(TINY.text_len, TINY.text_dim, generator=g).to(BF)


def _metadata(B, cache, step=0):
    return B.T2TAttentionMetadataBuilder().build(
        step, 50, cache, profile_name="manual", ns_base=NS, dense_prefix_steps=0, cq=CQ, ck=2048,
        step_profile=(1.0,) * 4, layer_profile=(1.0,) * 6, cfg_mult=(1.0, 1.0))


class OracleAttention:
    """Self-attention by the CPU oracle operator, with the backend's conventions: one state per
    layer, initialised with seed 2 * layer (first CFG branch) and the metadata's warm iterations."""

    def __init__(self, num_heads, head_size, causal, softmax_scale, prefix=""):
        self.layer = int(prefix.split(".")[1])
        self.state = None

    def forward(self, q, k, v, meta):
        qh, kh, vh = (t[0].transpose(0, 1).contiguous().cpu() for t in (q, k, v))      # [H, N, D]
        op = O.OracleOperator(qh.shape[0], N, CQ, s_frac=(NS + 0.5) / N)
        assert op.ns == NS
        if self.state is None:
            self.state = op.init_state(qh, kh, warm_iters=meta.warm_iters, seed=2 * self.layer)
        out = op.step(qh, kh, vh, self.state)
        return out.transpose(0, 1).unsqueeze(0).to(q.device)


class DenseAttention:
    def __init__(self, num_heads, head_size, causal, softmax_scale, prefix=""):
        self.scale = softmax_scale

    def forward(self, q, k, v, meta):
        out = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                               scale=self.scale)
        return out.transpose(1, 2).contiguous()


def _backend():
    from token2tile_b200 import t2t_attn as B
    B.clear_runtimes()
    B.set_backend_config({})
    B.set_forward_context(None)
    B.set_ulysses_world_size(1)
    return B


def test_step_with_the_real_backend_matches_the_step_with_the_oracle_operator():
    B = _backend()
    x, text = _inputs()
    xd, td = x.cuda(), text.cuda()
    real = DiTStep(TINY, device="cuda", seed=7)
    got = real.forward(xd, td, 500.0, _metadata(B, B.T2TRequestCache())).float().cpu()
    torch.cuda.synchronize()
    assert len(B._RUNTIMES) == 1
    for rt in B._RUNTIMES.values():
        assert rt.deploy.device_status() == 0
    want = DiTStep(TINY, device="cuda", seed=7, make_attn=OracleAttention).forward(
        xd, td, 500.0, _metadata(B, B.T2TRequestCache())).float().cpu()
    dense = DiTStep(TINY, device="cuda", seed=7, make_attn=DenseAttention).forward(xd, td, 500.0, None).float().cpu()
    rel = lambda a, b: float((a - b).norm() / b.norm())
    # The projections of the two runs agree to rounding, so a few near-tie labels may differ: the comparison is by
    # tolerance over the whole step.  Both stay close to the dense step, and much closer to each other.
    assert rel(got, want) < 1e-2, rel(got, want)
    assert rel(got, dense) < 5e-2 and rel(want, dense) < 5e-2
    assert rel(got, want) < 0.5 * rel(got, dense) + 1e-3
    B.clear_runtimes()


def _ulysses_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        B = _backend()
        B.set_ulysses_world_size(world)
        x, text = _inputs()
        n = N // world
        dev = torch.device("cuda", rank)
        model = DiTStep(TINY, device=dev, seed=7, group=dist.group.WORLD)
        out = model.forward(x[rank * n:(rank + 1) * n].to(dev), text.to(dev), 500.0, _metadata(B, B.T2TRequestCache()))
        torch.cuda.synchronize()
        q.put((rank, out.float().cpu().numpy().copy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_ulysses_step_equals_the_single_gpu_step():
    from conftest import run_gloo_ranks
    B = _backend()
    x, text = _inputs()
    whole = DiTStep(TINY, device="cuda", seed=7).forward(x.cuda(), text.cuda(), 500.0,
                                                         _metadata(B, B.T2TRequestCache())).float().cpu()
    torch.cuda.synchronize()
    B.clear_runtimes()
    parts = dict(run_gloo_ranks(_ulysses_worker, 2, timeout=300))
    got = torch.cat([torch.from_numpy(parts[0]), torch.from_numpy(parts[1])])
    # each rank runs six of the twelve heads: the operator's bits do not depend on the sharding, the GEMMs around it
    # see half the rows and may round differently
    assert float((got - whole).norm() / whole.norm()) < 1e-2
