"""The transformer-step harness on the CPU: a sequence-sharded step (two gloo
ranks, Ulysses all-to-all around self-attention) equals the unsharded step.  A
dense stand-in replaces the attention backend, which needs a GPU."""
import math
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from token2tile_b200.dit_step import DiTShape, DiTStep, all_to_all_bytes_per_block, flops_per_step, WAN_14B

TINY = DiTShape(blocks=2, dim=256, heads=2, head_dim=128, ffn=384, text_len=8, text_dim=64, freq_dim=32)


class DenseStandIn:
    """Same constructor and forward signature as the backend's implementation class."""

    def __init__(self, num_heads, head_size, causal, softmax_scale, prefix=""):
        self.scale = softmax_scale

    def forward(self, q, k, v, meta):
        out = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2),
                                                               v.transpose(1, 2), scale=self.scale)
        return out.transpose(1, 2).contiguous()


def _inputs(n=32):
    g = torch.Generator().manual_seed(1)
    return torch.randn(n, TINY.dim, generator=g), torch.randn(TINY.text_len, TINY.text_dim, generator=g)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, text = _inputs()
        n = x.shape[0] // world
        model = DiTStep(TINY, device="cpu", dtype=torch.float32, seed=7, make_attn=DenseStandIn,
                        group=dist.group.WORLD)
        out = model.forward(x[rank * n:(rank + 1) * n].contiguous(), text, 500.0, None)
        # by value: a tensor would travel as a shared-memory handle that dies with this process
        q.put((rank, out.numpy().copy()))
    finally:
        dist.destroy_process_group()


def test_sequence_sharded_step_equals_the_unsharded_step():
    x, text = _inputs()
    whole = DiTStep(TINY, device="cpu", dtype=torch.float32, seed=7, make_attn=DenseStandIn).forward(
        x, text, 500.0, None)
    assert whole.shape == x.shape and bool(torch.isfinite(whole).all())
    assert (whole - x).abs().max() > 1e-3          # the step does something
    from conftest import run_gloo_ranks
    parts = dict(run_gloo_ranks(_worker, 2))
    got = torch.cat([torch.from_numpy(parts[0]), torch.from_numpy(parts[1])])
    assert (got - whole).abs().max() <= 1e-4 * whole.abs().max()


def test_work_and_traffic_figures():
    # 40 blocks x 75,600 tokens: 2 * (6 * 5120^2 + 2 * 5120 * 13824) flops per token and block
    per_token = 2 * (6 * 5120 ** 2 + 2 * 5120 * 13824)
    assert math.isclose(flops_per_step(WAN_14B, 75600), 40 * (75600 * per_token + 512 * 4 * 5120 ** 2))
    assert all_to_all_bytes_per_block(WAN_14B, 75600, 1) == 0
    # each rank's [9450, 5120] bf16 slab, four times, 7/8 of it leaving the device
    assert all_to_all_bytes_per_block(WAN_14B, 75600, 8) == 4 * 9450 * 5120 * 2 * 7 // 8
