"""Multi-GPU plumbing around the operator: head-parallel sharding and the
Ulysses sequence <-> head all-to-all.

The operator itself never communicates: no kernel mixes heads, so a layer with
H heads runs as `world` independent operators over H / world heads each.  A
transformer block whose activations are sharded by sequence wraps it with two
all-to-alls (torch.distributed over NCCL on GPUs, gloo in the CPU tests); the
reference leaves this to its serving framework and only checks the head count
(integrations/sglang/backend/t2t_attn.py:1115-1125).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def head_range(rank: int, world: int, H: int):
    """Contiguous, balanced split of H heads over `world` ranks: [lo, hi)."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    base, rem = divmod(H, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def seq_to_head(x: torch.Tensor, group=None) -> torch.Tensor:
    """[N / P, H, D] (this rank's block of the sequence, all heads) ->
    [N, H / P, D] (whole sequence, this rank's heads)."""
    P = dist.get_world_size(group)
    n, H, D = x.shape
    if H % P:
        raise ValueError(f"{H} heads do not split over {P} ranks")
    send = x.view(n, P, H // P, D).permute(1, 0, 2, 3).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.view(P * n, H // P, D)


def head_to_seq(x: torch.Tensor, group=None) -> torch.Tensor:
    """Inverse of seq_to_head: [N, H / P, D] -> [N / P, H, D]."""
    P = dist.get_world_size(group)
    N, Hl, D = x.shape
    if N % P:
        raise ValueError(f"{N} tokens do not split over {P} ranks")
    send = x.view(P, N // P, Hl, D).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.permute(1, 0, 2, 3).reshape(N // P, P * Hl, D)
