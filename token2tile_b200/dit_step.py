"""One denoising step of a video diffusion transformer with the Wan2.1-14B
architecture, random-initialised, with Token2Tile self-attention.

This is a measurement harness, not a model port: the reference leaves the
transformer to its serving framework, so the block below is built from the
published shape alone (40 blocks, width 5120, 40 heads of 128, feed-forward
width 13824, cross-attention over 512 text tokens of width 4096, bfloat16).
Each block is

    x += gate_sa  * SelfAttn (modulate(LN(x), shift_sa, scale_sa))      Token2Tile
    x +=            CrossAttn(LN_affine(x), text)                        dense
    x += gate_ffn * FFN      (modulate(LN(x), shift_ffn, scale_ffn))     GELU(tanh)

with the six modulation vectors from the timestep embedding plus a learned
per-block table, and RMS-normalised queries and keys.  Rotary position
embedding is left out: it is elementwise work on q and k that changes neither
the shapes nor the communication pattern.

Sequence parallelism (Ulysses): every rank holds N / P tokens of the residual
stream and all weights.  Around self-attention the q, k, v projections are
exchanged by an all-to-all into [N, H / P, 128] (whole sequence, this rank's
heads), the attention backend runs on them, and the inverse all-to-all brings
the output back to [N / P, H, 128]: four all-to-alls per block over NCCL.
Cross-attention is sequence-local (every rank holds all 512 text tokens).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import parallel


@dataclass(frozen=True)
class DiTShape:
    blocks: int = 40
    dim: int = 5120
    heads: int = 40
    head_dim: int = 128
    ffn: int = 13824
    text_len: int = 512
    text_dim: int = 4096
    freq_dim: int = 256

    def __post_init__(self):
        if self.heads * self.head_dim != self.dim:
            raise ValueError("dim must equal heads * head_dim")


WAN_14B = DiTShape()


def _rms(x, weight, eps=1e-6):
    return F.rms_norm(x, x.shape[-1:], weight, eps)


def _modulate(x, shift, scale, eps=1e-6):
    """LayerNorm(x) * (1 + scale) + shift; the fused norm accumulates in fp32 internally."""
    return torch.addcmul(shift, F.layer_norm(x, x.shape[-1:], eps=eps), 1 + scale)


class _Linear:
    """y = x W^T + b with W [out, in]; plain tensors, no autograd."""

    def __init__(self, fan_in, fan_out, gen, device, dtype):
        w = torch.randn(fan_out, fan_in, generator=gen, dtype=torch.float32, device=device) / math.sqrt(fan_in)
        self.w = w.to(dtype)
        self.b = torch.zeros(fan_out, dtype=dtype, device=device)

    def __call__(self, x):
        return F.linear(x, self.w, self.b)


class DiTBlock:
    def __init__(self, shape: DiTShape, index: int, gen, device, dtype, make_attn):
        d = shape.dim
        lin = lambda i, o: _Linear(i, o, gen, device, dtype)
        self.shape, self.index = shape, index
        self.q, self.k, self.v, self.o = lin(d, d), lin(d, d), lin(d, d), lin(d, d)
        self.cq, self.ck, self.cv, self.co = lin(d, d), lin(d, d), lin(d, d), lin(d, d)
        self.up, self.down = lin(d, shape.ffn), lin(shape.ffn, d)
        ones = lambda n: torch.ones(n, dtype=dtype, device=device)
        self.norm_q, self.norm_k, self.norm_cq, self.norm_ck = ones(d), ones(d), ones(d), ones(d)
        self.norm3_w, self.norm3_b = ones(d), torch.zeros(d, dtype=dtype, device=device)
        self.modulation = (torch.randn(6, d, generator=gen, dtype=torch.float32, device=device)
                           / math.sqrt(d)).to(dtype)
        # self-attention implementation of this layer: (num_heads, head_size, causal, scale, prefix=) -> impl
        self.attn = make_attn(shape.heads, shape.head_dim, False, 1.0 / math.sqrt(shape.head_dim),
                              prefix=f"blocks.{index}.attn1")

    def forward(self, x, e6, text, attn_metadata, group):
        """x [n_local, dim]; e6 [6, dim] timestep modulation; text [text_len, dim]."""
        s = self.shape
        H, D = s.heads, s.head_dim
        mod = (self.modulation.float() + e6.float()).to(x.dtype)
        shift_sa, scale_sa, gate_sa, shift_ff, scale_ff, gate_ff = mod.unbind(0)

        h = _modulate(x, shift_sa, scale_sa)
        q = _rms(self.q(h), self.norm_q).view(-1, H, D)
        k = _rms(self.k(h), self.norm_k).view(-1, H, D)
        v = self.v(h).view(-1, H, D)
        if group is not None:
            q, k, v = (parallel.seq_to_head(t, group) for t in (q, k, v))
        a = self.attn.forward(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), attn_metadata)[0]
        if group is not None:
            a = parallel.head_to_seq(a.contiguous(), group)
        x = torch.addcmul(x, self.o(a.reshape(-1, H * D)), gate_sa)

        h = F.layer_norm(x, x.shape[-1:], self.norm3_w, self.norm3_b, 1e-6)
        cq = _rms(self.cq(h), self.norm_cq).view(-1, H, D).transpose(0, 1)
        ck = _rms(self.ck(text), self.norm_ck).view(-1, H, D).transpose(0, 1)
        cv = self.cv(text).view(-1, H, D).transpose(0, 1)
        c = F.scaled_dot_product_attention(cq, ck, cv).transpose(0, 1).reshape(-1, H * D)
        x = x + self.co(c)

        h = _modulate(x, shift_ff, scale_ff)
        y = self.down(F.gelu(self.up(h), approximate="tanh"))
        return torch.addcmul(x, y, gate_ff)


class DiTStep:
    """The transformer of one denoising step over this rank's tokens.

    make_attn: factory with the signature of the attention backend's
        implementation class (`T2TAttentionImpl` by default).
    group: the sequence-parallel process group, or None for a single device."""

    def __init__(self, shape: DiTShape = WAN_14B, *, device="cuda", dtype=torch.bfloat16, seed=0, make_attn=None,
                 group=None, blocks=None):
        if make_attn is None:
            from .t2t_attn import T2TAttentionImpl as make_attn
        self.shape, self.group = shape, group
        self.device, self.dtype = torch.device(device), dtype
        # a device generator: the same seed gives every rank (same device type) the same weights
        gen = torch.Generator(device=self.device).manual_seed(seed)
        d = shape.dim
        lin = lambda i, o: _Linear(i, o, gen, self.device, dtype)
        self.text_in, self.text_mid = lin(shape.text_dim, d), lin(d, d)
        self.time_in, self.time_mid, self.time_proj = lin(shape.freq_dim, d), lin(d, d), lin(d, 6 * d)
        self.blocks = [DiTBlock(shape, i, gen, self.device, dtype, make_attn)
                       for i in range(shape.blocks if blocks is None else blocks)]

    def weight_bytes(self) -> int:
        total = 0
        for obj in [self.text_in, self.text_mid, self.time_in, self.time_mid, self.time_proj] + \
                [getattr(b, n) for b in self.blocks for n in ("q", "k", "v", "o", "cq", "ck", "cv", "co", "up", "down")]:
            total += obj.w.numel() * obj.w.element_size()
        return total

    def _time_embedding(self, t: float):
        half = self.shape.freq_dim // 2
        freqs = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=self.device) / half)
        arg = float(t) * freqs
        emb = torch.cat((arg.cos(), arg.sin())).to(self.dtype)
        e = self.time_mid(F.silu(self.time_in(emb)))
        return self.time_proj(F.silu(e)).view(6, self.shape.dim)

    @torch.no_grad()
    def forward(self, x_local, text_tokens, timestep: float, attn_metadata):
        """x_local [N / P, dim]: this rank's block of the latent tokens;
        text_tokens [text_len, text_dim]; returns the block's new value."""
        e6 = self._time_embedding(timestep)
        text = self.text_mid(F.gelu(self.text_in(text_tokens), approximate="tanh"))
        x = x_local
        for block in self.blocks:
            x = block.forward(x, e6, text, attn_metadata, self.group)
        return x


def flops_per_step(shape: DiTShape, n_tokens: int) -> float:
    """Dense-GEMM FLOPs of one step over n_tokens (attention excluded)."""
    d = shape.dim
    per_token = 2 * (4 * d * d + 2 * d * d + 2 * d * shape.ffn)      # self qkvo, cross q + o, ffn
    per_text = 2 * (2 * d * d)                                        # cross k, v
    return shape.blocks * (n_tokens * per_token + shape.text_len * per_text)


def all_to_all_bytes_per_block(shape: DiTShape, n_tokens: int, world: int, elem: int = 2) -> int:
    """Bytes each rank sends per block: four all-to-alls of its [N / P, H, D]
    slab, of which the fraction (P - 1) / P leaves the device."""
    if world <= 1:
        return 0
    slab = n_tokens // world * shape.dim * elem
    return 4 * slab * (world - 1) // world
