"""A Llama-shaped prefill worker for measuring what KV transfer adds to time-to-first-token.

The framework itself has no model code (neither has the reference: it is a connector that a
serving engine calls).  To measure the one number a user of PD separation cares about, the time
to first token with and without shipping the KV away, something has to play the engine's model
runner: this module runs a random-initialised decoder of a given geometry over a prompt, writes
each layer's K and V into a paged NHD cache the way an attention backend does, and calls a
``save_kv_layer``-style hook after every layer on the forward stream.  The dense math is plain
library code (cuBLAS through ``torch.matmul``, ``scaled_dot_product_attention``); the part under
test is the transfer that overlaps it.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from llumnix_kv_b200.ops.layouts import AttnLayout, CacheShape


@dataclasses.dataclass(frozen=True)
class DecoderGeometry:
    name: str
    num_layers: int
    hidden: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int


LLAMA3_8B_GEOMETRY = DecoderGeometry("llama-3-8b", 32, 4096, 32, 8, 128, 14336, 128256)
TINY_GEOMETRY = DecoderGeometry("tiny", 2, 256, 4, 2, 64, 512, 1000)


class PrefillWorker:
    """Random-init decoder + paged NHD KV cache on one GPU."""

    def __init__(self, geo: DecoderGeometry, device, num_blocks: int, block_size: int = 16, seed: int = 0,
                 attn_chunk: int = 2048):
        self.geo, self.device, self.block_size = geo, torch.device(device), block_size
        self.attn_chunk = attn_chunk
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        dt = torch.bfloat16

        def w(*shape, scale):
            return (torch.randn(*shape, device=self.device, dtype=torch.float32, generator=g) * scale).to(dt)

        h, qd, kvd = geo.hidden, geo.num_heads * geo.head_dim, geo.num_kv_heads * geo.head_dim
        self.layers = []
        for _ in range(geo.num_layers):
            self.layers.append(dict(
                wqkv=w(h, qd + 2 * kvd, scale=h ** -0.5), wo=w(qd, h, scale=qd ** -0.5),
                wgu=w(h, 2 * geo.ffn, scale=h ** -0.5), wd=w(geo.ffn, h, scale=geo.ffn ** -0.5),
                n1=torch.ones(h, device=self.device, dtype=dt), n2=torch.ones(h, device=self.device, dtype=dt)))
        self.embed = w(geo.vocab, h, scale=1.0)
        self.lm_head = w(h, geo.vocab, scale=h ** -0.5)
        self.norm = torch.ones(h, device=self.device, dtype=dt)
        self.layout = AttnLayout(CacheShape.FLASH, num_blocks, block_size, geo.num_kv_heads, geo.head_dim, 2)
        self.kv_caches = [self.layout.alloc(self.device) for _ in range(geo.num_layers)]
        self._views = [self.layout.view(c, dt) for c in self.kv_caches]     # [block, kv, slot, head, dim]

    @staticmethod
    def _rms(x: torch.Tensor, wt: torch.Tensor) -> torch.Tensor:
        v = x.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5)).to(x.dtype) * wt

    def _rope(self, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        d = x.shape[-1]
        inv = 1.0 / (500000.0 ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
        ang = pos.float()[:, None] * inv[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        x1, x2 = x.float()[..., 0::2], x.float()[..., 1::2]
        out = torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1).flatten(-2)
        return out.to(x.dtype)

    @torch.no_grad()
    def prefill(self, token_ids: torch.Tensor, block_ids: torch.Tensor,
                after_layer: Optional[Callable[[int], None]] = None) -> torch.Tensor:
        """Runs the prompt, fills the paged cache, returns the first sampled token (device tensor).
        ``after_layer(i)`` is called on the forward stream right after layer i's KV has been
        written (the place where an engine calls ``save_kv_layer``)."""
        geo = self.geo
        T = token_ids.numel()
        pos = torch.arange(T, device=self.device)
        blk = block_ids[pos // self.block_size]
        slot = pos % self.block_size
        x = self.embed[token_ids]
        qd, kvd = geo.num_heads * geo.head_dim, geo.num_kv_heads * geo.head_dim
        for i, L in enumerate(self.layers):
            hdn = self._rms(x, L["n1"])
            qkv = hdn @ L["wqkv"]
            q = self._rope(qkv[:, :qd].view(T, geo.num_heads, geo.head_dim), pos)
            k = self._rope(qkv[:, qd:qd + kvd].view(T, geo.num_kv_heads, geo.head_dim), pos)
            v = qkv[:, qd + kvd:].view(T, geo.num_kv_heads, geo.head_dim)
            view = self._views[i]
            view[blk, 0, slot] = k
            view[blk, 1, slot] = v
            if after_layer is not None:
                after_layer(i)
            attn = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None],
                                                  v.transpose(0, 1)[None], is_causal=True, enable_gqa=True)
            x = x + attn[0].transpose(0, 1).reshape(T, qd) @ L["wo"]
            hdn = self._rms(x, L["n2"])
            gu = hdn @ L["wgu"]
            x = x + (F.silu(gu[:, :geo.ffn]) * gu[:, geo.ffn:]) @ L["wd"]
        last = self._rms(x[-1:], self.norm)
        return (last @ self.lm_head).argmax(-1)
