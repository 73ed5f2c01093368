"""KV-cache shapes of the model families the transfer engine serves.

The framework has no model code of its own (neither has the reference: it is a connector); what
it needs from a model is the geometry of its KV cache.  A ``KVSpec`` carries that geometry and
turns it, for one TP rank, into the layout descriptors the kernels and the planner use.
Families follow the cache shapes of kvtransfer/include/envcfg.h:25-52 and the argument builder
in blade_kvt/hybrid_connector/kvtbackend.py:709-1101.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

from llumnix_kv_b200.ops.layouts import AttnLayout, CacheShape, mla_layout


@dataclasses.dataclass(frozen=True)
class KVSpec:
    name: str
    num_layers: int
    num_kv_heads: int
    head_dim: int
    dtype_bytes: int = 2
    block_size: int = 16
    # MLA (DeepSeek-style): one latent+rope vector per token instead of K and V heads
    use_mla: bool = False
    kv_lora_rank: int = 0
    qk_rope_head_dim: int = 0
    indexer_dim: int = 0          # sparse-attention indexer keys (second tensor per layer)
    # hybrid (GDN / KDA) linear-attention state, per request rather than per token
    num_linear_layers: int = 0
    conv_state_shape: Optional[tuple] = None   # (rows, channels)
    ssm_state_shape: Optional[tuple] = None    # (heads, k_dim, v_dim)
    conv_channel_dims: Optional[tuple] = None  # (q, k, v) channel split of the conv state
    ssm_dtype_bytes: int = 4

    def heads_on_rank(self, tp: int) -> int:
        return 1 if self.use_mla else max(1, self.num_kv_heads // tp)

    def attn_layout(self, shape: CacheShape, num_blocks: int, tp: int = 1, mx_scaled: bool = False) -> AttnLayout:
        """Per-layer attention cache of one TP rank (GQA heads are replicated when tp > heads)."""
        if self.use_mla:
            width = (self.kv_lora_rank + self.qk_rope_head_dim) * (1 if mx_scaled else self.dtype_bytes)
            return mla_layout(num_blocks, self.block_size, width, mx_scaled)
        elem = 1 if mx_scaled else self.dtype_bytes
        return AttnLayout(CacheShape(shape), num_blocks, self.block_size, self.heads_on_rank(tp), self.head_dim, elem,
                          mx_scaled=mx_scaled)

    def token_bytes(self, tp: int = 1) -> int:
        """KV bytes of one token in one layer on one rank (what WorkerInfo.token_sizes carries)."""
        if self.use_mla:
            return (self.kv_lora_rank + self.qk_rope_head_dim) * self.dtype_bytes
        return 2 * self.heads_on_rank(tp) * self.head_dim * self.dtype_bytes

    def linear_state_bytes(self, tp: int = 1) -> int:
        """Bytes of one request's conv + recurrent state in one linear-attention layer on one rank."""
        if not self.num_linear_layers:
            return 0
        rows, ch = self.conv_state_shape
        h, k, v = self.ssm_state_shape
        return rows * (ch // tp) * self.dtype_bytes + (h // tp) * k * v * self.ssm_dtype_bytes


LLAMA3_8B = KVSpec("llama-3-8b", 32, 8, 128)
LLAMA3_70B = KVSpec("llama-3-70b", 80, 8, 128)
QWEN3_NEXT_80B = KVSpec("qwen3-next-80b-a3b", 12, 2, 256, num_linear_layers=36, conv_state_shape=(3, 8192),
                        ssm_state_shape=(32, 128, 128), conv_channel_dims=(2048, 2048, 4096))
DEEPSEEK_V32 = KVSpec("deepseek-v3.2", 61, 1, 576, use_mla=True, kv_lora_rank=512, qk_rope_head_dim=64,
                      indexer_dim=128, block_size=64)
KIMI_K3 = KVSpec("kimi-k3", 48, 1, 576, use_mla=True, kv_lora_rank=512, qk_rope_head_dim=64, num_linear_layers=36,
                 conv_state_shape=(3, 6144), ssm_state_shape=(48, 128, 128), conv_channel_dims=(2048, 2048, 2048))

SPECS = {s.name: s for s in (LLAMA3_8B, LLAMA3_70B, QWEN3_NEXT_80B, DEEPSEEK_V32, KIMI_K3)}


def spec_from_config(cfg) -> KVSpec:
    """KVSpec of the minimal engine's ``VllmConfig``."""
    mc, cc = cfg.model_config, cfg.cache_config
    return KVSpec(mc.name, mc.num_layers, mc.num_kv_heads, mc.head_dim, mc.dtype_bytes, cc.block_size,
                  use_mla=mc.use_mla, kv_lora_rank=mc.kv_lora_rank, qk_rope_head_dim=mc.qk_rope_head_dim)


def rank_attn_layout(cfg) -> AttnLayout:
    """Layout of every TP rank's per-layer attention cache under ``cfg`` (ranks are symmetric)."""
    cc = cfg.cache_config
    return spec_from_config(cfg).attn_layout(CacheShape(cc.cache_shape), cc.num_gpu_blocks,
                                             cfg.parallel_config.tensor_parallel_size, cc.mx_scaled)
