"""Engine configuration objects.

The reference control plane reads its settings from a forked vLLM's ``VllmConfig``
(``kv_transfer_config.kv_connector_extra_config``, ``parallel_config``, ``cache_config``,
``model_config`` ...; blade_kvt/hybrid_connector/__init__.py:599-678, kvtbackend.py:483-563,
engine_proxy.py:424-433).  This framework ships its own minimal engine, so the same fields
live in plain dataclasses with the same names.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Optional


@dataclasses.dataclass
class ModelConfig:
    num_layers: int = 2
    num_kv_heads: int = 8
    head_dim: int = 128
    dtype_bytes: int = 2
    is_hybrid: bool = False
    use_mla: bool = False
    kv_lora_rank: int = 0
    qk_rope_head_dim: int = 0
    indexer_token_bytes: int = 0   # sparse MLA: bytes per token of the indexer key cache (second tensor of a layer)
    vocab_size: int = 32000
    name: str = "mini"
    # hybrid (Qwen3-Next-like) models: layers repeat as [gdn x num_gdn_groups, attention]; layer i of
    # that pattern lives in KV-cache group i % (num_gdn_groups + 1) and in physical cache tensor
    # i // (num_gdn_groups + 1), which one GDN layer of every group and one attention layer share
    num_gdn_groups: int = 0
    gdn_conv_rows: int = 3
    gdn_conv_channel_dims: tuple = (32, 32, 64)     # q, k, v channels of the conv state, whole model
    gdn_ssm_shape: tuple = (4, 8, 8)                # (heads, k_dim, v_dim) of the recurrent state, whole model
    gdn_conv_elem_size: int = 2
    gdn_ssm_elem_size: int = 4

    def group_types(self) -> list:
        return ["gdn"] * self.num_gdn_groups + ["attn"] if self.is_hybrid else ["attn"]

    def layer_group(self, layer: int) -> int:
        return layer % (self.num_gdn_groups + 1) if self.is_hybrid else 0

    def layer_tensor(self, layer: int) -> int:
        return layer // (self.num_gdn_groups + 1) if self.is_hybrid else layer

    def is_gdn_layer(self, layer: int) -> bool:
        return self.is_hybrid and self.layer_group(layer) < self.num_gdn_groups

    def hybrid_kvt_kwargs_for(self, tp: int) -> dict:
        """Per-rank recurrent-state geometry in the form KVTransferClient / Server take it."""
        if not self.is_hybrid:
            return {}
        dims = [d // tp for d in self.gdn_conv_channel_dims]
        h, k, v = self.gdn_ssm_shape
        return dict(num_gdn_layers=self.num_gdn_groups, conv_state_shape=[1, self.gdn_conv_rows, sum(dims)],
                    ssm_state_shape=[1, max(1, h // tp), k, v], gdn_conv_channel_dims=dims,
                    gdn_conv_elem_size=self.gdn_conv_elem_size, gdn_ssm_elem_size=self.gdn_ssm_elem_size)


@dataclasses.dataclass
class CacheConfig:
    block_size: int = 16
    num_gpu_blocks: int = 64
    enable_prefix_caching: bool = False
    cache_shape: int = 2          # CacheShape id of this engine's paged cache
    mx_scaled: bool = False       # pages are block-scaled e4m3 (decode side of an fp8 transfer)
    mamba_cache_mode: str = "none"
    cache_dtype: str = "auto"


@dataclasses.dataclass
class ParallelConfig:
    tensor_parallel_size: int = 1
    data_parallel_rank: int = 0
    data_parallel_size: int = 1


@dataclasses.dataclass
class SpeculativeConfig:
    num_speculative_tokens: int = 0


@dataclasses.dataclass
class SchedulerConfig:
    max_num_batched_tokens: int = 8192
    max_num_seqs: int = 64


@dataclasses.dataclass
class KVTransferConfig:
    kv_connector: str = "HybridConnector"
    kv_role: str = "kv_both"      # kv_producer | kv_consumer | kv_both
    kv_connector_extra_config: dict = dataclasses.field(default_factory=dict)
    engine_available_port: int = 0

    @property
    def is_kv_producer(self) -> bool:
        return self.kv_role in ("kv_producer", "kv_both")

    @property
    def is_kv_consumer(self) -> bool:
        return self.kv_role in ("kv_consumer", "kv_both")

    def get_from_extra_config(self, key: str, default: Any = None) -> Any:
        return self.kv_connector_extra_config.get(key, default)


@dataclasses.dataclass
class VllmConfig:
    model_config: ModelConfig = dataclasses.field(default_factory=ModelConfig)
    cache_config: CacheConfig = dataclasses.field(default_factory=CacheConfig)
    parallel_config: ParallelConfig = dataclasses.field(default_factory=ParallelConfig)
    scheduler_config: SchedulerConfig = dataclasses.field(default_factory=SchedulerConfig)
    speculative_config: Optional[SpeculativeConfig] = None
    kv_transfer_config: Optional[KVTransferConfig] = None
    device: str = "cpu"           # "cpu" or "cuda:N" - where the paged cache lives
    instance_name: str = "inst"


@dataclasses.dataclass
class KVCacheGroupSpec:
    layer_names: list
    kv_cache_spec: Any = None


@dataclasses.dataclass
class KVCacheConfig:
    num_blocks: int = 0
    kv_cache_groups: list = dataclasses.field(default_factory=list)
