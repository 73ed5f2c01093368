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
    vocab_size: int = 32000
    name: str = "mini"


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
