"""Builders shared by the control-plane tests: a prefill engine and a decode engine in one process."""
import os

os.environ.setdefault("BLLM_KVTRANS_QUIET_ENV", "1")
os.environ.setdefault("LLUMNIX_KV_ABORT_ON_TASK_EXCEPTION", "0")

from llumnix_kv_b200.engine.config import (CacheConfig, KVTransferConfig, ModelConfig, ParallelConfig,
                                            SchedulerConfig, VllmConfig)
from llumnix_kv_b200.engine.core import MiniEngineCore
from llumnix_kv_b200.engine.types import EngineCoreRequest, SamplingParams


def make_cfg(role, name, tp=1, device="cpu", cache_shape=2, num_blocks=64, layers=2, heads=8, head_dim=32,
             max_batched=8192, backend="kvt", extra=None, mx_scaled=False, block_size=16, gdn_groups=0, mla=None):
    ex = {"backend": backend, "kvt_inst_id": name, "naming_url": "fake://", "rpc_port": 0}
    ex.update(extra or {})
    return VllmConfig(
        model_config=ModelConfig(num_layers=layers, num_kv_heads=heads, head_dim=head_dim, is_hybrid=gdn_groups > 0,
                                 num_gdn_groups=gdn_groups, **(dict(use_mla=True, kv_lora_rank=mla[0],
                                                                    qk_rope_head_dim=mla[1], indexer_token_bytes=mla[2])
                                                               if mla else {})),
        cache_config=CacheConfig(block_size=block_size, num_gpu_blocks=num_blocks, cache_shape=cache_shape,
                                 mx_scaled=mx_scaled),
        parallel_config=ParallelConfig(tensor_parallel_size=tp),
        scheduler_config=SchedulerConfig(max_num_batched_tokens=max_batched),
        kv_transfer_config=KVTransferConfig(kv_role=role, kv_connector_extra_config=ex),
        device=device, instance_name=name)


def make_req(rid, n_prompt, max_tokens=4, params=None, seed=0):
    toks = [(seed * 7919 + i * 104729) % 31999 + 1 for i in range(n_prompt)]
    sp = SamplingParams(max_tokens=max_tokens, extra_args={"kv_transfer_params": dict(params or {})})
    return EngineCoreRequest(request_id=rid, prompt_token_ids=toks, sampling_params=sp, eos_token_id=None)


def make_pd(p_kw=None, d_kw=None):
    p = MiniEngineCore(make_cfg("kv_producer", "P", **(p_kw or {})))
    d = MiniEngineCore(make_cfg("kv_consumer", "D", **(d_kw or {})))
    return p, d
