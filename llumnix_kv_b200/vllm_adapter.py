"""The connector in the shape stock vLLM loads: ``KVConnectorBase_V1`` + ``SupportsHMA``.

vLLM instantiates the class named by ``kv_transfer_config.kv_connector`` (module given by
``kv_connector_module_path``) once in the engine-core process with role SCHEDULER and once in
every worker with role WORKER, and calls the entry points of ``KVConnectorBase_V1`` on it.  The
reference derives its facade from the same base, but inside a fork of vLLM whose scheduler calls
further hooks (``on_add_req``, ``step``, ``pending_requests``, an engine seam for block
reservation: blade_kvt/hybrid_connector/__init__.py:1776-1937).  Stock vLLM has no such calls, so:

* the WORKER half is complete here: ``register_kv_caches``, ``bind_connector_metadata`` /
  ``clear_connector_metadata``, ``start_load_kv``, ``wait_for_layer_load``, ``save_kv_layer``,
  ``wait_for_save`` run the same ``HybridWorker`` as the in-repo engine does;
* the SCHEDULER half delegates the base-class entry points (``get_num_new_matched_tokens``,
  ``update_state_after_alloc``, ``build_connector_meta``, ``request_finished_all_groups``) to the
  ``HybridScheduler``, which needs an engine seam object (``engine_proxy.EngineProxy``).  A host
  engine hands it over through ``kv_connector_extra_config["engine_proxy"]`` (scheduler) and
  ``["worker_proxy"]`` (worker); without one the scheduler-role constructor says so.

``connector_class()`` builds the class on first use, so importing this module does not import
vLLM.  Configuration objects are read through the attribute names that vLLM's own config
classes use; ``adapt_config`` copies them into the dataclasses of ``engine/config.py``.
"""
from __future__ import annotations

from typing import Any, Optional

_cls = None


def _first(obj: Any, names: tuple, default: Any = None) -> Any:
    for n in names:
        v = getattr(obj, n, None)
        if callable(v):
            try:
                v = v()
            except TypeError:
                continue
        if v is not None:
            return v
    return default


def adapt_config(vllm_config: Any, device: Optional[str] = None):
    """A ``llumnix_kv_b200.engine.config.VllmConfig`` with the fields this package reads, taken
    from a vLLM ``VllmConfig`` (or an object with the same attribute names)."""
    from llumnix_kv_b200.engine import config as C

    if isinstance(vllm_config, C.VllmConfig):
        return vllm_config
    mc, cc, pc = vllm_config.model_config, vllm_config.cache_config, vllm_config.parallel_config
    ktc = vllm_config.kv_transfer_config
    hf = _first(mc, ("hf_text_config", "hf_config"))
    tp = int(getattr(pc, "tensor_parallel_size", 1))
    heads = None
    if hasattr(mc, "get_total_num_kv_heads"):
        heads = mc.get_total_num_kv_heads()
    heads = int(heads if heads is not None else _first(hf, ("num_key_value_heads", "num_attention_heads"), 1))
    head_dim = int(mc.get_head_size()) if hasattr(mc, "get_head_size") else int(_first(hf, ("head_dim",), 128))
    layers = int(_first(hf, ("num_hidden_layers",), 1))
    model = C.ModelConfig(num_layers=layers, num_kv_heads=heads, head_dim=head_dim)
    if hasattr(model, "use_mla"):
        model.use_mla = bool(getattr(mc, "use_mla", False))
    cache = C.CacheConfig(block_size=int(getattr(cc, "block_size", 16)), num_gpu_blocks=int(getattr(cc, "num_gpu_blocks", 0) or 0))
    if hasattr(cache, "enable_prefix_caching"):
        cache.enable_prefix_caching = bool(getattr(cc, "enable_prefix_caching", False))
    par = C.ParallelConfig()
    for name in ("tensor_parallel_size", "data_parallel_rank", "data_parallel_size", "pipeline_parallel_size"):
        if hasattr(par, name) and hasattr(pc, name):
            setattr(par, name, getattr(pc, name))
    par.tensor_parallel_size = tp
    extra = dict(getattr(ktc, "kv_connector_extra_config", {}) or {})
    kv = C.KVTransferConfig(kv_role=getattr(ktc, "kv_role", None), kv_connector_extra_config=extra)
    out = C.VllmConfig(model_config=model, cache_config=cache, parallel_config=par, scheduler_config=C.SchedulerConfig(),
                       kv_transfer_config=kv, device=device or "cuda", instance_name=str(extra.get("kvt_inst_id", "vllm")))
    return out


def connector_class():
    """``LlumnixKVConnector``, a subclass of vLLM's ``KVConnectorBase_V1`` and ``SupportsHMA``."""
    global _cls
    if _cls is not None:
        return _cls
    from vllm.distributed.kv_transfer.kv_connector.v1.base import (KVConnectorBase_V1, KVConnectorMetadata,
                                                                   KVConnectorRole as VRole, SupportsHMA)

    from llumnix_kv_b200.hybrid_connector import HybridConnector
    from llumnix_kv_b200.hybrid_connector.engine_proxy import KVConnectorRole

    class LlumnixKVConnector(KVConnectorBase_V1, SupportsHMA):
        def __init__(self, vllm_config, role, kv_cache_config=None):
            super().__init__(vllm_config, role, kv_cache_config)
            extra = dict(getattr(vllm_config.kv_transfer_config, "kv_connector_extra_config", {}) or {})
            cfg = adapt_config(vllm_config, device=extra.get("device"))
            if role == VRole.SCHEDULER:
                engine = extra.get("engine_proxy")
                if engine is None:
                    raise RuntimeError(
                        "the scheduler half needs an engine seam (kv_connector_extra_config['engine_proxy'], an "
                        "engine_proxy.EngineProxy): stock vLLM's scheduler has no calls for block reservation on "
                        "behalf of a connector; the worker half needs none")
                self._impl = HybridConnector(cfg, KVConnectorRole.SCHEDULER, kv_cache_config, engine=engine)
            else:
                self._impl = HybridConnector(cfg, KVConnectorRole.WORKER, kv_cache_config, worker=extra.get("worker_proxy"))

        # ---- worker ------------------------------------------------------------------------------
        def register_kv_caches(self, kv_caches):
            self._impl.register_kv_caches(kv_caches)

        def bind_connector_metadata(self, connector_metadata: KVConnectorMetadata) -> None:
            super().bind_connector_metadata(connector_metadata)
            self._impl.bind_connector_metadata(connector_metadata)

        def clear_connector_metadata(self) -> None:
            self._impl.clear_connector_metadata()
            super().clear_connector_metadata()

        def start_load_kv(self, forward_context, **kwargs) -> None:
            self._impl.start_load_kv(forward_context, **kwargs)

        def wait_for_layer_load(self, layer_name: str) -> None:
            self._impl.wait_for_layer_load(layer_name)

        def save_kv_layer(self, layer_name: str, kv_layer, attn_metadata=None, **kwargs) -> None:
            self._impl.save_kv_layer(layer_name, kv_layer, attn_metadata, **kwargs)

        def wait_for_save(self):
            self._impl.wait_for_save()

        def get_finished(self, finished_req_ids):
            # completions reach the scheduler half over its own RPC port (SAVE_DONE / LOAD_DONE), not through
            # the executor's return path
            return None, None

        # ---- scheduler ---------------------------------------------------------------------------
        def get_num_new_matched_tokens(self, request, num_computed_tokens):
            return self._impl.get_num_new_matched_tokens(request, num_computed_tokens)

        def update_state_after_alloc(self, request, blocks, num_external_tokens):
            return self._impl.update_state_after_alloc(request, blocks, num_external_tokens)

        def build_connector_meta(self, scheduler_output):
            return self._impl.build_connector_meta(scheduler_output)

        def request_finished(self, request, block_ids):
            return self._impl.request_finished_all_groups(request, (block_ids,))

        def request_finished_all_groups(self, request, block_ids):
            return self._impl.request_finished_all_groups(request, block_ids)

        def shutdown(self):
            sched = getattr(self._impl, "_sched", None)
            if sched is not None:
                sched.close_bypass()

        @property
        def hybrid(self) -> HybridConnector:
            """The facade with the hooks stock vLLM does not call (``on_add_req``, ``step``, ...)."""
            return self._impl

    _cls = LlumnixKVConnector
    return _cls


def __getattr__(name: str):
    # lets vLLM's factory find the class by name without this module importing vLLM at import time
    if name == "LlumnixKVConnector":
        return connector_class()
    raise AttributeError(name)
