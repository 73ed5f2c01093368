"""The connector class that stock vLLM can load: it derives from vLLM's own KVConnectorBase_V1 and
SupportsHMA, leaves no abstract method open, and its worker half runs the same HybridWorker as the
in-repo engine (a decode-side worker registers its caches and serves a prefill engine's push)."""
import types

import pytest
import torch

vllm_base = pytest.importorskip("vllm.distributed.kv_transfer.kv_connector.v1.base")

from pd_helpers import make_cfg, make_req

from llumnix_kv_b200 import vllm_adapter
from llumnix_kv_b200.hybrid_connector.engine_proxy import WorkerProxy


def test_class_fits_vllms_connector_interface():
    cls = vllm_adapter.connector_class()
    assert vllm_adapter.LlumnixKVConnector is cls                      # what vLLM's factory looks up by name
    assert issubclass(cls, vllm_base.KVConnectorBase_V1) and issubclass(cls, vllm_base.SupportsHMA)
    assert not getattr(cls, "__abstractmethods__", None)
    for name in ("register_kv_caches", "start_load_kv", "wait_for_layer_load", "save_kv_layer", "wait_for_save",
                 "get_num_new_matched_tokens", "update_state_after_alloc", "build_connector_meta",
                 "request_finished_all_groups", "bind_connector_metadata", "clear_connector_metadata"):
        assert name in cls.__dict__, name
    with pytest.raises(RuntimeError, match="engine seam"):
        cls(make_cfg("kv_producer", "S"), vllm_base.KVConnectorRole.SCHEDULER, None)


def test_config_fields_are_read_through_vllms_attribute_names():
    hf = types.SimpleNamespace(num_hidden_layers=32, num_key_value_heads=8, head_dim=128)
    mc = types.SimpleNamespace(hf_text_config=hf, get_total_num_kv_heads=lambda: 8, get_head_size=lambda: 128, use_mla=False)
    cc = types.SimpleNamespace(block_size=16, num_gpu_blocks=512, enable_prefix_caching=True)
    pc = types.SimpleNamespace(tensor_parallel_size=4, data_parallel_rank=1, data_parallel_size=2)
    ktc = types.SimpleNamespace(kv_role="kv_consumer", kv_connector_extra_config={"backend": "kvt", "kvt_inst_id": "dec"})
    cfg = vllm_adapter.adapt_config(types.SimpleNamespace(model_config=mc, cache_config=cc, parallel_config=pc,
                                                          kv_transfer_config=ktc))
    assert (cfg.model_config.num_layers, cfg.model_config.num_kv_heads, cfg.model_config.head_dim) == (32, 8, 128)
    assert (cfg.cache_config.block_size, cfg.cache_config.num_gpu_blocks, cfg.cache_config.enable_prefix_caching) == (16, 512, True)
    assert cfg.parallel_config.tensor_parallel_size == 4 and cfg.parallel_config.data_parallel_rank == 1
    assert cfg.kv_transfer_config.kv_role == "kv_consumer" and cfg.instance_name == "dec"
    assert cfg.kv_transfer_config.get_from_extra_config("backend", "") == "kvt"


def test_worker_half_serves_a_transfer_like_the_in_repo_worker():
    """A decode worker built WITHOUT its own connector gets the vLLM-shaped one: its
    register_kv_caches starts the transfer server, and a prefill engine's request lands in its cache."""
    from llumnix_kv_b200.engine.core import MiniEngineCore
    from llumnix_kv_b200.engine.worker import MiniWorker

    cls = vllm_adapter.connector_class()
    p = MiniEngineCore(make_cfg("kv_producer", "P"))
    d = MiniEngineCore(make_cfg("kv_consumer", "D"))
    try:
        # a second worker of the decode instance's shape whose connector is the adapter
        cfg = make_cfg("kv_consumer", "D2")
        w = MiniWorker(cfg, 0, with_connector=False)
        proxy = WorkerProxy(cfg, 0, "cpu")
        cfg.kv_transfer_config.kv_connector_extra_config["worker_proxy"] = proxy
        conn = cls(cfg, vllm_base.KVConnectorRole.WORKER, w.kv_cache_config)
        conn.register_kv_caches(w.kv_caches)
        assert conn.hybrid._worker is not None and not conn.has_connector_metadata()
        assert conn.get_finished(set()) == (None, None)
        conn.wait_for_layer_load("model.layers.0.attn")
        conn.wait_for_save()
        # the stock P -> D path still works next to it
        params = {"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()}
        d.add_request(make_req("r", 40, max_tokens=2, params=params))
        out = d.wait_finished("r", 30)
        assert out is not None and out.finish_reason is not None
    finally:
        d.shutdown()
        p.shutdown()


def test_scheduler_half_over_an_engine_seam():
    """With an engine seam object the scheduler-role instance is the same HybridScheduler the in-repo engine
    drives: vLLM's own entry points answer as the reference's do (no external tokens through that hook), and the
    hooks stock vLLM never calls are reachable through ``.hybrid``."""
    from llumnix_kv_b200.engine.core import MiniEngineCore
    from llumnix_kv_b200.engine.types import Request

    from llumnix_kv_b200.hybrid_connector.engine_proxy import EngineProxy

    cls = vllm_adapter.connector_class()
    plain = make_cfg("kv_producer", "H")
    plain.kv_transfer_config = None
    host = MiniEngineCore(plain)                                     # an engine without a connector of its own
    try:
        cfg = make_cfg("kv_producer", "S", extra={"rpc_port": 0})
        cfg.kv_transfer_config.kv_connector_extra_config["engine_proxy"] = EngineProxy(host, cfg)
        conn = cls(cfg, vllm_base.KVConnectorRole.SCHEDULER, None)
        req = Request("r", [1, 2, 3])
        assert conn.get_num_new_matched_tokens(req, 0) == (0, False)
        assert conn.request_finished(req, [1, 2]) == (False, None)
        assert conn.request_finished_all_groups(req, ([1, 2],)) == (False, None)
        assert conn.hybrid.has_requests() is False and conn.hybrid.step() is None or conn.hybrid.step() == {}
        conn.shutdown()
    finally:
        host.shutdown()
