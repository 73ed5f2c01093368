"""Worker half of the HybridConnector (one per TP rank).

The model-runner thread binds the step's metadata, calls ``start_load_kv`` once and
``save_kv_layer`` after each attention layer, then clears the metadata.  Backend generators
run on the connector's own event loop (*disaggw thread*); every request they finish is
reported to the scheduler half over the LOAD_DONE / SAVE_DONE RPC
(blade_kvt/hybrid_connector/__init__.py:1573-1772).
"""
from __future__ import annotations

import asyncio
import logging
import pickle
import struct
import time
from collections.abc import AsyncGenerator
from typing import Optional

import msgspec

from .backend import (GET_BYPASS_HANDLE, GET_BYPASS_HANDLE_RESP, LOAD_DONE_REQ, LOAD_DONE_RESP, SAVE_DONE_REQ,
                      SAVE_DONE_RESP, HybridMetadata, IoDoneReqs, get_backend_cls)
from .engine_proxy import KVConnectorRole, VllmConfig, WorkerProxy, scheduler_rpc_host, sched_rpc_server_port
from .utils import ConnPool, IoRet, kill_me_if_exception, spawn_task

logger = logging.getLogger("llumnix_kv_b200.hybrid_connector")


class _WSavingReq:
    def __init__(self):
        self._ready_layers: list = []


def _failure_as_text(obj):
    if isinstance(obj, BaseException):
        return f"{type(obj).__name__}: {obj}"
    raise NotImplementedError(f"objects of type {type(obj).__name__} do not travel in a completion report")


class HybridWorker:
    def __init__(self, vllm_config: VllmConfig, kv_cache_config, worker: WorkerProxy):
        self.closing = False          # set by the engine before it stops the scheduler's RPC server
        from llumnix_kv_b200 import envs

        self._cfg = vllm_config
        self._kv_cache_config = kv_cache_config
        self._wp = worker
        self.loop = worker.get_hybrid_worker_loop()
        self._meta: Optional[HybridMetadata] = None          # model-runner thread
        self._saving: dict[str, _WSavingReq] = {}             # disaggw thread
        self._connpool = ConnPool(scheduler_rpc_host(vllm_config), sched_rpc_server_port(vllm_config), 3)
        # A failure crosses the wire as text ("Type: message"): msgspec does not encode exception objects, and a worker
        # that tried used to end its process (the reference warns of exactly that next to IoRet.ex and never sets it).
        self._ioenc = msgspec.msgpack.Encoder(enc_hook=_failure_as_text)
        self._strdec = msgspec.msgpack.Decoder(str)
        BackendCls = get_backend_cls(vllm_config)
        self._backend = BackendCls(vllm_config, KVConnectorRole.WORKER, kv_cache_config, worker=worker, connector=self)
        self._num_layers: Optional[int] = None
        if envs.VLLM_ENABLE_BYPASS_TASK:
            asyncio.run_coroutine_threadsafe(self.start_bypass_task_loop(), self.loop)

    # ---- bypass: step metadata produced between engine steps ---------------------------------------
    async def _get_bypass_handle(self) -> str:
        host, port = scheduler_rpc_host(self._cfg), sched_rpc_server_port(self._cfg)
        last_log = 0.0
        while True:
            try:
                reader, writer = await asyncio.open_connection(host, port)
                writer.write(struct.pack("=I", GET_BYPASS_HANDLE))
                await writer.drain()
                head, n = struct.unpack("=II", await asyncio.wait_for(reader.readexactly(8), timeout=3.0))
                if head != GET_BYPASS_HANDLE_RESP:
                    raise RuntimeError(f"invalid resp head={head:#x}")
                handle = self._strdec.decode(await reader.readexactly(n))
                writer.close()
                return handle
            except RuntimeError:
                raise
            except Exception as ex:  # scheduler not up yet: say so once per VLLM_LOG_STATS_INTERVAL, not every 0.1 s
                if time.time() - last_log > envs.VLLM_LOG_STATS_INTERVAL:
                    logger.warning("failed to get bypass handle: %s", ex)
                    last_log = time.time()
                await asyncio.sleep(0.1)

    def _do_bypass_meta(self, meta: HybridMetadata) -> None:
        self._backend.bypass_bind(meta.reqs)
        self._backend.bypass_clear()
        if self._backend.async_load_kv is not None:
            spawn_task(self._async_load_kv(meta))

    @kill_me_if_exception
    async def start_bypass_task_loop(self):
        import zmq
        import zmq.asyncio

        addr = await self._get_bypass_handle()
        if not addr:
            return
        self._bypass_ctx = zmq.asyncio.Context()      # kept: see the publisher's note on teardown
        sock = self._bypass_ctx.socket(zmq.SUB)
        sock.setsockopt(zmq.LINGER, 0)
        sock.setsockopt_string(zmq.SUBSCRIBE, "")
        sock.connect(addr)
        while True:
            meta = pickle.loads(await sock.recv())
            assert isinstance(meta, HybridMetadata)
            self._do_bypass_meta(meta)

    # ---- model-runner thread ---------------------------------------------------------------------
    def bind_connector_metadata(self, meta: HybridMetadata) -> None:
        self._meta = meta
        self._backend.bind_backend_metadata(meta.reqs)

    def has_connector_metadata(self) -> bool:
        return self._meta is not None

    def clear_connector_metadata(self) -> None:
        self._backend.clear_backend_metadata()
        self._meta = None

    def wants_nan_flag(self) -> bool:
        """Whether the model runner should hand this step's ``isnan(hidden_states).any()`` tensor to
        ``set_nan_flag`` before it clears the metadata (v6d_object_backend.py:78-90)."""
        return self._meta is not None and self._meta.reqs.wants_nan_flag()

    def set_nan_flag(self, flag) -> None:
        if self._meta is not None:
            self._meta.reqs.set_nan_flag(flag)

    def register_kv_caches(self, kv_caches: dict) -> None:
        if self._kv_cache_config is not None and self._kv_cache_config.kv_cache_groups:
            self._num_layers = sum(len(g.layer_names) for g in self._kv_cache_config.kv_cache_groups)
            assert self._num_layers == len(kv_caches), \
                f"num_layers mismatch. expected {self._num_layers}, got {len(kv_caches)}"
        else:
            self._num_layers = len(kv_caches)
        logger.info("Registering kv_caches, num_layers=%s", self._num_layers)
        return self._backend.register_kv_caches(kv_caches)

    def start_load_kv(self, **kwargs) -> None:
        if self._backend.async_load_kv is None or self._meta is None:
            return
        asyncio.run_coroutine_threadsafe(self._async_load_kv(self._meta), self.loop)

    def save_kv_layer(self, layer_name: str, kv_layer, **kwargs) -> None:
        if self._meta is None:
            return
        gen = self._backend.async_save_kv_layer(layer_name, kv_layer, self._meta.reqs)
        if gen is None:
            return
        asyncio.run_coroutine_threadsafe(self._async_save_layer(layer_name, gen), self.loop)

    # ---- disaggw thread ----------------------------------------------------------------------------
    async def io_done_rpc(self, req: IoDoneReqs, head: int, reshead: int) -> None:
        body = self._ioenc.encode(req)
        msg = struct.pack("=II", head, len(body)) + body
        for attempt in range(2):
            writer = None
            try:
                reader, writer = await self._connpool._acquire(force_new=attempt > 0)
                writer.write(msg)
                await writer.drain()
                (resphead,) = struct.unpack("=I", await reader.readexactly(4))
                assert resphead == reshead
                self._connpool._release((reader, writer))
                return
            except (asyncio.IncompleteReadError, ConnectionError, OSError):
                if writer is not None:
                    writer.close()
                if attempt == 0:
                    continue
                if self.closing:
                    # the engine is shutting down and its scheduler no longer listens: the report has nobody to go to
                    logger.info("io done report dropped at shutdown: %s", req)
                    return
                raise

    @kill_me_if_exception
    async def _async_load_kv(self, m: HybridMetadata):
        tprank = self._wp.get_tensor_model_parallel_rank()
        async for ioret in self._backend.async_load_kv(m.reqs):
            await self.io_done_rpc(IoDoneReqs(worker_tprank=tprank, reqids=[ioret]), LOAD_DONE_REQ, LOAD_DONE_RESP)

    async def _on_req_saved(self, reqid: str, layer_name: str, source: str) -> None:
        state = self._saving.setdefault(reqid, _WSavingReq())
        state._ready_layers.append(layer_name)
        assert self._num_layers is not None
        if len(state._ready_layers) != self._num_layers:
            return
        tprank = self._wp.get_tensor_model_parallel_rank()
        await self.io_done_rpc(IoDoneReqs(worker_tprank=tprank, reqids=[IoRet(reqid=reqid, source=source)]),
                               SAVE_DONE_REQ, SAVE_DONE_RESP)
        self._saving.pop(reqid)

    @kill_me_if_exception
    async def _async_save_layer(self, layer_name: str, gen: AsyncGenerator):
        source = self._backend.save_done_source()
        assert source is not None, "async save producer must declare save_done_source"
        async for reqid in gen:
            await self._on_req_saved(reqid, layer_name, source)
