""""migration" backend: move a live request from one engine to another.

Roles in one migration (blade_kvt/hybrid_connector/migration/backend.py:232-372, 598-759):

  frontend / global scheduler   sends MIGRATE_TO (the request + where it runs now + how many
                                output tokens it had) to the *destination* engine
  destination                   admission control, then adds the request with a load from the
                                "migration" source; its load is ``_kvt_suspend``: if the request
                                had produced nothing yet, SUSPEND the source and prefill here;
                                otherwise KVT_SUSPEND: the source pushes all computed KV into
                                the blocks reserved here, then suspends, and answers with the
                                output tokens produced so far
  source                        ``do_suspend``: abort the request silently, wait until the engine
                                has really let go of it, report its output tokens

Engines also forward the outputs of requests that came from a migration-aware frontend to that
frontend's output server (NEW_OUTPUT), whichever engine the request ends up on.
"""
from __future__ import annotations

import asyncio
import logging
import struct
import threading
import time
from typing import Optional

import msgspec

from llumnix_kv_b200 import envs

from ..backend import PREALLOC_KEY, BackendMeta, HybridBackend, OperationPlan
from ..engine_proxy import (EngineCoreRequest, KVCacheBlocks, KVConnectorRole, Request, RequestStatus,
                            SchedulerOutput, VllmConfig, core_get_param, core_update_params, get_param, set_param)
from ..kvtbackend import (CODE_MIGRATE_REJECTED_BUSY, CODE_OK, CODE_REQNOTFOUND, TRANSFER_KV_RESP, KVTDInfo, KVTResp,
                          RKVTDInfo, get_inst_id)
from ..utils import ConnManager, ConnPool, DeclinedError, IoRet, kill_me_if_exception, spawn_task
from . import (ABORT_REQS_REQ, ABORT_REQS_RESP, KVT_SUSPEND_REQ, MIGRATE_TO_REQ, MIGRATE_TO_RESP, NEW_OUTPUT_REQ,
               NEW_OUTPUT_RESP, NEW_REQ_REQ, NEW_REQ_RESP, OUTPUT_TOKENS_N, SRC_INFO, SUSPEND_EVT, SUSPEND_REQ,
               SUSPEND_RESP, EngineCoreOutputs, MigrateResp, SuspendReq, SuspendResp, WireOutput, int2ipport,
               ipport2int, is_migration)

logger = logging.getLogger("llumnix_kv_b200.hybrid_connector")

_enc = msgspec.msgpack.Encoder()


def pack_msg(head: int, obj) -> bytes:
    body = _enc.encode(obj)
    return struct.pack("=II", head, len(body)) + body


async def read_body(reader) -> bytes:
    (n,) = struct.unpack("=I", await reader.readexactly(4))
    return await reader.readexactly(n)


class MigrationBackend(HybridBackend):
    SOURCE_LABEL = "migration"

    def __init__(self, vllm_config: VllmConfig, role: KVConnectorRole, kv_cache_config=None, dbackend=None, **kw):
        super().__init__(vllm_config, role, kv_cache_config, **kw)
        if role == KVConnectorRole.WORKER:
            return
        self._cfg = vllm_config
        self._loop = self._engine.get_hybrid_sched_loop()
        fake = vllm_config.kv_transfer_config.get_from_extra_config("naming_url", "fake://") == "fake://"
        self._inst_id = get_inst_id(vllm_config, fake_naming=fake)
        self._dbackend = dbackend            # decode half of a kvt+migration engine: knows this engine's WorkerInfo
        self._conn_mgr = ConnManager(envs.VLLM_PD_CONNMANAGER_CAP)
        srv = self._engine.sched_rpc_server()
        srv.register_method(ABORT_REQS_REQ, self._on_abort_reqs)
        srv.register_method(NEW_REQ_REQ, self._on_new_req)
        srv.register_method(MIGRATE_TO_REQ, self._on_migrate_to)
        srv.register_method(SUSPEND_REQ, self._on_suspend)
        self._engidx = ipport2int(envs.get_ip(), srv.port())
        assert is_migration(self._engidx)
        self._reqstate: dict[str, Request] = {}          # written by the core thread, read by the disagg thread
        self._front_outputs: dict[int, asyncio.Queue] = {}   # disagg thread
        self._reqdec = msgspec.msgpack.Decoder(EngineCoreRequest)
        self._susreqdec = msgspec.msgpack.Decoder(SuspendReq)
        self._susrespdec = msgspec.msgpack.Decoder(SuspendResp)
        self._kvtrespdec = msgspec.msgpack.Decoder(KVTResp)
        self._dec = msgspec.msgpack.Decoder()
        # admission control of incoming migrations
        self._mig_lock = threading.Lock()
        self._mig_in: dict[str, int] = {}                # reqid -> tokens it will occupy
        self._mig_out: set = set()
        self._arriving: set = set()                      # accepted over RPC, not yet seen by the core thread
        total_tokens = vllm_config.cache_config.num_gpu_blocks * vllm_config.cache_config.block_size
        ratio = float(vllm_config.kv_transfer_config.get_from_extra_config("max_block_ratio_mig_in", 1.0))
        self.max_migrate_in_tokens = min(envs.LLUMNIX_MAX_TOKEN_MIG_IN, int(total_tokens * ratio))

    # ---- source side ----------------------------------------------------------------------------------
    async def do_suspend(self, susreq: SuspendReq) -> SuspendResp:
        req = self._reqstate.get(susreq.reqid)
        if req is None:
            logger.info("suspend: already finished. reqid=%s", susreq.reqid)
            return SuspendResp(code=CODE_REQNOTFOUND)
        if get_param(req, SUSPEND_EVT) is not None:
            # someone else is already taking this request over: the second asker is told so and keeps its hands off
            logger.warning("suspend: already being suspended. reqid=%s", susreq.reqid)
            return SuspendResp(code=CODE_MIGRATE_REJECTED_BUSY)
        evt = asyncio.Event()
        set_param(req, SUSPEND_EVT, evt)
        self._mig_out.add(susreq.reqid)
        self._engine.core_abort_req(susreq.reqid, "migration.suspend", False)   # silent: no output to the client
        if self._reqstate.get(susreq.reqid) is None:
            evt.set()       # it finished between the lookup and the abort
        await evt.wait()
        self._mig_out.discard(susreq.reqid)
        # a request that ended by itself in the meantime has nothing left to migrate
        stopped = req.status in (RequestStatus.FINISHED_STOPPED, RequestStatus.FINISHED_LENGTH)
        logger.info("suspend end: reqid=%s stopped=%s outputs=%s", req.request_id, stopped, len(req.output_token_ids))
        if stopped:
            return SuspendResp(code=CODE_REQNOTFOUND)
        return SuspendResp(code=CODE_OK, output_token_ids=list(req.output_token_ids))

    async def _on_suspend(self, reader, writer):
        susreq = self._susreqdec.decode(await read_body(reader))
        writer.write(pack_msg(SUSPEND_RESP, await self.do_suspend(susreq)))
        await writer.drain()

    # core thread
    def _finish_req(self, reqid: str) -> None:
        req = self._reqstate.pop(reqid, None)
        if req is None:
            return
        evt: Optional[asyncio.Event] = get_param(req, SUSPEND_EVT)
        if evt is not None:
            self._loop.call_soon_threadsafe(evt.set)

    # ---- destination side ---------------------------------------------------------------------------------
    def _has_migrate_in_slots(self, req: EngineCoreRequest, prealloc: int) -> bool:
        with self._mig_lock:
            if len(self._mig_in) >= envs.LLUMNIX_MAX_REQ_MIG_IN:
                return False
            if envs.LLUMNIX_DETAILED_MIG_STATUS:
                if sum(self._mig_in.values()) + len(req.prompt_token_ids) + prealloc > self.max_migrate_in_tokens:
                    return False
        return True

    def migration_status(self) -> dict:
        with self._mig_lock:
            return {"migrate_in": dict(self._mig_in), "migrate_out": sorted(self._mig_out)}

    async def _on_migrate_to(self, reader, writer):
        req: EngineCoreRequest = self._reqdec.decode(await read_body(reader))
        prealloc = core_get_param(req, OUTPUT_TOKENS_N, 0)
        if not self._has_migrate_in_slots(req, prealloc):
            logger.warning("migrate_to rejected, no room: reqid=%s", req.request_id)
            writer.write(pack_msg(MIGRATE_TO_RESP, MigrateResp(code=CODE_MIGRATE_REJECTED_BUSY)))
            await writer.drain()
            return
        with self._mig_lock:
            known = req.request_id in self._mig_in or req.request_id in self._arriving
        if known or req.request_id in self._reqstate:
            # the request was here a moment ago (it is still being let go, or its end has not been booked yet) or is
            # already on its way in: taking it now would run two lives of one id side by side
            logger.warning("migrate_to rejected, the request is still known here: reqid=%s", req.request_id)
            writer.write(pack_msg(MIGRATE_TO_RESP, MigrateResp(code=CODE_MIGRATE_REJECTED_BUSY)))
            await writer.drain()
            return
        srcinfo = core_get_param(req, SRC_INFO)
        assert srcinfo is not None, "MIGRATE_TO without the source engine's address"
        core_update_params(req, {SRC_INFO: tuple(srcinfo), PREALLOC_KEY: prealloc,
                                 "migration_start_time": time.monotonic()})
        with self._mig_lock:
            self._mig_in[req.request_id] = len(req.prompt_token_ids) + prealloc
            self._arriving.add(req.request_id)
        writer.write(pack_msg(MIGRATE_TO_RESP, MigrateResp(code=CODE_OK)))
        self._engine.core_add_req(req)
        logger.info("migrate in. reqid=%s prealloc=%s src=%s", req.request_id, prealloc, srcinfo)
        await writer.drain()

    async def _on_abort_reqs(self, reader, writer):
        reqs = self._dec.decode(await read_body(reader))
        writer.write(struct.pack("=I", ABORT_REQS_RESP))
        for rid in reqs:
            self._engine.core_abort_req(rid, "migration.abort_req", True)
        await writer.drain()

    async def _on_new_req(self, reader, writer):
        req: EngineCoreRequest = self._reqdec.decode(await read_body(reader))
        writer.write(struct.pack("=I", NEW_REQ_RESP))
        with self._mig_lock:
            self._arriving.add(req.request_id)     # known from now on, although the core thread has yet to book it
        self._engine.core_add_req(req)
        await writer.drain()

    async def _peer_rpc(self, peer: tuple, msg: bytes, want_head: int, dec):
        for attempt in range(2):
            try:
                conn = await self._conn_mgr.acquire_conn(peer, attempt > 0)
                conn[1].write(msg)
                await conn[1].drain()
                head, n = struct.unpack("=II", await conn[0].readexactly(8))
                if head != want_head:
                    raise RuntimeError(f"invalid response head={head:#x}")
                resp = dec.decode(await conn[0].readexactly(n))
                self._conn_mgr.release_conn(peer, conn)
                return resp
            except (asyncio.IncompleteReadError, ConnectionError):
                logger.warning("migration rpc to %s failed (attempt %d)", peer, attempt)
            await asyncio.sleep(0)
        raise RuntimeError(f"migration rpc to {peer} failed")

    async def _kvt_suspend(self, srcinfo: tuple, req: Request, blocks: KVCacheBlocks) -> KVTResp:
        blockids = blocks.get_block_ids()
        bs = self._cfg.cache_config.block_size
        n_out = get_param(req, OUTPUT_TOKENS_N, 0)
        alltokens = n_out + len(req.prompt_token_ids)
        # the attention group (the longest one; hybrid models put their one-block state groups first) must hold it all
        assert max(len(g) for g in blockids) * bs >= alltokens
        t0 = time.monotonic()
        if n_out == 0:
            # still waiting (or prefilling) on the source: nothing worth moving, just take it over
            sus: SuspendResp = await self._peer_rpc(srcinfo, pack_msg(SUSPEND_REQ, SuspendReq(reqid=req.request_id)),
                                                    SUSPEND_RESP, self._susrespdec)
            resp = KVTResp(code=sus.code, cached=req.num_computed_tokens, computed=-1,
                           output_token_ids=sus.output_token_ids)
        else:
            pc = self._cfg.parallel_config
            winfos = list(self._dbackend._workers_info) if self._dbackend is not None else []
            dinfo = KVTDInfo(instid=f"{self._inst_id}|{pc.data_parallel_rank}|{pc.tensor_parallel_size}",
                             blkids=blockids, cached_tokens=req.num_computed_tokens, max_tokens=alltokens,
                             d_workers_info=winfos)
            self._engine.sched_discard_zero_block_ids(b for g in blockids for b in g)
            resp = await self._peer_rpc(srcinfo, pack_msg(KVT_SUSPEND_REQ, RKVTDInfo(reqid=req.request_id, dinfo=dinfo,
                                                                                   migration=True)),
                                        TRANSFER_KV_RESP, self._kvtrespdec)
        logger.info("migrate end kvt: dur_ms=%.2f reqid=%s cached=%s max=%s resp=%s", (time.monotonic() - t0) * 1000,
                    req.request_id, req.num_computed_tokens, alltokens, resp)
        if resp.code != CODE_OK:
            # the source kept the request (it does not know it yet or any more, it is busy letting it go to someone
            # else, or its transfer failed before it let go): nothing changed hands
            raise DeclinedError(f"migration declined by the source: {resp}")
        if resp.output_token_ids is None or not (req.num_computed_tokens <= resp.cached <= alltokens):
            raise RuntimeError(f"migration kvt rpc failed: {resp}")
        return resp

    # ---- scheduler half of the backend contract --------------------------------------------------------------
    def get_operations(self, req: Request) -> OperationPlan:
        assert req.request_id not in self._reqstate
        self._reqstate[req.request_id] = req
        with self._mig_lock:
            self._arriving.discard(req.request_id)
        load = int(get_param(req, SRC_INFO) is not None)
        return load, 0, (self.source_label(),) if load else (), ()

    def build_backend_meta(self, sout: SchedulerOutput) -> BackendMeta:
        for reqid in sout.finished_req_ids:
            self._finish_req(reqid)
        for reqid in list(self._engine.sched_get_finished_req_ids()):
            self._finish_req(reqid)
        return BackendMeta()

    async def async_get_num_new_matched_tokens(self, req: Request, num_computed_tokens: int) -> int:
        return 0

    async def async_update_state_after_alloc(self, req: Request, blocks: KVCacheBlocks,
                                             num_external_tokens: int) -> Optional[IoRet]:
        ioret = IoRet(n=None)
        srcinfo = get_param(req, SRC_INFO)
        try:
            resp = await self._kvt_suspend(tuple(srcinfo), req, blocks)
            for tok in resp.output_token_ids:
                req.append_output_token_ids(tok)
            req.num_computed_tokens = resp.cached
            assert req.num_computed_tokens <= req.num_tokens
            if req.num_computed_tokens >= req.num_tokens:
                # everything arrived: the last token(s) are recomputed here to produce the next one
                gamma = 0
                if self._cfg.speculative_config and self._cfg.speculative_config.num_speculative_tokens:
                    gamma = self._cfg.speculative_config.num_speculative_tokens
                req.num_computed_tokens -= 1 + gamma
            logger.info("migration end. reqid=%s duration_ms=%.2f", req.request_id,
                        (time.monotonic() - get_param(req, "migration_start_time", time.monotonic())) * 1000)
        except Exception as ex:
            logger.warning("migration load failed. reqid=%s src=%s ex=%r", req.request_id, srcinfo, ex)
            ioret.ex = ex
        finally:
            with self._mig_lock:
                self._mig_in.pop(req.request_id, None)
        return ioret

    async_load_kv = None  # type: ignore[assignment]

    # ---- output forwarding to migration-aware frontends --------------------------------------------------------
    async def _new_output_rpc(self, pool: ConnPool, outs: EngineCoreOutputs) -> None:
        msg = pack_msg(NEW_OUTPUT_REQ, outs)
        for attempt in range(2):
            try:
                reader, writer = await pool._acquire(force_new=attempt > 0)
                writer.write(msg)
                await writer.drain()
                (head,) = struct.unpack("=I", await reader.readexactly(4))
                if head != NEW_OUTPUT_RESP:
                    raise RuntimeError(f"invalid response head={head}")
                pool._release((reader, writer))
                return
            except (asyncio.IncompleteReadError, ConnectionError, OSError):
                logger.warning("new_output to frontend failed (attempt %d)", attempt)
            await asyncio.sleep(0)
        logger.error("dropping %d outputs: frontend unreachable", len(outs.outputs))

    @kill_me_if_exception
    async def _front_main(self, front: int, q: asyncio.Queue):
        ip, port = int2ipport(front)
        pool = ConnPool(ip, port, 1)
        while True:
            outs: EngineCoreOutputs = await q.get()
            while not q.empty():            # coalesce what piled up while the last RPC was in flight
                outs.outputs.extend(q.get_nowait().outputs)
            await self._new_output_rpc(pool, outs)

    def _append_q(self, items: list) -> None:   # disagg thread; not a coroutine so that order is kept
        for front, outs in items:
            q = self._front_outputs.get(front)
            if q is None:
                q = self._front_outputs[front] = asyncio.Queue()
                spawn_task(self._front_main(front, q))
            q.put_nowait(outs)

    # core thread: called by the engine with every batch of outputs before it publishes them
    def on_outputs(self, outputs: dict) -> None:
        mig = []
        for cli in [c for c in outputs if is_migration(c)]:
            outs = outputs.pop(cli)
            mig.append((cli, EngineCoreOutputs(engine_index=self._engidx, outputs=[
                WireOutput(o.request_id, list(o.new_token_ids), None if o.finish_reason is None else int(o.finish_reason),
                           o.kv_transfer_params, o.num_cached_tokens) for o in outs])))
        if mig:
            self._loop.call_soon_threadsafe(self._append_q, mig)
