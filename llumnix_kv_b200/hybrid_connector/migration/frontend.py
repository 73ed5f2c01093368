"""A migration-aware frontend for demos and tests.

It plays the part of the API server plus a trivial global scheduler
(blade_kvt/hybrid_connector/migration/frontend.py:65-309): requests are handed round-robin to
engines over NEW_REQ, outputs come back on this frontend's own NEW_OUTPUT server whichever
engine produced them, and, when ``migrate_after_first_token`` is set, every request is
deliberately moved to the next engine as soon as its first token has arrived, which exercises
the whole migration path on every request.
"""
from __future__ import annotations

import asyncio
import logging
import struct
import threading
from typing import Optional

import msgspec

from llumnix_kv_b200 import envs

from ..engine_proxy import EngineCoreRequest, core_update_params
from ..kvtbackend import CODE_OK
from ..utils import ConnManager, RpcServer, spawn_task, start_asyncio_thread
from . import (ABORT_REQS_REQ, ABORT_REQS_RESP, MIGRATE_TO_REQ, MIGRATE_TO_RESP, NEW_OUTPUT_REQ, NEW_OUTPUT_RESP,
               NEW_REQ_REQ, NEW_REQ_RESP, OUTPUT_TOKENS_N, SRC_INFO, EngineCoreOutputs, MigrateResp, int2ipport,
               ipport2int)
from .backend import pack_msg, read_body

logger = logging.getLogger("llumnix_kv_b200.hybrid_connector")


class _ReqState:
    def __init__(self, req: EngineCoreRequest, engine: tuple):
        self.req = req
        self.engine = engine            # (addr, port) of the engine it runs on now
        self.tokens: list = []
        self.finish_reason: Optional[int] = None
        self.migrations = 0
        self.engines_seen: list = [engine]
        self.done = threading.Event()


class MigrationCli:
    def __init__(self, engines: list, migrate_after_first_token: bool = False, name: str = "migfront"):
        assert engines, "at least one engine address"
        self.engines = [tuple(e) for e in engines]
        self.migrate_after_first_token = migrate_after_first_token
        self.loop = start_asyncio_thread(name)
        self.server = RpcServer(0, name)
        self.server.register_method(NEW_OUTPUT_REQ, self._on_new_output)
        self.server.start(self.loop)
        self.client_index = ipport2int(envs.get_ip(), self.server.port())
        self._conns = ConnManager(64)
        self._reqs: dict[str, _ReqState] = {}
        self._rr = 0
        self._outdec = msgspec.msgpack.Decoder(EngineCoreOutputs)
        self._migdec = msgspec.msgpack.Decoder(MigrateResp)
        self.rejected = 0

    # ---- public (any thread) -----------------------------------------------------------------------
    def add_request(self, req: EngineCoreRequest, engine: Optional[tuple] = None) -> None:
        if engine is None:
            engine = self.engines[self._rr % len(self.engines)]
            self._rr += 1
        req.client_index = self.client_index
        self._reqs[req.request_id] = _ReqState(req, tuple(engine))
        asyncio.run_coroutine_threadsafe(self._simple_rpc(tuple(engine), pack_msg(NEW_REQ_REQ, req), NEW_REQ_RESP),
                                         self.loop).result(30)

    def abort(self, reqid: str) -> None:
        st = self._reqs[reqid]
        asyncio.run_coroutine_threadsafe(self._simple_rpc(st.engine, pack_msg(ABORT_REQS_REQ, [reqid]), ABORT_REQS_RESP),
                                         self.loop).result(30)

    def migrate(self, reqid: str, dst: tuple) -> int:
        """Ask ``dst`` to take the request over from the engine it runs on; returns the response code."""
        return asyncio.run_coroutine_threadsafe(self._migrate(reqid, tuple(dst)), self.loop).result(60)

    def wait(self, reqid: str, timeout: float = 60.0) -> Optional[_ReqState]:
        st = self._reqs[reqid]
        return st if st.done.wait(timeout) else None

    def close(self) -> None:
        self.server.close(self.loop)

    # ---- frontend loop ----------------------------------------------------------------------------
    async def _simple_rpc(self, peer: tuple, msg: bytes, want_head: int) -> None:
        conn = await self._conns.acquire_conn(peer, False)
        conn[1].write(msg)
        await conn[1].drain()
        (head,) = struct.unpack("=I", await conn[0].readexactly(4))
        if head != want_head:
            raise RuntimeError(f"invalid response head={head}")
        self._conns.release_conn(peer, conn)

    async def _migrate(self, reqid: str, dst: tuple) -> int:
        st = self._reqs[reqid]
        if st.done.is_set() or dst == st.engine:
            return -1
        req = st.req
        core_update_params(req, {SRC_INFO: st.engine, OUTPUT_TOKENS_N: len(st.tokens), "ali_llumnix_disagg": False})
        conn = await self._conns.acquire_conn(dst, False)
        conn[1].write(pack_msg(MIGRATE_TO_REQ, req))
        await conn[1].drain()
        head, n = struct.unpack("=II", await conn[0].readexactly(8))
        if head != MIGRATE_TO_RESP:
            raise RuntimeError(f"invalid response head={head}")
        resp: MigrateResp = self._migdec.decode(await conn[0].readexactly(n))
        self._conns.release_conn(dst, conn)
        if resp.code == CODE_OK:
            st.engine = dst
            st.engines_seen.append(dst)
            st.migrations += 1
        else:
            self.rejected += 1
        return resp.code

    async def _on_new_output(self, reader, writer):
        outs: EngineCoreOutputs = self._outdec.decode(await read_body(reader))
        writer.write(struct.pack("=I", NEW_OUTPUT_RESP))
        src = int2ipport(outs.engine_index)
        for o in outs.outputs:
            st = self._reqs.get(o.request_id)
            if st is None:
                continue
            first = not st.tokens and bool(o.new_token_ids)
            st.tokens.extend(o.new_token_ids)
            if (src[0], src[1]) in self.engines:
                st.engine = (src[0], src[1])       # where it really runs: an accepted migration may yet be declined by the source
            if o.finish_reason is not None:
                st.finish_reason = o.finish_reason
                st.done.set()
            elif first and self.migrate_after_first_token and len(self.engines) > 1 and st.migrations == 0:
                here = (src[0], src[1])
                idx = self.engines.index(here) if here in self.engines else 0
                spawn_task(self._migrate(o.request_id, self.engines[(idx + 1) % len(self.engines)]))
        await writer.drain()


_g_is_frontend = False


def i_am_frontend() -> None:
    """Marks this process as the API-server side (blade_kvt/hybrid_connector/migration/frontend.py:314-321):
    code shared with the engines asks ``is_frontend()`` before it touches engine-only state."""
    global _g_is_frontend
    _g_is_frontend = True


def is_frontend() -> bool:
    return _g_is_frontend
