"""Control-plane plumbing: event-loop threads, the head-dispatch RPC server, connection pools,
peer discovery, and the per-request completion bookkeeping shared by save and load paths.

Behaviour follows blade_kvt/hybrid_connector/utils.py (RpcServer :88-146, ConnPool/ConnManager
:152-228, PeerInfo :231-268, PeerManager :271-409, IoRet/IoState/try_advance :412-552,
handle_done_req :561-627).
"""
from __future__ import annotations

import asyncio
import logging
import os
import random
import struct
import sys
import threading
import traceback
from collections import OrderedDict
from dataclasses import dataclass
from typing import Any, Callable, Coroutine, Optional

import msgspec

logger = logging.getLogger("llumnix_kv_b200.hybrid_connector")

# Tests flip this off so that a deliberately failing coroutine raises instead of taking the
# interpreter down.
ABORT_ON_TASK_EXCEPTION = os.environ.get("LLUMNIX_KV_ABORT_ON_TASK_EXCEPTION", "1") != "0"


def kill_me_if_exception(async_func):
    """Every coroutine that is the main of a task wears this: a control-plane bug must not leave
    a request silently stuck, so an unexpected exception ends the process."""

    async def wrapper(*args, **kwargs):
        try:
            loop = asyncio.get_running_loop()
            running = getattr(loop, "_kvx_running_tasks", None)
            if running is None:
                running = set()
                loop._kvx_running_tasks = running  # keeps tasks referenced until done
            task = asyncio.current_task()
            if task is not None:
                running.add(task)
                task.add_done_callback(running.discard)
            return await async_func(*args, **kwargs)
        except asyncio.CancelledError:
            raise
        except Exception:
            logger.exception("task %s failed", getattr(async_func, "__name__", async_func))
            if ABORT_ON_TASK_EXCEPTION:
                # the reason must be readable even where logging goes nowhere
                why = f"aborting: background task {getattr(async_func, '__name__', async_func)} failed\n{traceback.format_exc()}"
                sys.stderr.write(why)
                sys.stderr.flush()
                try:        # stderr may be captured or closed: leave the reason where it can be found afterwards
                    import tempfile
                    with open(os.path.join(tempfile.gettempdir(), f"llumnix_kv_abort.{os.getpid()}.txt"), "w") as f:
                        f.write(why)
                except OSError:
                    pass
                os.abort()
            raise

    wrapper.__name__ = getattr(async_func, "__name__", "wrapped")
    return wrapper


def start_asyncio_thread(name: str, device: Optional[str] = None) -> asyncio.AbstractEventLoop:
    """A daemon thread running its own event loop (uvloop when available)."""
    try:
        import uvloop

        loop = uvloop.new_event_loop()
    except Exception:  # pragma: no cover
        loop = asyncio.new_event_loop()

    def on_ex(_loop, context):
        logger.error("event loop %s exception: %s", name, context)
        if ABORT_ON_TASK_EXCEPTION and context.get("exception") is not None:
            os.abort()

    loop.set_exception_handler(on_ex)

    def main():
        if device is not None and device.startswith("cuda"):
            import torch

            torch.cuda.set_device(torch.device(device))
        asyncio.set_event_loop(loop)
        loop.run_forever()

    threading.Thread(target=main, name=name, daemon=True).start()
    return loop


_background_tasks: set = set()


def spawn_task(coro) -> "asyncio.Task":
    """``asyncio.ensure_future`` that keeps the task alive: the event loop only holds weak
    references to tasks, so a fire-and-forget task can be garbage collected in mid-flight."""
    task = asyncio.ensure_future(coro)
    _background_tasks.add(task)
    task.add_done_callback(_background_tasks.discard)
    return task


# ---- RPC: 4-byte head selects the handler, the handler reads its own body -----------------------
_RpcMethod = Callable[[asyncio.StreamReader, asyncio.StreamWriter], Coroutine[Any, Any, None]]


class RpcServer:
    def __init__(self, port: int, name: str):
        self._name, self._port = name, port
        self._methods: dict[int, _RpcMethod] = {}
        self._started = threading.Event()
        self._server: Optional[asyncio.AbstractServer] = None
        self._clients: set = set()           # writers of the accepted connections (loop thread only)
        self._client_tasks: set = set()      # and the tasks that serve them

    def register_method(self, head: int, cb: _RpcMethod) -> None:
        assert head not in self._methods, f"rpc head {head:#x} registered twice"
        self._methods[head] = cb

    def port(self) -> int:
        return self._port

    def start(self, loop: asyncio.AbstractEventLoop, wait: bool = True) -> None:
        asyncio.run_coroutine_threadsafe(self._main(), loop)
        if wait:
            self._started.wait(30)

    async def _client_main(self, reader, writer):
        self._clients.add(writer)
        me = asyncio.current_task()
        self._client_tasks.add(me)
        try:
            await self._serve_client(reader, writer)
        finally:
            self._client_tasks.discard(me)

    async def _serve_client(self, reader, writer):
        try:
            while True:
                (head,) = struct.unpack("=I", await reader.readexactly(4))
                cb = self._methods.get(head)
                if cb is None:
                    logger.warning("%s: rpc unknown head=%#x", self._name, head)
                    break
                await cb(reader, writer)
        except asyncio.IncompleteReadError as ex:
            if ex.partial:
                logger.warning("%s: connection closed mid-message", self._name)
        except (ConnectionResetError, BrokenPipeError):
            pass
        except Exception:
            # whatever a peer sent, or whatever broke while answering it, costs that peer its connection and
            # nothing else (blade_kvt/hybrid_connector/utils.py:109-137 logs and closes likewise)
            logger.exception("%s: rpc handler failed", self._name)
        self._clients.discard(writer)
        try:
            writer.close()
            await writer.wait_closed()
        except Exception:
            pass

    async def _main(self):
        self._task = asyncio.current_task()
        self._server = await asyncio.start_server(self._client_main, "0.0.0.0", self._port)
        if self._port == 0:
            self._port = self._server.sockets[0].getsockname()[1]
        logger.info("%s RPC server on port %s", self._name, self._port)
        self._started.set()
        async with self._server:
            await self._server.serve_forever()

    def close(self, loop: asyncio.AbstractEventLoop) -> None:
        """Stops listening and hangs up on every peer: one that waits for an answer sees the connection end, as it
        would when this process died, instead of waiting for a handler that will never finish."""
        def hang_up():
            if self._server is not None:
                self._server.close()
            task = getattr(self, "_task", None)
            if task is not None and not task.done():
                task.cancel()          # serve_forever would otherwise stay pending until the interpreter exits
            for w in list(self._clients):
                try:
                    w.close()
                except Exception:
                    pass
            self._clients.clear()
            for t in list(self._client_tasks):
                t.cancel()         # a handler may be waiting for something that will never come now

        loop.call_soon_threadsafe(hang_up)


Conn = tuple


class ConnPool:
    def __init__(self, host: str, port: int, max_conn: int):
        self._host, self._port, self._max = host, port, max_conn
        self._conns: list = []

    async def _acquire(self, force_new: bool = False):
        if not force_new and self._conns:
            return self._conns.pop()
        return await asyncio.open_connection(self._host, self._port)

    def _release(self, conn) -> None:
        if len(self._conns) >= self._max:
            if not conn[1].is_closing():
                conn[1].close()
            return
        self._conns.append(conn)

    acquire = _acquire
    release = _release

    def host(self):
        return self._host

    def port(self):
        return self._port

    def close(self):
        for _, w in self._conns:
            if not w.is_closing():
                w.close()
        self._conns.clear()


class ConnManager:
    """LRU of connection pools keyed by (addr, port)."""

    def __init__(self, capacity: int = 512):
        self._cap = capacity
        self._pools: "OrderedDict[tuple, ConnPool]" = OrderedDict()

    async def acquire_conn(self, addr_port: tuple, force_new: bool = False):
        pool = self._pools.get(addr_port)
        if pool is None:
            pool = ConnPool(addr_port[0], addr_port[1], 3)
            self._pools[addr_port] = pool
            while len(self._pools) > self._cap:
                _, old = self._pools.popitem(last=False)
                old.close()
        else:
            self._pools.move_to_end(addr_port)
        return await pool._acquire(force_new)

    def release_conn(self, addr_port: tuple, conn) -> None:
        pool = self._pools.get(addr_port)
        if pool is not None:
            pool._release(conn)

    def pop(self, addr_port, default=None):
        pool = self._pools.pop(addr_port, default)
        if isinstance(pool, ConnPool):
            pool.close()
        return pool


@dataclass
class PeerInfo:
    """``role:tpsize:ctime_us:addr:port:dprank`` as published under ``endpoint{dprank}``."""

    role: str = ""
    tpsize: int = -1
    ctime_us: int = -1
    addr: str = ""
    port: int = 33000
    dprank: int = 0

    def serialize(self) -> str:
        return f"{self.role}:{self.tpsize}:{self.ctime_us}:{self.addr}:{self.port}:{self.dprank}"

    @classmethod
    def deserialize(cls, data: str) -> "PeerInfo":
        p = data.split(":")
        if len(p) != 6:
            raise ValueError(f"PeerInfo.deserialize: BadVal={data}")
        return cls(role=p[0], tpsize=int(p[1]), ctime_us=int(p[2]), addr=p[3], port=int(p[4]), dprank=int(p[5]))


class PeerMap:
    def __init__(self):
        self._addr2id: dict = {}
        self._id2info: dict = {}

    def __bool__(self):
        return bool(self._id2info)

    def __setitem__(self, peerid: str, peer: PeerInfo):
        old = self._id2info.pop(peerid, None)
        if old is not None:
            self._addr2id.pop((old.addr, old.port), None)
        self._addr2id[(peer.addr, peer.port)] = peerid
        self._id2info[peerid] = peer

    def __getitem__(self, peerid: str) -> PeerInfo:
        return self._id2info[peerid]

    def get_peerid(self, addr: tuple) -> Optional[str]:
        return self._addr2id.get(addr)

    def items(self):
        return self._id2info.items()

    def keys(self, exclude: Optional[tuple] = None) -> list:
        if exclude is None:
            return list(self._id2info)
        return [i for i, p in self._id2info.items() if (p.addr, p.port) != tuple(exclude)]

    def pop(self, peerid: str, default=None):
        info = self._id2info.pop(peerid, default)
        if info is not None:
            self._addr2id.pop((info.addr, info.port), None)
        return info

    def update(self, infos: dict) -> None:
        for k, v in infos.items():
            self[k] = v


def get_peer_id(inst_id: str, dp_rank: int, tp_size: int) -> str:
    return f"{inst_id}|{dp_rank}|{tp_size}"


class PeerManager:
    """Polls the naming service, notices peers that left or restarted (``ctime_us`` changed) and
    drops their pooled connections; hands out a random live peer."""

    POLL_S = 7.0

    def __init__(self, naming_cli, interested_role: Optional[str], conn_mgr: ConnManager):
        self._naming, self._role, self._conn_mgr = naming_cli, interested_role, conn_mgr
        self._running = PeerMap()

    def _list_instance(self) -> list:
        out = []
        for inst in self._naming.list():
            for ep in self._naming.search(inst, "endpoint"):
                info = PeerInfo.deserialize(ep)
                if self._role is not None and info.role != self._role:
                    break
                out.append((get_peer_id(inst, info.dprank, info.tpsize), info))
        return out

    async def refresh(self) -> None:
        """One poll of the naming service.  A peer is identified by (instance, dp rank, tp size) and versioned by
        its creation time: a peer that disappeared, or came back with another creation time, loses its pooled
        connections before anybody is handed its address again."""
        seen = dict(self._list_instance())
        known = dict(self._running.items())
        departed = known.keys() - seen.keys()
        restarted = {pid for pid in known.keys() & seen.keys() if known[pid].ctime_us != seen[pid].ctime_us}
        arrived = seen.keys() - known.keys()
        for pid in departed | restarted:
            old = known[pid]
            self._conn_mgr.pop((old.addr, old.port), None)
            if pid in departed:
                self._running.pop(pid)
                logger.info("peer left: %s", old)
            else:
                self._running[pid] = seen[pid]
                logger.info("peer restarted: %s -> %s", old, seen[pid])
        if arrived:
            self._running.update({pid: seen[pid] for pid in arrived})
            logger.info("peers arrived: %s", {pid: seen[pid] for pid in arrived})

    @kill_me_if_exception
    async def _main(self):
        while True:
            try:
                await self.refresh()
            except Exception:
                logger.exception("PeerManager refresh failed")
            await asyncio.sleep(self.POLL_S)

    def start(self, loop) -> None:
        asyncio.run_coroutine_threadsafe(self._main(), loop)

    def get_peer(self, exclude: Optional[tuple] = None) -> Optional[tuple]:
        peers = self._running.keys(exclude)
        if not peers:
            return None
        info = self._running[random.choice(peers)]
        return (info.addr, info.port)


# ---- completion bookkeeping -----------------------------------------------------------------------
class IoRet(msgspec.Struct, array_like=True, omit_defaults=True, gc=False):
    """Outcome of one I/O on one worker: request id, failure, tokens moved, which backend."""

    reqid: Optional[str] = None
    ex: Optional[Any] = None      # exceptions never cross the wire: only in-process producers set it
    n: Optional[int] = None
    source: Optional[str] = None


class IoState:
    """Completion ledger of one request across the TP ranks of an instance.

    Every rank owes a quota of completion signals: one per name in ``expected_sources`` when the
    request is served by several backends at once, else ``signals_per_worker`` anonymous ones.  The
    ledger is kept incrementally: each accepted signal updates the rank's tally, the per-source
    tallies and a running summary (first failure, smallest token count), so completion and the
    summary are O(1) to read however many ranks report.  Same contract as the reference's
    per-request state (blade_kvt/hybrid_connector/utils.py: IoState / try_advance)."""

    def __init__(self, signals_per_worker: int = 1):
        self.signals_per_worker = signals_per_worker
        self.expected_sources: tuple = ()
        self.lock = threading.Lock()
        self._got: dict[int, set | int] = {}        # rank -> names seen (named mode) or count (anonymous mode)
        self._full_ranks = 0
        self._src_ranks: dict[str, int] = {}         # source -> ranks that reported it
        self._src_zero: set[str] = set()             # sources with a signal that moved nothing
        self._head: Optional[IoRet] = None           # first accepted signal: names the request in the summary
        self._failure: Optional[Any] = None
        self._fewest: Optional[int] = None
        self._uncounted = False                      # some signal carried no token count

    # -- writing (callers hold ``lock``) ----------------------------------------------------------
    def accept(self, rank: int, sig: IoRet) -> Optional[str]:
        """Books one signal; returns why it was refused, or None when it counted."""
        names = tuple(self.expected_sources or ())
        if names:
            if sig.source not in names:
                return "source not expected"
            seen = self._got.setdefault(rank, set())
            if sig.source in seen:
                return "source already reported by this rank"
            seen.add(sig.source)
            if len(seen) == len(names):
                self._full_ranks += 1
        else:
            have = self._got.get(rank, 0)
            if have >= self.signals_per_worker:
                return "rank already reported its quota"
            self._got[rank] = have + 1
            if have + 1 == self.signals_per_worker:
                self._full_ranks += 1
        if sig.source is not None:
            self._src_ranks[sig.source] = self._src_ranks.get(sig.source, 0) + 1
            if sig.n == 0:
                self._src_zero.add(sig.source)
        if self._head is None:
            self._head = sig
        if sig.ex is not None and self._failure is None:
            self._failure = sig.ex
        if sig.n is None:
            self._uncounted = True
        elif self._fewest is None or sig.n < self._fewest:
            self._fewest = sig.n
        return None

    # -- reading ------------------------------------------------------------------------------------
    def full_ranks(self) -> int:
        return self._full_ranks

    def ranks_reporting(self, source: str) -> int:
        return self._src_ranks.get(source, 0)

    def source_moved_nothing(self, source: str) -> bool:
        return source in self._src_zero

    def merge(self) -> IoRet:
        """The request's outcome: the first failure any rank reported; the token count every rank
        reached (the smallest), unknown as soon as one rank gave none."""
        assert self._head is not None, "no signal was accepted"
        return IoRet(reqid=self._head.reqid, ex=self._failure, n=None if self._uncounted else self._fewest,
                     source=self._head.source)


def try_advance(state_dict: dict, ioret: IoRet, worker_tprank: int, tpsize: int,
                on_signal_advanced: Optional[Callable[[Any, IoRet], None]] = None):
    """Books one completion signal in its request's ledger; returns the ledger when this signal
    completed the request (every one of ``tpsize`` ranks has met its quota), else None.
    ``on_signal_advanced(state, ioret)`` runs under the ledger's lock after an accepted signal."""
    assert ioret.reqid is not None
    state: Optional[IoState] = state_dict.get(ioret.reqid)
    if state is None:
        logger.warning("completion signal for a request that is not tracked: %s (rank %s)", ioret, worker_tprank)
        return None
    with state.lock:
        refused = state.accept(worker_tprank, ioret)
        if refused is not None:
            logger.warning("completion signal ignored (%s): %s (rank %s)", refused, ioret, worker_tprank)
            return None
        if on_signal_advanced is not None:
            on_signal_advanced(state, ioret)
        return state if state.full_ranks() >= tpsize else None


class DeclinedError(RuntimeError):
    """A load that the other side declined before anything changed hands: the request still lives (or has
    ended) where it was, so the copy that asked for it goes away without a word to the client.  The scheduler
    reads ``silent`` off a failed load's exception."""

    silent = True


class CodeError(Exception):
    def __init__(self, code: int, msg: str):
        super().__init__(f"{code}: {msg}")
        self.code, self.msg = code, msg


async def handle_done_req(reader, writer, cb: Callable[[int, IoRet], Any], respcode: int) -> None:
    """Parse the native engine's send-done body (the head has been consumed).

    ``worker_tp | flags : u32, n : u32`` then, version 2 (flag 0x40000000), per request
    ``plen, code, rlen : u32`` + reqid; version 1 is ``len, reqid`` per request followed, with
    flag 0x80000000, by one ``plen`` per request.
    """
    HAS_VER2, HAS_PLEN = 0x40000000, 0x80000000
    tprank, n = struct.unpack("=II", await reader.readexactly(8))
    ver2, has_plen = tprank & HAS_VER2, tprank & HAS_PLEN
    tprank &= 0xFFFF
    rets: list = []
    if ver2:
        for _ in range(n):
            plen, code, rlen = struct.unpack("=III", await reader.readexactly(12))
            reqid = (await reader.readexactly(rlen)).decode("utf-8")
            rets.append(IoRet(reqid=reqid, n=plen, ex=CodeError(code, "done req") if code else None))
    else:
        for _ in range(n):
            (rlen,) = struct.unpack("=I", await reader.readexactly(4))
            rets.append(IoRet(reqid=(await reader.readexactly(rlen)).decode("utf-8")))
        if has_plen:
            for r in rets:
                (r.n,) = struct.unpack("=I", await reader.readexactly(4))
    writer.write(struct.pack("=I", respcode))
    coros = []
    for r in rets:
        res = cb(tprank, r)
        if asyncio.iscoroutine(res):
            coros.append(res)
    if coros:
        await asyncio.gather(*coros)
    await writer.drain()


def pack_rpc(head: int, body: bytes) -> bytes:
    """``head:u32, len:u32, body`` - the framing of every msgpack-bodied RPC."""
    return struct.pack("=II", head, len(body)) + body
