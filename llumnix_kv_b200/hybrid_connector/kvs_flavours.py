"""The store backends the reference ships as adapters to external services, over the in-repo block store.

Each flavour keeps what defines its adapter towards the connector and at rest: how a block is named, when a
step's pages leave the GPU, who declares a block complete, and how a prefix is looked up.

``MooncakeKVSBackend`` (mooncake_kvsbackend.py:172-634 of the reference)
    name of a block: ``"{block_hash.hex()}_{tp_rank}"`` (:460-468); a request's blocks are saved once, when
    the step's last layer has run (``batch_save_kv_async`` of the whole step); a prefix matches as far as
    every TP rank's name exists (``batch_is_exist`` over ``tp_size`` names per block, :452-476).

``V6dObjectBackend`` (v6d_object_backend.py:97-658)
    blocks named by xxh64 of the engine's block hashes (kvsbackend.py:381-399 maps the 128-bit hashes to the
    64-bit ones the object store uses); the store of a step is deferred to ``clear_backend_metadata`` (one
    move of every layer after the forward pass, :285-316); the worker reports the outcome in its save-done
    (``n == 0``: failed, :317-329) and the SCHEDULER seals or discards the pending objects in
    ``async_cleanup`` (:572-618), after an aborted save has been drained on the worker (:344-368).

The Vineyard flavour is the base class (kvsbackend.py).
"""
from __future__ import annotations

import asyncio
import hashlib
import logging
from typing import Optional

from .backend import HB_SAVE_IORET, BackendMeta
from .engine_proxy import Request, get_param
from .kvsbackend import KVSBackend, KVSMeta, KVSReqMeta
from .utils import IoRet, kill_me_if_exception

logger = logging.getLogger("llumnix_kv_b200.hybrid_connector")


def mooncake_block_name(block_hash: bytes, tp_rank: int) -> str:
    """At-rest name of one block of one TP rank in a Mooncake store."""
    return f"{block_hash.hex()}_{tp_rank}"


def name_to_store_key(name: str) -> bytes:
    """The shared store indexes 16-byte keys: a named block is found under BLAKE2b-128 of its name."""
    return hashlib.blake2b(name.encode(), digest_size=16).digest()


class MooncakeKVSBackend(KVSBackend):
    SOURCE_LABEL = "kvs"
    FLAVOUR = "mooncake"
    NEEDS_BLOCK_HASHES = True

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self._per_step = True      # the step's blocks leave together, after the last layer

    def block_names(self, token_ids: list, block_hashes: list, n_blocks: int, tp_rank: int) -> list:
        assert len(block_hashes) >= n_blocks, "the Mooncake flavour names blocks by the engine's block hashes"
        return [mooncake_block_name(h, tp_rank) for h in block_hashes[:n_blocks]]

    def store_keys(self, token_ids: list, block_hashes: list, n_blocks: int, tp_rank: int) -> list:
        return [name_to_store_key(n) for n in self.block_names(token_ids, block_hashes, n_blocks, tp_rank)]

    def _matched_blocks(self, req: Request, max_blocks: int) -> int:
        """``batch_is_exist`` semantics: block by block, every TP rank's name must exist; stop at the first
        block that is missing anywhere."""
        if max_blocks <= 0:
            return 0
        if not self._open_index():
            return max_blocks
        hashes = self._hashes_of(req, max_blocks)
        per_rank = [self._index.lookup_prefix(b"".join(self.store_keys(req.prompt_token_ids, hashes, max_blocks, r)))
                    for r in range(self._tp)]
        return min(per_rank)


class V6dObjectBackend(KVSBackend):
    SOURCE_LABEL = "v6d_object"
    FLAVOUR = "v6d_object"
    NEEDS_BLOCK_HASHES = True

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self._per_step = True
        self._deferred: list = []          # worker: this step's save work, issued in clear_backend_metadata
        self._inflight: dict = {}          # worker: reqid -> asyncio tasks of stores in flight (drained on abort)
        self._pending_seal: dict = {}      # scheduler: reqid -> {tp_rank: [store keys]} waiting for async_cleanup

    def block_names(self, token_ids: list, block_hashes: list, n_blocks: int, tp_rank: int) -> list:
        import xxhash

        assert len(block_hashes) >= n_blocks
        return [xxhash.xxh64(h).intdigest() for h in block_hashes[:n_blocks]]

    # ---- scheduler half -----------------------------------------------------------------------------
    def _save_meta(self, reqid: str, scheduled: int) -> Optional[KVSReqMeta]:
        m = super()._save_meta(reqid, scheduled)
        if m is not None:
            # what the workers will leave pending: sealed (or discarded) here when the request is cleaned up
            per_rank = self._pending_seal.setdefault(reqid, {})
            for r in range(self._tp):
                keys = self.store_keys(m.token_ids, m.block_hashes, len(m.block_ids), r)[m.skip_blocks:]
                per_rank.setdefault(r, []).extend(keys)
        return m

    async def async_cleanup(self, req: Request) -> None:
        """Seal what the request's workers stored, or discard it when a worker reported a failed store
        (save-done with n == 0) or the save was aborted."""
        pending = self._pending_seal.pop(req.request_id, None)
        if not pending or not self._open_index():
            return
        ioret: Optional[IoRet] = get_param(req, HB_SAVE_IORET, None)
        failed = ioret is not None and ioret.n is not None and ioret.n == 0
        for rank, keys in pending.items():
            if failed:
                logger.warning("v6d_object: store failed for req %s: discarding %d pending blocks of rank %d",
                               req.request_id, len(keys), rank)
            for k in keys:
                # a key another request sealed meanwhile, or one the worker never reserved (store full), is left alone
                (self._index.discard if failed else self._index.seal)(k)

    # ---- worker half --------------------------------------------------------------------------------
    def async_save_kv_layer(self, layer_name: str, kv_layer, m: BackendMeta):
        """Nothing leaves during the forward pass: the first layer fixes the step's work, the store itself is
        issued when the metadata is cleared."""
        assert isinstance(m, KVSMeta)
        if self._layer_index[layer_name] == 0:
            self._drain_aborts(m)
            self._plan_step_saves(m)
            self._deferred = list(self._step_saves)
            self._step_saves = []
        return None

    def _drain_aborts(self, m: KVSMeta) -> None:
        """An aborted save may still have a store in flight: wait for it (bounded by the I/O timeout) before
        the scheduler discards the blocks it was writing."""
        for r in m.metas:
            if r.is_store and r.abort:
                tasks = self._inflight.pop(r.reqid, [])
                for t in tasks:
                    try:
                        t.result(timeout=self._io_timeout)
                    except Exception as ex:   # the store failed or timed out: the blocks are discarded either way
                        logger.warning("v6d_object: draining the aborted save of %s: %r", r.reqid, ex)

    def clear_backend_metadata(self) -> None:
        work, self._deferred = self._deferred, []
        gate = self._nan_gate
        super().clear_backend_metadata()
        if not work:
            return
        st = self._store
        after = None
        if st.device.type == "cuda":
            import torch

            after = torch.cuda.Event()
            after.record(torch.cuda.current_stream(st.device))
        blocks = [b for _, bl, _, _ in work for b in bl]
        slots = [s for _, _, sl, _ in work for s in sl]
        ev = st.save_layers(0, self._num_layers, blocks, slots, after=after)    # every layer of the step, one move
        fut = asyncio.run_coroutine_threadsafe(self._finish_step(work, ev, gate), self._connector.loop)
        for r, _, _, _ in work:
            self._inflight.setdefault(r.reqid, []).append(fut)

    @kill_me_if_exception
    async def _finish_step(self, work: list, ev, gate) -> None:
        failed = None
        try:
            await self._wait_event(ev)
            self._store.check_status()
        except Exception as ex:
            failed = ex
            logger.warning("v6d_object: store of a step failed: %r", ex)
        nan = False
        if gate is not None:
            flag = await asyncio.wait_for(asyncio.wrap_future(gate), self._io_timeout)
            nan = flag is not None and bool(flag.item())
        tprank = self._rank
        from .backend import IoDoneReqs, SAVE_DONE_REQ, SAVE_DONE_RESP

        for r, _, _, mine in work:
            if nan:
                self._nan_failed.add(r.reqid)
            bad = failed is not None or r.reqid in self._nan_failed
            if bad:
                self._wfailed.add(r.reqid)
            if r.is_last_chunk:
                # the blocks stay pending: the scheduler seals or discards them in async_cleanup
                ok = r.reqid not in self._wfailed
                self._wfailed.discard(r.reqid)
                self._nan_failed.discard(r.reqid)
                self._wpending.pop(r.reqid, None)
                self._inflight.pop(r.reqid, None)
                ioret = IoRet(reqid=r.reqid, n=(len(r.block_ids) if ok else 0), source=self.source_label())
                await self._connector.io_done_rpc(IoDoneReqs(worker_tprank=tprank, reqids=[ioret]), SAVE_DONE_REQ,
                                                  SAVE_DONE_RESP)

    def register_kv_caches(self, kv_caches: dict) -> None:
        super().register_kv_caches(kv_caches)
        self._wfailed: set = set()

    def save_done_source(self) -> Optional[str]:
        return self.source_label()


def flavour_class(name: str):
    """Store backend class of a ``kvs_backend`` / ``backend`` name."""
    table = {"pinned": KVSBackend, "kvs": KVSBackend, "vineyard": KVSBackend, "mooncake": MooncakeKVSBackend,
             "v6d_object": V6dObjectBackend}
    if name not in table:
        raise ValueError(f"unknown store flavour {name!r}")
    return table[name]
