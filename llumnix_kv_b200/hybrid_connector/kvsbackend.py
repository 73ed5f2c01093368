""""kvs" backend: prefix KV persisted in the node's shared host-DRAM block store.

The reference's kvs backends are adapters to external stores
(blade_kvt/hybrid_connector/kvsbackend.py:111-514 Vineyard, mooncake_kvsbackend.py:172-634,
v6d_object_backend.py:97-658); the contract they implement against the connector is kept:

  scheduler half  get_operations (load and save when the prompt is longer than
                  VLLM_KVS_ON_MIN_LENGTH), async_get_num_new_matched_tokens,
                  async_update_state_after_alloc (queues a load), build_backend_meta (loads +
                  per-step saves, chunked-prefill aware, ``is_last_chunk``), aborted saves are
                  released after the I/O timeout;
  worker half     async_load_kv yields IoRet(reqid, n = tokens actually loaded),
                  async_save_kv_layer returns a generator that yields a request once per layer
                  in the step of its last chunk.

Unlike the adapters, the store is in this repo (llumnix_kv_b200/kvstore): the scheduler half
looks prefixes up in the shared index before blocks are reserved (the Vineyard adapter cannot:
"no lookup support", kvsbackend.py:372-380), only full blocks are stored, keys are chained
block hashes salted per TP rank, entries are visible only once every layer has landed (seal)
and unfinished ones are discarded on abort.
"""
from __future__ import annotations

import asyncio
import dataclasses
import logging
from collections import deque
from collections.abc import AsyncGenerator
from typing import Optional

from llumnix_kv_b200 import envs

from .backend import HB_SAVE_SOURCES, BackendMeta, HCSchedOutput, HybridBackend, OperationPlan
from .engine_proxy import KVCacheBlocks, KVConnectorRole, Request, SchedulerOutput, VllmConfig, get_param
from .utils import IoRet, kill_me_if_exception

logger = logging.getLogger("llumnix_kv_b200.hybrid_connector")

KVS_NOSAVE = "kvs_nosave"     # per-request switch in kv_transfer_params
KVS_NOLOAD = "kvs_noload"


@dataclasses.dataclass
class KVSReqMeta:
    reqid: str
    is_store: bool
    token_ids: list            # the prefix whose full blocks are keyed
    block_ids: list            # engine block id of each of those blocks
    skip_blocks: int = 0       # load: blocks already present locally; save: blocks handled in earlier steps
    is_last_chunk: bool = False
    abort: bool = False        # save was aborted: drop what is not sealed
    trace: Optional[str] = None  # W3C traceparent of this I/O (child of the request's span), if the request carries one
    block_hashes: list = dataclasses.field(default_factory=list)   # engine block hashes of those blocks (hash-keyed flavours)


@dataclasses.dataclass
class KVSMeta(BackendMeta):
    metas: list = dataclasses.field(default_factory=list)
    nan_flag: object = None    # set by the model runner after the forward pass when the NaN check is on

    def __bool__(self):
        return bool(self.metas)

    def wants_nan_flag(self) -> bool:
        return any(m.is_store and not m.abort for m in self.metas)

    def set_nan_flag(self, flag) -> None:
        self.nan_flag = flag


def should_use(req: Request) -> bool:
    return req.num_prompt_tokens > envs.VLLM_KVS_ON_MIN_LENGTH + 1


class KVSBackend(HybridBackend):
    """The store backend, and its Vineyard flavour: keys made from the token ids (or, with
    VLLM_KVS_USE_REQUEST_HASH, from xxh64 of the engine's block hashes, as kvsbackend.py:381-399 of the
    reference maps them), every layer saved right after it ran with one CUDA event per layer
    (kvsbackend.py:111-514).  The flavours in kvs_flavours.py change the keys, when a step's pages leave,
    and who seals them."""

    SOURCE_LABEL = "kvs"
    FLAVOUR = "vineyard"
    NEEDS_BLOCK_HASHES = False     # the scheduler half ships the engine's block hashes with every request

    def __init__(self, vllm_config: VllmConfig, role: KVConnectorRole, kv_cache_config=None, **kw):
        super().__init__(vllm_config, role, kv_cache_config, **kw)
        kcfg = vllm_config.kv_transfer_config
        assert kcfg is not None
        self._cfg = vllm_config
        self._bs = vllm_config.cache_config.block_size
        self._tp = vllm_config.parallel_config.tensor_parallel_size
        self._name = kcfg.get_from_extra_config("kvs_name", f"kvx_store_{vllm_config.instance_name}")
        self._fp8 = bool(kcfg.get_from_extra_config("kvs_fp8", False))
        self._ttl_ms = int(float(kcfg.get_from_extra_config("kvs_ttl_s", envs.VLLM_KVS_TTL_SECONDS)) * 1000)
        self._slots_cfg = kcfg.get_from_extra_config("kvs_slots", None)
        self._model_tag = vllm_config.model_config.name
        self._io_timeout = envs.VLLM_KVS_IO_TIMEOUT_SECONDS
        # "layer": every layer's pages leave right after the layer ran (overlaps the forward pass);
        # "step": one move of all layers after the last one (fewer, larger transfers, the way the
        # reference's object-store adapter defers its store to the end of the step,
        # v6d_object_backend.py:97-658)
        self._per_step = kcfg.get_from_extra_config("kvs_save_granularity", "layer") == "step"
        # scheduler half
        self._loads: deque = deque()          # KVSReqMeta queued by the disagg thread
        self._index = None                    # KvStore handle used for lookups only
        self._salts: list = []
        self._saved_blocks: dict = {}         # reqid -> blocks already handed to the workers
        # worker half
        self._store = None
        self._wkeys: dict = {}                # reqid -> chained keys computed so far
        self._wpending: dict = {}             # reqid -> keys reserved by this worker and not sealed yet
        # NaN gate (the reference's VLLM_V6D_STORE_NAN_CHECK, v6d_object_backend.py:78-90,373-430):
        # blocks of a step are sealed only once the model runner's isnan flag of that step is known to
        # be clear; a request that saw a NaN stores nothing from then on
        self._nan_check = bool(envs.VLLM_KVS_STORE_NAN_CHECK)
        self._bound_meta = None
        self._nan_gate = None                 # concurrent Future of this step: resolves to the flag tensor or None
        self._nan_failed: set = set()
        # request context of the last store operations, "reqid[;traceparent][;op=start|end]" as the reference
        # hands it to its stores (kvsbackend.py:232-245,297-323); kept for logs and tests
        self.request_contexts: deque = deque(maxlen=256)

    # ---- geometry shared by both halves --------------------------------------------------------------
    def _geometry(self):
        from llumnix_kv_b200.kvstore import store_format
        from llumnix_kv_b200.models.kv_spec import rank_attn_layout

        layout = rank_attn_layout(self._cfg)
        slot_bytes, tag = store_format(layout, self._cfg.model_config.num_layers, self._fp8)
        n_slots = int(self._slots_cfg) if self._slots_cfg else max(1, envs.VLLM_KVS_CAPACITY_BYTES // slot_bytes)
        return layout, slot_bytes, tag, n_slots

    # ==================================================================================================
    # scheduler half
    # ==================================================================================================
    def get_operations(self, req: Request) -> OperationPlan:
        src = self.source_label()
        load = should_use(req) and not get_param(req, KVS_NOLOAD, False)
        save = should_use(req) and not get_param(req, KVS_NOSAVE, False)
        return int(load), int(save), (src,) if load else (), (src,) if save else ()

    def _open_index(self) -> bool:
        if self._index is not None:
            return True
        from llumnix_kv_b200 import load_ops
        from llumnix_kv_b200.kvstore import store_salt

        _, slot_bytes, tag, n_slots = self._geometry()
        try:
            self._index = load_ops().KvStore.open(self._name, slot_bytes, n_slots, 2, tag)
        except RuntimeError as ex:
            logger.warning("kvs: cannot open the store index (%s); loads are attempted blindly", ex)
            return False
        self._salts = [store_salt(self._model_tag, r, self._tp, tag) for r in range(self._tp)]
        return True

    def _matched_blocks(self, req: Request, max_blocks: int) -> int:
        """Leading full blocks that every TP rank has in the store."""
        from llumnix_kv_b200.kvstore import block_keys

        if max_blocks <= 0:
            return 0
        if not self._open_index():
            return max_blocks
        n = max_blocks
        hashes = self._hashes_of(req, n)
        for rank in range(self._tp):
            keys = self.store_keys(req.prompt_token_ids, hashes, n, rank)
            n = min(n, self._index.lookup_prefix(b"".join(keys)))
            if n == 0:
                break
        return n

    # ---- naming of blocks at rest (flavours override) -------------------------------------------------
    def _hashes_of(self, req: Request, n_blocks: int) -> list:
        if not (self.NEEDS_BLOCK_HASHES or envs.VLLM_KVS_USE_REQUEST_HASH):
            return []
        return list(req.compute_block_hashes(self._bs)[:n_blocks])

    def block_names(self, token_ids: list, block_hashes: list, n_blocks: int, tp_rank: int) -> list:
        """The flavour's own name of each of the first ``n_blocks`` blocks on ``tp_rank`` (what an external
        store of that kind would be asked for); None for the token-keyed default, which has no name but the key."""
        if envs.VLLM_KVS_USE_REQUEST_HASH and block_hashes:
            import xxhash

            return [xxhash.xxh64(h).intdigest() for h in block_hashes[:n_blocks]]
        return [None] * n_blocks

    def store_keys(self, token_ids: list, block_hashes: list, n_blocks: int, tp_rank: int) -> list:
        """16-byte keys of those blocks in the shared store."""
        import struct

        from llumnix_kv_b200.kvstore import block_keys, store_salt

        names = self.block_names(token_ids, block_hashes, n_blocks, tp_rank)
        if names and names[0] is not None:
            return [struct.pack("<QII", int(x) & 0xFFFFFFFFFFFFFFFF, tp_rank, self._tp) for x in names]
        _, _, tag, _ = self._geometry()
        return block_keys(token_ids, self._bs, n_blocks, store_salt(self._model_tag, tp_rank, self._tp, tag))

    async def async_get_num_new_matched_tokens(self, req: Request, num_computed_tokens: int) -> int:
        assert num_computed_tokens % self._bs == 0
        # the last prompt token is always computed locally: it produces the first output
        max_blocks = (req.num_prompt_tokens - 1) // self._bs
        matched = self._matched_blocks(req, max_blocks)
        return max(0, matched * self._bs - num_computed_tokens)

    async def async_update_state_after_alloc(self, request: Request, blocks: KVCacheBlocks,
                                             num_external_tokens: int) -> Optional[IoRet]:
        if num_external_tokens <= 0:
            return None
        upto = request.num_computed_tokens + num_external_tokens
        assert upto % self._bs == 0
        nblk = upto // self._bs
        block_ids = blocks.get_block_ids()[0][:nblk]
        assert len(block_ids) == nblk
        self._engine.sched_discard_zero_block_ids(block_ids)
        self._loads.append(KVSReqMeta(request.request_id, False, list(request.prompt_token_ids[:upto]), list(block_ids),
                                      skip_blocks=request.num_computed_tokens // self._bs,
                                      trace=request.trace_wrapper.traceparent("kv_load"),
                                      block_hashes=self._hashes_of(request, nblk)))
        return None   # the workers report LOAD_DONE with what they really loaded

    def _save_meta(self, reqid: str, scheduled: int) -> Optional[KVSReqMeta]:
        req = self.get_request(reqid)
        if req is None or self.source_label() not in get_param(req, HB_SAVE_SOURCES, ()):
            return None
        if req.num_computed_tokens >= req.num_prompt_tokens:
            return None   # decoding: the prompt's blocks were handled in earlier steps
        after = min(req.num_computed_tokens + scheduled, req.num_prompt_tokens)
        last = after >= req.num_prompt_tokens
        done_blocks = after // self._bs
        prev = self._saved_blocks.get(reqid, 0)
        if last:
            self._saved_blocks.pop(reqid, None)
        else:
            self._saved_blocks[reqid] = done_blocks
        if done_blocks <= prev and not last:
            return None
        block_ids = self._engine.sched_get_kvblk_ids(reqid)[0][:done_blocks]
        return KVSReqMeta(reqid, True, list(req.prompt_token_ids[:done_blocks * self._bs]), list(block_ids),
                          skip_blocks=prev, is_last_chunk=last, trace=req.trace_wrapper.traceparent("kv_save"),
                          block_hashes=self._hashes_of(req, done_blocks))

    def build_backend_meta(self, sout: SchedulerOutput) -> BackendMeta:
        assert isinstance(sout, HCSchedOutput)
        meta = KVSMeta()
        while self._loads:
            meta.metas.append(self._loads.popleft())
        if sout.hc_aborted_save:
            for req in sout.hc_aborted_save:
                self._saved_blocks.pop(req.request_id, None)
                meta.metas.append(KVSReqMeta(req.request_id, True, [], [], abort=True))
            asyncio.run_coroutine_threadsafe(self._release_aborted(list(sout.hc_aborted_save)),
                                             self._engine.get_hybrid_sched_loop())
        if sout.hc_parent is None:
            for nr in sout.scheduled_new_reqs:
                m = self._save_meta(nr.req_id, sout.num_scheduled_tokens[nr.req_id])
                if m is not None:
                    meta.metas.append(m)
            for rid in sout.scheduled_cached_reqs.req_ids:
                m = self._save_meta(rid, sout.num_scheduled_tokens[rid])
                if m is not None:
                    meta.metas.append(m)
        return meta

    @kill_me_if_exception
    async def _release_aborted(self, reqs: list):
        """An aborted save never reaches its last chunk: once the workers have had the time to
        drain what was in flight, declare it finished so that its block references unwind."""
        await asyncio.sleep(float(self._cfg.kv_transfer_config.get_from_extra_config("kvs_abort_grace_s", 0.2)))
        for req in reqs:
            self._connector.mark_backend_save_done(req, self.source_label())

    # ==================================================================================================
    # worker half
    # ==================================================================================================
    def register_kv_caches(self, kv_caches: dict) -> None:
        from llumnix_kv_b200.kvstore import PinnedKVStore

        from .kvtbackend import flatten_cache

        layers = [t[0] for t in flatten_cache(kv_caches)]
        layout, _, _, n_slots = self._geometry()
        assert layers[0].nbytes == layout.layer_bytes, "cache tensor does not match the configured cache shape"
        rank = self._rank = self._worker.get_tensor_model_parallel_rank()
        self._store = PinnedKVStore(self._name, layout, layers, rank, self._tp, n_slots, create="auto",
                                    ttl_ms=self._ttl_ms, fp8=self._fp8, model_tag=self._model_tag)
        self._layer_index = {name: i for i, name in enumerate(sorted(kv_caches, key=_layer_key))}
        self._num_layers = len(layers)
        self._step_saves: list = []          # this step's save work, fixed at the first layer
        logger.info("kvs: rank %d attached to store %s (%d slots of %d bytes, fp8=%s)", rank, self._name, n_slots,
                    self._store.slot_bytes, self._fp8)

    def bind_backend_metadata(self, meta: BackendMeta) -> None:
        self._bound_meta = meta
        if self._nan_check and isinstance(meta, KVSMeta) and meta.wants_nan_flag():
            import concurrent.futures

            self._nan_gate = concurrent.futures.Future()

    def clear_backend_metadata(self) -> None:
        gate, meta = self._nan_gate, self._bound_meta
        self._nan_gate = self._bound_meta = None
        if gate is not None:
            gate.set_result(getattr(meta, "nan_flag", None))    # the forward pass is over: the flag was set, or never will be

    def bypass_bind(self, meta: BackendMeta) -> None:
        return   # bypass substeps only carry loads; their metadata reaches async_load_kv directly

    def bypass_clear(self) -> None:
        return

    async def _wait_event(self, ev) -> None:
        if ev is not None:
            await asyncio.wait_for(asyncio.get_running_loop().run_in_executor(None, ev.synchronize), self._io_timeout)

    def _keys_for(self, m: KVSReqMeta) -> list:
        """Chained keys of the request's blocks, extended from what earlier steps computed."""
        n = len(m.block_ids)
        if m.block_hashes:       # hash-keyed flavours: nothing to chain, the engine's hashes already are
            return self.store_keys(m.token_ids, m.block_hashes, n, self._rank)
        have = self._wkeys.get(m.reqid, [])
        if len(have) < n:
            from llumnix_kv_b200.kvstore.store import block_keys

            have = block_keys(m.token_ids, self._bs, n, self._store.salt) if not have else \
                have + _extend_keys(have[-1], m.token_ids, self._bs, len(have), n, self._store.salt)
            self._wkeys[m.reqid] = have
        return have[:n]

    async def async_load_kv(self, m: BackendMeta) -> AsyncGenerator:
        assert isinstance(m, KVSMeta)
        for r in m.metas:
            if r.is_store:
                continue
            st = self._store
            self._note_context(r, None)
            keys = self._keys_for(r)
            self._wkeys.pop(r.reqid, None)
            slots = st.pin(keys)
            n = len(slots)
            loaded = max(0, n - r.skip_blocks) * self._bs
            try:
                ev = st.load_layers(0, self._num_layers, r.block_ids[r.skip_blocks:n], slots[r.skip_blocks:n])
                await self._wait_event(ev)
                st.check_status()
                ioret = IoRet(reqid=r.reqid, n=loaded, source=self.source_label())
            except Exception as ex:   # a miss, not a failed request: it falls back to computing everything itself
                logger.warning("kvs: load failed, the request computes its prompt. reqid=%s ex=%r", r.reqid, ex)
                ioret = IoRet(reqid=r.reqid, n=0, source=self.source_label())
            finally:
                st.unpin(keys[:n])
            yield ioret

    def _plan_step_saves(self, m: KVSMeta) -> None:
        """First layer of a forward pass: decide which blocks of which request go to which slot."""
        self._step_saves = []
        for r in m.metas:
            if not r.is_store:
                continue
            if r.abort:
                self._store.discard(self._wpending.pop(r.reqid, []))
                self._wkeys.pop(r.reqid, None)
                continue
            keys = self._keys_for(r)
            todo = keys[r.skip_blocks:]
            new, full = self._store.reserve(todo)
            if full:
                logger.info("kvs: store full, reqid=%s keeps %d of %d new blocks", r.reqid, len(new), len(todo))
            blocks = [r.block_ids[r.skip_blocks + i] for i, _ in new]
            slots = [s for _, s in new]
            mine = [todo[i] for i, _ in new]
            self._wpending.setdefault(r.reqid, []).extend(mine)
            self._step_saves.append((r, blocks, slots, mine))
            if r.is_last_chunk:
                self._wkeys.pop(r.reqid, None)

    def async_save_kv_layer(self, layer_name: str, kv_layer, m: BackendMeta) -> Optional[AsyncGenerator]:
        assert isinstance(m, KVSMeta)
        layer = self._layer_index[layer_name]
        if layer == 0:
            self._plan_step_saves(m)
        if not self._step_saves:
            return None
        st = self._store
        last_layer = layer == self._num_layers - 1
        ev = None
        if not self._per_step or last_layer:
            after = None
            if st.device.type == "cuda":
                import torch

                after = torch.cuda.Event()
                after.record(torch.cuda.current_stream(st.device))
            blocks = [b for _, bl, _, _ in self._step_saves for b in bl]
            slots = [s for _, _, sl, _ in self._step_saves for s in sl]
            lo = 0 if self._per_step else layer
            ev = st.save_layers(lo, layer + 1, blocks, slots, after=after)   # one launch for every request of the step
        work = list(self._step_saves)
        if layer == 0 or last_layer:
            for r, _, _, _ in work:
                self._note_context(r, "start" if layer == 0 else "end")
        gate = self._nan_gate if last_layer else None
        if last_layer:
            self._step_saves = []

        async def gen():
            failed = None
            try:
                await self._wait_event(ev)
                st.check_status()
            except Exception as ex:
                failed = ex
                logger.warning("kvs: save of layer %d failed: %r", layer, ex)
            nan = False
            if gate is not None:
                flag = await asyncio.wait_for(asyncio.wrap_future(gate), self._io_timeout)
                nan = flag is not None and bool(flag.item())    # the isnan kernel precedes the save event on the stream
                if nan:
                    logger.error("kvs: NaN in this step's hidden states: its %d request(s) store nothing", len(work))
            for r, _, _, mine in work:
                if last_layer:
                    pend = self._wpending.get(r.reqid, [])
                    if nan:
                        self._nan_failed.add(r.reqid)
                    if failed is None and r.reqid not in self._nan_failed:
                        st.seal(mine)             # every layer of these blocks has landed
                    else:
                        st.discard(mine)
                    for k in mine:
                        if k in pend:
                            pend.remove(k)
                    if r.is_last_chunk:
                        self._wpending.pop(r.reqid, None)
                        self._nan_failed.discard(r.reqid)
                if r.is_last_chunk:
                    yield r.reqid

        return gen()

    def _note_context(self, r: KVSReqMeta, op: Optional[str]) -> None:
        ctx = r.reqid
        if r.trace:
            ctx += f";{r.trace}"
            if op:
                ctx += f";op={op}"
        self.request_contexts.append(ctx)
        logger.debug("kvs: %s %s", "save" if r.is_store else "load", ctx)

    def stop(self) -> None:
        if self._store is not None:
            self._store.close()
            self._store = None


def _layer_key(name: str):
    from .kvtbackend import extract_layer_index

    return extract_layer_index(name)


def _extend_keys(prev: bytes, token_ids: list, bs: int, lo: int, hi: int, salt: bytes) -> list:
    import hashlib
    import struct

    out = []
    for i in range(lo, hi):
        h = hashlib.blake2b(prev, digest_size=16)
        h.update(struct.pack(f"<{bs}q", *token_ids[i * bs:(i + 1) * bs]))
        h.update(salt)
        prev = h.digest()
        out.append(prev)
    return out
