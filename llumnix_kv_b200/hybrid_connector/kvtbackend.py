"""PD-separation backends over the native KVT engine: ``PBackend`` (prefill, sender) and
``DBackend`` (decode, receiver).

Two ways a prefill engine learns where to send a request's KV
(blade_kvt/hybrid_connector/kvtbackend.py:1104-2157 for P, :2160-2791 for D):

* *push mode* - the decode engine sends the whole request to a prefill engine (PREFILL_REQ);
  P runs it with ``max_tokens=1`` and ``ignore_output`` and answers with a ``KVTResp`` once
  every TP rank has reported its send done;
* *dual-request mode* - a frontend sent the request to P (``do_remote_decode``) and to D
  (``do_remote_prefill`` + ``remote_host/port``) separately; D tells P where the KV goes with
  TRANSFER_KV_REQ.  The two can arrive in either order: P keeps finished prefills for a while
  (``_dual_req_done``), answers 404 for a request it has not seen yet (D retries with
  back-off) and 410 for one that is gone for good (aborted or timed out).

Per engine step the scheduler half turns the scheduler output into ``KVTPMeta``: which chunks
of which requests leave in this step (chunked prefill sends ``[seen, seen+new)`` per step; the
first chunk carries the block tables, later ones are deltas).  The worker half hands them to
``KVTransferClient`` before the forward pass, records one event per layer from
``save_kv_layer`` and closes the step afterwards.
"""
from __future__ import annotations

import asyncio
import logging
import os
import re
import struct
import threading
import time
import uuid
from collections import OrderedDict, defaultdict, deque
from dataclasses import dataclass, field
from typing import Optional

import msgspec

from llumnix_kv_b200 import envs

from .backend import BackendMeta, HCSchedOutput, HybridBackend, OperationPlan, has_setup_save, req_aborted
from .engine_proxy import (EngineCoreRequest, KVCacheBlocks, KVConnectorRole, Request, SchedulerOutput, VllmConfig,
                           core_get_param, core_update_params, get_p_node_pop_len, get_param,
                           sched_rpc_server_port, scheduler_rpc_host, set_param)
from .utils import (CodeError, ConnManager, IoRet, IoState, PeerInfo, PeerManager, handle_done_req,
                    kill_me_if_exception, try_advance)

logger = logging.getLogger("llumnix_kv_b200.hybrid_connector")

# ---- request parameters ----------------------------------------------------------------------------
D_DISAGG = "ali_llumnix_disagg"
P_REMOTE_DECODE = "do_remote_decode"
D_REMOTE_PREFILL = "do_remote_prefill"
D_PID = "_hbkvtpid"                # which prefill engine a decode request went to ("addr:port")
P_IGNORE_OUTPUTS = "ignore_output"
P_KVTD_INFO = "hbpkvtdinfo"
P_KVT_STATE = "hbpkvtstate"

# ---- RPC heads -------------------------------------------------------------------------------------
PREFILL_REQ = 0x20181218           # body: msgpack EngineCoreRequest
PREFILL_RESP = 0x81218102          # body: msgpack KVTResp
SEND_DONE_REQ = 0x20181219         # from the native send stubs
SEND_DONE_RESP = 0x91218102
TRANSFER_KV_REQ = 0x20210912       # body: msgpack RKVTDInfo
TRANSFER_KV_RESP = PREFILL_RESP
ABORT_REQS_REQ = 20250820          # body: msgpack list[str]
ABORT_REQS_RESP = 20250820
REGISTER_WORKER = 0x20181224       # body: msgpack "{rank}|{WorkerInfo}"
REGISTER_WORKER_RESP = 0x20181225

CODE_OK = 0
CODE_REQNOTFOUND = 404             # "not yet": D retries
CODE_REQGONE = 410                 # "never": D fails the load at once
CODE_INTERNALERROR = 500
CODE_MIGRATE_REJECTED_BUSY = 1001


class KVTDInfo(msgspec.Struct, array_like=True, omit_defaults=True, gc=False):
    """Where a request's KV goes: decode instance ``name|dprank|tpsize``, its block ids per group,
    what it already has, up to where it wants it, and its workers' WorkerInfo strings."""

    instid: str
    blkids: list[list[int]]
    cached_tokens: int
    max_tokens: int
    d_workers_info: list[str]


class RKVTDInfo(msgspec.Struct, array_like=True, omit_defaults=True, gc=False):
    reqid: str
    dinfo: KVTDInfo
    migration: bool = False


class KVTResp(msgspec.Struct, array_like=True, omit_defaults=True, gc=False):
    code: int
    cached: int
    computed: int
    output_token_ids: Optional[list[int]] = None


@dataclass
class KVTState:
    dinfo: KVTDInfo
    maxtokens: int
    untouched: bool = True      # no chunk of this request has been planned yet
    frozen: bool = False        # everything up to maxtokens left in one frozen step: nothing more to plan


@dataclass
class PReqMeta:
    """One chunk of one request for the worker.  With block ids it is a first submit, without it
    is a delta of a request submitted earlier."""

    reqid: str
    d_inst_id: str
    p_block_ids: list
    d_block_ids: list
    new_tokens: int
    has_last_token: bool
    seen_tokens: int
    d_workers_info: list = field(default_factory=list)
    has_freeze: bool = False


@dataclass
class KVTPMeta(BackendMeta):
    stepid: int = 0
    substepid: int = 0
    sched_tokens: int = 0
    freeze_metas: list = field(default_factory=list)      # data already complete: sent as frozen steps
    abort_metas: list = field(default_factory=list)       # zero-length closing deltas
    nonfreeze_metas: list = field(default_factory=list)   # chunks computed in this step

    def __bool__(self):
        return bool(self.freeze_metas or self.abort_metas or self.nonfreeze_metas)


class _SendingReq(IoState):
    def __init__(self, signals_per_worker: int = 1):
        super().__init__(signals_per_worker=signals_per_worker)
        self._fut = asyncio.get_running_loop().create_future()

    def try_mark_done(self, ioret: IoRet) -> None:
        if self._fut.done():
            logger.warning("mark done twice: ioret=%s", ioret)
            return
        self._fut.set_result(ioret)


class DualReq:
    def __init__(self, req: Request, pblkids: list, finished: bool = False):
        assert len(pblkids) > 0
        self.req, self.pblkids, self.finished = req, pblkids, finished
        self.insert_ts = time.time()


# ---- helpers ---------------------------------------------------------------------------------------
def get_inst_id(cfg: VllmConfig, fake_naming: bool = False) -> str:
    assert cfg.kv_transfer_config is not None
    r = cfg.kv_transfer_config.get_from_extra_config("kvt_inst_id", None)
    if r is None:
        pod = os.environ.get("POD_NAME")
        r = f"{pod}-{sched_rpc_server_port(cfg)}-{envs.get_ip()}" if fake_naming else pod
    return r if r is not None else str(uuid.uuid4())


def reg_naming(naming_cli, cfg: VllmConfig) -> None:
    assert cfg.kv_transfer_config is not None
    info = PeerInfo(role="prefill" if cfg.kv_transfer_config.is_kv_producer else "decode",
                    tpsize=cfg.parallel_config.tensor_parallel_size, ctime_us=int(time.time_ns() // 1000),
                    addr=envs.get_ip(), dprank=cfg.parallel_config.data_parallel_rank, port=sched_rpc_server_port(cfg))
    logger.info("register naming: %s", info)
    naming_cli.store(f"endpoint{info.dprank}", info.serialize())


def _worker_process_envs(cfg) -> None:
    """A worker that owns its process (one engine worker per process, as vLLM runs them) publishes its cache
    shape and the scheduler's send-done address through the environment, where the process-global engine
    functions of the reference binding look for them (``kvt_args.set_worker_envs``).  Off by default: several
    engines can share a process here, and each client is given its address explicitly; switched on with
    ``kv_connector_extra_config["kvt_worker_process_envs"]``."""
    if not cfg.kv_transfer_config.get_from_extra_config("kvt_worker_process_envs", False):
        return
    from .kvt_args import set_worker_envs

    set_worker_envs(cfg.cache_config.cache_shape, scheduler_rpc_host(cfg), sched_rpc_server_port(cfg))


def multicast_kwargs(layers) -> dict:
    """Server arguments that advertise the worker's NVLink multicast group, when every cache tensor it
    registers lives in a ``parallel.nvls.MulticastKVCache`` of this process (the decode group allocated
    its caches symmetrically); empty otherwise."""
    import torch

    from llumnix_kv_b200.parallel.nvls import multicast_address_of

    rows = [[layer] if isinstance(layer, torch.Tensor) else list(layer) for layer in layers]
    found = [[multicast_address_of(t) if t.is_cuda else None for t in row] for row in rows]
    if not found or any(f is None for row in found for f in row):
        return {}
    sizes = {f[1] for row in found for f in row}
    if len(sizes) != 1 or next(iter(sizes)) < 2:
        return {}
    return {"mc_layers": [[f[0] for f in row] for row in found], "mc_size": next(iter(sizes))}


def choose_relay(reqid: str, dist: list, total_kv_heads: int, src_tpsize: int) -> Optional[int]:
    """Index into ``dist`` (the decode workers this prefill rank would serve one by one) of the worker
    that receives the request for all of them, or None when each must be served separately.

    A relay needs: several targets; the same bytes for every one of them, which is the case when the
    prefill rank holds a single KV head or the MLA latent (``total_kv_heads <= src_tpsize``: the decode
    ranks it serves all replicate that head); every target advertising a multicast group that covers
    them (``mcn`` in its worker info); ``VLLM_KVT_NVLS_FANOUT`` not switched off.  The choice is a pure
    function of the request id, so every chunk of a request takes the same relay."""
    import zlib

    if len(dist) < 2 or not envs.VLLM_KVT_NVLS_FANOUT or total_kv_heads <= 0 or total_kv_heads > src_tpsize:
        return None
    for _, _, winfo in dist:
        if not isinstance(winfo, str) or ";mcn=" not in winfo and ":mcn=" not in winfo:
            return None
        try:
            group = int(winfo.split("mcn=", 1)[1].split(";", 1)[0])
        except ValueError:
            return None
        if group < len(dist):
            return None
    return zlib.crc32(reqid.encode()) % len(dist)


def get_dist(d_inst_id: str, src_tprank: int, src_tpsize: int) -> list:
    """(dst instance, dst worker id, dst tp rank) targets of this prefill rank.  One target, except
    P TP < D TP where one rank fans out to D_tp / P_tp ranks.  Empty: TP sizes do not divide."""
    name, dprank, tpsize = d_inst_id.rsplit("|", 2)
    d_dp, d_tp = int(dprank), int(tpsize)
    base = d_dp * d_tp
    if d_tp == src_tpsize:
        return [(name, base + src_tprank, src_tprank)]
    if src_tpsize > d_tp:
        g = src_tpsize // d_tp
        if d_tp * g != src_tpsize:
            return []
        return [(name, base + src_tprank // g, src_tprank // g)]
    g = d_tp // src_tpsize
    if src_tpsize * g != d_tp:
        return []
    return [(name, base + src_tprank * g + j, src_tprank * g + j) for j in range(g)]


def get_distinfo(meta: PReqMeta, src_tprank: int, src_tpsize: int) -> list:
    out = []
    for name, wid, d_rank in get_dist(meta.d_inst_id, src_tprank, src_tpsize):
        winfo = None
        if meta.d_workers_info:
            if d_rank >= len(meta.d_workers_info):
                return []
            winfo = meta.d_workers_info[d_rank]
        out.append((name, wid, winfo))
    return out


def handle_hybrid_blocks(grouped_blks: list, gamma: int, num_gdn_layers: int, num_kv_cache_groups: int,
                         has_null_prefix_block: bool, ple_group_index: Optional[int] = None) -> list:
    """Recurrent-state groups (GDN, PLE) own [null?] + 1 runtime block + gamma speculative work
    blocks; only the runtime block holds state worth transferring."""
    assert num_kv_cache_groups > num_gdn_layers > 0
    assert len(grouped_blks) == num_kv_cache_groups
    idx = 1 if has_null_prefix_block else 0
    out = []
    for g, blocks in enumerate(grouped_blks):
        if g < num_gdn_layers or g == ple_group_index:
            assert len(blocks) >= idx + 1, f"state group {g} has {len(blocks)} blocks"
            out.append(blocks[idx:idx + 1])
        else:
            out.append(blocks)
    return out


def extract_layer_index(layer_name: str) -> int:
    nums = re.findall(r"\.(\d+)\.", f".{layer_name}.")
    assert len(nums) == 1, f"layer name {layer_name!r} must contain exactly one integer component"
    return int(nums[0])


def turboquant_last_dim_bytes(packed_key_dim: int, head_size: int, fast: bool) -> int:
    """Bytes of one (token, head) row of a TurboQuant cache: the packed indices plus the per-row scale
    block (one fp16 per 128 dims in the fast variant, 16 bytes otherwise;
    blade_kvt/hybrid_connector/kvtbackend.py:122-139)."""
    return packed_key_dim + (head_size // 128 * 2 if fast else 16)


def resolve_raw_cache_tensors(kv_caches: dict) -> dict:
    """Cache objects that wrap views of one raw buffer -> that buffer as a flat int8 tensor.

    A TurboQuant cache hands the connector an object whose ``key_cache.indices`` and
    ``value_cache.indices`` are slices of one allocation ``[blocks, 2, block_size, heads * row_bytes]``;
    the transfer moves raw bytes, so it wants the allocation itself
    (blade_kvt/hybrid_connector/kvtbackend.py:141-171).  Plain tensors pass through."""
    import torch

    out = {}
    for name, cache in kv_caches.items():
        key, val = getattr(cache, "key_cache", None), getattr(cache, "value_cache", None)
        if isinstance(cache, torch.Tensor) or key is None or val is None:
            out[name] = cache
            continue
        ks, vs = key.indices.untyped_storage(), val.indices.untyped_storage()
        assert ks.data_ptr() == vs.data_ptr(), f"layer {name}: key and value indices do not share one allocation"
        raw = torch.tensor([], dtype=torch.int8, device=key.indices.device)
        raw.set_(ks, 0, (ks.nbytes(),))
        out[name] = raw
    return out


def flatten_cache(kv_caches: dict) -> list:
    """layer index -> [cache tensors of that layer] (sparse-MLA models register two per layer)."""
    by_index: dict = defaultdict(list)
    for name in kv_caches:
        by_index[extract_layer_index(name)].append(name)
    return [[kv_caches[n] for n in sorted(by_index[i])] for i in sorted(by_index)]


def build_kvt_args(backend: "HybridBackend", kv_caches: dict, tp_rank: int) -> dict:
    """Constructor arguments of KVTransferClient / KVTransferServer for this worker."""
    from llumnix_kv_b200.kv_transfer_impl import KVTransferProtocolType as PT

    cfg = backend._vllm_config
    mc, cc = cfg.model_config, cfg.cache_config
    tp = cfg.parallel_config.tensor_parallel_size
    dp = cfg.parallel_config.data_parallel_rank
    kv_caches = resolve_raw_cache_tensors(kv_caches)
    layers = flatten_cache(kv_caches)
    derived = None
    kcc = backend._kv_cache_config
    hf = getattr(mc, "hf_text_config", None)
    if backend.is_hybrid and kcc is not None and getattr(kcc, "kv_cache_tensors", None) and hf is not None:
        # an engine that registers its caches the way vLLM does (recurrent state as lists, attention pages as
        # views of shared physical tensors, a KV-cache configuration that says who shares what): everything the
        # native engine needs is worked out from those objects (kvt_args.py)
        from .kvt_args import derive_hybrid_kvt_args

        derived = derive_hybrid_kvt_args(kv_caches, kcc, hf, tp, cc.block_size, getattr(cc, "attn_pack_size", 1),
                                         kda_page_stride=getattr(cc, "kda_page_stride", 0),
                                         kda_conv_dim_first=bool(getattr(mc, "kda_conv_dim_first", False)))
        layers = [[t] for t in derived.physical_tensors.values()]
        backend.hybrid_model_send_layer = list(derived.send_layers)
    elif backend.is_hybrid:
        # Several logical layers (one GDN layer of each group and one attention layer) share a
        # physical cache tensor.  Each tensor is registered once, and the transfer of a tensor
        # starts when the last logical layer that writes into it has run.
        order = sorted(kv_caches, key=extract_layer_index)
        seen: dict = {}
        for name in order:
            seen[kv_caches[name].data_ptr()] = (extract_layer_index(name), kv_caches[name])
        phys = sorted(seen.values(), key=lambda it: it[0])
        layers = [[t] for _, t in phys]
        backend.hybrid_model_send_layer = [idx for idx, _ in phys]
    n_tensors = len(layers[0])
    block_bytes, token_bytes = [], []
    if derived is not None:
        block_bytes, token_bytes = list(derived.block_bytes), list(derived.token_bytes)
    else:
        for t in range(n_tensors):
            nbytes = layers[0][t].nbytes
            assert nbytes % cc.num_gpu_blocks == 0
            bb = nbytes // cc.num_gpu_blocks
            block_bytes.append(bb)
            token_bytes.append(bb // cc.block_size)
    proto = envs.VLLM_KV_TRANS_PROTOCOL or cfg.kv_transfer_config.get_from_extra_config("kvt_protocol", "")
    protocols = [PT.to_protocol_type(p) for p in proto.split(",") if p] if proto else []
    args = dict(inst_id=backend._inst_id, tp_size=tp, worker_id=dp * tp + tp_rank, worker_tp_rank=tp_rank,
                block_bytes=block_bytes, token_bytes=token_bytes, naming_url=backend._naming_url, layers=layers,
                protocols=protocols, num_kv_heads=1 if mc.use_mla else mc.num_kv_heads, cache_shape=cc.cache_shape)
    if derived is not None:
        args.update(derived.kwargs)
    elif backend.is_hybrid:
        args.update(mc.hybrid_kvt_kwargs_for(tp))
    return args


# ======================================================================================================
class PBackend(HybridBackend):
    SOURCE_LABEL = "kvt"
    _GONE_REQS_MAX = 8192

    def __init__(self, vllm_config: VllmConfig, role: KVConnectorRole, kv_cache_config=None, **kw):
        super().__init__(vllm_config, role, kv_cache_config, **kw)
        kcfg = vllm_config.kv_transfer_config
        assert kcfg is not None
        self._cfg = vllm_config
        self._naming_url = kcfg.get_from_extra_config("naming_url", "fake://")
        fake = self._naming_url == "fake://"
        self._inst_id = get_inst_id(vllm_config, fake_naming=fake)
        self._naming_cli = None
        if not fake:
            from llumnix_kv_b200.kv_transfer_impl import connect_naming

            self._naming_cli = connect_naming(self._inst_id, self._naming_url)
        self._gamma = get_p_node_pop_len(vllm_config) - 1
        self._kvt_cli = None
        if role == KVConnectorRole.WORKER:
            # where this worker's native send stubs report finished requests (the scheduler half)
            self._send_done_addr = f"{scheduler_rpc_host(vllm_config)}:{sched_rpc_server_port(vllm_config)}"
            return
        if self._naming_cli is not None:
            reg_naming(self._naming_cli, vllm_config)
        srv = self._engine.sched_rpc_server()
        srv.register_method(TRANSFER_KV_REQ, self._on_transfer_kv)
        srv.register_method(PREFILL_REQ, self._on_prefill)
        srv.register_method(SEND_DONE_REQ, self._on_send_done)
        srv.register_method(ABORT_REQS_REQ, self._on_abort_reqs)
        self._sending: dict[str, _SendingReq] = {}
        self._reqdec = msgspec.msgpack.Decoder(EngineCoreRequest)
        self._dec = msgspec.msgpack.Decoder()
        self._enc = msgspec.msgpack.Encoder()
        self._kvtreqdec = msgspec.msgpack.Decoder(RKVTDInfo)
        self._dual_req_done: "OrderedDict[str, DualReq]" = OrderedDict()
        self._dual_timer_armed = False     # a wake-up is scheduled for the oldest finished prefill half
        self._infly_kvt: dict[str, PReqMeta] = {}
        self._dinfoq: deque = deque()
        self._gone_reqs: "OrderedDict[str, float]" = OrderedDict()

    # ---- scheduler side: bookkeeping ---------------------------------------------------------------
    def naming_cli(self):
        return self._naming_cli

    def _tp_size(self) -> int:
        return self._cfg.parallel_config.tensor_parallel_size

    def _loop(self):
        return self._engine.get_hybrid_sched_loop()

    def _total_kv_heads(self) -> int:
        mc = self._cfg.model_config
        return 1 if getattr(mc, "use_mla", False) else int(getattr(mc, "num_kv_heads", 0) or 0)

    def _kvt_signals_per_worker(self, dinfo: KVTDInfo) -> int:
        """A prefill rank that fans out to several decode ranks reports once per target."""
        try:
            d_tp = int(dinfo.instid.rsplit("|", 2)[2])
        except (IndexError, ValueError):
            return 1
        p_tp = self._tp_size()
        return d_tp // p_tp if d_tp > p_tp and d_tp % p_tp == 0 else 1

    def _do_send_done(self, worker_tprank: int, ioret: IoRet) -> None:
        if ioret.source is None:
            ioret.source = self.source_label()
        state: Optional[_SendingReq] = try_advance(self._sending, ioret, worker_tprank, self._tp_size())
        if state is not None:
            state.try_mark_done(state.merge())

    async def _on_send_done(self, reader, writer):
        await handle_done_req(reader, writer, self._do_send_done, SEND_DONE_RESP)

    def _mark_gone(self, reqid: str, reason: str) -> None:
        ttl = envs.VLLM_KVT_GONE_REQ_TTL_S
        if ttl <= 0:
            return
        self._gone_reqs.pop(reqid, None)
        self._gone_reqs[reqid] = time.time()
        while len(self._gone_reqs) > self._GONE_REQS_MAX:
            self._gone_reqs.popitem(last=False)
        logger.info("mark gone reqid. reqid=%s reason=%s gone_size=%s", reqid, reason, len(self._gone_reqs))

    def _is_gone(self, reqid: str) -> bool:
        ttl = envs.VLLM_KVT_GONE_REQ_TTL_S
        ts = self._gone_reqs.get(reqid) if ttl > 0 else None
        if ts is None:
            return False
        if time.time() - ts > ttl:
            self._gone_reqs.pop(reqid, None)
            return False
        return True

    def _check_kvtdinfo(self, info: KVTDInfo) -> bool:
        assert info.cached_tokens < info.max_tokens
        if self._naming_cli is None:
            assert info.d_workers_info and all(info.d_workers_info), "fake naming needs the workers' info"
        return True

    def _get_kvblk_ids(self, reqid: str, blks: Optional[list] = None) -> list:
        if blks is None:
            blks = self._engine.sched_get_kvblk_ids(reqid)
        if self.is_hybrid and self._num_gdn_layers > 0:
            blks = handle_hybrid_blocks(blks, self._gamma, self._num_gdn_layers, self._num_kv_cache_groups,
                                        self._cfg.cache_config.mamba_cache_mode == "light", self._ple_group_index)
        return blks

    # ---- scheduler side: RPC handlers (disagg thread) ------------------------------------------------
    async def _wait_kvt_state(self, reqid: str, state: _SendingReq) -> KVTResp:
        t0 = time.monotonic()
        ioret: IoRet = await state._fut
        code = CODE_OK
        if ioret.ex is not None:
            code = ioret.ex.code if isinstance(ioret.ex, CodeError) else CODE_INTERNALERROR
        req = self.get_request(reqid)
        computed = req.num_computed_tokens if req is not None else -1
        logger.info("disagg kvt done. kvt_dur_ms=%.2f reqid=%s cached=%s computed=%s code=%s",
                    (time.monotonic() - t0) * 1000, reqid, ioret.n, computed, code)
        self._sending.pop(reqid, None)
        return KVTResp(code=code, cached=ioret.n or 0, computed=computed, output_token_ids=[])

    async def submit_transfer_kv(self, req: RKVTDInfo) -> KVTResp:
        logger.info("disagg start kvt. reqid=%s peer=%s computed=%s max=%s", req.reqid, req.dinfo.instid,
                    req.dinfo.cached_tokens, req.dinfo.max_tokens)
        assert self._check_kvtdinfo(req.dinfo)
        if req.migration:
            known = self.get_request(req.reqid)
            if req.reqid in self._sending or (known is not None and (get_param(known, P_KVT_STATE) is not None
                                                                      or has_setup_save(known))):
                # This request's KV has been shipped from here before, for a migration that did not take it away
                # in the end (or one is under way).  Its save cannot be set up a second time: the asker is told to
                # keep its hands off instead of tripping the engine over it.
                logger.warning("transfer for migration refused, the request was shipped before: reqid=%s", req.reqid)
                return KVTResp(code=CODE_MIGRATE_REJECTED_BUSY, cached=0, computed=known.num_computed_tokens if known else 0,
                               output_token_ids=[])
        assert req.reqid not in self._sending
        state = _SendingReq(self._kvt_signals_per_worker(req.dinfo))
        self._sending[req.reqid] = state
        self._dinfoq.append(req)
        if len(self._dinfoq) == 1:
            self._connector.wakeup_scheduler()
        return await self._wait_kvt_state(req.reqid, state)

    async def _reply(self, writer, head: int, obj) -> None:
        body = self._enc.encode(obj)
        writer.write(struct.pack("=II", head, len(body)) + body)
        await writer.drain()

    async def _on_transfer_kv(self, reader, writer):
        (n,) = struct.unpack("=I", await reader.readexactly(4))
        req: RKVTDInfo = self._kvtreqdec.decode(await reader.readexactly(n))
        await self._reply(writer, TRANSFER_KV_RESP, await self.submit_transfer_kv(req))

    async def _on_prefill(self, reader, writer):
        (n,) = struct.unpack("=I", await reader.readexactly(4))
        req: EngineCoreRequest = self._reqdec.decode(await reader.readexactly(n))
        raw = core_get_param(req, P_KVTD_INFO)
        assert raw is not None
        dinfo = KVTDInfo(*raw) if not isinstance(raw, KVTDInfo) else raw
        assert self._check_kvtdinfo(dinfo)
        assert dinfo.max_tokens == len(req.prompt_token_ids) - (self._gamma + 1)
        assert len(req.prompt_token_ids) > 1
        logger.info("disagg start prefill. reqid=%s peer=%s computed=%s max=%s", req.request_id, dinfo.instid,
                    dinfo.cached_tokens, dinfo.max_tokens)
        assert req.request_id not in self._sending
        state = _SendingReq(self._kvt_signals_per_worker(dinfo))
        self._sending[req.request_id] = state
        assert req.sampling_params is not None
        req.sampling_params.min_tokens = 0
        req.sampling_params.max_tokens = 1
        core_update_params(req, {P_KVT_STATE: KVTState(dinfo=dinfo, maxtokens=dinfo.max_tokens),
                                 P_IGNORE_OUTPUTS: True, P_KVTD_INFO: None})
        self._engine.core_add_req(req)
        await self._reply(writer, PREFILL_RESP, await self._wait_kvt_state(req.request_id, state))

    def _mark_send_done(self, ioret: IoRet) -> None:
        if ioret.source is None:
            ioret.source = self.source_label()
        state = self._sending.get(ioret.reqid)
        if state is None:
            logger.info("send done: no state: ioret=%s", ioret)
            return
        state.try_mark_done(ioret)

    async def _on_abort_reqs(self, reader, writer):
        (n,) = struct.unpack("=I", await reader.readexactly(4))
        body = await reader.readexactly(n)
        writer.write(struct.pack("=I", ABORT_REQS_RESP))
        reqs = self._dec.decode(body)
        for rid in reqs:
            self._engine.core_abort_req(rid, "pbackend.abort_req", True)
        logger.info("abort reqs=%s", reqs)
        await writer.drain()

    # ---- scheduler side: per-step planning (core thread) ----------------------------------------------
    def _freeze_meta(self, reqid: str, pblkids: list, kvtstate: KVTState) -> PReqMeta:
        d = kvtstate.dinfo
        kvtstate.frozen = True
        return PReqMeta(reqid=reqid, d_inst_id=d.instid, p_block_ids=pblkids, d_block_ids=d.blkids,
                        seen_tokens=d.cached_tokens, new_tokens=kvtstate.maxtokens - d.cached_tokens,
                        has_last_token=True, d_workers_info=d.d_workers_info, has_freeze=True)

    def _dual_req_finish(self, reqid: str, ret: list) -> None:
        dual = self._dual_req_done.get(reqid)
        if dual is None or dual.finished:
            return
        dual.finished = True
        kvtstate: Optional[KVTState] = get_param(dual.req, P_KVT_STATE)
        if kvtstate is None:
            return   # D has not asked yet: keep the finished prefill around
        self._dual_req_done.pop(reqid)
        if kvtstate.untouched:
            kvtstate.untouched = False
            ret.append(self._freeze_meta(reqid, dual.pblkids, kvtstate))

    def _dual_req_get(self, reqid: str) -> tuple:
        dual = self._dual_req_done.get(reqid)
        if dual is None:
            return self.get_request(reqid), False
        return dual.req, dual.finished

    def _step_dinfoq(self, ret: list) -> set:
        """Destination infos that arrived since the last step (dual-request mode, migration)."""
        substep_news: set = set()
        loop = self._loop()
        while self._dinfoq:
            rd: RKVTDInfo = self._dinfoq.popleft()
            dinfo = rd.dinfo
            req, isdone = self._dual_req_get(rd.reqid)
            if req is None:
                gone = self._is_gone(rd.reqid)
                err = CodeError(CODE_REQGONE if gone else CODE_REQNOTFOUND, "req gone" if gone else "req not found")
                loop.call_soon_threadsafe(self._mark_send_done, IoRet(reqid=rd.reqid, ex=err))
                continue
            assert get_param(req, P_KVT_STATE) is None
            maxcomputed = req.max_computed_tokens()
            maxtokens = min(req.num_tokens, dinfo.max_tokens)
            if maxcomputed is not None:
                maxtokens = min(maxtokens, maxcomputed)
            kvtstat = KVTState(dinfo=dinfo, maxtokens=maxtokens, untouched=False)
            set_param(req, P_KVT_STATE, kvtstat)
            if maxcomputed is not None and maxcomputed <= dinfo.cached_tokens:
                # D already holds everything this engine would compute: nothing to send
                loop.call_soon_threadsafe(self._mark_send_done, IoRet(reqid=req.request_id, n=dinfo.cached_tokens))
                self._connector.mark_backend_save_done(req, source=self.source_label())
                self._dual_req_done.pop(req.request_id, None)
                continue
            if not isdone:
                if rd.migration:
                    assert self._connector.try_setup_save(req, source=self.source_label())
                    ret.append(self._freeze_meta(req.request_id, self._get_kvblk_ids(req.request_id), kvtstat))
                else:
                    kvtstat.untouched = True   # still prefilling: chunks leave as they are computed
                    substep_news.add(req.request_id)
                continue
            if dinfo.max_tokens > req.num_prompt_tokens:
                reason = f"reqid={req.request_id} dinfo.max_tokens={dinfo.max_tokens} prompt_len={req.num_prompt_tokens}"
                logger.error("Aborting request due to token mismatch: %s", reason)
                self._engine.core_abort_req(req.request_id, reason, True)
                continue
            dual = self._dual_req_done.pop(req.request_id)
            ret.append(self._freeze_meta(req.request_id, dual.pblkids, kvtstat))
        return substep_news

    def _update_dual_req_done(self, req: Request, islast: bool, pblkids: Optional[list], finished: bool = False):
        if not get_param(req, P_REMOTE_DECODE) or not islast or req.request_id in self._dual_req_done:
            return
        if pblkids is None:
            pblkids = self._get_kvblk_ids(req.request_id)
        self._dual_req_done[req.request_id] = DualReq(req, pblkids, finished)

    def _update_infly_kvt(self, meta: PReqMeta) -> None:
        if meta.d_block_ids:
            assert meta.reqid not in self._infly_kvt
            if not meta.has_last_token:
                self._infly_kvt[meta.reqid] = meta
            return
        assert meta.reqid in self._infly_kvt
        if meta.has_last_token:
            self._infly_kvt.pop(meta.reqid)
        else:
            self._infly_kvt[meta.reqid] = meta

    def _step_finished_reqs(self, sout: SchedulerOutput, kvtpmeta: KVTPMeta) -> None:
        if not self._infly_kvt and not self._dual_req_done:
            return
        for reqid in sout.finished_req_ids:
            meta = self._infly_kvt.pop(reqid, None)
            if meta is None:
                self._dual_req_finish(reqid, kvtpmeta.freeze_metas)
                continue
            # finished (aborted) in the middle of a chunked transfer: close it on the workers
            kvtpmeta.abort_metas.append(PReqMeta(reqid=meta.reqid, d_inst_id="", p_block_ids=[], d_block_ids=[],
                                                 new_tokens=0, has_last_token=True,
                                                 seen_tokens=meta.seen_tokens + meta.new_tokens,
                                                 d_workers_info=meta.d_workers_info))

    def _step_aborting(self, sout: HCSchedOutput) -> None:
        for areq in sout.hc_aborted_save:
            kvstate: Optional[KVTState] = get_param(areq, P_KVT_STATE)
            if kvstate is not None and not kvstate.untouched:
                continue   # chunks are in flight: the workers' send-done closes it
            self._dual_req_done.pop(areq.request_id, None)
            self._mark_gone(areq.request_id, "abort_save")
            if kvstate is not None:
                err = CodeError(CODE_INTERNALERROR, "aborted")
                self._loop().call_soon_threadsafe(self._mark_send_done, IoRet(reqid=areq.request_id, ex=err))
            self._connector.mark_backend_save_done(areq, source=self.source_label())

    def on_queued_req_aborted(self, req: Request) -> None:
        # a decode engine that pushed this request here is waiting for its answer: nothing will ever be sent
        if req.request_id in self._sending:
            self._mark_gone(req.request_id, "abort_queued")
            err = CodeError(CODE_REQGONE, "aborted before it was scheduled")
            self._loop().call_soon_threadsafe(self._mark_send_done, IoRet(reqid=req.request_id, ex=err))

    def _step_stop0(self, sout: HCSchedOutput) -> None:
        for req in sout.hc_stop0:
            assert get_param(req, P_KVT_STATE) is None and req.request_id not in self._dual_req_done
            self._update_dual_req_done(req, True, None, True)

    def _step_dual_req_done(self) -> None:
        now, timeout_s = time.time(), envs.VLLM_PD_TRY_CONNECT_TIMEOUT_SECONDS
        for reqid, dual in list(self._dual_req_done.items()):
            if not dual.finished:
                continue
            if dual.insert_ts + timeout_s > now:
                # Its time is checked where the engine steps; an idle engine does not step.  One timer wakes the
                # scheduler when the oldest parked half is due, so its blocks come back on time either way.
                if not self._dual_timer_armed:
                    self._dual_timer_armed = True
                    delay = dual.insert_ts + timeout_s - now + 0.05
                    loop = self._loop()
                    loop.call_soon_threadsafe(lambda: loop.call_later(delay, self._dual_timer_fired))
                break
            self._engine.core_abort_req(reqid, "dual_req_done.timeout", True)

    def _dual_timer_fired(self) -> None:     # backend loop
        self._dual_timer_armed = False
        self._connector.wakeup_scheduler()

    def _plan_chunk(self, req: Request, reqid: str, seen: int, end: int, p_block_ids: Optional[list], ret: list,
                    substep_mode: bool) -> None:
        """One scheduled request: decide which token range leaves in this step."""
        num_tokens = req.max_computed_tokens()
        if num_tokens is None:
            num_tokens = req.num_prompt_tokens
        has_last = end >= num_tokens
        kvtstate: Optional[KVTState] = get_param(req, P_KVT_STATE)
        if kvtstate is None:
            assert not substep_mode
            self._update_dual_req_done(req, has_last, p_block_ids)
            return
        d_computed = kvtstate.dinfo.cached_tokens
        if end <= d_computed or kvtstate.frozen:
            return   # (a migrating request keeps decoding here until it is suspended)
        has_last = end >= kvtstate.maxtokens
        if substep_mode and not has_last:
            return
        if has_last:
            end = kvtstate.maxtokens
        if kvtstate.untouched:
            seen = 0
        if seen <= d_computed:
            # first chunk that reaches past what D has: carries the block tables
            kvtstate.untouched = False
            meta = PReqMeta(reqid=reqid, d_inst_id=kvtstate.dinfo.instid,
                            p_block_ids=p_block_ids if p_block_ids is not None else self._get_kvblk_ids(reqid),
                            d_block_ids=kvtstate.dinfo.blkids, new_tokens=end - d_computed, has_last_token=has_last,
                            seen_tokens=d_computed, d_workers_info=kvtstate.dinfo.d_workers_info)
        elif seen < kvtstate.maxtokens:
            assert not substep_mode
            meta = PReqMeta(reqid=reqid, d_inst_id="", p_block_ids=[], d_block_ids=[], new_tokens=end - seen,
                            has_last_token=has_last, seen_tokens=seen)
        else:
            return
        ret.append(meta)
        self._update_infly_kvt(meta)

    def _step_sched_req(self, sout: SchedulerOutput, ret: list, substep_news: Optional[set] = None) -> None:
        substep_mode = substep_news is not None
        for rd in sout.scheduled_new_reqs:
            if substep_mode and rd.req_id not in substep_news:
                continue
            req = self.get_request(rd.req_id)
            if req is None:
                continue
            end = sout.num_scheduled_tokens[rd.req_id] + rd.num_computed_tokens
            self._plan_chunk(req, rd.req_id, rd.num_computed_tokens, end, self._get_kvblk_ids(rd.req_id, rd.block_ids),
                             ret, substep_mode)
        cached = sout.scheduled_cached_reqs
        for i, reqid in enumerate(cached.req_ids):
            if substep_mode and reqid not in substep_news:
                continue
            req = self.get_request(reqid)
            if req is None:
                continue
            seen = cached.num_computed_tokens[i]
            self._plan_chunk(req, reqid, seen, seen + sout.num_scheduled_tokens[reqid], None, ret, substep_mode)

    async_get_num_new_matched_tokens = None  # type: ignore[assignment]  (a prefill engine never loads)

    def get_operations(self, req: Request) -> OperationPlan:
        if self._cfg.model_config.is_hybrid:
            # a hybrid model's last gamma+1 prompt tokens are recomputed on the decode side
            if len(req.prompt_token_ids) <= self._gamma + 1:
                return 0, 0, (), ()
            req.prompt_token_ids = req.prompt_token_ids[:-(self._gamma + 1)]
            req._all_token_ids = list(req.prompt_token_ids)
            req.num_prompt_tokens = len(req.prompt_token_ids)
        if get_param(req, P_KVT_STATE) is not None:
            return 0, 1, (), (self.source_label(),)
        if get_param(req, P_REMOTE_DECODE):
            if req.num_prompt_tokens <= 1:
                return 0, 0, (), ()
            return 0, 1, (), (self.source_label(),)
        return 0, 0, (), ()

    def build_backend_meta(self, sout: SchedulerOutput) -> BackendMeta:
        assert isinstance(sout, HCSchedOutput)
        meta = KVTPMeta(stepid=sout.hc_stepid, substepid=sout.hc_substepid,
                        sched_tokens=sout.total_num_scheduled_tokens)
        self._step_stop0(sout)
        self._step_aborting(sout)
        substep_news = self._step_dinfoq(meta.freeze_metas)
        self._step_finished_reqs(sout, meta)
        self._step_dual_req_done()
        if sout.hc_parent is None:
            self._step_sched_req(sout, meta.nonfreeze_metas)
            if substep_news:
                # infos that arrived for requests scheduled in this very step were handled above;
                # nothing more to do: their chunks are in nonfreeze_metas
                pass
        elif substep_news and envs.VLLM_ENABLE_BYPASS_SUBSTEP:
            self._step_sched_req(sout.hc_parent, meta.nonfreeze_metas, substep_news=substep_news)
        return meta

    # ---- worker side ---------------------------------------------------------------------------------
    def register_kv_caches(self, kv_caches: dict) -> None:
        import llumnix_kv_b200
        from llumnix_kv_b200.kv_transfer_impl import KVTransferClient

        llumnix_kv_b200.set_envs()
        _worker_process_envs(self._cfg)
        args = build_kvt_args(self, kv_caches, self._worker.get_tensor_model_parallel_rank())
        self._kvt_cli = KVTransferClient(send_done_addr=self._send_done_addr, **args)
        self._layer_index = {name: extract_layer_index(name) for name in kv_caches}
        # a layer with several cache tensors (latent + indexer keys) is announced once, by the tensor
        # that is written last
        last_of: dict = {}
        for name in sorted(kv_caches):
            last_of[self._layer_index[name]] = name
        self._announcing = set(last_of.values())
        logger.info("register_kv_caches (prefill). worker_id=%s winfo=%s", args["worker_id"],
                    self._kvt_cli.worker_info())

    def _send_error_done_in_loop(self, reqids: list) -> None:
        if not reqids:
            return

        async def do_send():
            try:
                await self._kvt_cli.send_error_done_req(reqids)
            except Exception:
                logger.exception("_send_error_done_in_loop: failed")

        asyncio.run_coroutine_threadsafe(do_send(), self._worker.get_hybrid_worker_loop())

    def _build_req_send_batch(self, metas: list, expect_freeze: bool) -> tuple:
        from llumnix_kv_b200.kv_transfer_impl import ReqMeta

        rank, tp = self._worker.get_tensor_model_parallel_rank(), self._tp_size()
        out, failed = [], []
        for m in metas:
            assert m.has_freeze == expect_freeze
            assert m.has_last_token and m.d_block_ids and m.d_inst_id
            dist = get_distinfo(m, rank, tp)
            if not dist:
                logger.warning("get_distinfo failed req=%s", m)
                failed.append(m.reqid)
                continue
            for name, wid, winfo in dist:
                r = ReqMeta()
                r.dst_inst, r.dst_worker, r.reqid = name, wid, m.reqid
                r.seen_tokens, r.new_tokens = m.seen_tokens, m.new_tokens
                r.src_block_ids, r.dst_block_ids, r.dst_worker_info = m.p_block_ids, m.d_block_ids, winfo
                out.append(r)
        return out, failed

    def _bind_prologue(self, meta: BackendMeta) -> Optional[tuple]:
        assert isinstance(meta, KVTPMeta)
        if self._kvt_cli is None:
            assert not meta
            return None
        failed: list = []
        if meta.freeze_metas:
            batch, failed = self._build_req_send_batch(meta.freeze_metas, True)
            if batch:
                self._kvt_cli.start_req_send(batch, meta.stepid, meta.substepid)
        return meta, failed

    def bind_backend_metadata(self, meta: BackendMeta) -> None:
        pro = self._bind_prologue(meta)
        if pro is None:
            return
        meta, failed = pro
        assert meta.substepid == 0, "bind_backend_metadata is the main step path"
        rank, tp = self._worker.get_tensor_model_parallel_rank(), self._tp_size()
        for m in meta.abort_metas:
            assert m.new_tokens == 0 and m.has_last_token and not m.has_freeze
            self._kvt_cli.submit_delta_send(m.reqid, m.seen_tokens, m.new_tokens, m.has_last_token, stepid=meta.stepid)
        for m in meta.nonfreeze_metas:
            assert not m.has_freeze
            if not m.d_block_ids:
                self._kvt_cli.submit_delta_send(m.reqid, m.seen_tokens, m.new_tokens, m.has_last_token,
                                                stepid=meta.stepid)
                continue
            dist = get_distinfo(m, rank, tp)
            if not dist:
                logger.warning("bind_backend_metadata: get_distinfo failed req=%s", m)
                failed.append(m.reqid)
                continue
            try:
                relay = choose_relay(m.reqid, dist, self._total_kv_heads(), tp)
                if relay is not None:
                    # one decode worker receives the request and stores it to its group through NVSwitch:
                    # this rank's link carries the bytes once instead of len(dist) times
                    name, wid, winfo = dist[relay]
                    self._kvt_cli.submit_req_send2(name, wid, m.reqid, m.seen_tokens, m.new_tokens, m.has_last_token,
                                                   m.p_block_ids, m.d_block_ids, winfo, stepid=meta.stepid, fanout=len(dist))
                    continue
                for name, wid, winfo in dist:
                    self._kvt_cli.submit_req_send2(name, wid, m.reqid, m.seen_tokens, m.new_tokens, m.has_last_token,
                                                   m.p_block_ids, m.d_block_ids, winfo, stepid=meta.stepid)
            except Exception:
                logger.exception("bind_backend_metadata: submit_req_send2 failed req=%s", m)
                failed.append(m.reqid)
        if failed:
            self._send_error_done_in_loop(failed)
        self._kvt_cli.start_send_step(stepid=meta.stepid, sched_tokens=meta.sched_tokens)

    def bypass_bind(self, meta: BackendMeta) -> None:
        pro = self._bind_prologue(meta)
        if pro is None:
            return
        meta, failed = pro
        assert meta.substepid != 0 and not meta.abort_metas
        if meta.nonfreeze_metas:
            batch, f2 = self._build_req_send_batch(meta.nonfreeze_metas, False)
            failed.extend(f2)
            if batch:
                self._kvt_cli.start_send_substep(meta.stepid, meta.substepid, batch)
        if failed:
            self._send_error_done_in_loop(failed)

    def clear_backend_metadata(self) -> None:
        if self._kvt_cli is not None:
            self._kvt_cli.flush_send_step()

    def bypass_clear(self) -> None:
        return

    async_load_kv = None  # type: ignore[assignment]

    def async_save_kv_layer(self, layer_name: str, kv_layer, m: BackendMeta):
        """The layer's KV has been enqueued on the current stream: record its event so the transfer
        of this layer can start while the forward pass goes on."""
        if self._kvt_cli is None:
            return None
        idx = self._layer_index.get(layer_name)
        if idx is None:
            idx = extract_layer_index(layer_name)
        elif layer_name not in self._announcing:
            return None
        if self.is_hybrid:
            if idx not in self.hybrid_model_send_layer:
                return None
            idx = self.hybrid_model_send_layer.index(idx)
        stream = None
        if self._kvt_cli._device_id >= 0:
            import torch

            stream = torch.cuda.current_stream()
        self._kvt_cli.record_event(idx, stream)
        return None


# ======================================================================================================
class DBackend(HybridBackend):
    SOURCE_LABEL = "kvt"

    def __init__(self, vllm_config: VllmConfig, role: KVConnectorRole, kv_cache_config=None, **kw):
        super().__init__(vllm_config, role, kv_cache_config, **kw)
        kcfg = vllm_config.kv_transfer_config
        assert kcfg is not None
        self._cfg = vllm_config
        self._naming_url = kcfg.get_from_extra_config("naming_url", "fake://")
        fake = self._naming_url == "fake://"
        self._inst_id = get_inst_id(vllm_config, fake_naming=fake)
        self._naming_cli = None
        if not fake:
            from llumnix_kv_b200.kv_transfer_impl import connect_naming

            self._naming_cli = connect_naming(self._inst_id, self._naming_url)
        self._gamma = get_p_node_pop_len(vllm_config) - 1
        self._kvt_srv = None
        self._delay_s_list = self._generate_delay_list()
        if role == KVConnectorRole.WORKER:
            self._loop = self._worker.get_hybrid_worker_loop()
            return
        self._loop = self._engine.get_hybrid_sched_loop()
        self.my_addr_port = (envs.get_ip(), sched_rpc_server_port(vllm_config))
        interested: Optional[str] = "prefill"
        if kcfg.get_from_extra_config("backend", None) in ("kvt+migration", "migration+kvt"):
            interested = None
        self._conn_mgr = ConnManager(envs.VLLM_PD_CONNMANAGER_CAP)
        self._workers_info: list = []
        self._workers_info_lock = threading.Lock()
        self._workers_info_event = threading.Event()
        self._enc = msgspec.msgpack.Encoder()
        self._kvtrespdec = msgspec.msgpack.Decoder(KVTResp)
        self._strdec = msgspec.msgpack.Decoder(str)
        if self._naming_cli is not None:
            self._pmgr: Optional[PeerManager] = PeerManager(self._naming_cli, interested, self._conn_mgr)
            self._pmgr.start(self._loop)
            reg_naming(self._naming_cli, vllm_config)
            self._workers_info_event.set()
        else:
            self._pmgr = None
            self._workers_info = [""] * self._tp_size()
            self._engine.sched_rpc_server().register_method(REGISTER_WORKER, self._on_register_worker)

    def _generate_delay_list(self) -> list:
        """Back-off of the dual-request 404 retry: 1, 3, 7, 11, 17 ms, then 100 ms doubling, the sum
        capped by VLLM_KVT_MAX_DELAY_MS."""
        cap = envs.VLLM_KVT_MAX_DELAY_MS
        out, total = [], 0.0
        for d in (1, 3, 7, 11, 17):
            if total + d >= cap:
                break
            out.append(d)
            total += d
        step = 100.0
        while total < cap:
            d = min(step, cap - total)
            out.append(d)
            total += d
            step *= 2
        return [d / 1000.0 for d in out]

    def _tp_size(self) -> int:
        return self._cfg.parallel_config.tensor_parallel_size

    def naming_cli(self):
        return self._naming_cli

    def wait_workers_registered(self, timeout: Optional[float] = None) -> bool:
        """Without a naming service the scheduler half learns its workers' WorkerInfo through
        REGISTER_WORKER; requests can only be served once every rank has registered."""
        return self._workers_info_event.wait(timeout)

    async def _on_register_worker(self, reader, writer):
        (n,) = struct.unpack("=I", await reader.readexactly(4))
        body = await reader.readexactly(n)
        writer.write(struct.pack("=I", REGISTER_WORKER_RESP))
        text = self._strdec.decode(body)
        parts = text.split("|", 1)   # the WorkerInfo itself contains '|'
        if len(parts) != 2:
            raise RuntimeError(f"Invalid worker registration format: {text}")
        rank, winfo = int(parts[0]), parts[1]
        with self._workers_info_lock:
            if rank < len(self._workers_info):
                self._workers_info[rank] = winfo
                logger.info("DBackend registered worker %d with winfo: %s", rank, winfo)
                if all(self._workers_info) and not self._workers_info_event.is_set():
                    self._workers_info_event.set()
            else:
                logger.error("Worker rank %d exceeds tp_size %d", rank, self._tp_size())
        await writer.drain()

    def get_peer(self, hint: Optional[tuple] = None, exclude: Optional[tuple] = None) -> Optional[tuple]:
        if hint is not None:
            return hint
        return None if self._pmgr is None else self._pmgr.get_peer(exclude)

    async def _kvt_rpc(self, req: Request, msg: bytes, peer_hint: Optional[tuple]) -> KVTResp:
        peer: Optional[tuple] = None
        for retry in range(2):
            try:
                peer = self.get_peer(hint=peer_hint, exclude=self.my_addr_port)
                logger.info("disagg start kvt. reqid=%s retry=%s hint=%s peer=%s msglen=%s", req.request_id, retry,
                            peer_hint, peer, len(msg))
                if peer is None:
                    raise RuntimeError("no p")
                set_param(req, D_PID, f"{peer[0]}:{peer[1]}")
                if req_aborted(req):
                    raise RuntimeError("req aborted")
                conn = await self._conn_mgr.acquire_conn(peer, retry > 0)
                conn[1].write(msg)
                await conn[1].drain()
                head, n = struct.unpack("=II", await conn[0].readexactly(8))
                if head != PREFILL_RESP:
                    raise RuntimeError(f"invalid resp head={head:#x}")
                resp: KVTResp = self._kvtrespdec.decode(await conn[0].readexactly(n))
                self._conn_mgr.release_conn(peer, conn)
                return resp
            except (asyncio.IncompleteReadError, ConnectionError):
                logger.warning("do kvt failed (stale connection?). peer=%s retry=%s", peer, retry)
            await asyncio.sleep(0)
        raise RuntimeError("kvt rpc failed")

    def _get_kvblk_ids(self, reqid: str) -> list:
        blks = self._engine.sched_get_kvblk_ids(reqid)
        if self.is_hybrid and self._num_gdn_layers > 0:
            blks = handle_hybrid_blocks(blks, self._gamma, self._num_gdn_layers, self._num_kv_cache_groups,
                                        self._cfg.cache_config.mamba_cache_mode == "light", self._ple_group_index)
        return blks

    def _make_dinfo(self, req: Request) -> KVTDInfo:
        blockids = self._get_kvblk_ids(req.request_id)
        self._engine.sched_discard_zero_block_ids(b for g in blockids for b in g)
        pc = self._cfg.parallel_config
        return KVTDInfo(instid=f"{self._inst_id}|{pc.data_parallel_rank}|{pc.tensor_parallel_size}", blkids=blockids,
                        cached_tokens=req.num_computed_tokens, max_tokens=req.num_prompt_tokens - (self._gamma + 1),
                        d_workers_info=list(self._workers_info))

    @staticmethod
    def _peer_hint(req: Request) -> Optional[tuple]:
        host, port = get_param(req, "remote_host"), get_param(req, "remote_port")
        return (host, int(port)) if host is not None and port is not None else None

    async def _prefill_rpc(self, req: Request, blocks: KVCacheBlocks) -> int:
        corereq = self._engine.req2corereq(req)
        dinfo = self._make_dinfo(req)
        core_update_params(corereq, {P_KVTD_INFO: dinfo})
        body = msgspec.msgpack.encode(corereq)
        t0 = time.monotonic()
        resp = await self._kvt_rpc(req, struct.pack("=II", PREFILL_REQ, len(body)) + body, self._peer_hint(req))
        logger.info("disagg end prefill. reqid=%s prompt=%s dur_ms=%.2f kvtresp=%s", req.request_id,
                    req.num_prompt_tokens, (time.monotonic() - t0) * 1000, resp)
        if resp.code != CODE_OK:
            raise RuntimeError(f"bad resp code={resp.code}")
        return resp.cached

    async def _dual_req_prefill_rpc(self, req: Request, blocks: KVCacheBlocks) -> int:
        body = self._enc.encode(RKVTDInfo(reqid=req.request_id, dinfo=self._make_dinfo(req)))
        msg = struct.pack("=II", TRANSFER_KV_REQ, len(body)) + body
        hint = self._peer_hint(req)
        assert hint is not None
        for retry, delay in enumerate(self._delay_s_list):
            if req_aborted(req):
                raise RuntimeError("req aborted")
            t0 = time.monotonic()
            resp = await self._kvt_rpc(req, msg, hint)
            logger.info("disagg end dual_req prefill. reqid=%s dur_ms=%.2f kvtresp=%s retry=%s", req.request_id,
                        (time.monotonic() - t0) * 1000, resp, retry)
            if resp.code == CODE_OK:
                return resp.cached
            if resp.code == CODE_REQNOTFOUND:
                await asyncio.sleep(delay)   # P may simply not have received its half yet
                continue
            if resp.code == CODE_REQGONE:
                raise RuntimeError(f"kv gone on P (reqid={req.request_id}, peer={hint}, retry={retry})")
            raise RuntimeError(f"bad resp code={resp.code}")
        raise RuntimeError("bad 404 resp")

    async def _abort_rpc(self, addr_port_str: str, reqids: list) -> None:
        addr, port = addr_port_str.rsplit(":", 1)
        peer = (addr, int(port))
        body = self._enc.encode(reqids)
        msg = struct.pack("=II", ABORT_REQS_REQ, len(body)) + body
        for retry in range(2):
            try:
                conn = await self._conn_mgr.acquire_conn(peer, retry > 0)
                conn[1].write(msg)
                await conn[1].drain()
                (head,) = struct.unpack("=I", await conn[0].readexactly(4))
                if head != ABORT_REQS_RESP:
                    raise RuntimeError(f"invalid resp head={head}")
                self._conn_mgr.release_conn(peer, conn)
                logger.info("abort rpc end. peer=%s reqids=%s", addr_port_str, reqids)
                return
            except Exception:
                logger.exception("abort rpc failed. peer=%s reqids=%s", addr_port_str, reqids)
            await asyncio.sleep(0)

    @kill_me_if_exception
    async def _abort_prefill(self, reqs: list):
        by_peer: dict = defaultdict(list)
        for req in reqs:
            peer = get_param(req, D_PID, None)
            if peer is None:
                logger.info("abort prefill: reqid=%s peer=None", req.request_id)
                continue
            by_peer[peer].append(req.request_id)
        await asyncio.gather(*(self._abort_rpc(p, ids) for p, ids in by_peer.items()))

    async def async_get_num_new_matched_tokens(self, req: Request, local_tokens: int) -> int:
        assert local_tokens % self._cfg.cache_config.block_size == 0 and local_tokens <= req.num_prompt_tokens
        left = req.num_prompt_tokens - local_tokens
        gamma = 0
        if self._cfg.speculative_config and self._cfg.speculative_config.num_speculative_tokens:
            gamma = self._cfg.speculative_config.num_speculative_tokens
        # the last gamma+1 prompt tokens are always computed locally (they produce the first output)
        return 0 if left <= gamma + 1 else left - (gamma + 1)

    async def async_update_state_after_alloc(self, request: Request, blocks: KVCacheBlocks, rmt_tokens: int):
        if rmt_tokens <= 0:
            return None
        ioret = IoRet(n=0)
        try:
            if get_param(request, D_REMOTE_PREFILL):
                cached = await self._dual_req_prefill_rpc(request, blocks)
            else:
                cached = await self._prefill_rpc(request, blocks)
            ioret.n = min(cached - request.num_computed_tokens, rmt_tokens)
        except Exception as e:
            logger.warning("load fail. req=%s ex=%r", request.request_id, e)
            ioret.ex = e
        return ioret

    def get_operations(self, req: Request) -> OperationPlan:
        if req.num_prompt_tokens <= 1:
            return 0, 0, (), ()
        if get_param(req, D_REMOTE_PREFILL):
            assert get_param(req, "remote_host") is not None and get_param(req, "remote_port") is not None
            return 1, 0, (self.source_label(),), ()
        if not get_param(req, D_DISAGG, True):
            return 0, 0, (), ()
        return 1, 0, (self.source_label(),), ()

    def build_backend_meta(self, sout: SchedulerOutput) -> BackendMeta:
        assert isinstance(sout, HCSchedOutput)
        if sout.hc_aborted_load:
            asyncio.run_coroutine_threadsafe(self._abort_prefill(list(sout.hc_aborted_load)), self._loop)
        return BackendMeta()

    # ---- worker side -----------------------------------------------------------------------------------
    def register_kv_caches(self, kv_caches: dict) -> None:
        import llumnix_kv_b200
        from llumnix_kv_b200.kv_transfer_impl import KVTransferServer

        llumnix_kv_b200.set_envs()
        _worker_process_envs(self._cfg)
        rank = self._worker.get_tensor_model_parallel_rank()
        args = build_kvt_args(self, kv_caches, rank)
        args.update(multicast_kwargs(args["layers"]))
        self._kvt_srv = KVTransferServer(mx_scaled=self._cfg.cache_config.mx_scaled, **args)
        winfo = self._kvt_srv.worker_info()
        logger.info("register_kv_caches (decode). worker_id=%s winfo=%s", args["worker_id"], winfo)
        if self._naming_cli is not None:
            self._naming_cli.store(f"worker_{args['worker_id']}", winfo)
        else:
            asyncio.run_coroutine_threadsafe(self._register_worker_rpc(rank, winfo), self._loop)

    async def _register_worker_rpc(self, rank: int, winfo: str) -> None:
        body = msgspec.msgpack.encode(f"{rank}|{winfo}")
        msg = struct.pack("=II", REGISTER_WORKER, len(body)) + body
        host, port = scheduler_rpc_host(self._cfg), sched_rpc_server_port(self._cfg)
        while True:
            try:
                reader, writer = await asyncio.open_connection(host, port)
                writer.write(msg)
                await writer.drain()
                (head,) = struct.unpack("=I", await asyncio.wait_for(reader.readexactly(4), timeout=3.0))
                if head != REGISTER_WORKER_RESP:
                    raise RuntimeError(f"invalid response head={head:#x}")
                writer.close()
                logger.info("DBackend worker %d registered via RPC", rank)
                return
            except RuntimeError:
                raise
            except Exception as e:   # scheduler not listening yet
                logger.debug("worker registration retry: %s", e)
                await asyncio.sleep(0.1)

    async_load_kv = None  # type: ignore[assignment]  (data lands by itself; completion comes from P)

    def stop(self) -> None:
        if self._kvt_srv is not None:
            self._kvt_srv.stop()
