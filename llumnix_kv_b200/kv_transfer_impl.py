"""``KVTransferClient`` / ``KVTransferServer``: Python face of the native engine.

Signatures follow ``blade_kvt/kv_transfer_impl.py:141-700``.  Differences that matter:

* cache tensors may be CUDA tensors (device transports: NVLink, plus TCP / shared memory with
  kernel gather/scatter) or CPU tensors (host transports only; used for CPU-only plumbing);
* ``cache_shape`` names the paged layout of *this* worker (the reference has one process-wide
  ``BLLM_KVTRANS_CACHE_SHAPE``); it travels to the peer so that a prefill worker with a
  FlashAttention NHD cache can fill a decode worker's FlashInfer HND cache;
* several clients / servers can exist in one process (``process_global=False``).
"""
from __future__ import annotations

import asyncio
import enum
import logging
import os
import struct
from typing import List, Optional, Union

import torch

from llumnix_kv_b200 import load_ops

_K = load_ops()
ReqMeta = _K.ReqMeta
TransferProtocol = _K.TransferProtocol

logger = logging.getLogger("llumnix_kv_b200")

DEFAULT_STEPID = 1024
DEFAULT_SUBSTEPID = 0
EMPTY_STEP_ID = 9223372036854775807

SEND_DONE_REQ = 0x20181219
SEND_DONE_RESP = 0x91218102
SAVE_DONE2_REQ = 0x20181223
SEND_DONE_HEAD_KIND = 1
SEND_SAVE_DONE_HEAD_KIND = 2
CODE_INTERNALERROR = 500


def _get_send_done_addr() -> Optional[tuple]:
    addr = os.environ.get("BLLM_KVTRANS_SEND_DONE_ADDR")
    if not addr:
        return None
    parts = addr.split(":")
    if len(parts) != 2:
        return None
    return parts[0], int(parts[1])


def _get_send_done_head_kind() -> int:
    val = os.environ.get("BLLM_KVTRANS_SDH_KIND")
    return SEND_SAVE_DONE_HEAD_KIND if val is None else int(val)


@enum.unique
class KVTransferProtocolType(enum.Enum):
    RDMA_DIRECT = enum.auto()
    TCP = enum.auto()
    UNKNOWN = enum.auto()
    NVLINK = enum.auto()
    SHM = enum.auto()

    def to_ops_protocol(self):
        kind = {
            KVTransferProtocolType.RDMA_DIRECT: TransferProtocol.Kind.RDMA_DIRECT,
            KVTransferProtocolType.TCP: TransferProtocol.Kind.TCP,
            KVTransferProtocolType.NVLINK: TransferProtocol.Kind.NVLINK,
            KVTransferProtocolType.SHM: TransferProtocol.Kind.SHM,
        }.get(self)
        if kind is None:
            raise RuntimeError("unknown protocol type: " + self.name)
        return TransferProtocol(kind)

    @classmethod
    def to_protocol_type(cls, protocol_kind: str) -> "KVTransferProtocolType":
        return {"rdma": cls.RDMA_DIRECT, "tcp": cls.TCP, "nvlink": cls.NVLINK, "shm": cls.SHM}.get(
            protocol_kind, cls.UNKNOWN)


def support_transfers_protocols() -> List[KVTransferProtocolType]:
    out = []
    for p in _K.lib_support_transfer_protocols():
        out.append(KVTransferProtocolType.to_protocol_type(p.to_string()))
    return out


def connect_naming(inst_id: str, url: str):
    return _K.connect_naming(inst_id, url)


def current_worker_info(kind: str = "any") -> str:
    return _K.current_worker_info(kind)


class _DeviceBuffer:
    """Owner of one ``cudaMalloc`` allocation, exposed to torch through the CUDA array interface."""

    def __init__(self, nbytes: int, device_index: int):
        with torch.cuda.device(device_index):
            self.ptr = _K.kvt_malloc(nbytes)
        self.nbytes, self.device_index = nbytes, device_index
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (self.ptr, False), "version": 3,
                                         "strides": None}

    def __del__(self):
        try:
            with torch.cuda.device(self.device_index):
                _K.kvt_free(self.ptr)
        except Exception:  # interpreter shutdown: the driver reclaims it
            pass


def alloc_phy_cont_mem(nbytes: int, device_index: int = 0) -> torch.Tensor:
    """KV-cache storage from the framework instead of the engine's caching allocator: one whole
    ``cudaMalloc`` allocation, so its CUDA IPC handle covers exactly this cache and peers can map it
    (the hook the reference offers for RDMA-registrable memory, kvtransfer/src/barex_protocol.cpp:808-830,
    blade_kvt/hybrid_connector/kvtbackend.py:330-364).  Returns a flat uint8 tensor that keeps the
    allocation alive."""
    buf = _DeviceBuffer(int(nbytes), device_index)
    t = torch.as_tensor(buf, device=torch.device("cuda", device_index))
    t._kvx_owner = buf        # the tensor does not own the memory: tie the owner's life to it
    return t


def alloc_kv_cache_peer_mappable(cache: torch.Tensor) -> torch.Tensor:
    """Same shape / dtype / strides as ``cache`` but backed by :func:`alloc_phy_cont_mem` (the
    engine swaps its cache tensor for the returned one before registering it)."""
    flat = alloc_phy_cont_mem(cache.untyped_storage().nbytes(), cache.device.index or 0)
    out = flat.view(cache.dtype).as_strided(cache.size(), cache.stride(), cache.storage_offset())
    out._kvx_owner = flat
    return out


def _get_layer_num_blocks(layers: List[torch.Tensor], block_bytes: int) -> int:
    if block_bytes <= 0:
        raise ValueError(f"block_bytes must be positive, got {block_bytes}")
    first = layers[0]
    sig0 = (first.shape, first.stride(), first.dtype, first.device, first.nbytes)
    for idx, layer in enumerate(layers):
        sig = (layer.shape, layer.stride(), layer.dtype, layer.device, layer.nbytes)
        if sig != sig0:
            raise ValueError("All registered KV layers must have identical layout; "
                             f"layer_idx={idx}, expected={sig0}, actual={sig}")
        if layer.nbytes % block_bytes != 0:
            raise ValueError("KV layer size is not divisible by block_bytes; "
                             f"layer_idx={idx}, nbytes={layer.nbytes}, block_bytes={block_bytes}")
    return first.nbytes // block_bytes


def _normalise(block_bytes, token_bytes, layers):
    if isinstance(block_bytes, int) and isinstance(token_bytes, int):
        block_bytes, token_bytes = [block_bytes], [token_bytes]
        layers = [[layer] for layer in layers]
    elif not isinstance(block_bytes, list) or not isinstance(token_bytes, list):
        raise TypeError("block_bytes and token_bytes must both be int or list")
    if any(len(layer) != len(layers[0]) for layer in layers):
        raise ValueError("All layers must have the same number of cache tensors")
    if not len(block_bytes) == len(token_bytes) == len(layers[0]):
        raise ValueError("block_bytes and token_bytes must align with the number of cache tensors per layer")
    nblocks = [_get_layer_num_blocks([layer[i] for layer in layers], block_bytes[i]) for i in range(len(block_bytes))]
    if not all(n == nblocks[0] for n in nblocks):
        raise ValueError(f"All cache tensors in one layer must have the same number of blocks, got {nblocks}")
    dev = layers[0][0].device
    device_id = dev.index if dev.type == "cuda" else -1
    if dev.type == "cuda" and device_id is None:
        device_id = torch.cuda.current_device()
    return block_bytes, token_bytes, layers, nblocks[0], device_id


def _hybrid_kwargs(num_kv_heads, num_gdn_layers, indexer_blk_ntpb, hybrid_indexer_token_size, gdn_conv_elem_size,
                   gdn_ssm_elem_size, conv_state_shape, ssm_state_shape, gdn_conv_channel_dims, kda_conv_dim_first,
                   hybrid_attn_token_size, kda_page_stride, attn_pack_size, num_ple_layers, ple_block_group,
                   ple_conv_elem_size, ple_conv_state_shape, ple_conv_channel_dims):
    return dict(
        num_kv_heads=num_kv_heads, num_gdn_layers=num_gdn_layers, indexer_blk_ntpb=indexer_blk_ntpb,
        hybrid_indexer_token_size=hybrid_indexer_token_size, gdn_conv_elem_size=gdn_conv_elem_size,
        gdn_ssm_elem_size=gdn_ssm_elem_size, conv_state_shape=list(conv_state_shape or []),
        ssm_state_shape=list(ssm_state_shape or []), gdn_conv_channel_dims=list(gdn_conv_channel_dims or []),
        kda_conv_dim_first=kda_conv_dim_first, hybrid_attn_token_size=hybrid_attn_token_size,
        kda_page_stride=kda_page_stride, attn_pack_size=attn_pack_size, num_ple_layers=num_ple_layers,
        ple_block_group=ple_block_group, ple_conv_elem_size=ple_conv_elem_size,
        ple_conv_state_shape=list(ple_conv_state_shape or []),
        ple_conv_channel_dims=list(ple_conv_channel_dims or []))


class KVTransferClient:
    """Sender side: submit request chunks, open a step, record one event per layer, flush."""

    def __init__(self, inst_id: str, tp_size: int, worker_id: int, worker_tp_rank: int,
                 block_bytes: Union[List[int], int], token_bytes: Union[List[int], int], naming_url: str,
                 layers: Union[List[List[torch.Tensor]], List[torch.Tensor]],
                 protocols: List[KVTransferProtocolType], num_kv_heads: int = -1, num_gdn_layers: int = 3,
                 indexer_blk_ntpb: int = 0, hybrid_indexer_token_size: int = 0, gdn_conv_elem_size: int = 1,
                 gdn_ssm_elem_size: int = 1, conv_state_shape=None, ssm_state_shape=None,
                 gdn_conv_channel_dims=None, kda_conv_dim_first: bool = False, hybrid_attn_token_size: int = 0,
                 kda_page_stride: int = 0, attn_pack_size: int = 1, num_ple_layers: int = 0,
                 ple_block_group: int = 0, ple_conv_elem_size: int = 1, ple_conv_state_shape=None,
                 ple_conv_channel_dims=None, cache_shape: int = -1, process_global: bool = False,
                 send_done_addr: Optional[str] = None, mc_layers=None, mc_size: int = 0):
        """``mc_layers`` / ``mc_size``: this worker's GPU is bound to the NVLink multicast object of a decode
        group's caches (it is a member of the same symmetric allocation, with memory of its own that only
        absorbs the echo), and ``mc_layers`` gives ITS mapping of the multicast address of every decode cache
        tensor, shaped like ``layers``.  Requests submitted with ``fanout=k`` to a worker of that group then
        leave as multicast stores from this GPU: no decode worker has to receive and relay them."""
        block_bytes, token_bytes, layers, layer_num_blocks, device_id = _normalise(block_bytes, token_bytes, layers)
        self._num_layers = len(layers)
        self._device_id = device_id
        self._init_events()
        layer_addrs = [[t.data_ptr() for t in layer] for layer in layers]
        kw = _hybrid_kwargs(num_kv_heads, num_gdn_layers, indexer_blk_ntpb, hybrid_indexer_token_size,
                            gdn_conv_elem_size, gdn_ssm_elem_size, conv_state_shape, ssm_state_shape,
                            gdn_conv_channel_dims, kda_conv_dim_first, hybrid_attn_token_size, kda_page_stride,
                            attn_pack_size, num_ple_layers, ple_block_group, ple_conv_elem_size,
                            ple_conv_state_shape, ple_conv_channel_dims)
        if mc_layers is not None and mc_size > 1:
            mc = [[int(a)] if isinstance(a, int) else [int(x) for x in a] for a in mc_layers]
            assert len(mc) == len(layer_addrs) and all(len(a) == len(b) for a, b in zip(mc, layer_addrs))
            kw["mc_layers"], kw["mc_size"] = mc, int(mc_size)
        ops_protocols = [p.to_ops_protocol() for p in protocols]
        logger.info("init kvt client: instid=%s tpsize=%s wid=%s wrank=%s blockbytes=%s tokenbytes=%s naming=%s "
                    "protocols=%s device_id=%s num_blocks=%s num_layers=%s cache_shape=%s", inst_id, tp_size,
                    worker_id, worker_tp_rank, block_bytes, token_bytes, naming_url, protocols, device_id,
                    layer_num_blocks, len(layers), cache_shape)
        self._global = process_global
        if process_global:
            _K.init_kv_transfer_client(inst_id, tp_size, worker_id, worker_tp_rank, device_id, block_bytes,
                                       token_bytes, layer_num_blocks, naming_url, self._event_addrs, layer_addrs,
                                       ops_protocols, cache_shape=cache_shape, **kw)
            self._c = None
        else:
            self._c = _K.KvClient(inst_id, tp_size, worker_id, worker_tp_rank, device_id, block_bytes, token_bytes,
                                  layer_num_blocks, naming_url, self._event_addrs, layer_addrs, ops_protocols,
                                  cache_shape, send_done_addr=send_done_addr, **kw)
        self._send_done_addr = None
        if send_done_addr:
            h, p = send_done_addr.rsplit(':', 1)
            self._send_done_addr = (h, int(p))
        self._layers = layers  # keep the tensors alive as long as the engine holds their addresses
        self._inited = True
        self._cur_step_id: Optional[int] = None
        self._worker_tp_rank = worker_tp_rank
        self._async_sched_warned = False

    def _init_events(self):
        if self._device_id >= 0:
            with torch.cuda.device(self._device_id):
                # interprocess: a decode worker that pulls this cache orders its streams after these events
                # (CUDA IPC event handles), so nobody's host waits for the forward pass
                self._events = [torch.cuda.Event(interprocess=True) for _ in range(self._num_layers)]
                for ev in self._events:
                    ev.record()
            self._event_addrs = [ev.cuda_event for ev in self._events]
        else:
            self._events = []
            self._event_addrs = []

    # ---- engine calls ---------------------------------------------------------------------
    def _call(self, name, *args):
        if self._c is not None:
            return getattr(self._c, name)(*args)
        return getattr(_K, name)(*args)

    def add_worker(self, inst_id, worker_id, start_layer, num_layers, protocol=None):
        if not self._inited:
            raise RuntimeError("KVTransferClient not inited")
        _K.add_target(inst_id, worker_id, start_layer, num_layers, protocol)

    def record_event(self, layer_id: int, stream=None):
        """Mark that layer ``layer_id``'s KV has been enqueued on ``stream`` (call once per layer, in order)."""
        if self._cur_step_id is None:
            return  # warm-up forward passes before the first step are ignored
        if self._events:
            self._events[layer_id].record(stream)
        self._call("notify_event_record", self._cur_step_id)

    def submit_req_send(self, dst_inst_id, dst_worker_id, req_id, new_tokens, has_last_token, src_block_ids,
                        dst_block_ids, dst_worker_info=None):
        return self.submit_req_send2(dst_inst_id, dst_worker_id, req_id, 0, new_tokens, has_last_token,
                                     src_block_ids, dst_block_ids, dst_worker_info)

    def start_req_send(self, metas, stepid: int = DEFAULT_STEPID, substepid: int = DEFAULT_SUBSTEPID):
        if not self._inited:
            raise RuntimeError("KVTransferClient not inited")
        self._call("start_req_send", metas, stepid, substepid)

    def submit_req_send2(self, dst_inst_id, dst_worker_id, req_id, seen_tokens, new_tokens, has_last_token,
                         src_block_ids, dst_block_ids, dst_worker_info=None, stepid: int = DEFAULT_STEPID,
                         fanout: int = 0):
        """Queue tokens ``[seen, seen+new)`` of a request for the coming step (does not start any transfer).

        ``fanout=k`` (k > 1) asks the destination worker to relay the bytes to k workers of its NVLink
        multicast group (itself included) instead of this rank sending k copies: for data that those
        workers hold identically, at the same block ids (MLA latent caches, replicated KV heads).  The
        destination must advertise a group of at least k (``mc_layers`` / ``mc_size`` of its server);
        the send-done report then counts k completions."""
        if not self._inited:
            raise RuntimeError("KVTransferClient not inited")
        if isinstance(src_block_ids, list) and src_block_ids and isinstance(src_block_ids[0], int):
            assert isinstance(dst_block_ids, list) and dst_block_ids and isinstance(dst_block_ids[0], int)
            src_block_ids, dst_block_ids = [src_block_ids], [dst_block_ids]
        self._call("submit_req_send2", dst_inst_id, dst_worker_id, req_id, seen_tokens, new_tokens, has_last_token,
                   src_block_ids, dst_block_ids, dst_worker_info, stepid, 0, int(fanout))

    def submit_delta_send(self, req_id, seen_tokens, new_tokens, has_last_token, stepid: int = DEFAULT_STEPID):
        if not self._inited:
            raise RuntimeError("KVTransferClient not inited")
        self._call("submit_delta_send", req_id, seen_tokens, new_tokens, has_last_token, stepid, 0)

    def start_send_step(self, stepid: int = DEFAULT_STEPID, sched_tokens: int = 1):
        """Open the step: everything submitted since the last step starts moving layer by layer."""
        if not self._inited:
            raise RuntimeError("KVTransferClient not inited")
        if self._cur_step_id is not None:
            raise RuntimeError("start_send_step has been called multiple times")
        step_id = self._call("start_send", stepid, sched_tokens)
        if step_id != EMPTY_STEP_ID:
            assert step_id == stepid
            self._cur_step_id = step_id

    def start_send_substep(self, stepid: int, substepid: int, metas) -> None:
        if not self._inited:
            raise RuntimeError("KVTransferClient not inited")
        self._call("start_send_substep", stepid, substepid, metas)

    def flush_send_step(self):
        """Close the step after the forward pass (all layer events recorded)."""
        if not self._inited:
            raise RuntimeError("KVTransferClient not inited")
        if self._cur_step_id is None:
            return
        if self._events and not self._events[-1].query() and not self._async_sched_warned:
            self._async_sched_warned = True
            # The reference warns here because its step protocol cannot run ahead of the GPU.  Device-ordered
            # transports (NVLINK) order themselves after each layer's event, so this is only worth a note.
            logger.info("flush_send_step called before the last layer event is ready: host-staged transports "
                        "will wait for the events, device-ordered ones already queue behind them")
        self._call("flush_send", self._cur_step_id)
        self._cur_step_id = None

    def drain(self):
        """Block until every batch handed to the engine has been processed."""
        if self._c is not None:
            self._c.drain()

    def wait_inflight(self, max_batches: int = 0, timeout_s: float = 30.0) -> bool:
        """Block until at most ``max_batches`` batches of this client are still in flight (handed to the
        sender threads and not yet finished).  Over the NVLINK transport "finished" means that the batch's
        completion record, written by the GPU into mapped host memory behind the last transfer kernel, has
        been read: no stream is synchronised.  ``wait_inflight(0)`` after a step waits for that step;
        ``wait_inflight(1)`` lets the engine run one step ahead of the transfers.  False on timeout."""
        if self._c is None:
            self.drain()
            return True
        return bool(self._c.wait_inflight(max_batches, timeout_s))

    def inflight(self) -> int:
        return int(self._c.inflight()) if self._c is not None else 0

    def failed_batches(self) -> int:
        """Batches of this client that finished without their data having arrived (unreachable
        destination, refused plan, kernel status, missing completion record).  Their requests were
        reported as failed to the scheduler; this counter lets a caller without one notice."""
        return int(self._c.failed_batches()) if self._c is not None else 0

    def worker_info(self) -> str:
        return self._c.worker_info() if self._c is not None else _K.current_worker_info("client")

    async def send_error_done_req(self, reqids: List[str], plen: int = 0):
        """Tell the scheduler that ``reqids`` failed on this worker before they reached the engine.

        Same bytes as the engine's own send-done message with code 500 (kv_transfer_impl.py:502-573
        of the reference re-implements tx_stub.cpp:324-386 the same way).
        """
        if not reqids:
            return
        addr = self._send_done_addr or _get_send_done_addr()
        assert addr is not None, "send_error_done_req: BLLM_KVTRANS_SEND_DONE_ADDR not set"
        body = encode_send_done(self._worker_tp_rank, [(r, plen, CODE_INTERNALERROR) for r in reqids],
                                _get_send_done_head_kind())
        respsize = 8 if _get_send_done_head_kind() == SEND_SAVE_DONE_HEAD_KIND else 4
        reader, writer = await asyncio.open_connection(*addr)
        writer.write(body)
        await writer.drain()
        await reader.readexactly(respsize)
        writer.close()
        await writer.wait_closed()


def encode_send_done(worker_tp_rank: int, reqs, head_kind: int) -> bytes:
    """``reqs``: iterable of (reqid, plen, code)."""
    assert worker_tp_rank < 0xFFFF
    body = bytearray(struct.pack("=III", SEND_DONE_REQ, worker_tp_rank | 0x40000000, len(reqs)))
    for reqid, plen, code in reqs:
        rb = reqid.encode("utf-8")
        body += struct.pack("=III", plen, code, len(rb)) + rb
    if head_kind == SEND_SAVE_DONE_HEAD_KIND:
        n = len(body)
        body.extend(body)
        struct.pack_into("=I", body, n, SAVE_DONE2_REQ)
    return bytes(body)


class KVTransferServer:
    """Receiver side: exposes this worker's cache to senders (sockets, shared memory, NVLink)."""

    def __init__(self, inst_id: str, tp_size: int, worker_id: int, worker_tp_rank: int,
                 block_bytes: Union[List[int], int], token_bytes: Union[List[int], int], naming_url: str,
                 layers: Union[List[List[torch.Tensor]], List[torch.Tensor]],
                 protocols: List[KVTransferProtocolType], num_kv_heads: int = -1, num_gdn_layers: int = 3,
                 indexer_blk_ntpb: int = 0, hybrid_indexer_token_size: int = 0, gdn_conv_elem_size: int = 1,
                 gdn_ssm_elem_size: int = 1, conv_state_shape=None, ssm_state_shape=None,
                 gdn_conv_channel_dims=None, kda_conv_dim_first: bool = False, hybrid_attn_token_size: int = 0,
                 kda_page_stride: int = 0, attn_pack_size: int = 1, num_ple_layers: int = 0,
                 ple_block_group: int = 0, ple_conv_elem_size: int = 1, ple_conv_state_shape=None,
                 ple_conv_channel_dims=None, cache_shape: int = -1, mx_scaled: bool = False,
                 process_global: bool = False, mc_layers=None, mc_size: int = 0):
        """``mc_layers`` / ``mc_size``: this worker's cache tensors are members of an NVLink multicast
        group of ``mc_size`` workers (a tensor-parallel decode group whose caches live in one symmetric
        allocation, ``parallel.nvls.MulticastKVCache``); ``mc_layers`` gives the multicast address of
        every tensor, shaped like ``layers``.  A sender may then hand this worker a request for the
        whole group (``submit_req_send2(..., fanout=k)``)."""
        block_bytes, token_bytes, layers, layer_num_blocks, device_id = _normalise(block_bytes, token_bytes, layers)
        layer_addrs = [[t.data_ptr() for t in layer] for layer in layers]
        kw = _hybrid_kwargs(num_kv_heads, num_gdn_layers, indexer_blk_ntpb, hybrid_indexer_token_size,
                            gdn_conv_elem_size, gdn_ssm_elem_size, conv_state_shape, ssm_state_shape,
                            gdn_conv_channel_dims, kda_conv_dim_first, hybrid_attn_token_size, kda_page_stride,
                            attn_pack_size, num_ple_layers, ple_block_group, ple_conv_elem_size,
                            ple_conv_state_shape, ple_conv_channel_dims)
        if mc_layers is not None and mc_size > 1:
            mc = [[int(a)] if isinstance(a, int) else [int(x) for x in a] for a in mc_layers]
            assert len(mc) == len(layer_addrs) and all(len(a) == len(b) for a, b in zip(mc, layer_addrs))
            kw["mc_layers"], kw["mc_size"] = mc, int(mc_size)
        ops_protocols = [p.to_ops_protocol() for p in protocols]
        logger.info("init kvt server: instid=%s tpsize=%s wid=%s wrank=%s blockbytes=%s tokenbytes=%s naming=%s "
                    "protocols=%s device_id=%s num_blocks=%s num_layers=%s cache_shape=%s", inst_id, tp_size,
                    worker_id, worker_tp_rank, block_bytes, token_bytes, naming_url, protocols, device_id,
                    layer_num_blocks, len(layers), cache_shape)
        if process_global:
            _K.init_kv_transfer_server(inst_id, tp_size, worker_id, worker_tp_rank, device_id, block_bytes,
                                       token_bytes, layer_num_blocks, naming_url, layer_addrs, ops_protocols,
                                       cache_shape=cache_shape, mx_scaled=mx_scaled, **kw)
            self._s = None
        else:
            self._s = _K.KvServer(inst_id, tp_size, worker_id, worker_tp_rank, device_id, block_bytes, token_bytes,
                                  layer_num_blocks, naming_url, layer_addrs, ops_protocols, cache_shape, mx_scaled,
                                  **kw)
        self._layers = layers
        self._inited = True

    def worker_info(self) -> str:
        return self._s.worker_info() if self._s is not None else _K.current_worker_info("server")

    def port(self) -> int:
        return self._s.port() if self._s is not None else 0

    def stop(self):
        if self._s is not None:
            self._s.stop()
