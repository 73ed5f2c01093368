"""One rank's window onto the shared host-DRAM block store.

A store *slot* holds every layer of one KV block of one TP rank as ``num_layers`` consecutive
pages; a page is block-major ``[kv, slot, head, dim]`` whatever the engine's own cache layout
is, optionally block-scaled fp8 (e4m3 codes followed by one UE8M0 exponent per 32 values).  The
per-block page is the same thing the reference's demo store writes per block and layer
(blade_kvt/hybrid_connector/file_backend.py:258-284 saves ``kvcache[:, blkid]``), so an NHD
engine can save what an HND engine loads.

On a GPU the move is the fused transfer kernel with the slot arena (registered, mapped host
memory) as its destination (save) or source (load): block-table walk, layout conversion and
the optional bf16<->fp8 conversion happen in that one pass over PCIe.  On a CPU "device" (the
control-plane tests) the same move is a strided torch copy.

Keys are chained: key_i = H(key_{i-1} || tokens of block i || salt), so a key identifies the
whole prefix up to its block (the property vLLM block hashes have and the reference's KVS
adapters rely on, blade_kvt/hybrid_connector/kvsbackend.py:381-399).
"""
from __future__ import annotations

import os

import ctypes
import dataclasses
import hashlib
import struct
from typing import List, Optional, Sequence, Tuple

import torch

from llumnix_kv_b200.ops.layouts import AttnLayout, CacheShape

RESERVE_NEW, RESERVE_EXISTS, RESERVE_BUSY, RESERVE_FULL = 0, 1, 2, 3


def block_keys(token_ids: Sequence[int], block_size: int, n_blocks: int, salt: bytes = b"") -> List[bytes]:
    """16-byte chained keys of the first ``n_blocks`` full blocks of ``token_ids``."""
    assert n_blocks * block_size <= len(token_ids)
    keys, prev = [], b"\0" * 16
    for i in range(n_blocks):
        chunk = token_ids[i * block_size:(i + 1) * block_size]
        h = hashlib.blake2b(prev, digest_size=16)
        h.update(struct.pack(f"<{block_size}q", *chunk))
        h.update(salt)
        prev = h.digest()
        keys.append(prev)
    return keys


def store_page_layout(engine: AttnLayout, n_slots: int, num_layers: int, fp8: bool = False) -> AttnLayout:
    """Layout of one layer's pages inside the slot arena (block stride = whole slot)."""
    if fp8:
        assert engine.elem_bytes == 2 and not engine.mx_scaled, "fp8 pages are made from a 16-bit cache"
    elem = 1 if fp8 else engine.elem_bytes
    dense = AttnLayout(CacheShape.QWEN3_NEXT_FLASH, n_slots, engine.ntpb, engine.num_heads, engine.head_dim, elem,
                       kv_count=engine.kv_count, mx_scaled=fp8 or engine.mx_scaled)
    return dataclasses.replace(dense, block_stride_override=dense.block_bytes * num_layers)


def store_format(engine: AttnLayout, num_layers: int, fp8: bool = False) -> Tuple[int, str]:
    """(slot_bytes, format tag) of a store serving caches of this geometry; every opener of one
    store must agree on both."""
    page = store_page_layout(engine, 1, num_layers, fp8)
    tag = (f"v1;L={num_layers};T={engine.ntpb};H={engine.num_heads};D={engine.head_dim};"
           f"E={page.elem_bytes};kv={engine.kv_count};mx={int(page.mx_scaled)}")
    return page.block_bytes * num_layers, tag


def store_salt(model_tag: str, tp_rank: int, tp_size: int, tag: str) -> bytes:
    """What distinguishes the keys of one rank / model from another's inside a shared store."""
    return f"{model_tag};{tp_rank}/{tp_size};{tag}".encode()


class PinnedKVStore:
    def __init__(self, name: str, engine_layout: AttnLayout, layers: Sequence[torch.Tensor], tp_rank: int,
                 tp_size: int, n_slots: int, create, ttl_ms: int = 0, fp8: bool = False,
                 model_tag: str = ""):
        from llumnix_kv_b200 import load_ops

        self.K = load_ops()
        self.engine_layout = engine_layout
        self.layers = list(layers)
        self.num_layers = len(self.layers)
        self.device = self.layers[0].device
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self.ttl_ms = ttl_ms
        # CTAs of the gather / scatter launches.  The copies are PCIe-bound: a quarter of a CTA per SM moves
        # as much as four per SM (measured 50.0 / 51.3 GB/s save / load with 37 CTAs, 49.1 / 51.3 with 592) and
        # leaves the SMs to the forward pass the save overlaps with.  BLLM_KVSTORE_CTAS overrides.
        self.grid = int(os.environ.get("BLLM_KVSTORE_CTAS", "0"))
        if self.grid <= 0 and self.device.type == "cuda":
            self.grid = max(1, self.K.kvt_sm_count(self.device.index or 0) // 4)
        self.fp8 = fp8
        self.page = store_page_layout(engine_layout, n_slots, self.num_layers, fp8)
        self.page_bytes = self.page.block_bytes
        self.slot_bytes = self.page_bytes * self.num_layers
        slot_bytes, tag = store_format(engine_layout, self.num_layers, fp8)
        assert slot_bytes == self.slot_bytes
        # create: False = attach, True = create (replacing), "auto" = attach or create
        mode = 2 if create == "auto" else int(bool(create))
        self.kv = self.K.KvStore.open(name, self.slot_bytes, n_slots, mode, tag)
        self.salt = store_salt(model_tag, tp_rank, tp_size, tag)
        n = self.kv.data_bytes
        self._buf = (ctypes.c_ubyte * n).from_address(self.kv.data_ptr)
        self.host = torch.frombuffer(self._buf, dtype=torch.uint8)   # the arena as a CPU tensor
        self._registered = False
        self._save_xfer = self._load_xfer = None
        self.stream: Optional[torch.cuda.Stream] = None
        if self.device.type == "cuda":
            from llumnix_kv_b200.ops.p2d_attn import MODE_BF16_TO_MXFP8, MODE_COPY, MODE_MXFP8_TO_BF16, AttnTransfer

            with torch.cuda.device(self.device):
                dev_ptr = self.K.kvt_host_register(self.kv.data_ptr, n)
                self._registered = True
                self.stream = torch.cuda.Stream(self.device)
                eng_ptrs = [t.data_ptr() for t in self.layers]
                page_ptrs = [dev_ptr + i * self.page_bytes for i in range(self.num_layers)]
                # BLLM_KVSTORE_TMA=1: tiles travel through the TMA engine (tensor maps over the mapped host arena)
                # instead of the SIMT warps; bf16 pages only (the fp8 pages are written by the quantiser)
                tma = os.environ.get("BLLM_KVSTORE_TMA", "0") not in ("0", "") and not fp8
                self.uses_tma = tma
                self._save_xfer = AttnTransfer(engine_layout, self.page, eng_ptrs, page_ptrs, self.device,
                                               mode=MODE_BF16_TO_MXFP8 if fp8 else MODE_COPY, use_tma=tma, simt_tile=2)
                self._load_xfer = AttnTransfer(self.page, engine_layout, page_ptrs, eng_ptrs, self.device,
                                               mode=MODE_MXFP8_TO_BF16 if fp8 else MODE_COPY, use_tma=tma, simt_tile=2)
                self.uses_tma = tma and self._save_xfer.use_tma and self._load_xfer.use_tma

    # ---- index ----------------------------------------------------------------------------------
    def keys(self, token_ids: Sequence[int], n_blocks: int) -> List[bytes]:
        return block_keys(token_ids, self.engine_layout.ntpb, n_blocks, self.salt)

    def lookup(self, keys: Sequence[bytes]) -> int:
        return self.kv.lookup_prefix(b"".join(keys)) if keys else 0

    def reserve(self, keys: Sequence[bytes]) -> Tuple[List[Tuple[int, int]], bool]:
        """Reserves a slot for every key that is not stored yet.  Returns ([(index, slot)], full):
        ``full`` says that the store ran out of evictable slots before the end of the list."""
        out = []
        for i, k in enumerate(keys):
            code, slot = self.kv.reserve(k, self.ttl_ms)
            if code == RESERVE_NEW:
                out.append((i, slot))
            elif code == RESERVE_FULL:
                return out, True
        return out, False

    def seal(self, keys: Sequence[bytes]) -> None:
        for k in keys:
            self.kv.seal(k)

    def discard(self, keys: Sequence[bytes]) -> None:
        for k in keys:
            self.kv.discard(k)

    def pin(self, keys: Sequence[bytes]) -> List[int]:
        return list(self.kv.pin_prefix(b"".join(keys))) if keys else []

    def unpin(self, keys: Sequence[bytes]) -> None:
        if keys:
            self.kv.unpin(b"".join(keys))

    # ---- data -----------------------------------------------------------------------------------
    def _page_view(self, layer: int, dtype: torch.dtype) -> torch.Tensor:
        flat = self.host[layer * self.page_bytes:]
        return self.page.view(flat, dtype)

    def _move(self, save: bool, layer_begin: int, layer_end: int, blocks: Sequence[int], slots: Sequence[int],
              after: Optional["torch.cuda.Event"]) -> Optional["torch.cuda.Event"]:
        assert len(blocks) == len(slots)
        if not blocks:
            return None
        ntpb = self.engine_layout.ntpb
        if self.device.type == "cuda":
            from llumnix_kv_b200.ops.p2d_attn import ReqChunk

            xfer = self._save_xfer if save else self._load_xfer
            chunk = ReqChunk(blocks, slots, 0, len(blocks) * ntpb) if save else \
                ReqChunk(slots, blocks, 0, len(blocks) * ntpb)
            with torch.cuda.device(self.device), torch.cuda.stream(self.stream):
                if after is not None:
                    self.stream.wait_event(after)
                plan = xfer.plan([chunk], stream=self.stream)
                xfer.launch(plan, layer_begin, layer_end, stream=self.stream, grid=self.grid)
                done = torch.cuda.Event()
                done.record(self.stream)
            done._keepalive = plan      # the plan's device buffers must outlive the kernel
            return done
        # CPU "device": same page format through strided views
        assert not self.fp8, "the fp8 page format needs the GPU kernel"
        dt = torch.uint8 if self.engine_layout.elem_bytes == 1 else torch.int16
        b = torch.as_tensor(list(blocks), dtype=torch.long)
        s = torch.as_tensor(list(slots), dtype=torch.long)
        for layer in range(layer_begin, layer_end):
            ev, pv = self.engine_layout.view(self.layers[layer], dt), self._page_view(layer, dt)
            if save:
                pv[s] = ev[b]
            else:
                ev[b] = pv[s]
            if self.page.mx_scaled:
                es = self.engine_layout.scale_view(self.layers[layer])
                ps = self.page.scale_view(self.host[layer * self.page_bytes:])
                if save:
                    ps[s] = es[b]
                else:
                    es[b] = ps[s]
        return None

    def save_layers(self, layer_begin: int, layer_end: int, blocks: Sequence[int], slots: Sequence[int],
                    after=None):
        """Engine cache -> store pages for layers [begin, end).  ``after``: event on the forward
        stream that says the layers' KV has been written.  Returns an event (GPU) or None."""
        return self._move(True, layer_begin, layer_end, blocks, slots, after)

    def load_layers(self, layer_begin: int, layer_end: int, blocks: Sequence[int], slots: Sequence[int], after=None):
        return self._move(False, layer_begin, layer_end, blocks, slots, after)

    def check_status(self) -> None:
        for x in (self._save_xfer, self._load_xfer):
            if x is not None:
                code, detail = x.check_status()
                if code != 0:
                    raise RuntimeError(f"kv store transfer kernel reported status {code} (detail {detail})")

    def stats(self) -> dict:
        return dict(self.kv.stats())

    def close(self) -> None:
        if self._registered:
            with torch.cuda.device(self.device):
                torch.cuda.synchronize()
                self.K.kvt_host_unregister(self.kv.data_ptr)
            self._registered = False
        self._save_xfer = self._load_xfer = None
        self.host = None
        self._buf = None
        self.kv = None
