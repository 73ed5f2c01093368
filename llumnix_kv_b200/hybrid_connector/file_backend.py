""""local_file" backend: the smallest complete HybridBackend, persisting blocks as files.

Same at-rest format as the reference demo backend (blade_kvt/hybrid_connector/file_backend.py:
31-60, 258-284): one directory per block named after the block's token ids joined by ``_``,
one ``<tprank>.<layer name>.data`` file per layer written with ``torch.save`` and holding the
block as ``[kv, slot, head, dim]``, and an empty ``ready`` marker written after the last layer.
It exists to show the backend contract (every request both loads and saves) and as the file
half of the ``kv_both`` composite; it is not meant for production traffic.
"""
from __future__ import annotations

import asyncio
import dataclasses
import logging
import os
from collections import deque
from collections.abc import AsyncGenerator
from contextlib import suppress
from typing import Optional

import torch

from .backend import BackendMeta, HybridBackend, OperationPlan
from .engine_proxy import KVCacheBlocks, KVConnectorRole, Request, SchedulerOutput, VllmConfig
from .utils import IoRet

logger = logging.getLogger("llumnix_kv_b200.hybrid_connector")


def block_dirname(tokens: list) -> str:
    return "_".join(str(t) for t in tokens)


def block_ready(path: str) -> bool:
    return os.path.isfile(os.path.join(path, "ready"))


@dataclasses.dataclass
class FileReqMeta:
    reqid: str
    is_store: bool
    blks: list      # [(engine block id, directory name)]


@dataclasses.dataclass
class FileMeta(BackendMeta):
    reqs: list = dataclasses.field(default_factory=list)

    def __bool__(self):
        return bool(self.reqs)


class FileBackend(HybridBackend):
    SOURCE_LABEL = "local_file"

    def __init__(self, vllm_config: VllmConfig, role: KVConnectorRole, kv_cache_config=None, **kw):
        super().__init__(vllm_config, role, kv_cache_config, **kw)
        self._cfg = vllm_config
        self._dir = vllm_config.kv_transfer_config.get_from_extra_config("cachedir", "/tmp")
        self._bs = vllm_config.cache_config.block_size
        self._num_layers = vllm_config.model_config.num_layers
        self._load_req: deque = deque()     # filled by the disagg thread, drained by the core thread
        self._kv_caches: dict = {}
        self._rank = 0
        logger.warning("the local_file backend is a demonstration of the backend contract, not a production store")

    # ---- scheduler half ----------------------------------------------------------------------------
    def get_operations(self, req: Request) -> OperationPlan:
        s = self.source_label()
        return 1, 1, (s,), (s,)

    def _full_blocks(self, tokens: list, first: int = 0):
        for i in range(first, len(tokens) // self._bs):
            yield i, block_dirname(tokens[i * self._bs:(i + 1) * self._bs])

    async def async_get_num_new_matched_tokens(self, req: Request, num_computed_tokens: int) -> int:
        assert num_computed_tokens % self._bs == 0
        matched = 0
        # never the whole prompt: its last token is computed here and produces the first output
        usable = req.prompt_token_ids[:req.num_prompt_tokens - 1]
        for _, name in self._full_blocks(usable, num_computed_tokens // self._bs):
            if not block_ready(os.path.join(self._dir, name)):
                break
            matched += 1
        return matched * self._bs

    async def async_update_state_after_alloc(self, req: Request, blocks: KVCacheBlocks,
                                             num_external_tokens: int) -> Optional[IoRet]:
        if num_external_tokens <= 0:
            return None
        ids = blocks.get_block_ids()
        assert len(ids) == 1, "the file backend handles single-group caches"
        lo = req.num_computed_tokens // self._bs
        hi = (req.num_computed_tokens + num_external_tokens) // self._bs
        blks = [(ids[0][i], block_dirname(req.prompt_token_ids[i * self._bs:(i + 1) * self._bs])) for i in range(lo, hi)]
        self._engine.sched_discard_zero_block_ids(b for b, _ in blks)
        self._load_req.append(FileReqMeta(req.request_id, False, blks))
        return None

    def build_backend_meta(self, sout: SchedulerOutput) -> BackendMeta:
        meta = FileMeta()
        while self._load_req:
            meta.reqs.append(self._load_req.popleft())
        if getattr(sout, "hc_parent", None) is not None:
            return meta
        computed = {nr.req_id: nr.num_computed_tokens for nr in sout.scheduled_new_reqs}
        cached = sout.scheduled_cached_reqs
        computed.update(dict(zip(cached.req_ids, cached.num_computed_tokens)))
        for rid, before in computed.items():
            req = self.get_request(rid)
            if req is None or before >= req.num_prompt_tokens:
                continue
            if before + sout.num_scheduled_tokens[rid] < req.num_prompt_tokens:
                continue   # not the step that completes the prompt
            blkids = self._engine.sched_get_kvblk_ids(rid)[0]
            blks = [(blkids[i], name) for i, name in self._full_blocks(req.prompt_token_ids)]
            meta.reqs.append(FileReqMeta(rid, True, blks))
        for req in getattr(sout, "hc_aborted_save", ()):
            # an aborted request never reaches its last step: nothing was or will be written
            self._connector.mark_backend_save_done(req, self.source_label())
        return meta

    # ---- worker half -------------------------------------------------------------------------------
    def register_kv_caches(self, kv_caches: dict) -> None:
        from llumnix_kv_b200.models.kv_spec import rank_attn_layout

        self._kv_caches = dict(kv_caches)
        self._rank = self._worker.get_tensor_model_parallel_rank()
        self._layout = rank_attn_layout(self._cfg)
        self._dtype = torch.uint8 if self._layout.elem_bytes == 1 else torch.bfloat16
        from .kvtbackend import extract_layer_index

        self._last_layer = max(kv_caches, key=extract_layer_index)

    def _block_view(self, layer: str) -> torch.Tensor:
        return self._layout.view(self._kv_caches[layer], self._dtype)     # [block, kv, slot, head, dim]

    async def async_load_kv(self, m: BackendMeta) -> AsyncGenerator:
        assert isinstance(m, FileMeta)
        loop = asyncio.get_running_loop()
        for r in m.reqs:
            if r.is_store:
                continue

            def load(r=r):
                for blkid, name in r.blks:
                    d = os.path.join(self._dir, name)
                    assert block_ready(d), d
                    for layer in self._kv_caches:
                        blk = torch.load(os.path.join(d, f"{self._rank}.{layer}.data"))
                        view = self._block_view(layer)
                        assert tuple(blk.shape) == tuple(view.shape[1:]), (blk.shape, view.shape)
                        view[blkid] = blk.to(view.device)

            try:
                await loop.run_in_executor(None, load)
                yield IoRet(reqid=r.reqid, source=self.source_label())
            except Exception as ex:
                # a cache that cannot deliver is a miss, not a failed request: nothing counts as loaded and the engine
                # computes the prompt itself (as the reference's store backends report fewer tokens, never a failure)
                logger.warning("local_file: load failed, the request computes its prompt. reqid=%s ex=%r", r.reqid, ex)
                yield IoRet(reqid=r.reqid, n=0, source=self.source_label())

    def async_save_kv_layer(self, layer_name: str, kv_layer, m: BackendMeta) -> Optional[AsyncGenerator]:
        assert isinstance(m, FileMeta)
        todo = [r for r in m.reqs if r.is_store]
        if not todo:
            return None
        # copy the blocks out now, on the model-runner thread, in stream order with the forward pass
        view = self._block_view(layer_name)
        staged = []
        for r in todo:
            blks = []
            for blkid, name in r.blks:
                d = os.path.join(self._dir, name)
                if not block_ready(d):
                    blks.append((d, view[blkid].cpu()))
            staged.append((r.reqid, blks))
        last = layer_name == self._last_layer

        async def gen():
            loop = asyncio.get_running_loop()

            def write(blks):
                for d, data in blks:
                    with suppress(FileExistsError):
                        os.mkdir(d)
                    torch.save(data, os.path.join(d, f"{self._rank}.{layer_name}.data"))
                    if last:
                        # the block is ready once every TP rank has written its last layer
                        open(os.path.join(d, f"{self._rank}.ready"), "w").close()
                        tp = self._cfg.parallel_config.tensor_parallel_size
                        if all(os.path.isfile(os.path.join(d, f"{r}.ready")) for r in range(tp)):
                            open(os.path.join(d, "ready"), "w").close()

            for reqid, blks in staged:
                await loop.run_in_executor(None, write, blks)
                yield reqid

        return gen()
