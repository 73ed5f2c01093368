"""Worker side of the minimal engine: one ``MiniWorker`` per TP rank owns that rank's paged KV
cache and runs the "model".

The model is a stand-in whose KV is a closed-form function of (token id, position, layer,
K/V, global head, dim), written into the paged cache exactly where a real attention layer
would write it.  That makes every transfer checkable: a decode engine can recompute what any
slot must contain, whatever layout, TP split or dtype path the bytes took to get there.
The forward pass drives the connector the way a model runner does: bind metadata,
``start_load_kv``, ``save_kv_layer`` after each layer, clear.
"""
from __future__ import annotations

from typing import Optional

import torch

from llumnix_kv_b200 import envs
from llumnix_kv_b200.hybrid_connector import HybridConnector
from llumnix_kv_b200.hybrid_connector.engine_proxy import KVConnectorRole, WorkerProxy
from llumnix_kv_b200.ops.layouts import AttnLayout, CacheShape

from .config import KVCacheConfig, KVCacheGroupSpec, VllmConfig
from .types import SchedulerOutput


def layer_name(i: int, gdn: bool = False) -> str:
    return f"model.layers.{i}.linear_attn" if gdn else f"model.layers.{i}.self_attn.attn"


def indexer_name(i: int) -> str:
    return f"model.layers.{i}.self_attn.indexer"


def synthetic_rows(token_ids: torch.Tensor, positions: torch.Tensor, layer: int, tensor_idx: int,
                   width: int) -> torch.Tensor:
    """[tokens, width] uint8 rows of a head-less cache (MLA latent + rope, indexer keys): the same
    on every TP rank, a function of (token, position, layer, tensor, byte)."""
    t = token_ids.to(torch.int64).view(-1, 1)
    p = positions.to(torch.int64).view(-1, 1)
    b = torch.arange(width, device=token_ids.device).view(1, -1)
    return ((t * 37 + p * 11 + layer * 5 + tensor_idx * 101 + b * 3) % 251 + 1).to(torch.uint8)


def make_kv_cache_config(cfg: VllmConfig) -> KVCacheConfig:
    """KV-cache groups in physical order: one group per GDN position of the layer pattern, then
    the attention group (a plain model has the attention group only)."""
    mc = cfg.model_config
    groups = [[] for _ in mc.group_types()]
    for i in range(mc.num_layers):
        groups[mc.layer_group(i)].append(layer_name(i, mc.is_gdn_layer(i)))
        if mc.use_mla and mc.indexer_token_bytes:
            groups[mc.layer_group(i)].append(indexer_name(i))
    return KVCacheConfig(num_blocks=cfg.cache_config.num_gpu_blocks,
                         kv_cache_groups=[KVCacheGroupSpec(g) for g in groups])


def synthetic_state(token_ids: list, upto: int, layer: int, col0: int, cols: int, rows: int, dtype: torch.dtype,
                    device, row0: int = 0) -> torch.Tensor:
    """[rows, cols] recurrent-state values that depend on the whole prefix ``token_ids[:upto]``, on the
    layer and on the GLOBAL row / column index, so that any TP slicing of the state can be recomputed."""
    digest = (sum((j + 1) * t for j, t in enumerate(token_ids[:upto])) + 7919 * upto) % 100003
    r = (torch.arange(rows, device=device) + row0).view(-1, 1)
    c = (torch.arange(cols, device=device) + col0).view(1, -1)
    code = (digest + layer * 131 + r * 17 + c * 3) % 251
    return ((code - 125).to(torch.float32) / 16.0).to(dtype)


def synthetic_kv(token_ids: torch.Tensor, positions: torch.Tensor, layer: int, head0: int, n_heads: int,
                 head_dim: int, dtype: torch.dtype) -> torch.Tensor:
    """[tokens, 2(K/V), heads, dim] values in a range every cache dtype represents exactly enough
    to compare bit-for-bit (multiples of 1/64 below 8)."""
    dev = token_ids.device
    t = token_ids.to(torch.int64).view(-1, 1, 1, 1)
    p = positions.to(torch.int64).view(-1, 1, 1, 1)
    kv = torch.arange(2, device=dev).view(1, 2, 1, 1)
    h = (torch.arange(n_heads, device=dev) + head0).view(1, 1, -1, 1)
    d = torch.arange(head_dim, device=dev).view(1, 1, 1, -1)
    code = (t * 131 + p * 31 + layer * 17 + kv * 7 + h * 5 + d * 3) % 509
    return ((code - 254).to(torch.float32) / 64.0).to(dtype)


class MiniWorker:
    def __init__(self, cfg: VllmConfig, tp_rank: int, device: Optional[str] = None, with_connector: bool = True):
        self.cfg = cfg
        self.tp_rank = tp_rank
        self.device = torch.device(device or cfg.device)
        mc, cc = cfg.model_config, cfg.cache_config
        tp = cfg.parallel_config.tensor_parallel_size
        self.heads = max(1, mc.num_kv_heads // tp)
        self.head0 = (tp_rank * mc.num_kv_heads // tp) if mc.num_kv_heads >= tp else tp_rank * mc.num_kv_heads // tp
        self.dtype = torch.bfloat16 if mc.dtype_bytes == 2 else torch.uint8
        elem = 1 if cc.mx_scaled else mc.dtype_bytes
        self.layout = AttnLayout(CacheShape(cc.cache_shape), cc.num_gpu_blocks, cc.block_size, self.heads, mc.head_dim,
                                 elem, mx_scaled=cc.mx_scaled)
        # hybrid models: one physical tensor per repetition of the layer pattern, shared by its layers
        n_tensors = mc.layer_tensor(mc.num_layers - 1) + 1
        self._tensors = [self.layout.alloc(self.device) for _ in range(n_tensors)]
        self.names = [layer_name(i, mc.is_gdn_layer(i)) for i in range(mc.num_layers)]
        self.kv_caches = {self.names[i]: self._tensors[mc.layer_tensor(i)] for i in range(mc.num_layers)}
        self.row_widths: list = []
        if mc.use_mla:
            # head-less caches, identical on every TP rank: [blocks, slots, width] rows per tensor
            self.row_widths = [(mc.kv_lora_rank + mc.qk_rope_head_dim) * mc.dtype_bytes]
            if mc.indexer_token_bytes:
                self.row_widths.append(mc.indexer_token_bytes)
            self.kv_caches = {}
            self._rows = []          # per layer: one [blocks, slots, width] uint8 tensor per cache tensor
            for i in range(mc.num_layers):
                ts = [torch.zeros(cc.num_gpu_blocks, cc.block_size, w, dtype=torch.uint8, device=self.device)
                      for w in self.row_widths]
                self._rows.append(ts)
                self.kv_caches[layer_name(i)] = ts[0].view(-1)
                if len(ts) > 1:
                    self.kv_caches[indexer_name(i)] = ts[1].view(-1)
        self.kv_cache_config = make_kv_cache_config(cfg)
        if mc.is_hybrid:
            tp_ = cfg.parallel_config.tensor_parallel_size
            self._conv_dims = [d // tp_ for d in mc.gdn_conv_channel_dims]
            self._ssm_heads = max(1, mc.gdn_ssm_shape[0] // tp_)
            conv_b = mc.gdn_conv_rows * sum(self._conv_dims) * mc.gdn_conv_elem_size
            ssm_b = self._ssm_heads * mc.gdn_ssm_shape[1] * mc.gdn_ssm_shape[2] * mc.gdn_ssm_elem_size
            assert conv_b + ssm_b <= self.layout.block_bytes, "recurrent state does not fit in one cache page"
        self.connector: Optional[HybridConnector] = None
        self.proxy: Optional[WorkerProxy] = None
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        if with_connector and cfg.kv_transfer_config is not None:
            self.proxy = WorkerProxy(cfg, tp_rank, str(self.device))
            self.connector = HybridConnector(cfg, KVConnectorRole.WORKER, self.kv_cache_config, worker=self.proxy)
            self.connector.register_kv_caches(self.kv_caches)
        self._req_state: dict = {}   # reqid -> (prompt tokens, block ids of group 0)
        self.forward_passes = 0
        self.hidden_states_hook = None    # callable(forward pass number) -> the pass's hidden states (NaN-check tests)

    # ---- the "model" ---------------------------------------------------------------------------
    def expected_rows(self, layer: int, tensor_idx: int, token_ids: list, lo: int, hi: int) -> torch.Tensor:
        return synthetic_rows(torch.tensor(token_ids[lo:hi], device=self.device), torch.arange(lo, hi, device=self.device),
                              layer, tensor_idx, self.row_widths[tensor_idx])

    def read_rows(self, layer: int, tensor_idx: int, blocks: list, lo: int, hi: int) -> torch.Tensor:
        bs = self.cfg.cache_config.block_size
        blk = torch.tensor([blocks[p // bs] for p in range(lo, hi)], device=self.device)
        return self._rows[layer][tensor_idx][blk, torch.arange(lo, hi, device=self.device) % bs]

    def _write_layer(self, layer: int, tokens: torch.Tensor, positions: torch.Tensor, blocks: list) -> None:
        if self.cfg.model_config.use_mla:
            bs = self.cfg.cache_config.block_size
            blk = torch.tensor([blocks[int(p) // bs] for p in positions.tolist()], device=self.device)
            for t, w in enumerate(self.row_widths):
                self._rows[layer][t][blk, positions % bs] = synthetic_rows(tokens, positions, layer, t, w)
            return
        if self.cfg.cache_config.mx_scaled:
            return  # a block-scaled fp8 cache is only ever filled by transfers in this engine
        lay = self.layout
        kv = synthetic_kv(tokens, positions, layer, self.head0, self.heads, lay.head_dim, self.dtype)
        view = lay.view(self.kv_caches[self.names[layer]], self.dtype)   # [block, kv, slot, head, dim]
        blk = torch.tensor([blocks[int(p) // lay.ntpb] for p in positions.tolist()], device=self.device)
        slot = (positions % lay.ntpb).to(self.device)
        view[blk, :, slot] = kv

    # ---- recurrent (GDN) state of hybrid models: one page per request and GDN group -----------------------
    def expected_state(self, layer: int, token_ids: list, upto: int) -> tuple:
        """(conv [rows, q+k+v channels of this rank] bf16, ssm [heads of this rank, k*v] fp32) after
        the first ``upto`` tokens.  A rank holds a contiguous slice of each of q, k, v and of the heads."""
        mc = self.cfg.model_config
        parts, g0 = [], 0
        for dim_rank, dim_all in zip(self._conv_dims, mc.gdn_conv_channel_dims):
            parts.append(synthetic_state(token_ids, upto, layer, g0 + self.tp_rank * dim_rank, dim_rank,
                                         mc.gdn_conv_rows, torch.bfloat16, self.device))
            g0 += dim_all
        _h, k, v = mc.gdn_ssm_shape
        ssm = synthetic_state(token_ids, upto, layer + 1000, 0, k * v, self._ssm_heads, torch.float32, self.device,
                              row0=self.tp_rank * self._ssm_heads)
        return torch.cat(parts, dim=1), ssm

    def _state_regions(self, layer: int, block: int) -> tuple:
        mc = self.cfg.model_config
        flat = self._tensors[mc.layer_tensor(layer)]
        cols = sum(self._conv_dims)
        conv_b = mc.gdn_conv_rows * cols * 2
        ssm_b = self._ssm_heads * mc.gdn_ssm_shape[1] * mc.gdn_ssm_shape[2] * 4
        off = block * self.layout.block_bytes
        conv = flat[off:off + conv_b].view(torch.bfloat16).view(mc.gdn_conv_rows, cols)
        ssm = flat[off + conv_b:off + conv_b + ssm_b].view(torch.float32).view(self._ssm_heads, -1)
        return conv, ssm

    def _write_state(self, layer: int, token_ids: list, upto: int, block: int) -> None:
        conv, ssm = self._state_regions(layer, block)
        c, s = self.expected_state(layer, token_ids, upto)
        conv.copy_(c)
        ssm.copy_(s)

    def read_state(self, layer: int, block: int) -> tuple:
        conv, ssm = self._state_regions(layer, block)
        return conv.clone(), ssm.clone()

    def expected_kv(self, layer: int, token_ids: list, lo: int, hi: int, dtype=None) -> torch.Tensor:
        toks = torch.tensor(token_ids[lo:hi], device=self.device)
        pos = torch.arange(lo, hi, device=self.device)
        return synthetic_kv(toks, pos, layer, self.head0, self.heads, self.layout.head_dim, dtype or self.dtype)

    def read_kv(self, layer: int, blocks: list, lo: int, hi: int) -> torch.Tensor:
        lay = self.layout
        view = lay.view(self.kv_caches[self.names[layer]], self.dtype)
        pos = torch.arange(lo, hi, device=self.device)
        blk = torch.tensor([blocks[p // lay.ntpb] for p in range(lo, hi)], device=self.device)
        return view[blk, :, pos % lay.ntpb]

    def read_kv_mx(self, layer: int, blocks: list, lo: int, hi: int):
        """(codes, UE8M0 exponents) of a block-scaled fp8 cache for prompt positions [lo, hi)."""
        lay = self.layout
        flat = self.kv_caches[self.names[layer]]
        pos = torch.arange(lo, hi, device=self.device)
        blk = torch.tensor([blocks[p // lay.ntpb] for p in range(lo, hi)], device=self.device)
        return lay.view(flat, torch.uint8)[blk, :, pos % lay.ntpb], lay.scale_view(flat)[blk, :, pos % lay.ntpb]

    def execute_model(self, sout: SchedulerOutput) -> dict:
        """One forward pass over the scheduled tokens; returns {reqid: sampled token}."""
        if self.device.type == "cuda":
            # the connector records its per-layer events on this device's current stream
            with torch.cuda.device(self.device):
                return self._execute_model(sout)
        return self._execute_model(sout)

    def _execute_model(self, sout: SchedulerOutput) -> dict:
        self.forward_passes += 1
        conn = self.connector
        meta = sout.kv_connector_metadata
        if conn is not None and meta is not None:
            conn.bind_connector_metadata(meta)
            conn.start_load_kv(None)
        for nr in sout.scheduled_new_reqs:
            self._req_state[nr.req_id] = [list(nr.prompt_token_ids), [list(g) for g in nr.block_ids]]
        cached = sout.scheduled_cached_reqs
        for rid, new_blocks in zip(cached.req_ids, cached.new_block_ids):
            st = self._req_state.get(rid)
            if st is not None:
                for g, extra in zip(st[1], new_blocks):
                    g.extend(extra)
        work = []
        computed = {nr.req_id: nr.num_computed_tokens for nr in sout.scheduled_new_reqs}
        computed.update(dict(zip(cached.req_ids, cached.num_computed_tokens)))
        for rid, n in sout.num_scheduled_tokens.items():
            st = self._req_state.get(rid)
            if st is None or n <= 0:
                continue
            lo = computed[rid]
            toks = st[0]
            hi = min(lo + n, len(toks))
            if hi > lo:
                work.append((torch.tensor(toks[lo:hi], device=self.device), torch.arange(lo, hi, device=self.device),
                             st[1][-1] if len(st[1]) > 1 else st[1][0], st, hi))
        mc = self.cfg.model_config
        for layer in range(mc.num_layers):
            for toks, pos, blocks, st, hi in work:
                if mc.is_gdn_layer(layer):
                    # the recurrent state after this step's tokens, in the request's page of the layer's group
                    self._write_state(layer, st[0], hi, st[1][mc.layer_group(layer)][0])
                else:
                    self._write_layer(layer, toks, pos, blocks)
            if conn is not None and meta is not None:
                conn.save_kv_layer(self.names[layer], self.kv_caches[self.names[layer]], None)
                if len(self.row_widths) > 1:
                    conn.save_kv_layer(indexer_name(layer), self.kv_caches[indexer_name(layer)], None)
        if conn is not None and meta is not None:
            if envs.VLLM_KVS_STORE_NAN_CHECK and conn.wants_nan_flag():
                # on the forward stream, so the check precedes anything recorded after the last layer
                hidden = self.hidden_states_hook(self.forward_passes) if self.hidden_states_hook is not None \
                    else torch.zeros(8, device=self.device)
                conn.set_nan_flag(torch.isnan(hidden).any())
            conn.clear_connector_metadata()
        sampled = {}
        for rid, n in sout.num_scheduled_tokens.items():
            st = self._req_state.get(rid)
            if st is not None:
                sampled[rid] = (sum(st[0][-4:]) * 7 + len(st[0])) % self.cfg.model_config.vocab_size
        for rid in sout.finished_req_ids:
            self._req_state.pop(rid, None)
        return sampled

    def append_token(self, rid: str, tok: int) -> None:
        st = self._req_state.get(rid)
        if st is not None:
            st[0].append(tok)
