"""Deriving the transfer engine's constructor arguments from what an engine registers.

``KVTransferClient`` / ``KVTransferServer`` describe a worker's cache to the native engine with numbers:
bytes per token and block of every cache tensor, the number of KV heads, and for hybrid models the geometry
of the recurrent-state pages.  The engine itself hands the connector none of these: it registers cache
tensors by layer name and a KV-cache configuration (groups of layers with a spec each, physical tensors
shared by several layers).  This module works the numbers out, the way ``_build_kvt_args`` of the reference
does (blade_kvt/hybrid_connector/kvtbackend.py:709-1101), and picks the cache-shape id and the send-done
address a worker needs before it creates its client or server (``_set_worker_envs``, :524-563).

The inputs are duck-typed after vLLM's objects:
  kv_caches          {layer name: Tensor | [conv_state, ssm_state] | [short_conv_state]}
  kv_cache_config    .kv_cache_groups[i].layer_names / .kv_cache_spec (block_size, num_kv_heads, head_size, dtype)
                     .kv_cache_tensors[j].shared_by  (layer names that live in physical tensor j, in page order)
  hf_text_config     linear_num_key_heads, linear_key_head_dim, linear_num_value_heads, linear_value_head_dim
"""
from __future__ import annotations

import dataclasses
import os
import re
from typing import Any, Optional

import torch


def extract_layer_index(layer_name: str) -> int:
    nums = re.findall(r"\.(\d+)\.", f".{layer_name}.")
    assert len(nums) == 1, f"layer name {layer_name!r} must contain exactly one integer component"
    return int(nums[0])


def _is_indexer(name: str) -> bool:
    return "indexer" in name


@dataclasses.dataclass
class HybridKVTArgs:
    kwargs: dict                 # hybrid keyword arguments of KVTransferClient / KVTransferServer
    physical_tensors: dict       # {last attention layer of the pack: flat view of the physical page tensor}
    send_layers: list            # layer index whose completion releases each physical tensor, ascending
    token_bytes: list
    block_bytes: list


def group_roles(kv_caches: dict, kv_cache_config: Any) -> list:
    """Role of every KV-cache group, in group (= block-table) order: "gdn" (recurrent state: conv + ssm),
    "ple" (short-conv state only), "indexer", "attn"."""
    roles = []
    for g in kv_cache_config.kv_cache_groups:
        names = list(g.layer_names)
        cache = kv_caches[names[0]]
        if isinstance(cache, (list, tuple)):
            roles.append("gdn" if len(cache) == 2 else "ple")
        elif all(_is_indexer(n) for n in names):
            roles.append("indexer")
        else:
            roles.append("attn")
    return roles


def derive_hybrid_kvt_args(kv_caches: dict, kv_cache_config: Any, hf_text_config: Any, tp_size: int,
                           block_size: int, attn_pack_size: int = 1, kda_page_stride: int = 0,
                           kda_conv_dim_first: bool = False) -> HybridKVTArgs:
    assert attn_pack_size >= 1
    roles = group_roles(kv_caches, kv_cache_config)
    num_gdn = sum(r == "gdn" for r in roles)
    num_ple = sum(r == "ple" for r in roles)
    assert num_gdn > 0, "a hybrid model has at least one recurrent-state group"
    # block-table order the native planner expects: [gdn ... | indexer? | attn | ple?]
    assert roles[:num_gdn] == ["gdn"] * num_gdn, f"recurrent-state groups must come first: {roles}"
    kw: dict = dict(attn_pack_size=attn_pack_size, num_gdn_layers=num_gdn, num_ple_layers=num_ple,
                    ple_block_group=roles.index("ple") if num_ple else 0)
    key_dim = hf_text_config.linear_num_key_heads * hf_text_config.linear_key_head_dim // tp_size
    value_dim = hf_text_config.linear_num_value_heads * hf_text_config.linear_value_head_dim // tp_size
    kw["gdn_conv_channel_dims"] = [key_dim, key_dim, value_dim]
    if kda_page_stride:
        kw["kda_page_stride"] = kda_page_stride
    if kda_conv_dim_first:
        kw["kda_conv_dim_first"] = True
    for g, role in zip(kv_cache_config.kv_cache_groups, roles):
        if role == "indexer":
            spec = g.kv_cache_spec
            kw["indexer_blk_ntpb"] = spec.block_size
            kw["hybrid_indexer_token_size"] = spec.num_kv_heads * spec.head_size * torch.empty((), dtype=spec.dtype).element_size()
    physical: dict = {}
    send_layers: list = []
    layer_cache: Optional[torch.Tensor] = None
    for tensor_group in kv_cache_config.kv_cache_tensors:
        shared_by = list(tensor_group.shared_by)
        attn = [(i, n) for i, n in enumerate(shared_by)
                if isinstance(kv_caches[n], torch.Tensor) and not n.endswith(".indexer.k_cache")]
        assert 0 < len(attn) <= attn_pack_size, f"expected 1..{attn_pack_size} attention layers per physical tensor, got {attn}"
        pos = [i for i, _ in attn]
        assert pos == list(range(pos[0], pos[0] + len(pos))), f"an attention pack must be contiguous in the page: {shared_by}"
        idxs = [extract_layer_index(n) for _, n in attn]
        assert idxs == sorted(idxs), f"attention pack layers must ascend: {idxs}"
        first, last = attn[0][1], attn[-1][1]
        send_layers.append(extract_layer_index(last))
        first_view, last_view = kv_caches[first], kv_caches[last]
        assert first_view.untyped_storage().data_ptr() == last_view.untyped_storage().data_ptr(), \
            f"pack members {first!r} and {last!r} do not share one allocation"
        assert first_view.storage_offset() == 0, f"{first!r} must start its physical page tensor"
        storage = first_view.untyped_storage()
        flat = torch.empty(0, dtype=first_view.dtype, device=first_view.device)
        flat.set_(storage, 0, (storage.nbytes() // first_view.element_size(),), (1,))
        physical[last] = flat          # registered once per pack, under the layer whose completion releases it
        if layer_cache is None:
            layer_cache = first_view
        attn_names = {n for _, n in attn}
        for name in shared_by:
            cache = kv_caches[name]
            if isinstance(cache, torch.Tensor):
                assert name in attn_names or name.endswith(".indexer.k_cache"), f"unexpected tensor cache {name}"
                continue
            assert isinstance(cache, (list, tuple)), f"recurrent state of {name} must be a list"
            if len(cache) == 2:
                conv, ssm = cache
                assert conv.dim() == 3 and ssm.dim() == 4, (conv.shape, ssm.shape)
                if "conv_state_shape" not in kw:
                    kw.update(conv_state_shape=list(conv.shape), ssm_state_shape=list(ssm.shape),
                              gdn_conv_elem_size=conv.element_size(), gdn_ssm_elem_size=ssm.element_size())
                    channels = conv.shape[1] if kda_conv_dim_first else conv.shape[2]
                    assert 2 * key_dim + value_dim == channels, \
                        f"2 * key_dim + value_dim = {2 * key_dim + value_dim}, conv state has {channels} channels"
            else:
                assert len(cache) == 1, f"unexpected recurrent state of {name}: {len(cache)} tensors"
                (conv,) = cache
                assert conv.dim() == 3, conv.shape
                if "ple_conv_state_shape" not in kw:
                    kw.update(ple_conv_state_shape=list(conv.shape), ple_conv_elem_size=conv.element_size(),
                              ple_conv_channel_dims=[conv.shape[2]])
    if num_ple:
        assert "ple_conv_state_shape" in kw, "a PLE group exists but no short-conv state was registered"
    assert send_layers == sorted(send_layers) and len(set(send_layers)) == len(send_layers), send_layers
    assert layer_cache is not None and layer_cache.dim() == 5, "attention caches are [2, blocks, slots, heads, dim] (or a permutation)"
    # the full-attention page sizes every block; state pages are padded to it
    token_bytes = [2 * layer_cache.shape[3] * layer_cache.shape[4] * layer_cache.element_size()]
    block_bytes = [t * block_size * attn_pack_size for t in token_bytes]
    return HybridKVTArgs(kw, physical, send_layers, token_bytes, block_bytes)


def plain_token_bytes(kv_caches: dict) -> list:
    """Bytes per token of every cache tensor of a layer, non-hybrid models: one 5-D attention cache, one 3-D
    MLA cache, or the two 3-D tensors of a sparse-MLA layer (indexer keys + latent), in shape order of first use."""
    by_shape: dict = {}
    for name, t in kv_caches.items():
        by_shape.setdefault(tuple(t.shape), t)
    if len(by_shape) == 1:
        (shape, t), = by_shape.items()
        if len(shape) == 5:
            return [2 * shape[3] * shape[4] * t.element_size()]
        assert len(shape) == 3, f"unknown cache tensor shape {shape}"
        return [shape[2] * t.element_size()]
    out = []
    for shape, t in by_shape.items():
        assert len(shape) == 3, f"several tensors per layer are supported for sparse MLA only; got {shape}"
        out.append(shape[2] * t.element_size())
    return out


def choose_cache_shape(use_mla: bool, use_sparse_mla: bool, is_hybrid: bool, use_flashinfer: bool,
                       use_turboquant: bool, sm_major: int = 10) -> int:
    """Cache-shape id (kvtransfer/include/envcfg.h:25-52) by attention backend and GPU generation."""
    if use_mla:
        return 4 if use_sparse_mla else 1
    if use_flashinfer:
        if sm_major == 10:
            return 7 if is_hybrid else 5
        if sm_major == 12 and is_hybrid:
            return 3
        raise ValueError(f"no FlashInfer cache shape for SM {sm_major}.x" + ("" if is_hybrid else " non-hybrid"))
    if is_hybrid:
        return 3
    return 6 if use_turboquant else 2


def set_worker_envs(cache_shape: int, scheduler_host: str, rpc_port: int) -> None:
    """Defaults a worker sets before it creates its client / server: the engine settings of ``set_envs``, its
    cache shape, and where the native send stubs report finished requests (the scheduler's RPC port)."""
    import llumnix_kv_b200

    llumnix_kv_b200.set_envs()
    os.environ.setdefault("BLLM_KVTRANS_CACHE_SHAPE", str(cache_shape))
    os.environ.setdefault("BLLM_KVTRANS_SEND_DONE_ADDR", f"{scheduler_host}:{rpc_port}")
