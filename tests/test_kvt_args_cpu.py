"""The transfer engine's constructor arguments derived from a vLLM-shaped hybrid KV-cache configuration."""
import os
import types

import pytest
import torch

from llumnix_kv_b200.hybrid_connector.kvt_args import (choose_cache_shape, derive_hybrid_kvt_args, group_roles,
                                                     plain_token_bytes, set_worker_envs)

NS = types.SimpleNamespace


def fake_hybrid(pack=1, indexer=False, ple=False, tp=2, n_tensors=2):
    """A Qwen3-Next-like model: per physical tensor 3 GDN layers + `pack` attention layers (+ a PLE short conv);
    heads 4 x 64 per rank; GDN conv 3 rows x (2 * key + value) channels, SSM 8 x 16 x 16 fp32."""
    hf = NS(linear_num_key_heads=8, linear_key_head_dim=32, linear_num_value_heads=16, linear_value_head_dim=32)
    key, val = 8 * 32 // tp, 16 * 32 // tp
    blocks, slots, heads, dim = 6, 16, 4, 64
    kv_caches, tensors = {}, []
    gdn_groups = [[], [], []]
    attn_group, idx_group, ple_group = [], [], []
    layer = 0
    for _ in range(n_tensors):
        page = torch.zeros(pack * 2 * blocks * slots * heads * dim, dtype=torch.bfloat16)
        shared = []
        for g in range(3):
            name = f"model.layers.{layer}.linear_attn"
            kv_caches[name] = [torch.zeros(blocks, 3, 2 * key + val, dtype=torch.bfloat16),
                               torch.zeros(blocks, 8 // tp, 16, 16, dtype=torch.float32)]
            gdn_groups[g].append(name)
            shared.append(name)
            layer += 1
        for p in range(pack):
            name = f"model.layers.{layer}.self_attn.attn"
            per = 2 * blocks * slots * heads * dim
            kv_caches[name] = torch.as_strided(page, (2, blocks, slots, heads, dim),
                                               (blocks * slots * heads * dim, slots * heads * dim, heads * dim, dim, 1),
                                               storage_offset=0 if p == 0 else p * per)
            attn_group.append(name)
            shared.append(name)
            layer += 1
        if indexer:                      # the indexer keys of the pack's layers follow the attention pages
            for p in range(pack):
                iname = f"model.layers.{layer - pack + p}.self_attn.indexer.k_cache"
                kv_caches[iname] = torch.zeros(blocks, 64, 132, dtype=torch.uint8)
                idx_group.append(iname)
                shared.append(iname)
        if ple:
            name = f"model.layers.{layer}.ple_conv"
            kv_caches[name] = [torch.zeros(blocks, 2, 48, dtype=torch.bfloat16)]
            ple_group.append(name)
            shared.append(name)
            layer += 1
        tensors.append(NS(shared_by=shared))
    groups = [NS(layer_names=g, kv_cache_spec=NS(block_size=16)) for g in gdn_groups]
    if indexer:
        groups.append(NS(layer_names=idx_group, kv_cache_spec=NS(block_size=64, num_kv_heads=1, head_size=132, dtype=torch.uint8)))
    groups.append(NS(layer_names=attn_group, kv_cache_spec=NS(block_size=16)))
    if ple:
        groups.append(NS(layer_names=ple_group, kv_cache_spec=NS(block_size=16)))
    return kv_caches, NS(kv_cache_groups=groups, kv_cache_tensors=tensors), hf, (key, val)


def test_plain_hybrid_model():
    kv, cfg, hf, (key, val) = fake_hybrid()
    assert group_roles(kv, cfg) == ["gdn", "gdn", "gdn", "attn"]
    a = derive_hybrid_kvt_args(kv, cfg, hf, tp_size=2, block_size=16)
    assert a.kwargs == dict(attn_pack_size=1, num_gdn_layers=3, num_ple_layers=0, ple_block_group=0,
                            gdn_conv_channel_dims=[key, key, val], conv_state_shape=[6, 3, 2 * key + val],
                            ssm_state_shape=[6, 4, 16, 16], gdn_conv_elem_size=2, gdn_ssm_elem_size=4)
    assert a.send_layers == [3, 7]                       # the attention layer closes each physical tensor
    assert a.token_bytes == [2 * 4 * 64 * 2] and a.block_bytes == [2 * 4 * 64 * 2 * 16]
    assert list(a.physical_tensors) == ["model.layers.3.self_attn.attn", "model.layers.7.self_attn.attn"]
    t = a.physical_tensors["model.layers.3.self_attn.attn"]
    assert t.dim() == 1 and t.data_ptr() == kv["model.layers.3.self_attn.attn"].data_ptr()


def test_attention_packs_indexer_and_ple():
    kv, cfg, hf, _ = fake_hybrid(pack=2, indexer=True, ple=True)
    assert group_roles(kv, cfg) == ["gdn", "gdn", "gdn", "indexer", "attn", "ple"]
    a = derive_hybrid_kvt_args(kv, cfg, hf, tp_size=2, block_size=16, attn_pack_size=2)
    k = a.kwargs
    assert k["attn_pack_size"] == 2 and k["num_ple_layers"] == 1 and k["ple_block_group"] == 5
    assert k["indexer_blk_ntpb"] == 64 and k["hybrid_indexer_token_size"] == 132
    assert k["ple_conv_state_shape"] == [6, 2, 48] and k["ple_conv_elem_size"] == 2 and k["ple_conv_channel_dims"] == [48]
    # one tensor per pack, named after the pack's LAST layer, covering the whole physical page of both layers
    assert a.send_layers == [4, 10]
    t = a.physical_tensors["model.layers.4.self_attn.attn"]
    assert t.numel() == 2 * 2 * 6 * 16 * 4 * 64
    assert a.block_bytes == [2 * 4 * 64 * 2 * 16 * 2]     # a physical page holds both layers of the pack


def test_inconsistent_configurations_are_refused():
    kv, cfg, hf, _ = fake_hybrid()
    hf.linear_num_value_heads = 8                          # conv channels no longer add up
    with pytest.raises(AssertionError):
        derive_hybrid_kvt_args(kv, cfg, hf, tp_size=2, block_size=16)
    kv, cfg, hf, _ = fake_hybrid(pack=2)
    with pytest.raises(AssertionError):
        derive_hybrid_kvt_args(kv, cfg, hf, tp_size=2, block_size=16, attn_pack_size=1)   # two attention layers per tensor


def test_plain_models_token_bytes():
    assert plain_token_bytes({"l.0.a": torch.zeros(2, 4, 16, 8, 128, dtype=torch.bfloat16)}) == [2 * 8 * 128 * 2]
    assert plain_token_bytes({"l.0.a": torch.zeros(4, 64, 576, dtype=torch.bfloat16)}) == [576 * 2]
    both = {"l.0.indexer": torch.zeros(4, 64, 132, dtype=torch.uint8), "l.0.kv": torch.zeros(4, 64, 656, dtype=torch.uint8)}
    assert plain_token_bytes(both) == [132, 656]


def test_cache_shape_choice_and_worker_envs(monkeypatch):
    assert choose_cache_shape(False, False, False, False, False) == 2
    assert choose_cache_shape(False, False, True, False, False) == 3
    assert choose_cache_shape(True, True, False, False, False) == 4
    assert choose_cache_shape(True, False, False, False, False) == 1
    assert choose_cache_shape(False, False, False, True, False, sm_major=10) == 5
    assert choose_cache_shape(False, False, True, True, False, sm_major=10) == 7
    assert choose_cache_shape(False, False, True, True, False, sm_major=12) == 3
    assert choose_cache_shape(False, False, False, False, True) == 6
    with pytest.raises(ValueError):
        choose_cache_shape(False, False, False, True, False, sm_major=12)
    for k in ("BLLM_KVTRANS_CACHE_SHAPE", "BLLM_KVTRANS_SEND_DONE_ADDR", "BLLM_KVTRANS_RDMA_SP"):
        monkeypatch.delenv(k, raising=False)
    set_worker_envs(7, "10.0.0.5", 41000)
    assert os.environ["BLLM_KVTRANS_CACHE_SHAPE"] == "7" and os.environ["BLLM_KVTRANS_SEND_DONE_ADDR"] == "10.0.0.5:41000"
    assert os.environ["BLLM_KVTRANS_RDMA_SP"] == "2"
    monkeypatch.setenv("BLLM_KVTRANS_CACHE_SHAPE", "3")
    set_worker_envs(7, "10.0.0.5", 41000)
    assert os.environ["BLLM_KVTRANS_CACHE_SHAPE"] == "3"      # an operator's setting wins
