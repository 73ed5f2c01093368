"""Host-DRAM store on a B200: the fused kernel gathers engine blocks into registered host pages
and scatters them back (copy and block-scaled fp8 pages), and the kvs backend end to end."""
import os
import time

import pytest
import torch

from llumnix_kv_b200 import load_ops
from llumnix_kv_b200.kvstore import PinnedKVStore
from llumnix_kv_b200.ops.layouts import AttnLayout, CacheShape
from llumnix_kv_b200.ops.p2d_attn import mx_dequantize_reference, mx_quantize_reference

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("src_shape,dst_shape", [(CacheShape.FLASH, CacheShape.FLASHINFER),
                                                 (CacheShape.FLASHINFER, CacheShape.FLASH)])
def test_save_then_load_across_layouts(src_shape, dst_shape):
    name = f"kvx_g_{os.getpid()}"
    src_l = AttnLayout(src_shape, 40, 16, 8, 128, 2)
    dst_l = AttnLayout(dst_shape, 40, 16, 8, 128, 2)
    L = 3
    src = [src_l.alloc(DEV, fill="normal", seed=i) for i in range(L)]
    dst = [dst_l.alloc(DEV) for _ in range(L)]
    a = PinnedKVStore(name, src_l, src, 0, 1, 32, create=True)
    b = PinnedKVStore(name, dst_l, dst, 0, 1, 32, create=False)
    try:
        toks = list(range(7, 7 + 16 * 9))
        keys = a.keys(toks, 9)
        new, full = a.reserve(keys)
        assert not full and len(new) == 9
        blocks = [3, 9, 1, 30, 12, 5, 39, 20, 8]
        fwd = torch.cuda.Event()
        fwd.record(torch.cuda.current_stream())
        for layer in range(L):                       # per layer, as save_kv_layer issues it
            ev = a.save_layers(layer, layer + 1, blocks, [s for _, s in new], after=fwd)
        ev.synchronize()
        a.check_status()
        a.seal(keys)
        # the host pages hold [kv, slot, head, dim] whatever the source layout was
        page0 = a._page_view(1, torch.int16)[new[0][1]]
        assert torch.equal(page0, src_l.view(src[1], torch.int16)[blocks[0]].cpu())
        slots = b.pin(keys)
        into = [2, 4, 6, 8, 10, 12, 14, 16, 18]
        b.load_layers(0, L, into, slots).synchronize()
        b.check_status()
        b.unpin(keys)
        for layer in range(L):
            assert torch.equal(src_l.view(src[layer], torch.int16)[blocks], dst_l.view(dst[layer], torch.int16)[into])
    finally:
        a.close()
        b.close()
        load_ops().KvStore.unlink(name)


def test_fp8_pages_halve_the_footprint():
    name = f"kvx_g8_{os.getpid()}"
    lay = AttnLayout(CacheShape.FLASH, 24, 16, 8, 128, 2)
    src = [lay.alloc(DEV, fill="normal", seed=3)]
    dst = [lay.alloc(DEV)]
    a = PinnedKVStore(name, lay, src, 0, 1, 16, create=True, fp8=True)
    b = PinnedKVStore(name, lay, dst, 0, 1, 16, create=False, fp8=True)
    try:
        assert a.slot_bytes == lay.block_bytes // 2 + lay.block_bytes // 2 // 32
        keys = a.keys(list(range(64)), 4)
        new, _ = a.reserve(keys)
        a.save_layers(0, 1, [5, 6, 7, 8], [s for _, s in new]).synchronize()
        a.check_status()
        a.seal(keys)
        b.load_layers(0, 1, [1, 2, 3, 4], b.pin(keys)).synchronize()
        b.check_status()
        x = lay.view(src[0], torch.bfloat16)[[5, 6, 7, 8]].float()
        y = lay.view(dst[0], torch.bfloat16)[[1, 2, 3, 4]]
        codes, exps = mx_quantize_reference(x)
        assert torch.equal(y, mx_dequantize_reference(codes, exps))
    finally:
        a.close()
        b.close()
        load_ops().KvStore.unlink(name)


def test_kvs_backend_on_gpu():
    from pd_helpers import make_cfg
    from test_kvs_cpu import run, spy, wait_free
    from llumnix_kv_b200.engine.core import MiniEngineCore

    name = f"kvx_ge_{os.getpid()}"
    e = MiniEngineCore(make_cfg("kv_both", "G", backend="kvs", device=DEV, layers=4, head_dim=128, num_blocks=96,
                                extra={"kvs_name": name, "kvs_slots": 64}))
    try:
        cap = spy(e)
        r1 = run(e, "a", 300)
        assert wait_free(e, 95) == 95
        for t in e.workers[0].kv_caches.values():
            t.zero_()
        r2 = run(e, "b", 300)
        computed, blocks = cap["b"]
        assert computed == 288
        w = e.workers[0]
        for layer in range(4):
            assert torch.equal(w.read_kv(layer, blocks[0], 0, 288), w.expected_kv(layer, r2.prompt_token_ids, 0, 288))
    finally:
        e.shutdown()
        load_ops().KvStore.unlink(name)
