"""Two-GPU path in one process: the destination cache lives on a peer GPU and the kernel on the
source GPU stores into it over NVLink (plain peer stores, no multicast)."""
import random

import pytest
import torch

from llumnix_kv_b200.ops.layouts import AttnLayout, CacheShape
from llumnix_kv_b200.ops.p2d_attn import AttnTransfer, ReqChunk, reference_transfer

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


@pytest.mark.parametrize("use_tma", [True, False])
def test_push_to_peer_gpu(ops, use_tma):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    if not ops.kvt_can_access_peer(0, 1):
        pytest.skip("no peer access between GPU 0 and 1")
    ops.kvt_enable_peer_access(0, 1)
    rng = random.Random(21)
    src_l = AttnLayout(CacheShape.FLASH, 64, 16, 8, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 64, 16, 8, 128, 2)
    src = [src_l.alloc("cuda:0", "normal", seed=i) for i in range(2)]
    dst = [dst_l.alloc("cuda:1") for _ in range(2)]
    chunks = []
    for _ in range(4):
        nb = rng.randint(1, 7)
        chunks.append(ReqChunk(rng.sample(range(64), nb), rng.sample(range(64), nb), 0, nb * 16 - rng.randint(0, 9)))
    # distinct destination blocks across requests
    used = set()
    for c in chunks:
        c.dst_blocks = [b for b in c.dst_blocks]
        for i, b in enumerate(c.dst_blocks):
            while b in used:
                b = (b + 1) % 64
            used.add(b)
            c.dst_blocks[i] = b
    flag = torch.zeros(2, dtype=torch.int64, device="cuda:1")
    with torch.cuda.device(0):
        xfer = AttnTransfer(src_l, dst_l, [s.data_ptr() for s in src], [d.data_ptr() for d in dst], "cuda:0",
                            use_tma=use_tma)
        xfer.launch(xfer.plan(chunks), flag_ptr=flag.data_ptr(), flag_value=7)
        torch.cuda.synchronize(0)
        assert xfer.check_status() == (0, 0)
    torch.cuda.synchronize(1)
    assert flag[0].item() == 7
    for i in range(2):
        expect = torch.zeros_like(src[i])
        reference_transfer(src_l, dst_l, src[i], expect, chunks)
        assert torch.equal(dst[i].to("cuda:0"), expect)


def test_framework_allocated_cache_storage(ops):
    """alloc_phy_cont_mem: a whole cudaMalloc allocation wrapped as a tensor; its IPC handle starts at
    the tensor, and a cache swapped onto it keeps shape and strides."""
    from llumnix_kv_b200.kv_transfer_impl import alloc_kv_cache_peer_mappable, alloc_phy_cont_mem

    t = alloc_phy_cont_mem(1 << 20, 0)
    assert t.dtype == torch.uint8 and t.numel() == 1 << 20 and t.is_cuda
    t.fill_(7)
    _h, base, size = ops.kvt_ipc_get_handle(t.data_ptr())
    assert base == t.data_ptr() and size >= 1 << 20
    cache = torch.zeros(2, 8, 16, 4, 64, dtype=torch.bfloat16, device="cuda:0")
    swapped = alloc_kv_cache_peer_mappable(cache)
    assert swapped.shape == cache.shape and swapped.stride() == cache.stride() and swapped.dtype == cache.dtype
    swapped.copy_(torch.ones_like(cache))
    assert float(swapped.float().sum()) == cache.numel()
    del t, swapped
    torch.cuda.synchronize()
