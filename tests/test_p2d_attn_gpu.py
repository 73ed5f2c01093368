"""GPU numerics of the fused transfer kernel against the plain-PyTorch oracle.

Source and destination caches sit on the same GPU here (the kernel does not care whose
memory the destination pointer names); the two-GPU path is covered in test_peer_gpu.py.
"""
import random

import pytest
import torch

from llumnix_kv_b200.ops.layouts import AttnLayout, CacheShape, mla_layout
from llumnix_kv_b200.ops.p2d_attn import (MODE_BF16_TO_MXFP8, MODE_COPY, MODE_MXFP8_TO_BF16, AttnTransfer, HeadMap,
                                          ReqChunk, mx_dequantize_reference, reference_transfer)

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _rand_chunks(rng, n_req, src_nb, dst_nb, ntpb, max_blocks, partial=True, pad_tail=False):
    src_free = list(range(1, src_nb))
    dst_free = list(range(1, dst_nb))
    rng.shuffle(src_free)
    rng.shuffle(dst_free)
    chunks = []
    for _ in range(n_req):
        nb = rng.randint(1, max_blocks)
        sb = [src_free.pop() for _ in range(nb)]
        db = [dst_free.pop() for _ in range(nb)]
        total = nb * ntpb
        if partial:
            seen = rng.randint(0, total - 1)
            new = rng.randint(1, total - seen)
        else:
            seen, new = 0, total
        chunks.append(ReqChunk(sb, db, seen, new, pad_tail=pad_tail))
    return chunks


def _run(src_l, dst_l, chunks, n_layers=3, head_map=None, mode=MODE_COPY, use_tma=True, grid=0, threads=0,
         layer_range=None, dst_remote=False):
    src = [src_l.alloc(DEV, "normal", seed=10 + i) for i in range(n_layers)]
    dst = [dst_l.alloc(DEV, "normal", seed=100 + i) for i in range(n_layers)]
    if mode == MODE_MXFP8_TO_BF16:
        # make the source scales sane exponents
        for s in src:
            src_l.scale_view(s).copy_(torch.randint(120, 134, src_l.scale_view(s).shape, dtype=torch.uint8, device=DEV))
    expect = [d.clone() for d in dst]
    xfer = AttnTransfer(src_l, dst_l, [s.data_ptr() for s in src], [d.data_ptr() for d in dst], DEV,
                        head_map=head_map, mode=mode, use_tma=use_tma, dst_remote=dst_remote)
    if use_tma and mode == MODE_COPY:
        assert xfer.use_tma, "tensor maps must encode on a GPU machine"
    plan = xfer.plan(chunks)
    lb, le = layer_range or (0, n_layers)
    xfer.launch(plan, lb, le, grid=grid, threads=threads)
    torch.cuda.synchronize()
    assert xfer.check_status() == (0, 0)
    for i in range(lb, le):
        reference_transfer(src_l, dst_l, src[i], expect[i], chunks, head_map, mode)
    return src, dst, expect


@pytest.mark.parametrize("use_tma", [True, False])
@pytest.mark.parametrize("partial", [False, True])
def test_nhd_to_hnd_copy(use_tma, partial):
    rng = random.Random(1)
    src_l = AttnLayout(CacheShape.FLASH, 64, 16, 8, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 80, 16, 8, 128, 2)
    chunks = _rand_chunks(rng, 5, 64, 80, 16, 8, partial=partial)
    _, dst, expect = _run(src_l, dst_l, chunks, use_tma=use_tma)
    for d, e in zip(dst, expect):
        assert torch.equal(d, e)


@pytest.mark.parametrize("shapes", [
    (CacheShape.FLASH, CacheShape.FLASH),
    (CacheShape.FLASHINFER, CacheShape.FLASH),
    (CacheShape.RAGGED_FLASH, CacheShape.FLASHINFER),
    (CacheShape.QWEN3_NEXT_FLASH, CacheShape.QWEN3_NEXT_FLASHINFER),
    (CacheShape.FLASHINFER, CacheShape.RAGGED_FLASH),
])
@pytest.mark.parametrize("use_tma", [True, False])
def test_layout_pairs(shapes, use_tma):
    rng = random.Random(2)
    src_l = AttnLayout(shapes[0], 40, 16, 4, 64, 2)
    dst_l = AttnLayout(shapes[1], 48, 16, 4, 64, 2)
    chunks = _rand_chunks(rng, 4, 40, 48, 16, 6)
    _, dst, expect = _run(src_l, dst_l, chunks, n_layers=2, use_tma=use_tma)
    for d, e in zip(dst, expect):
        assert torch.equal(d, e)


@pytest.mark.parametrize("use_tma", [True, False])
def test_p_gt_d_head_reshard(use_tma):
    # prefill TP=4 (2 heads per rank) -> decode TP=2 (4 heads per rank); this is prefill rank 1 / 3
    rng = random.Random(3)
    src_l = AttnLayout(CacheShape.FLASH, 32, 16, 2, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 32, 16, 4, 128, 2)
    chunks = _rand_chunks(rng, 3, 32, 32, 16, 6)
    hm = HeadMap(0, 2, 2)
    _, dst, expect = _run(src_l, dst_l, chunks, head_map=hm, use_tma=use_tma)
    for d, e in zip(dst, expect):
        assert torch.equal(d, e)


@pytest.mark.parametrize("use_tma", [True, False])
def test_p_lt_d_head_slice(use_tma):
    # prefill TP=1 (8 heads) fans out to decode TP=4 (2 heads each); this is decode rank 2
    rng = random.Random(4)
    src_l = AttnLayout(CacheShape.FLASHINFER, 32, 16, 8, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 32, 16, 2, 128, 2)
    chunks = _rand_chunks(rng, 3, 32, 32, 16, 6)
    hm = HeadMap(4, 0, 2)
    _, dst, expect = _run(src_l, dst_l, chunks, head_map=hm, use_tma=use_tma)
    for d, e in zip(dst, expect):
        assert torch.equal(d, e)


def test_different_block_sizes_and_pad_tail():
    rng = random.Random(5)
    src_l = AttnLayout(CacheShape.FLASH, 64, 16, 4, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 24, 64, 4, 128, 2)
    # request of 100 tokens: 7 src blocks, 2 dst blocks, tail of the 2nd dst block zeroed
    chunks = [ReqChunk([3, 9, 4, 20, 21, 33, 60], [5, 7], 0, 100, pad_tail=True),
              ReqChunk([40, 41, 42, 43], [11], 10, 50, pad_tail=False)]
    for use_tma in (True, False):
        _, dst, expect = _run(src_l, dst_l, chunks, n_layers=2, use_tma=use_tma)
        for d, e in zip(dst, expect):
            assert torch.equal(d, e)
        v = dst_l.view(dst[0], torch.int16)
        assert int(v[7, :, 100 - 64:, :, :].abs().max()) == 0


def test_mla_single_tensor():
    rng = random.Random(6)
    src_l = mla_layout(48, 64, 656)
    dst_l = mla_layout(40, 64, 656)
    chunks = _rand_chunks(rng, 4, 48, 40, 64, 5)
    for use_tma in (True, False):
        _, dst, expect = _run(src_l, dst_l, chunks, n_layers=2, use_tma=use_tma)
        for d, e in zip(dst, expect):
            assert torch.equal(d, e)


def test_layer_range_only_touches_those_layers():
    rng = random.Random(7)
    src_l = AttnLayout(CacheShape.FLASH, 32, 16, 8, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 32, 16, 8, 128, 2)
    chunks = _rand_chunks(rng, 3, 32, 32, 16, 4, partial=False)
    _, dst, expect = _run(src_l, dst_l, chunks, n_layers=4, layer_range=(1, 3))
    for d, e in zip(dst, expect):
        assert torch.equal(d, e)


@pytest.mark.parametrize("partial", [False, True])
@pytest.mark.parametrize("heads", [(2, 4, HeadMap(0, 2, 2)), (8, 8, None)])
def test_bf16_to_mxfp8_staged_for_a_remote_destination(heads, partial):
    """dst_remote=True makes the quantiser stage full HND tiles in shared memory and send them as bulk
    stores (the form used over NVLink); tiles it cannot stage (too large: 8 heads; ragged edges) take the
    direct stores.  Same bytes as the oracle either way."""
    rng = random.Random(18)
    src_h, dst_h, hm = heads
    src_l = AttnLayout(CacheShape.FLASH, 40, 16, src_h, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 48, 16, dst_h, 128, 1, mx_scaled=True)
    chunks = _rand_chunks(rng, 6, 40, 48, 16, 5, partial=partial)
    _, dst, expect = _run(src_l, dst_l, chunks, n_layers=3, head_map=hm, mode=MODE_BF16_TO_MXFP8, use_tma=False,
                          dst_remote=True)
    for d, e in zip(dst, expect):
        assert torch.equal(d, e)


@pytest.mark.parametrize("heads", [(1, 1, None), (2, 2, None)])
def test_bf16_to_mxfp8_staged_with_256_wide_heads(heads):
    """Rows of 256 values carry eight scale bytes: one head x 16 tokens fits the staging buffer (bulk
    stores), two heads do not (direct stores).  Scales must land chunk by chunk in both."""
    rng = random.Random(19)
    src_h, dst_h, hm = heads
    src_l = AttnLayout(CacheShape.FLASH, 24, 16, src_h, 256, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 24, 16, dst_h, 256, 1, mx_scaled=True)
    chunks = _rand_chunks(rng, 4, 24, 24, 16, 4, partial=False)
    _, dst, expect = _run(src_l, dst_l, chunks, n_layers=2, head_map=hm, mode=MODE_BF16_TO_MXFP8, use_tma=False,
                          dst_remote=True)
    for d, e in zip(dst, expect):
        assert torch.equal(d, e)


@pytest.mark.parametrize("form", [(0, 0), (1, 0), (1, 1), (0, 1)])
@pytest.mark.parametrize("stages", [0, 1, 2])
def test_tma_tile_orders_and_store_forms(form, stages):
    """Every way a TMA tile can sit in shared memory and leave it moves the same bytes: tokens or heads
    outermost, a tensor store or one linear bulk store (legal where the destination holds the tile
    contiguously: HND pages with heads outermost, NHD pages with tokens outermost), with an L2 policy or not."""
    order, flat = form
    rng = random.Random(31)
    src_l = AttnLayout(CacheShape.FLASH if order else CacheShape.FLASHINFER, 64, 16, 8, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER if order else CacheShape.FLASH, 80, 16, 8, 128, 2)
    chunks = _rand_chunks(rng, 5, 64, 80, 16, 8, partial=True)
    for hint in (0, 1):
        src = [src_l.alloc(DEV, "normal", seed=10 + i) for i in range(2)]
        dst = [dst_l.alloc(DEV, "normal", seed=100 + i) for i in range(2)]
        expect = [d.clone() for d in dst]
        xfer = AttnTransfer(src_l, dst_l, [s.data_ptr() for s in src], [d.data_ptr() for d in dst], DEV,
                            tile_order=order, store_form=flat, tma_stages=stages, cache_hint=hint)
        assert xfer.use_tma
        xfer.launch(xfer.plan(chunks))
        torch.cuda.synchronize()
        assert xfer.check_status() == (0, 0)
        for i in range(2):
            reference_transfer(src_l, dst_l, src[i], expect[i], chunks)
            assert torch.equal(dst[i], expect[i])


def test_linear_store_is_refused_where_the_tile_is_not_contiguous():
    src_l = AttnLayout(CacheShape.FLASH, 16, 16, 8, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 16, 16, 8, 128, 2)
    with pytest.raises(ValueError):
        AttnTransfer(src_l, dst_l, [0], [0], DEV, tile_order=0, store_form=1, use_tma=False)
    # P>D reshard into a slice of the heads of an HND page: still one run (heads are adjacent)
    x = AttnTransfer(AttnLayout(CacheShape.FLASH, 16, 16, 2, 128, 2), AttnLayout(CacheShape.FLASHINFER, 16, 16, 4, 128, 2),
                     [0], [0], DEV, head_map=HeadMap(0, 2, 2), use_tma=False)
    assert (x.tile_order, x.store_form) == (1, 1)


@pytest.mark.parametrize("dst_shape", [CacheShape.FLASHINFER, CacheShape.QWEN3_NEXT_FLASH])
def test_bf16_to_mxfp8(dst_shape):
    rng = random.Random(8)
    src_l = AttnLayout(CacheShape.FLASH, 32, 16, 2, 128, 2)
    dst_l = AttnLayout(dst_shape, 32, 16, 4, 128, 1, mx_scaled=True)
    chunks = _rand_chunks(rng, 4, 32, 32, 16, 5)
    hm = HeadMap(0, 2, 2)
    src, dst, expect = _run(src_l, dst_l, chunks, n_layers=2, head_map=hm, mode=MODE_BF16_TO_MXFP8, use_tma=False)
    for d, e in zip(dst, expect):
        assert torch.equal(d, e)
    # round trip error of the block-scaled format: relative to the group's amax, e4m3 with a
    # power-of-two scale is good to 2^-3 of the largest value's binade
    c = chunks[0]
    t = c.seen_tokens
    sb, ss = c.src_blocks[t // 16], t % 16
    db, ds = c.dst_blocks[t // 16], t % 16
    x = src_l.view(src[0], torch.bfloat16)[sb, :, ss, :, :].float()
    y = mx_dequantize_reference(dst_l.view(dst[0], torch.uint8)[db, :, ds, 2:4, :],
                                dst_l.scale_view(dst[0])[db, :, ds, 2:4, :]).float()
    amax = x.abs().reshape(2, 2, 4, 32).amax(-1, keepdim=True).expand(2, 2, 4, 32).reshape(2, 2, 128)
    assert float(((x - y).abs() / amax).max()) <= 0.0715


def test_mxfp8_to_bf16():
    rng = random.Random(9)
    src_l = AttnLayout(CacheShape.FLASHINFER, 32, 16, 4, 128, 1, mx_scaled=True)
    dst_l = AttnLayout(CacheShape.FLASH, 32, 16, 4, 128, 2)
    chunks = _rand_chunks(rng, 4, 32, 32, 16, 5)
    src = [src_l.alloc(DEV) for _ in range(2)]
    for i, s in enumerate(src):
        g = torch.Generator(device=DEV)
        g.manual_seed(i)
        codes = torch.randint(0, 256, src_l.view(s, torch.uint8).shape, dtype=torch.uint8, device=DEV, generator=g)
        # no NaN codes (0x7f / 0xff)
        codes = torch.where((codes & 0x7F) == 0x7F, codes - 1, codes)
        src_l.view(s, torch.uint8).copy_(codes)
        src_l.scale_view(s).copy_(torch.randint(118, 134, src_l.scale_view(s).shape, dtype=torch.uint8,
                                                device=DEV, generator=g))
    dst = [dst_l.alloc(DEV, "normal", seed=50 + i) for i in range(2)]
    expect = [d.clone() for d in dst]
    xfer = AttnTransfer(src_l, dst_l, [s.data_ptr() for s in src], [d.data_ptr() for d in dst], DEV,
                        mode=MODE_MXFP8_TO_BF16)
    xfer.launch(xfer.plan(chunks))
    torch.cuda.synchronize()
    assert xfer.check_status() == (0, 0)
    for i in range(2):
        reference_transfer(src_l, dst_l, src[i], expect[i], chunks, None, MODE_MXFP8_TO_BF16)
        assert torch.equal(dst[i], expect[i])


def test_bad_block_id_sets_status_and_skips():
    src_l = AttnLayout(CacheShape.FLASH, 16, 16, 8, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 16, 16, 8, 128, 2)
    src = [src_l.alloc(DEV, "normal", seed=1)]
    dst = [dst_l.alloc(DEV)]
    for use_tma in (True, False):
        xfer = AttnTransfer(src_l, dst_l, [src[0].data_ptr()], [dst[0].data_ptr()], DEV, use_tma=use_tma)
        chunks = [ReqChunk([1, 2], [3, 4], 0, 32), ReqChunk([5, 999], [6, 7], 0, 32)]
        xfer.launch(xfer.plan(chunks))
        torch.cuda.synchronize()
        code, _ = xfer.check_status()
        assert code == 1
        # the good request and the good block still arrived
        sv, dv = src_l.view(src[0], torch.int16), dst_l.view(dst[0], torch.int16)
        assert torch.equal(dv[3], sv[1]) and torch.equal(dv[4], sv[2])
        assert torch.equal(dv[6], sv[5])
        assert int(dv[7].abs().max()) == 0


def test_completion_flag_in_mapped_host_memory(ops):
    src_l = AttnLayout(CacheShape.FLASH, 16, 16, 8, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 16, 16, 8, 128, 2)
    src = [src_l.alloc(DEV, "normal", seed=1)]
    dst = [dst_l.alloc(DEV)]
    host, dev = ops.kvt_host_alloc_mapped(64)
    try:
        import ctypes

        flag = ctypes.c_uint64.from_address(host)
        flag.value = 0
        xfer = AttnTransfer(src_l, dst_l, [src[0].data_ptr()], [dst[0].data_ptr()], DEV)
        for step in (1, 2, 3):
            xfer.launch(xfer.plan([ReqChunk([1, 2, 3], [4, 5, 6], 0, 48)]), flag_ptr=dev, flag_value=step)
            torch.cuda.synchronize()
            assert flag.value == step
        # bounded device-side wait: nothing will set 99, the kernel gives up and reports
        status = torch.zeros(4, dtype=torch.int32, device=DEV)
        ops.kvt_launch_wait_flag(dev, 99, 50_000_000, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert status[0].item() == 4
        status.zero_()
        ops.kvt_launch_wait_flag(dev, 3, 50_000_000, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert status[0].item() == 0
    finally:
        ops.kvt_host_free(host)


def test_gather_to_pinned_host_and_scatter_back(ops):
    """KVStore path: GPU paged cache -> contiguous pinned host pages -> another paged cache."""
    rng = random.Random(11)
    gpu_l = AttnLayout(CacheShape.FLASHINFER, 48, 16, 8, 128, 2)
    n_host_blocks = 12
    host_l = AttnLayout(CacheShape.FLASHINFER, n_host_blocks, 16, 8, 128, 2)
    host, hdev = ops.kvt_host_alloc_mapped(host_l.layer_bytes * 2)
    try:
        src = [gpu_l.alloc(DEV, "normal", seed=3 + i) for i in range(2)]
        blocks = rng.sample(range(1, 48), n_host_blocks)
        host_ptrs = [hdev, hdev + host_l.layer_bytes]
        save = AttnTransfer(gpu_l, host_l, [s.data_ptr() for s in src], host_ptrs, DEV)
        chunk = [ReqChunk(blocks, list(range(n_host_blocks)), 0, n_host_blocks * 16)]
        save.launch(save.plan(chunk))
        torch.cuda.synchronize()
        assert save.check_status() == (0, 0)
        back = [gpu_l.alloc(DEV) for _ in range(2)]
        blocks2 = rng.sample(range(1, 48), n_host_blocks)
        load = AttnTransfer(host_l, gpu_l, host_ptrs, [b.data_ptr() for b in back], DEV)
        load.launch(load.plan([ReqChunk(list(range(n_host_blocks)), blocks2, 0, n_host_blocks * 16)]))
        torch.cuda.synchronize()
        assert load.check_status() == (0, 0)
        for i in range(2):
            sv, bv = gpu_l.view(src[i], torch.int16), gpu_l.view(back[i], torch.int16)
            assert torch.equal(bv[blocks2], sv[blocks])
    finally:
        ops.kvt_host_free(host)


def test_state_segments_and_copy_blocks(ops):
    # GDN-like page: conv rows split in 3 channel segments interleaved for group_n=2, then SSM
    rows, segs, ssm = 3, (32, 32, 64), 4096
    row_p = sum(segs)
    conv_p = rows * row_p
    g_n, g_off = 2, 1
    src_bs = conv_p + ssm
    dst_bs = g_n * (conv_p + ssm)
    nb = 10
    src = torch.randint(0, 255, (2, nb * src_bs), dtype=torch.uint8, device=DEV)
    dst = torch.zeros((2, nb * dst_bs), dtype=torch.uint8, device=DEV)
    rules, pre = [], 0
    for s in segs:
        rules.append(ops.KvtSegRule(pre, g_n * pre + g_off * s, row_p, g_n * row_p, s, rows))
        pre += s
    rules.append(ops.KvtSegRule(conv_p, g_n * conv_p + g_off * ssm, 0, 0, ssm, 1))
    rules_t = torch.frombuffer(bytearray(b"".join(r.pack() for r in rules)), dtype=torch.uint8).to(DEV)
    sblk = torch.tensor([1, 4, 7], dtype=torch.int32, device=DEV)
    dblk = torch.tensor([2, 3, 9], dtype=torch.int32, device=DEV)
    layers_s = torch.tensor([src[0].data_ptr(), src[1].data_ptr()], dtype=torch.int64, device=DEV)
    layers_d = torch.tensor([dst[0].data_ptr(), dst[1].data_ptr()], dtype=torch.int64, device=DEV)
    status = torch.zeros(4, dtype=torch.int32, device=DEV)
    ops.kvt_launch_p2d_state(layers_s.data_ptr(), layers_d.data_ptr(), 0, 2, src_bs, dst_bs, nb, nb,
                             sblk.data_ptr(), dblk.data_ptr(), 3, rules_t.data_ptr(), len(rules),
                             status.data_ptr(), 0, 0, 0, 8, 256, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status[0].item() == 0
    for l in range(2):
        for sb, db in zip([1, 4, 7], [2, 3, 9]):
            s_page = src[l, sb * src_bs:(sb + 1) * src_bs]
            d_page = dst[l, db * dst_bs:(db + 1) * dst_bs]
            pre = 0
            for s in segs:
                for r in range(rows):
                    a = s_page[r * row_p + pre: r * row_p + pre + s]
                    b = d_page[r * g_n * row_p + g_n * pre + g_off * s: r * g_n * row_p + g_n * pre + g_off * s + s]
                    assert torch.equal(a, b)
                pre += s
            assert torch.equal(s_page[conv_p:], d_page[g_n * conv_p + g_off * ssm: g_n * conv_p + (g_off + 1) * ssm])
    # descriptor-driven copy with odd alignments
    a = torch.randint(0, 255, (1 << 16,), dtype=torch.uint8, device=DEV)
    b = torch.zeros(1 << 16, dtype=torch.uint8, device=DEV)
    trip = [(0, 16, 4096), (5000, 9001, 777), (10000, 20004, 1024), (30000, 40000, 3)]
    t = torch.tensor([x for tr in trip for x in tr], dtype=torch.int64, device=DEV)
    ops.kvt_launch_copy_blocks(a.data_ptr(), b.data_ptr(), t.data_ptr(), len(trip), a.numel(), b.numel(),
                               status.data_ptr(), 4, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status[0].item() == 0
    for so, do, ln in trip:
        assert torch.equal(a[so:so + ln], b[do:do + ln])
    # out-of-range descriptor is reported, not executed
    t2 = torch.tensor([0, (1 << 16) - 8, 64], dtype=torch.int64, device=DEV)
    ops.kvt_launch_copy_blocks(a.data_ptr(), b.data_ptr(), t2.data_ptr(), 1, a.numel(), b.numel(),
                               status.data_ptr(), 4, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status[0].item() == 1


def test_copy_blocks_long_mixed_and_multi_tensor(ops):
    """The descriptor copy splits long runs into 4 KiB segments laid out by the FIRST descriptor's
    length: lists whose later entries are longer or shorter than the first, and several tensors with
    their own bases in one launch, must still move exactly the listed bytes."""
    st = torch.zeros(4, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device=DEV).manual_seed(3)
    n = 3 << 20
    for trip in ([(16, 64, 41984), (100000, 50000, 41984), (300000, 200000, 41984 * 3), (900000, 700000, 100)],
                 [(0, 0, 100), (4096, 8192, 1 << 20), (2 << 20, 1200000, 4097)],
                 [(48, 1, 65536 + 5)]):
        a = torch.randint(0, 255, (n,), dtype=torch.uint8, device=DEV, generator=g)
        b = torch.zeros(n, dtype=torch.uint8, device=DEV)
        t = torch.tensor([x for tr in trip for x in tr], dtype=torch.int64, device=DEV)
        ops.kvt_launch_copy_blocks(a.data_ptr(), b.data_ptr(), t.data_ptr(), len(trip), n, n, st.data_ptr(), 0, stream)
        torch.cuda.synchronize()
        assert st[0].item() == 0
        want = torch.zeros_like(b)
        for so, do, ln in trip:
            want[do:do + ln] = a[so:so + ln]
        assert torch.equal(b, want)
    # three tensors, one launch; the second tensor's list is empty, the third has short runs
    srcs = [torch.randint(0, 255, (1 << 20,), dtype=torch.uint8, device=DEV, generator=g) for _ in range(3)]
    dsts = [torch.zeros(1 << 20, dtype=torch.uint8, device=DEV) for _ in range(3)]
    lists = [[(0, 4096, 41984), (50000, 100000, 41984)], [], [(8, 24, 132 * 64), (9000, 20000, 132 * 64), (30000, 500000, 7)]]
    flat = [x for lst in lists for tr in lst for x in tr]
    first, count = [0, 2, 2], [2, 0, 3]
    t = torch.tensor(flat, dtype=torch.int64, device=DEV)
    ops.kvt_launch_copy_blocks_multi([x.data_ptr() for x in srcs], [x.data_ptr() for x in dsts], [1 << 20] * 3,
                                     [1 << 20] * 3, first, count, t.data_ptr(), st.data_ptr(), 0, stream)
    torch.cuda.synchronize()
    assert st[0].item() == 0
    for a, b, lst in zip(srcs, dsts, lists):
        want = torch.zeros_like(b)
        for so, do, ln in lst:
            want[do:do + ln] = a[so:so + ln]
        assert torch.equal(b, want)
    # two entries that share ONE descriptor range: the same pages of two layers in one launch
    dsts2 = [torch.zeros(1 << 20, dtype=torch.uint8, device=DEV) for _ in range(2)]
    ops.kvt_launch_copy_blocks_multi([srcs[0].data_ptr(), srcs[2].data_ptr()], [x.data_ptr() for x in dsts2], [1 << 20] * 2,
                                     [1 << 20] * 2, [0, 0], [2, 2], t.data_ptr(), st.data_ptr(), 0, stream)
    torch.cuda.synchronize()
    assert st[0].item() == 0
    for a, b in zip((srcs[0], srcs[2]), dsts2):
        want = torch.zeros_like(b)
        for so, do, ln in lists[0]:
            want[do:do + ln] = a[so:so + ln]
        assert torch.equal(b, want)
    # a descriptor outside its own tensor is reported with its index and skipped
    t_bad = torch.tensor([0, 0, 64, 0, (1 << 20) - 8, 64], dtype=torch.int64, device=DEV)
    ops.kvt_launch_copy_blocks_multi([srcs[0].data_ptr(), srcs[1].data_ptr()], [dsts[0].data_ptr(), dsts[1].data_ptr()],
                                     [1 << 20] * 2, [1 << 20] * 2, [0, 1], [1, 1], t_bad.data_ptr(), st.data_ptr(), 0, stream)
    torch.cuda.synchronize()
    assert st[0].item() == 1 and st[1].item() == 1


def test_bulk_copy_moves_aligned_runs_by_tma_and_the_rest_by_simt(ops):
    """kvt_copy_blocks_bulk: pages (16-byte aligned, whole 16-byte words) go through the TMA engine, odd
    runs and tails through the SIMT warps; entries whose later descriptors are longer than the first
    need more rounds; peers of the plain kernel's checks (range report) hold."""
    st = torch.zeros(4, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device=DEV).manual_seed(11)
    n = 4 << 20
    cases = [
        # MLA-like pages of two tensors
        ([[(0, 41984 * 3, 41984), (41984 * 5, 41984, 41984), (41984 * 9, 41984 * 20, 41984)],
          [(0, 8448 * 2, 8448), (8448 * 7, 8448 * 40, 8448)]]),
        # unaligned starts, odd lengths, a tail that is not a multiple of 16, a run longer than the first
        ([[(16, 32, 100), (4096, 100000, 8192 * 3 + 40), (500001, 300003, 5000), (1 << 20, 2 << 20, 1 << 20)],
          [(8, 8, 16), (1000, 2000, 12345)]]),
    ]
    for lists in cases:
        srcs = [torch.randint(0, 255, (n,), dtype=torch.uint8, device=DEV, generator=g) for _ in lists]
        dsts = [torch.zeros(n, dtype=torch.uint8, device=DEV) for _ in lists]
        flat = [x for lst in lists for tr in lst for x in tr]
        first, count, pos, rounds = [], [], 0, 1
        for lst in lists:
            first.append(pos)
            count.append(len(lst))
            pos += len(lst)
            rounds = max(rounds, ops.kvt_bulk_rounds(lst[0][2], max(tr[2] for tr in lst)))
        t = torch.tensor(flat, dtype=torch.int64, device=DEV)
        ops.kvt_launch_copy_blocks_multi([x.data_ptr() for x in srcs], [x.data_ptr() for x in dsts], [n] * len(lists),
                                         [n] * len(lists), first, count, t.data_ptr(), st.data_ptr(), 0, stream,
                                         bulk_rounds=rounds)
        torch.cuda.synchronize()
        assert st[0].item() == 0
        for a, b, lst in zip(srcs, dsts, lists):
            want = torch.zeros_like(b)
            for so, do, ln in lst:
                want[do:do + ln] = a[so:so + ln]
            assert torch.equal(b, want)
    assert ops.kvt_bulk_rounds(41984, 41984) == 1 and ops.kvt_bulk_rounds(100, 8192 * 3 + 40) == 4
    # a descriptor outside its tensor is reported and skipped
    a = torch.zeros(1 << 16, dtype=torch.uint8, device=DEV)
    t_bad = torch.tensor([0, 0, 64, 0, (1 << 16) - 8, 64], dtype=torch.int64, device=DEV)
    ops.kvt_launch_copy_blocks_multi([a.data_ptr()], [a.data_ptr()], [1 << 16], [1 << 16], [0], [2], t_bad.data_ptr(),
                                     st.data_ptr(), 0, stream, bulk_rounds=1)
    torch.cuda.synchronize()
    assert st[0].item() == 1 and st[1].item() == 1


def test_gather_with_unscaled_bf16_to_e4m3_cast(ops):
    """kvt_copy_blocks_cast: every bf16 bit pattern converts like the host routine (which matches torch's
    cast where e4m3 can hold the value and saturates beyond); descriptors with odd alignments and long
    runs land where they are told."""
    st = torch.zeros(4, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    bits = torch.arange(0, 1 << 16, dtype=torch.int32).to(torch.int16)
    src = torch.cat([bits, bits.flip(0), bits[1:5000]]).to(DEV)          # bf16 words
    nvals = src.numel()
    dst = torch.zeros(nvals + 64, dtype=torch.uint8, device=DEV)
    trip = [(0, 0, 65536), (65536 * 2, 65536, 65536), (65536 * 4 + 2, 65536 * 2 + 3, 4998), (10, 65536 * 2 + 5003, 1)]
    t = torch.tensor([x for tr in trip for x in tr], dtype=torch.int64, device=DEV)
    ops.kvt_launch_copy_blocks_cast(src.data_ptr(), dst.data_ptr(), t.data_ptr(), len(trip), nvals * 2, dst.numel(),
                                    st.data_ptr(), 0, stream)
    torch.cuda.synchronize()
    assert st[0].item() == 0
    table = torch.tensor([ops.kvt_bf16_to_e4m3(b) for b in range(1 << 16)], dtype=torch.uint8)
    words = src.cpu().to(torch.int32) & 0xFFFF
    got = dst.cpu()
    for so, do, n in trip:
        want = table[words[so // 2: so // 2 + n].long()]
        assert torch.equal(got[do:do + n], want), (so, do, n)
    finite = bits.view(torch.bfloat16).float().abs() <= 448
    assert torch.equal(got[:65536][finite], bits.view(torch.bfloat16)[finite].to(torch.float8_e4m3fn).view(torch.uint8))
    # a run whose 2 x n source bytes leave the tensor is reported
    t_bad = torch.tensor([nvals * 2 - 8, 0, 8], dtype=torch.int64, device=DEV)
    ops.kvt_launch_copy_blocks_cast(src.data_ptr(), dst.data_ptr(), t_bad.data_ptr(), 1, nvals * 2, dst.numel(),
                                    st.data_ptr(), 0, stream)
    torch.cuda.synchronize()
    assert st[0].item() == 1


def test_per_layer_launches_replay_from_a_cuda_graph(ops):
    """The launch is fixed-shape and touches no host state, so a step's per-layer launches can be
    captured once and replayed; new block tables reach the kernel through the plan buffer."""
    src_l = AttnLayout(CacheShape.FLASH, 40, 16, 8, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 40, 16, 8, 128, 2)
    L = 4
    src = [src_l.alloc("cuda", "normal", seed=40 + i) for i in range(L)]
    dst = [dst_l.alloc("cuda") for _ in range(L)]
    xfer = AttnTransfer(src_l, dst_l, [t.data_ptr() for t in src], [t.data_ptr() for t in dst], "cuda")
    first = [ReqChunk([3, 9, 12], [7, 1, 30], 0, 48), ReqChunk([5], [8], 0, 11)]
    second = [ReqChunk([20, 21, 22], [2, 3, 4], 0, 48), ReqChunk([33], [35], 0, 11)]   # same shape, other blocks
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        plan = xfer.plan(first, stream=s)
        for layer in range(L):                      # warm-up outside capture (module load, attributes)
            xfer.launch(plan, layer, layer + 1, stream=s)
    s.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        for layer in range(L):
            xfer.launch(plan, layer, layer + 1, stream=s)
    for d in dst:
        d.zero_()
    g.replay()
    torch.cuda.synchronize()
    for i in range(L):
        expect = torch.zeros_like(dst[i])
        reference_transfer(src_l, dst_l, src[i], expect, first)
        assert torch.equal(dst[i], expect)
    # next step: overwrite the plan buffer in place, replay the same graph
    plan2 = xfer.plan(second)
    torch.cuda.synchronize()
    assert plan2.nbytes == plan.nbytes and plan2.total_tiles == plan.total_tiles
    plan.dev.copy_(plan2.dev)
    for d in dst:
        d.zero_()
    g.replay()
    torch.cuda.synchronize()
    for i in range(L):
        expect = torch.zeros_like(dst[i])
        reference_transfer(src_l, dst_l, src[i], expect, second)
        assert torch.equal(dst[i], expect)
    assert xfer.check_status() == (0, 0)
