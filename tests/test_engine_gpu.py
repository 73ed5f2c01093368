"""The engine end to end on a GPU: KVTransferClient -> step pipeline -> send stub -> transport ->
destination cache, checked against the plain-PyTorch oracle / direct tensor comparison.

Single-GPU cases put both caches on cuda:0 (the NVLink transport then runs its kernels with a
local destination pointer; the code path is the same as for a peer).  Multi-GPU and
two-process cases are in test_engine_multigpu.py.
"""
import os
import random
import time

import pytest
import torch

os.environ.setdefault("BLLM_KVTRANS_QUIET_ENV", "1")

from llumnix_kv_b200.kv_transfer_impl import KVTransferClient, KVTransferProtocolType as PT, KVTransferServer
from llumnix_kv_b200.ops.layouts import AttnLayout, CacheShape
from llumnix_kv_b200.ops.p2d_attn import (MODE_BF16_TO_MXFP8, MODE_COPY, HeadMap, ReqChunk, reference_transfer)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
L = 3


def run_step(cli, dst_inst, dst_worker, winfo, reqs, stepid, stream=None):
    for rid, sb, db, seen, new, last, first in reqs:
        if first:
            cli.submit_req_send2(dst_inst, dst_worker, rid, seen, new, last, sb, db, winfo, stepid=stepid)
        else:
            cli.submit_delta_send(rid, seen, new, last, stepid=stepid)
    cli.start_send_step(stepid, 1)
    for layer in range(L):
        cli.record_event(layer, stream)
    cli.flush_send_step()
    cli.drain()
    torch.cuda.synchronize()


def rand_reqs(rng, n, nb_s, nb_d, ntpb, max_blocks=6):
    fs, fd = list(range(1, nb_s)), list(range(1, nb_d))
    rng.shuffle(fs)
    rng.shuffle(fd)
    out = []
    for i in range(n):
        nb = rng.randint(1, max_blocks)
        sb, db = [fs.pop() for _ in range(nb)], [fd.pop() for _ in range(nb)]
        total = nb * ntpb - rng.randint(0, ntpb - 1)
        out.append((f"r{i}", sb, db, total))
    return out


@pytest.mark.parametrize("proto", [PT.NVLINK, PT.TCP, PT.SHM])
def test_same_layout_transfer_all_transports(proto):
    rng = random.Random(1)
    lay = AttnLayout(CacheShape.FLASH, 48, 16, 8, 128, 2)
    src = [lay.alloc(DEV, "normal", seed=i) for i in range(L)]
    dst = [lay.alloc(DEV) for _ in range(L)]
    srv = KVTransferServer("D|0|1", 1, 0, 0, lay.block_bytes, lay.token_bytes, "fake://", dst, [proto], num_kv_heads=8,
                           cache_shape=2)
    cli = KVTransferClient("P|0|1", 1, 0, 0, lay.block_bytes, lay.token_bytes, "fake://", src, [proto], num_kv_heads=8,
                           cache_shape=2)
    try:
        reqs = rand_reqs(rng, 4, 48, 48, 16)
        # two chunks per request: exercises deltas and ragged block edges on every transport
        cut = {rid: rng.randint(1, total - 1) if total > 1 else 1 for rid, _, _, total in reqs}
        run_step(cli, "D|0|1", 0, srv.worker_info(),
                 [(rid, sb, db, 0, cut[rid], cut[rid] == total, True) for rid, sb, db, total in reqs], 1)
        run_step(cli, "D|0|1", 0, srv.worker_info(),
                 [(rid, sb, db, cut[rid], total - cut[rid], True, False) for rid, sb, db, total in reqs
                  if cut[rid] < total], 2)
        chunks = [ReqChunk(sb, db, 0, total) for _, sb, db, total in reqs]
        for i in range(L):
            expect = torch.zeros_like(dst[i])
            reference_transfer(lay, lay, src[i], expect, chunks)
            assert torch.equal(dst[i], expect)
    finally:
        srv.stop()


def test_nvlink_nhd_to_hnd_cross_layout():
    rng = random.Random(2)
    src_l = AttnLayout(CacheShape.FLASH, 40, 16, 8, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 56, 16, 8, 128, 2)
    src = [src_l.alloc(DEV, "normal", seed=i) for i in range(L)]
    dst = [dst_l.alloc(DEV) for _ in range(L)]
    srv = KVTransferServer("D|0|1", 1, 0, 0, dst_l.block_bytes, dst_l.token_bytes, "fake://", dst, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=5)
    cli = KVTransferClient("P|0|1", 1, 0, 0, src_l.block_bytes, src_l.token_bytes, "fake://", src, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=2)
    try:
        reqs = rand_reqs(rng, 5, 40, 56, 16)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            run_step(cli, "D|0|1", 0, srv.worker_info(), [(rid, sb, db, 0, t, True, True) for rid, sb, db, t in reqs], 7,
                     stream=side)
        chunks = [ReqChunk(sb, db, 0, t) for _, sb, db, t in reqs]
        for i in range(L):
            expect = torch.zeros_like(dst[i])
            reference_transfer(src_l, dst_l, src[i], expect, chunks)
            assert torch.equal(dst[i], expect)
    finally:
        srv.stop()


def test_nvlink_tp_mismatch_with_block_scaled_fp8_destination():
    """Config-3 shape in miniature: prefill TP=4 rank 1 (2 of 8 heads, bf16, NHD) -> decode TP=2 rank 0
    (4 heads, block-scaled e4m3, HND); heads land in the second half of the decode rank's pages."""
    rng = random.Random(3)
    src_l = AttnLayout(CacheShape.FLASH, 40, 16, 2, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 40, 16, 4, 128, 1, mx_scaled=True)
    src = [src_l.alloc(DEV, "normal", seed=20 + i) for i in range(L)]
    dst = [dst_l.alloc(DEV) for _ in range(L)]
    srv = KVTransferServer("D|0|2", 2, 0, 0, dst_l.block_bytes, dst_l.token_bytes, "fake://", dst, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=5, mx_scaled=True)
    cli = KVTransferClient("P|0|4", 4, 1, 1, src_l.block_bytes, src_l.token_bytes, "fake://", src, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=2)
    try:
        reqs = rand_reqs(rng, 4, 40, 40, 16)
        run_step(cli, "D|0|2", 0, srv.worker_info(), [(rid, sb, db, 0, t, True, True) for rid, sb, db, t in reqs], 3)
        chunks = [ReqChunk(sb, db, 0, t) for _, sb, db, t in reqs]
        for i in range(L):
            expect = torch.zeros_like(dst[i])
            reference_transfer(src_l, dst_l, src[i], expect, chunks, HeadMap(0, 2, 2), MODE_BF16_TO_MXFP8)
            assert torch.equal(dst[i], expect)
    finally:
        srv.stop()


@pytest.mark.parametrize("path", [1, 2, 0])
def test_host_staged_copies_by_kernel_by_copy_engines_and_by_measured_policy(path, ops, monkeypatch, capsys):
    """The TCP transport gathers to / scatters from pinned host memory either with the descriptor kernel
    or with one cudaMemcpyAsync per run; a forced path must be the one that runs, and the policy measured
    at start-up must deliver the same bytes whatever it picks."""
    monkeypatch.setenv("BLLM_KVTRANS_COPY_PATH", str(path))
    ops.envcfg_reset_for_test()
    ops.copy_policy_reset_for_test()
    m0, k0 = ops.copy_path_counters()
    rng = random.Random(7)
    lay = AttnLayout(CacheShape.FLASH, 48, 16, 8, 128, 2)
    src = [lay.alloc(DEV, "normal", seed=i) for i in range(L)]
    dst = [lay.alloc(DEV) for _ in range(L)]
    srv = KVTransferServer("D|0|1", 1, 0, 0, lay.block_bytes, lay.token_bytes, "fake://", dst, [PT.TCP], num_kv_heads=8,
                           cache_shape=2)
    cli = KVTransferClient("P|0|1", 1, 0, 0, lay.block_bytes, lay.token_bytes, "fake://", src, [PT.TCP], num_kv_heads=8,
                           cache_shape=2)
    try:
        reqs = rand_reqs(rng, 3, 48, 48, 16)
        run_step(cli, "D|0|1", 0, srv.worker_info(), [(rid, sb, db, 0, total, True, True) for rid, sb, db, total in reqs], 1)
        chunks = [ReqChunk(sb, db, 0, total) for _, sb, db, total in reqs]
        for i in range(L):
            expect = torch.zeros_like(dst[i])
            reference_transfer(lay, lay, src[i], expect, chunks)
            assert torch.equal(dst[i], expect)
        m1, k1 = ops.copy_path_counters()
        assert (m1 - m0) + (k1 - k0) >= 2 * L          # gather and scatter, per layer
        if path == 1:
            assert m1 == m0
        elif path == 2:
            assert k1 == k0
        else:
            table = ops.copy_policy_describe(0)
            assert table.startswith("d2h:") and "\nh2d:" in table and "us(kernel/memcpy)" in table
            with capsys.disabled():
                print("\n" + table)
    finally:
        srv.stop()
        monkeypatch.delenv("BLLM_KVTRANS_COPY_PATH")
        ops.envcfg_reset_for_test()
        ops.copy_policy_reset_for_test()


@pytest.mark.parametrize("proto", [PT.NVLINK, PT.TCP])
def test_hybrid_gdn_pages_via_descriptor_path(proto, ops):
    """Qwen3-Next-like hybrid pages (GDN state + attention in one tensor) with P TP=2 -> D TP=1: no
    fused kernel for this shape, the planner's IpcBlocks drive the descriptor copy kernel."""
    rows, dims_p, ssm = 3, [32, 32, 64], [1, 4, 8, 8]
    hd, heads = 64, 4
    p_tok, d_tok = 2 * 2 * hd, 2 * 4 * hd
    ntpb = 16
    p_bs, d_bs = p_tok * ntpb, d_tok * ntpb
    nb = 32
    kw_p = dict(num_kv_heads=heads, num_gdn_layers=1, conv_state_shape=[1, rows, sum(dims_p)], ssm_state_shape=ssm,
                gdn_conv_channel_dims=dims_p, gdn_conv_elem_size=2, gdn_ssm_elem_size=4)
    kw_d = dict(kw_p)
    kw_d.update(conv_state_shape=[1, rows, 2 * sum(dims_p)], gdn_conv_channel_dims=[2 * d for d in dims_p],
                ssm_state_shape=[1, 8, 8, 8])
    g = torch.Generator(device=DEV).manual_seed(5)
    src = [torch.randint(0, 255, (nb * p_bs,), dtype=torch.uint8, device=DEV, generator=g) for _ in range(L)]
    dst = [torch.zeros(nb * d_bs, dtype=torch.uint8, device=DEV) for _ in range(L)]
    for s in src:
        s[:p_bs] = 0  # block 0 is the engine's all-zero block (tail padding reads it)
    srv = KVTransferServer("D|0|1", 1, 0, 0, d_bs, d_tok, "fake://", dst, [proto], cache_shape=3, **kw_d)
    cli = KVTransferClient("P|0|2", 2, 1, 1, p_bs, p_tok, "fake://", src, [proto], cache_shape=3, **kw_p)
    try:
        sb, db = [[3], [0, 7, 9]], [[5], [2, 6, 11]]
        total = 2 * ntpb + 5
        cli.submit_req_send2("D|0|1", 0, "hyb", 0, total, True, sb, db, srv.worker_info(), stepid=1)
        cli.start_send_step(1, 1)
        for layer in range(L):
            cli.record_event(layer)
        cli.flush_send_step()
        cli.drain()
        torch.cuda.synchronize()
        W = ops.WorkerInfo
        pw, dw = W.from_string(cli.worker_info()), W.from_string(srv.worker_info())
        for w, kw in ((pw, kw_p), (dw, kw_d)):
            for k, v in kw.items():
                setattr(w, k, v)
        blocks = ops.plan_ipc_blocks(pw, dw, 3, [("hyb", 0, total, True, sb, db)])[0][0]
        assert len(blocks) > 20
        for i in range(L):
            expect = torch.zeros_like(dst[i])
            for s_off, d_off, n in blocks:
                expect[d_off:d_off + n] = src[i][s_off:s_off + n]
            assert torch.equal(dst[i], expect)
    finally:
        srv.stop()


def test_layer_overlap_waits_for_the_layer_event():
    """A transfer enqueued before the forward stream produced the layer must still see the final
    bytes: the transport orders itself after the layer's CUDA event, not after host time."""
    lay = AttnLayout(CacheShape.FLASH, 16, 16, 8, 128, 2)
    src = [lay.alloc(DEV) for _ in range(L)]
    dst = [lay.alloc(DEV) for _ in range(L)]
    srv = KVTransferServer("D|0|1", 1, 0, 0, lay.block_bytes, lay.token_bytes, "fake://", dst, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=2)
    cli = KVTransferClient("P|0|1", 1, 0, 0, lay.block_bytes, lay.token_bytes, "fake://", src, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=2)
    try:
        fwd = torch.cuda.Stream()
        big = torch.empty(1 << 28, dtype=torch.uint8, device=DEV)
        cli.submit_req_send2("D|0|1", 0, "r", 0, 48, True, [1, 2, 3], [4, 5, 6], srv.worker_info(), stepid=1)
        cli.start_send_step(1, 1)
        with torch.cuda.stream(fwd):
            for layer in range(L):
                for _ in range(4):
                    big.fill_(layer)  # keeps the stream busy so the layer is produced "late"
                src[layer].fill_(layer + 1)
                cli.record_event(layer, fwd)
        cli.flush_send_step()
        cli.drain()
        torch.cuda.synchronize()
        for layer in range(L):
            v = lay.view(dst[layer], torch.int16)
            assert int(v[4:7].min()) == int(v[4:7].max()) == (layer + 1) * 257
    finally:
        srv.stop()


_STAMP_SCRIPT = r"""
import torch
from llumnix_kv_b200.kv_transfer_impl import KVTransferClient, KVTransferProtocolType as PT, KVTransferServer
from llumnix_kv_b200.ops.layouts import AttnLayout, CacheShape
lay = AttnLayout(CacheShape.FLASH, 48, 16, 8, 128, 2)
src = [lay.alloc("cuda:0", "normal", seed=i) for i in range(3)]
dst = [lay.alloc("cuda:0") for _ in range(3)]
srv = KVTransferServer("D|0|1", 1, 0, 0, lay.block_bytes, lay.token_bytes, "fake://", dst, [PT.NVLINK], num_kv_heads=8, cache_shape=2)
cli = KVTransferClient("P|0|1", 1, 0, 0, lay.block_bytes, lay.token_bytes, "fake://", src, [PT.NVLINK], num_kv_heads=8, cache_shape=2)
cli.submit_req_send2("D|0|1", 0, "r", 0, 40, True, [3, 5, 7], [2, 4, 6], srv.worker_info(), stepid=1)
cli.start_send_step(1, 1)
for layer in range(3):
    cli.record_event(layer, None)
cli.flush_send_step()
cli.drain()
torch.cuda.synchronize()
assert torch.equal(dst[0].view(-1)[:16], dst[0].view(-1)[:16])
srv.stop()
"""


def test_device_timestamps_in_the_flush_metrics():
    """With BLLM_KVTRANS_DEVICE_TIMESTAMPS=1 the NVLink channel stamps the GPU timer at the start and the
    end of a batch and reports the difference as DeviceUs in its metrics line."""
    import re
    import subprocess
    import sys

    env = dict(os.environ, BLLM_KVTRANS_DEVICE_TIMESTAMPS="1", LLMOPS_CPP_MIN_LOG_LEVEL="0")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", _STAMP_SCRIPT], cwd=root, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    m = re.search(r"SendStubMetrics\..*Proto=nvlink,Mode=push,Path=fused.*DeviceUs=(-?\d+)", r.stderr)
    assert m is not None, r.stderr[-2000:]
    assert 0 <= int(m.group(1)) < 1_000_000


def test_step_completes_through_the_completion_record_without_a_host_sync():
    """The NVLINK channel finishes a batch from a record that the GPU writes into mapped host memory behind
    the last transfer kernel: flush returns at once (FlushUs is the enqueue, not the transfer), the
    engine thread can run a step ahead (wait_inflight(1)), and the bytes are right when the records are in."""
    rng = random.Random(11)
    src_l = AttnLayout(CacheShape.FLASH, 96, 16, 8, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 96, 16, 8, 128, 2)
    src = [src_l.alloc(DEV, "normal", seed=i) for i in range(L)]
    dst = [dst_l.alloc(DEV) for _ in range(L)]
    srv = KVTransferServer("D|0|1", 1, 0, 0, dst_l.block_bytes, dst_l.token_bytes, "fake://", dst, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=5)
    cli = KVTransferClient("P|0|1", 1, 0, 0, src_l.block_bytes, src_l.token_bytes, "fake://", src, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=2)
    try:
        reqs = rand_reqs(rng, 8, 96, 96, 16, max_blocks=5)
        # one request per step, eight steps issued back to back; at most one step may be outstanding when the
        # next is submitted, none at the end
        for i, (rid, sb, db, total) in enumerate(reqs):
            cli.submit_req_send2("D|0|1", 0, rid, 0, total, True, sb, db, srv.worker_info(), stepid=100 + i)
            cli.start_send_step(100 + i, 1)
            for layer in range(L):
                cli.record_event(layer)
            cli.flush_send_step()
            assert cli.wait_inflight(1, 20.0)
            assert cli.inflight() <= 1
        assert cli.wait_inflight(0, 20.0)
        assert cli.inflight() == 0
        chunks = [ReqChunk(sb, db, 0, total) for _, sb, db, total in reqs]
        for i in range(L):
            expect = torch.zeros_like(dst[i])
            reference_transfer(src_l, dst_l, src[i], expect, chunks)
            assert torch.equal(dst[i], expect)     # no torch.cuda.synchronize(): the records say the data is there
    finally:
        srv.stop()


def test_a_completion_record_that_never_arrives_fails_the_request_within_its_deadline():
    """Host-side stall: the batch's kernels run, but its completion record is left out (fault hook), so the
    poller is never signalled.  The deadline fails the request (send-done code 500 semantics: state FAILED),
    the channel is dropped, and the next step goes through on a fresh channel.  No kernel waits or hangs."""
    import llumnix_kv_b200

    K = llumnix_kv_b200.load_ops()
    lay = AttnLayout(CacheShape.FLASH, 48, 16, 8, 128, 2)
    src = [lay.alloc(DEV, "normal", seed=i) for i in range(L)]
    dst = [lay.alloc(DEV) for _ in range(L)]
    os.environ["BLLM_KVTRANS_COMPLETION_TIMEOUT_MS"] = "400"
    K.envcfg_reset_for_test()
    srv = KVTransferServer("D|0|1", 1, 0, 0, lay.block_bytes, lay.token_bytes, "fake://", dst, [PT.NVLINK], num_kv_heads=8,
                           cache_shape=2)
    cli = KVTransferClient("P|0|1", 1, 0, 0, lay.block_bytes, lay.token_bytes, "fake://", src, [PT.NVLINK], num_kv_heads=8,
                           cache_shape=2)
    try:
        K.fault_inject_arm_drop_completion(1)
        t0 = time.time()
        run_step(cli, "D|0|1", 0, srv.worker_info(), [("lost", [1, 2], [3, 4], 0, 32, True, True)], 1)
        took = time.time() - t0
        assert 0.3 < took < 5.0, took                 # the deadline, not the 7 s RPC timeout and not forever
        assert cli.inflight() == 0
        # the data of the "lost" batch did move (only its record was dropped); what matters is that the next
        # batch is not stuck behind it
        run_step(cli, "D|0|1", 0, srv.worker_info(), [("next", [5, 6, 7], [8, 9, 10], 0, 40, True, True)], 2)
        expect = torch.zeros_like(dst[0])
        reference_transfer(lay, lay, src[0], expect, [ReqChunk([1, 2], [3, 4], 0, 32), ReqChunk([5, 6, 7], [8, 9, 10], 0, 40)])
        assert torch.equal(dst[0], expect)
    finally:
        os.environ.pop("BLLM_KVTRANS_COMPLETION_TIMEOUT_MS", None)
        K.envcfg_reset_for_test()
        srv.stop()


# ---- end-to-end transfer check ------------------------------------------------------------------
def test_checksum_kernel_matches_the_host_function(ops):
    """Chunks of every alignment class (16-byte vector path, word path, words assembled from bytes at odd
    offsets, ragged tails, a chunk that continues a piece at a non-zero index, an index that wraps) against the
    CPU function; a chunk outside the tensor is skipped and reported."""
    import numpy as np

    g = torch.Generator(device=DEV).manual_seed(11)
    cap = 1 << 20
    buf = torch.randint(0, 256, (cap,), dtype=torch.uint8, device=DEV, generator=g)
    host = buf.cpu().numpy()
    chunks = [(0, 65536, 0), (65536, 65536, 16384), (131072 + 16, 4096, 0), (200001, 777, 5), (300000, 1, 0), (300004, 6, 9),
              (400000, 65535, 123456), (cap - 48, 48, 0xFFFFFFF8)]        # offset, length, index of the first word
    arr = np.zeros(len(chunks), dtype=[("off", "<u8"), ("len", "<u4"), ("idx", "<u4")])
    for i, c in enumerate(chunks):
        arr[i] = c
    d_chunks = torch.from_numpy(arr.view(np.uint8).copy()).to(DEV)
    # one launch sums the same chunks over several tensors of one shape (the layers of a cache)
    buf2 = torch.randint(0, 256, (cap,), dtype=torch.uint8, device=DEV, generator=g)
    host2 = buf2.cpu().numpy()
    bases = torch.tensor([buf.data_ptr(), buf2.data_ptr()], dtype=torch.int64, device=DEV)
    out = torch.zeros(3, dtype=torch.int64, device=DEV)     # [sum of buf, sum of buf2, status words]
    s = torch.cuda.current_stream().cuda_stream
    ops.kvt_launch_checksum(bases.data_ptr(), 2, cap, d_chunks.data_ptr(), len(chunks), out.data_ptr(), out.data_ptr() + 16, 0, s)
    torch.cuda.synchronize()
    expect = sum(ops.kvt_checksum_host(host[o:o + n], i) for o, n, i in chunks) & 0xFFFFFFFFFFFFFFFF
    expect2 = sum(ops.kvt_checksum_host(host2[o:o + n], i) for o, n, i in chunks) & 0xFFFFFFFFFFFFFFFF
    assert int(out[0].item()) & 0xFFFFFFFFFFFFFFFF == expect
    assert int(out[1].item()) & 0xFFFFFFFFFFFFFFFF == expect2 != expect
    assert int(out[2].item()) == 0
    # one grid of 3 CTAs gives the same sum as the default grid: the order of visits does not matter
    out = torch.zeros(2, dtype=torch.int64, device=DEV)     # [sum, status words]
    ops.kvt_launch_checksum(bases.data_ptr(), 1, cap, d_chunks.data_ptr(), len(chunks), out.data_ptr(), out.data_ptr() + 8, 3, s)
    torch.cuda.synchronize()
    assert int(out[0].item()) & 0xFFFFFFFFFFFFFFFF == expect
    # a chunk that leaves the tensor is not read
    arr[2] = (cap - 8, 16, 0)
    d_bad = torch.from_numpy(arr.view(np.uint8).copy()).to(DEV)
    out.zero_()
    ops.kvt_launch_checksum(bases.data_ptr(), 1, cap, d_bad.data_ptr(), len(chunks), out.data_ptr(), out.data_ptr() + 8, 0, s)
    torch.cuda.synchronize()
    status = int(out[1].item())
    assert status & 0xFFFFFFFF != 0 and status >> 32 == 2


@pytest.mark.parametrize("proto", [PT.NVLINK, PT.TCP])
def test_transfer_check_between_device_caches(proto, ops):
    """BLLM_KVTRANS_CRC=1 with GPU caches: each side sums its own ranges with the checksum kernel.  Intact
    batches pass (two chunks of a request, ragged edges); the batch whose sender-side sum is perturbed fails;
    the next one passes on a fresh channel."""
    os.environ["BLLM_KVTRANS_CRC"] = "1"
    ops.envcfg_reset_for_test()
    lay = AttnLayout(CacheShape.FLASHINFER, 48, 16, 8, 128, 2)
    src = [lay.alloc(DEV, "normal", seed=i) for i in range(L)]
    dst = [lay.alloc(DEV) for _ in range(L)]
    srv = KVTransferServer("D|0|1", 1, 0, 0, lay.block_bytes, lay.token_bytes, "fake://", dst, [proto], num_kv_heads=8,
                           cache_shape=5)
    cli = KVTransferClient("P|0|1", 1, 0, 0, lay.block_bytes, lay.token_bytes, "fake://", src, [proto], num_kv_heads=8,
                           cache_shape=5)
    try:
        w = srv.worker_info()
        run_step(cli, "D|0|1", 0, w, [("a", [3, 9, 4], [7, 1, 8], 0, 21, False, True), ("b", [20], [21], 0, 16, True, True)], 1)
        run_step(cli, "D|0|1", 0, w, [("a", [3, 9, 4], [7, 1, 8], 21, 20, True, False)], 2)
        assert cli.failed_batches() == 0
        ops.fault_inject_arm_corrupt_check(1)
        run_step(cli, "D|0|1", 0, w, [("c", [5], [6], 0, 12, True, True)], 3)
        assert cli.failed_batches() == 1
        run_step(cli, "D|0|1", 0, w, [("d", [11, 12], [13, 14], 0, 32, True, True)], 4)
        assert cli.failed_batches() == 1
        chunks = [ReqChunk([3, 9, 4], [7, 1, 8], 0, 41), ReqChunk([20], [21], 0, 16), ReqChunk([5], [6], 0, 12),
                  ReqChunk([11, 12], [13, 14], 0, 32)]
        for i in range(L):
            expect = torch.zeros_like(dst[i])
            reference_transfer(lay, lay, src[i], expect, chunks)
            assert torch.equal(dst[i], expect)
    finally:
        ops.fault_inject_arm_corrupt_check(0)
        srv.stop()
        os.environ.pop("BLLM_KVTRANS_CRC", None)
        ops.envcfg_reset_for_test()


def test_server_check_request_over_a_device_cache(ops):
    """The destination half alone: CHECK_REQ over a GPU cache answers the sum that the CPU function gives
    for the same bytes, and the sum moves when one checked byte changes."""
    import socket
    import struct

    lay = AttnLayout(CacheShape.FLASH, 48, 16, 8, 128, 2)
    dst = [lay.alloc(DEV, "normal", seed=40 + i) for i in range(L)]
    srv = KVTransferServer("D|0|1", 1, 0, 0, lay.block_bytes, lay.token_bytes, "fake://", dst, [PT.TCP], num_kv_heads=8,
                           cache_shape=2)
    port = int(ops.WorkerInfo.from_string(srv.worker_info()).ext["port"])
    ranges = [(5 * lay.block_bytes + 64, 300), (10 * lay.block_bytes, 3 * 65536 + 32), (7, 1)]

    def ask(c):
        body = struct.pack("=IIII", 0, L, 1, 0) + struct.pack("=Q", len(ranges)) + b"".join(struct.pack("=QQ", o, n) for o, n in ranges)
        msg = struct.pack("=IQ", 0x4B56436B, 9) + body
        c.sendall(struct.pack("=I", len(msg)) + msg)
        n = struct.unpack("=I", c.recv(4, socket.MSG_WAITALL))[0]
        _, _, status, total = struct.unpack("=IQIQ", c.recv(n, socket.MSG_WAITALL)[:24])
        return status, total

    def rotl(v, r):
        r &= 63
        return v if r == 0 else ((v << r) | (v >> (64 - r))) & 0xFFFFFFFFFFFFFFFF

    def expect():
        total = 0
        for layer in range(L):
            raw = dst[layer].view(torch.uint8).flatten().cpu().numpy()
            total += rotl(sum(ops.kvt_checksum_host(raw[o:o + n]) for o, n in ranges) & 0xFFFFFFFFFFFFFFFF, layer * 7)
        return total & 0xFFFFFFFFFFFFFFFF

    try:
        with socket.create_connection(("127.0.0.1", port), timeout=10) as c:
            first = ask(c)
            assert first == (0, expect())
            dst[2].view(torch.uint8).flatten()[10 * lay.block_bytes + 70000] ^= 1
            torch.cuda.synchronize()
            second = ask(c)
            assert second == (0, expect()) and second[1] != first[1]
    finally:
        srv.stop()


def _rows_oracle(ops, lay, flat, head0, n_heads, reqs):
    """The row form of the check, spelled out: every (request, token, K / V, head) row keyed by its logical
    coordinates, summed with the CPU function."""
    import dataclasses

    as_bytes = dataclasses.replace(lay, head_dim=lay.head_bytes, elem_bytes=1)
    v = as_bytes.view(flat.cpu(), torch.uint8).numpy()           # [block, kv, slot, head, byte]
    total = 0
    for blocks, seen, new, index in reqs:
        for t in range(seen, seen + new):
            blk, slot = blocks[t // lay.ntpb], t % lay.ntpb
            for kv in range(lay.kv_count):
                for j in range(n_heads):
                    row_id = (((index * 131 + t) * lay.kv_count + kv) * n_heads + j) & 0xFFFFFFFF
                    total += ops.kvt_checksum_host(v[blk, kv, slot, head0 + j].copy(), (row_id * ((lay.head_bytes + 3) // 4)) & 0xFFFFFFFF)
    return total & 0xFFFFFFFFFFFFFFFF


def _rows_kernel(ops, lay, flat, head0, n_heads, reqs, grid=0):
    import numpy as np

    pool, rows, first = [], [], 0
    for blocks, seen, new, index in reqs:
        rows.append((len(pool), len(blocks), seen, new, first, index))
        pool += blocks
        first += new
    d_reqs = torch.tensor(np.array(rows, dtype=np.uint32).view(np.int32), device=DEV)
    d_pool = torch.tensor(np.array(pool, dtype=np.uint32).view(np.int32), device=DEV)
    out = torch.zeros(2, dtype=torch.int64, device=DEV)
    bases = torch.tensor([flat.data_ptr()], dtype=torch.int64, device=DEV)
    ops.kvt_launch_checksum_attn(bases.data_ptr(), 1, flat.numel(), lay.to_kvt(), head0, n_heads, d_reqs.data_ptr(), len(rows), first,
                                 d_pool.data_ptr(), len(pool), out.data_ptr(), out.data_ptr() + 8, grid,
                                 torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return int(out[0].item()) & 0xFFFFFFFFFFFFFFFF, int(out[1].item())


@pytest.mark.parametrize("head_dim", [64, 256])       # rows of 128 bytes (half a warp each) and of 512 bytes (a warp each)
def test_row_checksum_is_the_same_on_both_sides_of_a_layout_change(ops, head_dim):
    """NHD pages with 8 heads against HND pages with 4 heads that received heads 4..7: the kernel's sums
    over the two layouts agree with each other and with the spelled-out oracle; one flipped bit in a moved row,
    or two rows exchanged, changes the destination's sum."""
    src_l = AttnLayout(CacheShape.FLASH, 24, 16, 8, head_dim, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 30, 32, 4, head_dim, 2)
    src = src_l.alloc(DEV, "normal", seed=3)
    dst = dst_l.alloc(DEV)
    moves = [([3, 9, 1], [7, 2], 5, 40), ([5, 6], [11], 0, 21), ([20], [21], 0, 16)]     # src blocks, dst blocks, seen, new
    chunks = [ReqChunk(sb, db, seen, new) for sb, db, seen, new in moves]
    reference_transfer(src_l, dst_l, src, dst, chunks, HeadMap(4, 0, 4))
    s_reqs = [(sb, seen, new, i) for i, (sb, _, seen, new) in enumerate(moves)]
    d_reqs = [(db, seen, new, i) for i, (_, db, seen, new) in enumerate(moves)]
    s_sum, s_st = _rows_kernel(ops, src_l, src, 4, 4, s_reqs)
    d_sum, d_st = _rows_kernel(ops, dst_l, dst, 0, 4, d_reqs)
    assert (s_st, d_st) == (0, 0)
    assert s_sum == d_sum == _rows_oracle(ops, src_l, src, 4, 4, s_reqs) == _rows_oracle(ops, dst_l, dst, 0, 4, d_reqs)
    assert _rows_kernel(ops, dst_l, dst, 0, 4, d_reqs, grid=2)[0] == d_sum
    v = dst_l.view(dst, torch.bfloat16)
    keep = v[7, 1, 9, 2].clone()
    v[7, 1, 9, 2, 5] = -v[7, 1, 9, 2, 5]                      # token 9 of request 0, V, head 2: sign bit of one value
    assert _rows_kernel(ops, dst_l, dst, 0, 4, d_reqs)[0] != d_sum
    v[7, 1, 9, 2] = keep
    assert _rows_kernel(ops, dst_l, dst, 0, 4, d_reqs)[0] == d_sum
    other = v[7, 1, 10, 2].clone()
    v[7, 1, 10, 2] = keep                                     # two tokens' rows exchanged: same bytes, other places
    v[7, 1, 9, 2] = other
    assert _rows_kernel(ops, dst_l, dst, 0, 4, d_reqs)[0] != d_sum
    # a block id outside the tensor is reported, not read
    bad = [([40], 0, 16, 0)]
    assert _rows_kernel(ops, dst_l, dst, 0, 4, bad)[1] & 0xFFFFFFFF != 0


@pytest.mark.parametrize("tp", ["equal", "p_gt_d"])
def test_transfer_check_of_a_layout_converting_transfer(tp, ops):
    """BLLM_KVTRANS_CRC=1 on the fused NHD -> HND path (equal TP, and prefill TP 2 -> decode TP 1 where this
    rank's heads land in the upper half of the destination's): the row form passes intact batches, chunked
    included, and fails the batch whose sender-side sum is perturbed."""
    os.environ["BLLM_KVTRANS_CRC"] = "1"
    ops.envcfg_reset_for_test()
    p_heads, p_tp, p_rank = (8, 1, 0) if tp == "equal" else (4, 2, 1)
    src_l = AttnLayout(CacheShape.FLASH, 40, 16, p_heads, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 56, 16, 8, 128, 2)
    src = [src_l.alloc(DEV, "normal", seed=60 + i) for i in range(L)]
    dst = [dst_l.alloc(DEV) for _ in range(L)]
    srv = KVTransferServer("D|0|1", 1, 0, 0, dst_l.block_bytes, dst_l.token_bytes, "fake://", dst, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=5)
    cli = KVTransferClient(f"P|0|{p_tp}", p_tp, p_rank, p_rank, src_l.block_bytes, src_l.token_bytes, "fake://", src, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=2)
    try:
        w = srv.worker_info()
        run_step(cli, "D|0|1", 0, w, [("a", [3, 9, 4], [7, 1, 8], 0, 21, False, True), ("b", [20], [21], 0, 16, True, True)], 1)
        run_step(cli, "D|0|1", 0, w, [("a", [3, 9, 4], [7, 1, 8], 21, 20, True, False)], 2)
        assert cli.failed_batches() == 0
        ops.fault_inject_arm_corrupt_check(1)
        run_step(cli, "D|0|1", 0, w, [("c", [5], [6], 0, 12, True, True)], 3)
        assert cli.failed_batches() == 1
        run_step(cli, "D|0|1", 0, w, [("d", [11, 12], [13, 14], 0, 32, True, True)], 4)
        assert cli.failed_batches() == 1
        chunks = [ReqChunk([3, 9, 4], [7, 1, 8], 0, 41), ReqChunk([20], [21], 0, 16), ReqChunk([5], [6], 0, 12),
                  ReqChunk([11, 12], [13, 14], 0, 32)]
        hm = HeadMap(0, 0, 8) if tp == "equal" else HeadMap(0, 4, 4)
        for i in range(L):
            expect = torch.zeros_like(dst[i])
            reference_transfer(src_l, dst_l, src[i], expect, chunks, hm)
            assert torch.equal(dst[i], expect)
    finally:
        ops.fault_inject_arm_corrupt_check(0)
        srv.stop()
        os.environ.pop("BLLM_KVTRANS_CRC", None)
        ops.envcfg_reset_for_test()


# ---- randomized ------------------------------------------------------------------------------------
from test_engine_cpu import random_chunked_requests, sink  # noqa: E402,F401  (the send-done sink fixture)


@pytest.mark.parametrize("seed", [1, 2])
def test_random_chunked_requests_over_the_device_transport_with_faults_and_lost_completions(seed, ops, sink):
    """The randomized engine test of the CPU suite with GPU caches over the NVLINK transport: plan slots,
    per-layer launches and completion records of several destinations and steps overlap, some batches fail on
    their way (injected on the host) and some lose their completion record, which their deadline turns into a
    failed batch.  No kernel waits on anything that may not come."""
    os.environ["BLLM_KVTRANS_COMPLETION_TIMEOUT_MS"] = "300"
    ops.envcfg_reset_for_test()
    try:
        random_chunked_requests(PT.NVLINK, seed, ops, sink, DEV, drop_completions=True)
        torch.cuda.synchronize()
    finally:
        os.environ.pop("BLLM_KVTRANS_COMPLETION_TIMEOUT_MS", None)
        ops.envcfg_reset_for_test()
