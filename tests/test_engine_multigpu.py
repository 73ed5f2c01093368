"""Engine over NVLink between two GPUs: inside one process (peer access) and between two
processes (CUDA IPC handles fetched from the destination's server).  Plain peer stores only."""
import multiprocessing as mp
import os
import random

import pytest
import torch

os.environ.setdefault("BLLM_KVTRANS_QUIET_ENV", "1")

from llumnix_kv_b200.kv_transfer_impl import KVTransferClient, KVTransferProtocolType as PT, KVTransferServer
from llumnix_kv_b200.ops.layouts import AttnLayout, CacheShape
from llumnix_kv_b200.ops.p2d_attn import ReqChunk, reference_transfer

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
L = 2
SRC_L = AttnLayout(CacheShape.FLASH, 48, 16, 8, 128, 2)
DST_L = AttnLayout(CacheShape.FLASHINFER, 48, 16, 8, 128, 2)


def _requests():
    rng = random.Random(5)
    fs, fd = list(range(1, 48)), list(range(1, 48))
    rng.shuffle(fs)
    rng.shuffle(fd)
    reqs = []
    for i in range(5):
        nb = rng.randint(1, 7)
        reqs.append((f"r{i}", [fs.pop() for _ in range(nb)], [fd.pop() for _ in range(nb)], nb * 16 - rng.randint(0, 15)))
    return reqs


def _send(cli, dst_inst, winfo, reqs):
    for rid, sb, db, total in reqs:
        cli.submit_req_send2(dst_inst, 0, rid, 0, total, True, sb, db, winfo, stepid=1)
    cli.start_send_step(1, 1)
    for layer in range(L):
        cli.record_event(layer)
    cli.flush_send_step()
    cli.drain()


def test_two_gpus_one_process():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    src = [SRC_L.alloc("cuda:0", "normal", seed=i) for i in range(L)]
    dst = [DST_L.alloc("cuda:1") for _ in range(L)]
    srv = KVTransferServer("D|0|1", 1, 0, 0, DST_L.block_bytes, DST_L.token_bytes, "fake://", dst, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=5)
    cli = KVTransferClient("P|0|1", 1, 0, 0, SRC_L.block_bytes, SRC_L.token_bytes, "fake://", src, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=2)
    try:
        reqs = _requests()
        _send(cli, "D|0|1", srv.worker_info(), reqs)
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)
        chunks = [ReqChunk(sb, db, 0, t) for _, sb, db, t in reqs]
        for i in range(L):
            expect = torch.zeros_like(src[i])
            reference_transfer(SRC_L, DST_L, src[i], expect, chunks)
            assert torch.equal(dst[i].to("cuda:0"), expect)
    finally:
        srv.stop()


def test_two_gpus_fp8_destination_takes_the_staged_quantiser():
    """Prefill TP=4 rank 1 on cuda:0 (2 of 8 heads, bf16, NHD) -> decode TP=2 rank 0 on cuda:1 (4 heads,
    block-scaled e4m3, HND).  The channel marks the destination remote, so full tiles leave through the
    quantiser's shared-memory staging and bulk stores; the bytes must equal the oracle's."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from llumnix_kv_b200.ops.layouts import AttnLayout, CacheShape
    from llumnix_kv_b200.ops.p2d_attn import MODE_BF16_TO_MXFP8, HeadMap

    src_l = AttnLayout(CacheShape.FLASH, 40, 16, 2, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 40, 16, 4, 128, 1, mx_scaled=True)
    src = [src_l.alloc("cuda:0", "normal", seed=40 + i) for i in range(L)]
    dst = [dst_l.alloc("cuda:1") for _ in range(L)]
    srv = KVTransferServer("D|0|2", 2, 0, 0, dst_l.block_bytes, dst_l.token_bytes, "fake://", dst, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=5, mx_scaled=True)
    cli = KVTransferClient("P|0|4", 4, 1, 1, src_l.block_bytes, src_l.token_bytes, "fake://", src, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=2)
    try:
        reqs = [("a", [3, 9, 1], [7, 2, 30], 48), ("b", [5, 6], [11, 4], 21), ("c", [20], [21], 16)]
        _send(cli, "D|0|2", srv.worker_info(), reqs)
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)
        chunks = [ReqChunk(sb, db, 0, t) for _, sb, db, t in reqs]
        for i in range(L):
            expect = torch.zeros_like(dst[i], device="cuda:0")
            reference_transfer(src_l, dst_l, src[i], expect, chunks, HeadMap(0, 2, 2), MODE_BF16_TO_MXFP8)
            assert torch.equal(dst[i].to("cuda:0"), expect)
    finally:
        srv.stop()


def _decode_proc(naming_dir, ready, go, result):
    os.environ["BLLM_KVTRANS_QUIET_ENV"] = "1"
    # no NVLS / multicast anywhere in this test: plain peer stores, so that a peer process leaving
    # between steps cannot affect the other GPU
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch as t2
    from llumnix_kv_b200.kv_transfer_impl import KVTransferProtocolType as P2, KVTransferServer as Srv
    t2.cuda.set_device(1)
    dst = [DST_L.alloc("cuda:1") for _ in range(L)]
    srv = Srv("D|0|1", 1, 0, 0, DST_L.block_bytes, DST_L.token_bytes, f"file:{naming_dir}", dst, [P2.NVLINK],
              num_kv_heads=8, cache_shape=5)
    ready.set()
    go.wait(120)
    t2.cuda.synchronize()
    result.put([d.cpu().numpy().copy() for d in dst])
    srv.stop()


def test_two_gpus_two_processes_cuda_ipc(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    ready, go, result = ctx.Event(), ctx.Event(), ctx.Queue()
    p = ctx.Process(target=_decode_proc, args=(str(tmp_path), ready, go, result))
    p.start()
    try:
        assert ready.wait(180)
        torch.cuda.set_device(0)
        src = [SRC_L.alloc("cuda:0", "normal", seed=i) for i in range(L)]
        cli = KVTransferClient("P|0|1", 1, 0, 0, SRC_L.block_bytes, SRC_L.token_bytes, f"file:{tmp_path}", src,
                               [PT.NVLINK], num_kv_heads=8, cache_shape=2)
        reqs = _requests()
        _send(cli, "D|0|1", None, reqs)
        torch.cuda.synchronize()
        go.set()
        got = [torch.from_numpy(a) for a in result.get(timeout=120)]
        chunks = [ReqChunk(sb, db, 0, t) for _, sb, db, t in reqs]
        for i in range(L):
            expect = torch.zeros_like(src[i])
            reference_transfer(SRC_L, DST_L, src[i], expect, chunks)
            assert torch.equal(got[i], expect.cpu())
    finally:
        go.set()
        p.join(60)
        if p.is_alive():
            p.kill()


# ---- which GPU runs the kernels ---------------------------------------------------------------------
# The mode is read from the environment once per process, so each mode runs in a process of its own:
# it repeats the one-process and the two-process transfer above and prints the transport's metrics.
_MODE_SCRIPT = r"""
import os, sys
sys.path.insert(0, os.path.join(os.getcwd(), "tests"))
import multiprocessing as mp
import torch
import test_engine_multigpu as T

def main():
    # one process, two devices
    src = [T.SRC_L.alloc("cuda:0", "normal", seed=i) for i in range(T.L)]
    dst = [T.DST_L.alloc("cuda:1") for _ in range(T.L)]
    srv = T.KVTransferServer("D|0|1", 1, 0, 0, T.DST_L.block_bytes, T.DST_L.token_bytes, "fake://", dst, [T.PT.NVLINK],
                             num_kv_heads=8, cache_shape=5)
    cli = T.KVTransferClient("P|0|1", 1, 0, 0, T.SRC_L.block_bytes, T.SRC_L.token_bytes, "fake://", src, [T.PT.NVLINK],
                             num_kv_heads=8, cache_shape=2)
    reqs = T._requests()
    chunks = [T.ReqChunk(sb, db, 0, t) for _, sb, db, t in reqs]
    for step in (1, 2, 3):          # several batches through one session
        for d in dst:
            d.zero_()
        torch.cuda.synchronize(1)
        for rid, sb, db, total in reqs:
            cli.submit_req_send2("D|0|1", 0, f"{rid}.{step}", 0, total, True, sb, db, srv.worker_info(), stepid=step)
        cli.start_send_step(step, 1)
        for layer in range(T.L):
            cli.record_event(layer)
        cli.flush_send_step()
        assert cli.wait_inflight(0, 30.0) and cli.failed_batches() == 0
        for i in range(T.L):
            expect = torch.zeros_like(src[i])
            T.reference_transfer(T.SRC_L, T.DST_L, src[i], expect, chunks)
            assert torch.equal(dst[i].to("cuda:0"), expect), (step, i)
    srv.stop()
    print("one-process ok", flush=True)

    # two processes: CUDA IPC memory and event handles
    import tempfile
    tmp = tempfile.mkdtemp()
    ctx = mp.get_context("spawn")
    ready, go, result = ctx.Event(), ctx.Event(), ctx.Queue()
    p = ctx.Process(target=T._decode_proc, args=(tmp, ready, go, result))
    p.start()
    try:
        assert ready.wait(180)
        cli2 = T.KVTransferClient("P2|0|1", 1, 0, 0, T.SRC_L.block_bytes, T.SRC_L.token_bytes, f"file:{tmp}", src,
                                  [T.PT.NVLINK], num_kv_heads=8, cache_shape=2)
        for rid, sb, db, total in reqs:
            cli2.submit_req_send2("D|0|1", 0, rid, 0, total, True, sb, db, None, stepid=1)
        cli2.start_send_step(1, 1)
        for layer in range(T.L):
            cli2.record_event(layer)
        cli2.flush_send_step()
        assert cli2.wait_inflight(0, 30.0) and cli2.failed_batches() == 0
        # a relayed request (fanout) to a worker that advertises no multicast group fails cleanly, on the host,
        # and the channel keeps serving
        cli2.submit_req_send2("D|0|1", 0, "fan", 0, 16, True, [1], [2], None, stepid=2, fanout=2)
        cli2.start_send_step(2, 1)
        for layer in range(T.L):
            cli2.record_event(layer)
        cli2.flush_send_step()
        assert cli2.wait_inflight(0, 30.0) and cli2.failed_batches() == 1
        rid, sb, db, total = reqs[0]
        cli2.submit_req_send2("D|0|1", 0, rid + ".again", 0, total, True, sb, db, None, stepid=3)
        cli2.start_send_step(3, 1)
        for layer in range(T.L):
            cli2.record_event(layer)
        cli2.flush_send_step()
        assert cli2.wait_inflight(0, 30.0) and cli2.failed_batches() == 1
        go.set()
        got = [torch.from_numpy(a) for a in result.get(timeout=120)]
        for i in range(T.L):
            expect = torch.zeros_like(src[i])
            T.reference_transfer(T.SRC_L, T.DST_L, src[i], expect, chunks)
            assert torch.equal(got[i], expect.cpu()), i
    finally:
        go.set()
        p.join(60)
        if p.is_alive():
            p.kill()
    print("two-process ok", flush=True)

if __name__ == "__main__":
    main()
"""


@pytest.mark.parametrize("pull", [1, 0])
def test_kernels_on_the_decode_gpu_or_on_the_prefill_gpu(pull):
    """Pull (default between two worker processes): a session on the decode worker's server maps the
    prefill cache and its layer events and runs the kernels there, loading over NVLink.  Push: the
    prefill GPU stores; two workers inside one process always push.  Same bytes either way; the
    metrics line names the mode.  The run has the end-to-end check on (BLLM_KVTRANS_CRC=1)."""
    import re
    import subprocess
    import sys

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, BLLM_KVTRANS_NVLINK_PULL=str(pull), LLMOPS_CPP_MIN_LOG_LEVEL="0", NCCL_NVLS_ENABLE="0",
               BLLM_KVTRANS_CRC="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", _MODE_SCRIPT], cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    assert "one-process ok" in r.stdout and "two-process ok" in r.stdout
    modes = re.findall(r"SendStubMetrics\..*Proto=nvlink,Mode=(\w+),Path=fused", r.stderr)
    assert modes[:3] == ["push"] * 3 and len(modes) >= 4, modes
    assert set(modes[3:]) == {"pull" if pull else "push"}, modes
    # with the end-to-end check on, every batch that moved data was compared across the two GPUs (each summing its
    # own cache in its own layout) before it was reported
    checks = re.findall(r"SendStubMetrics\..*Check=(\w+)", r.stderr)
    assert len(checks) >= 5 and set(checks) == {"ok"}, checks


def _send_step(cli, stepid, reqs, tag):
    for rid, sb, db, total in reqs:
        cli.submit_req_send2("D|0|1", 0, f"{rid}.{tag}", 0, total, True, sb, db, None, stepid=stepid)
    cli.start_send_step(stepid, 1)
    for layer in range(L):
        cli.record_event(layer)
    cli.flush_send_step()


def test_decode_worker_leaves_between_steps_and_a_new_one_takes_over(tmp_path):
    """The decode worker's process ends between two steps, with nothing in flight.  The prefill worker's next
    step fails on the host (its requests are reported failed, the wait returns well inside its limit, nothing
    hangs); a new decode worker that registers under the same name serves the step after that."""
    import time

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    torch.cuda.set_device(0)
    src = [SRC_L.alloc("cuda:0", "normal", seed=i) for i in range(L)]
    cli = KVTransferClient("P|0|1", 1, 0, 0, SRC_L.block_bytes, SRC_L.token_bytes, f"file:{tmp_path}", src, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=2)
    reqs = _requests()
    chunks = [ReqChunk(sb, db, 0, t) for _, sb, db, t in reqs]

    def expect_ok(got):
        for i in range(L):
            want = torch.zeros_like(src[i])
            reference_transfer(SRC_L, DST_L, src[i], want, chunks)
            assert torch.equal(got[i], want.cpu()), i

    procs = []
    try:
        # ---- first decode worker: one good step, then it leaves ------------------------------------------
        ready, go, result = ctx.Event(), ctx.Event(), ctx.Queue()
        a = ctx.Process(target=_decode_proc, args=(str(tmp_path), ready, go, result))
        a.start()
        procs.append((a, go))
        assert ready.wait(180)
        _send_step(cli, 1, reqs, "one")
        assert cli.wait_inflight(0, 30.0) and cli.failed_batches() == 0
        go.set()
        expect_ok([torch.from_numpy(x) for x in result.get(timeout=120)])
        a.join(60)
        assert not a.is_alive()
        # ---- nobody there: the step fails, quickly and on the host ------------------------------------------
        t0 = time.time()
        _send_step(cli, 2, reqs, "two")
        assert cli.wait_inflight(0, 60.0)
        assert cli.failed_batches() == 1 and time.time() - t0 < 30.0
        # ---- a new worker under the same name -----------------------------------------------------------
        ready2, go2, result2 = ctx.Event(), ctx.Event(), ctx.Queue()
        b = ctx.Process(target=_decode_proc, args=(str(tmp_path), ready2, go2, result2))
        b.start()
        procs.append((b, go2))
        assert ready2.wait(180)
        _send_step(cli, 3, reqs, "three")
        assert cli.wait_inflight(0, 60.0) and cli.failed_batches() == 1
        go2.set()
        expect_ok([torch.from_numpy(x) for x in result2.get(timeout=120)])
    finally:
        for p, g in procs:
            g.set()
            p.join(60)
            if p.is_alive():
                p.kill()


def _prefill_proc(naming_dir, seed0, done, result):
    """A prefill worker's whole life: register, one step to D|0|1, report, exit."""
    os.environ["BLLM_KVTRANS_QUIET_ENV"] = "1"
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch as t2
    from llumnix_kv_b200.kv_transfer_impl import KVTransferClient as Cli, KVTransferProtocolType as P2
    t2.cuda.set_device(0)
    src = [SRC_L.alloc("cuda:0", "normal", seed=seed0 + i) for i in range(L)]
    cli = Cli("P|0|1", 1, 0, 0, SRC_L.block_bytes, SRC_L.token_bytes, f"file:{naming_dir}", src, [P2.NVLINK], num_kv_heads=8,
              cache_shape=2)
    _send_step(cli, 1, _requests(), f"s{seed0}")
    ok = cli.wait_inflight(0, 30.0) and cli.failed_batches() == 0
    t2.cuda.synchronize()
    result.put(bool(ok))
    done.wait(60)          # stays until the decode side has looked at its cache, then leaves with nothing in flight


def test_prefill_worker_leaves_and_another_connects_to_the_same_decode_worker(tmp_path):
    """The decode worker outlives its senders: a prefill worker's process does a step and ends; its pull session
    goes with the connection and the mapping of its cache is released; the next prefill worker is served
    by a new session."""
    import time

    from llumnix_kv_b200 import load_ops

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    K = load_ops()
    torch.cuda.set_device(1)
    dst = [DST_L.alloc("cuda:1") for _ in range(L)]
    srv = KVTransferServer("D|0|1", 1, 0, 0, DST_L.block_bytes, DST_L.token_bytes, f"file:{tmp_path}", dst, [PT.NVLINK],
                           num_kv_heads=8, cache_shape=5)
    ctx = mp.get_context("spawn")
    reqs = _requests()
    chunks = [ReqChunk(sb, db, 0, t) for _, sb, db, t in reqs]
    procs = []
    try:
        for seed0 in (300, 700):
            for d in dst:
                d.zero_()
            torch.cuda.synchronize(1)
            done, result = ctx.Event(), ctx.Queue()
            p = ctx.Process(target=_prefill_proc, args=(str(tmp_path), seed0, done, result))
            p.start()
            procs.append((p, done))
            assert result.get(timeout=240) is True
            torch.cuda.synchronize(1)
            for i in range(L):
                src_i = SRC_L.alloc("cuda:1", "normal", seed=seed0 + i)
                want = torch.zeros_like(dst[i])
                reference_transfer(SRC_L, DST_L, src_i, want, chunks)
                assert torch.equal(dst[i], want), (seed0, i)
            assert K.ipc_mappings_open() >= 1                    # the sender's cache is mapped here while its session lives
            done.set()
            p.join(60)
            assert not p.is_alive()
            t0 = time.time()
            while K.ipc_mappings_open() != 0 and time.time() - t0 < 20:
                time.sleep(0.05)
            assert K.ipc_mappings_open() == 0                    # gone with the connection
    finally:
        for p, done in procs:
            done.set()
            p.join(30)
            if p.is_alive():
                p.kill()
        srv.stop()
