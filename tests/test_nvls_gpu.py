"""NVLS fan-out (multimem.st through NVSwitch) of replicated KV blocks inside a TP group.

Child processes, one per GPU (2 to 4).  Every rank runs the same sequence of collective steps and
only records what it finds wrong, so that no rank leaves while its memory is still bound to the
multicast object; the parent asserts on what the ranks reported."""
import os
import socket
import traceback

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

LAYERS, NUM_BLOCKS, STRIDE = 3, 16, 4096 + 512          # a block of 4608 bytes: not a power of two, 16-byte aligned


def _expected(seed: int, n: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 256, (n,), dtype=torch.uint8, generator=g)


def _child(rank: int, world: int, port: int, q) -> None:
    errors = []
    cache = None
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      BLLM_KVTRANS_QUIET_ENV="1")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    try:
        from llumnix_kv_b200.parallel.nvls import MulticastKVCache

        cache = MulticastKVCache(LAYERS, NUM_BLOCKS * STRIDE, dist.group.WORLD, dev)

        def block(layer, b):
            return cache.layers[layer][b * STRIDE:(b + 1) * STRIDE]

        # ---- 1. in place: rank 0 holds blocks 3, 7, 1 of every layer; everybody gets them ------------------
        ids = [3, 7, 1]
        if rank == 0:
            for layer in range(LAYERS):
                for b in ids:
                    block(layer, b).copy_(_expected(100 * layer + b, STRIDE))
            torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            cache.fanout(ids, STRIDE, NUM_BLOCKS, flag_value=1)
            torch.cuda.synchronize()
            try:
                cache.check_status()
            except Exception as ex:
                errors.append(f"in-place status: {ex}")
        elif not cache.wait(1, timeout_s=5.0, slots=[0]):
            errors.append("in-place: the completion word never arrived")
        for layer in range(LAYERS):
            for b in range(NUM_BLOCKS):
                want = _expected(100 * layer + b, STRIDE) if b in ids else torch.zeros(STRIDE, dtype=torch.uint8)
                if not torch.equal(block(layer, b).cpu(), want):
                    errors.append(f"in-place: layer {layer} block {b} differs on rank {rank}")
        dist.barrier()

        # ---- 2. from a landing buffer, part of a block, other block ids and another stride ---------------
        l_stride, l_blocks = 2048, 4
        landing = torch.zeros(LAYERS * l_blocks * l_stride, dtype=torch.uint8, device=dev)
        src_ptrs = torch.tensor([landing.data_ptr() + i * l_blocks * l_stride for i in range(LAYERS)], dtype=torch.int64,
                                device=dev)
        if rank == 0:
            landing.copy_(_expected(7, landing.numel()))
            torch.cuda.synchronize()
            cache.fanout([9, 4], STRIDE, NUM_BLOCKS, block_off=64, block_len=1024, layers=(1, 3), flag_value=2,
                         src_layers=src_ptrs, src_block_ids=[2, 0], src_block_stride=l_stride, src_num_blocks=l_blocks)
            torch.cuda.synchronize()
            try:
                cache.check_status()
            except Exception as ex:
                errors.append(f"landing status: {ex}")
        elif not cache.wait(2, timeout_s=5.0, slots=[0]):
            errors.append("landing: the completion word never arrived")
        land = _expected(7, landing.numel())
        for layer in range(LAYERS):
            for db, sb in ((9, 2), (4, 0)):
                got = block(layer, db).cpu()
                want = torch.zeros(STRIDE, dtype=torch.uint8)
                if layer >= 1:
                    o = (layer * l_blocks + sb) * l_stride + 64
                    want[64:64 + 1024] = land[o:o + 1024]
                if not torch.equal(got, want):
                    errors.append(f"landing: layer {layer} block {db} differs on rank {rank}")
        dist.barrier()

        # ---- 3. a wait that nothing satisfies runs out and leaves the context usable -----------------------
        if rank == world - 1:
            if cache.wait(99, timeout_s=0.2, slots=[0]):
                errors.append("bounded wait: returned True although nothing set the word")
            probe = torch.ones(4, device=dev).sum().item()
            if probe != 4.0:
                errors.append("bounded wait: context unusable afterwards")
        dist.barrier()

        # ---- 3b. every member relays its share from its own landing buffer; everybody waits for all words ----
        all_ids = [12, 2, 14, 6, 10, 8, 13, 11][:2 * world]
        share = all_ids[2 * rank:2 * rank + 2]
        mine = torch.zeros(LAYERS * 2 * STRIDE, dtype=torch.uint8, device=dev)
        mine.copy_(_expected(500 + rank, mine.numel()))
        mine_ptrs = torch.tensor([mine.data_ptr() + i * 2 * STRIDE for i in range(LAYERS)], dtype=torch.int64, device=dev)
        torch.cuda.synchronize()
        dist.barrier()
        cache.fanout(share, STRIDE, NUM_BLOCKS, flag_value=5, src_layers=mine_ptrs, src_block_ids=[0, 1],
                     src_block_stride=STRIDE, src_num_blocks=2)
        if not cache.wait(5, timeout_s=5.0):
            errors.append("scatter: a completion word never arrived")
        for r in range(world):
            theirs = _expected(500 + r, mine.numel())
            for layer in range(LAYERS):
                for i, b in enumerate(all_ids[2 * r:2 * r + 2]):
                    o = (layer * 2 + i) * STRIDE
                    if not torch.equal(block(layer, b).cpu(), theirs[o:o + STRIDE]):
                        errors.append(f"scatter: layer {layer} block {b} (share of rank {r}) differs on rank {rank}")
        dist.barrier()

        # ---- 4. a block id outside the tensor is reported and skipped ------------------------------------
        if rank == 0:
            cache.fanout([5, NUM_BLOCKS + 3], STRIDE, NUM_BLOCKS)
            torch.cuda.synchronize()
            try:
                cache.check_status()
                errors.append("range check: no status for a block id outside the tensor")
            except RuntimeError:
                pass
        dist.barrier()
    except Exception:
        errors.append(f"rank {rank}: {traceback.format_exc()}")
    finally:
        try:
            if cache is not None:
                cache.close()
            else:
                dist.barrier()
        except Exception:
            errors.append(f"rank {rank} teardown: {traceback.format_exc()}")
        q.put((rank, errors))
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_multicast_fanout_reaches_every_member():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    world = min(n, 4)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_child, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    reports = {}
    try:
        for _ in range(world):
            rank, errors = q.get(timeout=300)
            reports[rank] = errors
    finally:
        for p in procs:
            p.join(120)
    assert sorted(reports) == list(range(world))
    assert all(not e for e in reports.values()), reports


# ---- the relay inside the transport ----------------------------------------------------------------
# Rank 0 is a prefill worker (TP 1), ranks 1..k the tensor-parallel workers of ONE decode instance whose MLA-like
# caches (two tensors per layer, identical on every rank) live in symmetric allocations bound to a multicast
# group.  The prefill worker hands each request to ONE decode worker with fanout=k; that worker's pull session
# loads the bytes over NVLink and stores them to the whole group.  Every decode rank must end up with both
# requests, the prefill worker's link having carried each of them once.
R_LAYERS, R_TOKS, R_NTPB, R_BLOCKS = 3, [132, 656], 64, 24
R_SIZES = [t * R_NTPB for t in R_TOKS]


def _relay_src(layer: int, t: int, dev) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(1000 + 10 * layer + t)
    return torch.randint(1, 255, (R_SIZES[t] * R_BLOCKS,), dtype=torch.uint8, generator=g).to(dev)


def _relay_requests(k: int):
    # (request id, relay worker, tokens, prefill blocks, decode blocks)
    return [("ra", 0, 150, [3, 9, 4], [7, 2, 11]), ("rb", 1 % k, 64 + 17, [12, 1], [5, 20]), ("rc", (k - 1), 40, [6], [15])]


def _relay_child(rank: int, world: int, port: int, tmp: str, q, sender_in_group: bool = False) -> None:
    errors = []
    caches, srv, cli = [], None, None
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      BLLM_KVTRANS_QUIET_ENV="1")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    import datetime

    limit = datetime.timedelta(seconds=120)
    dist.init_process_group("nccl", device_id=dev, timeout=limit)
    host = dist.new_group(backend="gloo", timeout=limit)   # ranks wait for one another on the host, never inside a NCCL kernel
    k = world - 1
    # sender_in_group: the prefill GPU is bound to the multicast object too (memory of its own that only absorbs
    # the echo), holds a mapping of it, and stores to the group itself; no pull session, no relay
    d_group = dist.group.WORLD if sender_in_group else dist.new_group(list(range(1, world)))
    if sender_in_group and rank == 0:
        os.environ["BLLM_KVTRANS_NVLINK_PULL"] = "0"     # a relay would need a pull session: only the multicast path is left
    try:
        from llumnix_kv_b200.kv_transfer_impl import KVTransferClient, KVTransferProtocolType as PT, KVTransferServer
        from llumnix_kv_b200.parallel.nvls import MulticastKVCache

        inst = f"D|0|{k}"
        if rank > 0:
            caches = [MulticastKVCache(R_LAYERS, R_SIZES[t] * R_BLOCKS, d_group, dev) for t in range(2)]
            layers = [[caches[t].layers[layer] for t in range(2)] for layer in range(R_LAYERS)]
            mc = [[caches[t].mc_ptr + layer * caches[t].layer_bytes for t in range(2)] for layer in range(R_LAYERS)]
            srv = KVTransferServer(inst, k, rank - 1, rank - 1, list(R_SIZES), list(R_TOKS), f"file:{tmp}", layers, [PT.NVLINK],
                                   cache_shape=4, num_kv_heads=1, mc_layers=mc, mc_size=world if sender_in_group else k)
        elif sender_in_group:
            caches = [MulticastKVCache(R_LAYERS, R_SIZES[t] * R_BLOCKS, d_group, dev) for t in range(2)]
        dist.barrier(group=host)
        if rank == 0:
            src = [[_relay_src(layer, t, dev) for t in range(2)] for layer in range(R_LAYERS)]
            extra = {}
            if sender_in_group:
                extra = dict(mc_layers=[[caches[t].mc_ptr + layer * caches[t].layer_bytes for t in range(2)]
                                        for layer in range(R_LAYERS)], mc_size=world)
            cli = KVTransferClient("P|0|1", 1, 0, 0, list(R_SIZES), list(R_TOKS), f"file:{tmp}", src, [PT.NVLINK], cache_shape=4,
                                   num_kv_heads=1, **extra)
            for rid, relay, tokens, sb, db in _relay_requests(k):
                cli.submit_req_send2(inst, relay, rid, 0, tokens, True, [sb], [db], None, stepid=1, fanout=k)
            cli.start_send_step(1, 1)
            for layer in range(R_LAYERS):
                cli.record_event(layer)
            cli.flush_send_step()
            if not cli.wait_inflight(0, 30.0):
                errors.append("the relayed step did not complete")
            if cli.failed_batches():
                errors.append(f"{cli.failed_batches()} batches failed")
        dist.barrier(group=host)
        if rank > 0:
            torch.cuda.synchronize()
            for layer in range(R_LAYERS):
                for t in range(2):
                    want = torch.zeros(R_SIZES[t] * R_BLOCKS, dtype=torch.uint8, device=dev)
                    ref = _relay_src(layer, t, dev)
                    for _, _, tokens, sb, db in _relay_requests(k):
                        for i, (s, d) in enumerate(zip(sb, db)):
                            n = min(R_NTPB, tokens - i * R_NTPB) * R_TOKS[t]
                            want[d * R_SIZES[t]:d * R_SIZES[t] + n] = ref[s * R_SIZES[t]:s * R_SIZES[t] + n]
                    if not torch.equal(caches[t].layers[layer], want):
                        bad = (caches[t].layers[layer] != want).nonzero()
                        errors.append(f"rank {rank} layer {layer} tensor {t}: {bad.numel()} bytes differ, first at {int(bad[0])}")
        dist.barrier(group=host)
    except Exception:
        errors.append(f"rank {rank}: {traceback.format_exc()}")
    finally:
        try:
            if srv is not None:
                srv.stop()
            dist.barrier(group=host)
            for c in caches:
                c.close()
        except Exception:
            errors.append(f"rank {rank} teardown: {traceback.format_exc()}")
        q.put((rank, errors))
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("sender_in_group", [False, True])
def test_transport_relays_a_request_through_the_decode_groups_multicast(tmp_path, sender_in_group):
    """sender_in_group=False: one decode worker pulls the request and relays it.  True: the prefill GPU is bound
    to the group's multicast object and stores to every decode cache itself (`kvt_walk_multicast`)."""
    n = torch.cuda.device_count()
    if n < 3:
        pytest.skip("needs three GPUs: a prefill worker and a decode group of two")
    world = min(n, 4)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_relay_child, args=(r, world, port, str(tmp_path), q, sender_in_group)) for r in range(world)]
    for p in procs:
        p.start()
    reports = {}
    try:
        for _ in range(world):
            rank, errors = q.get(timeout=300)
            reports[rank] = errors
    finally:
        for p in procs:
            p.join(150)
            if p.is_alive():
                p.kill()
    assert sorted(reports) == list(range(world))
    assert all(not e for e in reports.values()), reports
