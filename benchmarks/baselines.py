"""Library baselines, bandwidth ceilings measured inside a run, and the store-form probe.

Everything here times on the device with CUDA events and reports the maximum over ranks.

* ``measure_ceilings``   what the copy engines of this box deliver right now: one large
                         ``cudaMemcpyAsync`` into the peer GPU (or inside the one GPU), and pinned
                         host <-> device copies.  These are the denominators of the roofline fractions.
* ``memcpy_peer_arm``    the reference's planner-then-copy architecture with the copy engine doing the
                         moving: the CPU planner's merged IpcBlocks, one ``cudaMemcpyAsync`` each, straight
                         into the peer cache (NHD -> NHD: byte ranges cannot change the layout).  The
                         reference's own loop of this kind is kvtransfer/src/copy_kernels.cpp:267-294.
* ``nccl_arm``           gather kernel -> NCCL send / recv of the staging buffer -> scatter kernel.
* ``link_probe``         the transfer kernel's tiles leaving in each store form, pipeline depth and grid.
"""
from __future__ import annotations

import statistics
from typing import Callable, Dict, List

import torch

from llumnix_kv_b200.ops.layouts import AttnLayout, CacheShape
from llumnix_kv_b200.ops.p2d_attn import AttnTransfer, ReqChunk

from . import hostsync as HS
from .support import BLOCK, HEAD_DIM, KV_HEADS, PDBenchPair


def _dist():
    import torch.distributed as dist

    return dist


def timed_reps(run_step: Callable[[int], None], steps: int, warmup: int, stream, world: int, dev, measures: bool,
               min_seconds: float = 1.0, max_reps: int = 400, sampler_factory=None, end_region=None):
    """Times ``steps`` calls of ``run_step`` as one region (CUDA events on ``stream``, a barrier and
    a device synchronisation on both sides, maximum over ranks), and repeats the region until
    ``min_seconds`` of device time have been measured.  Returns (list of region ms, clock record)."""
    dist = _dist()

    def barrier():
        if world > 1:
            HS.barrier()
        torch.cuda.synchronize()

    for i in range(warmup):
        run_step(i)
    if end_region is not None:
        end_region()
    barrier()
    sampler = sampler_factory() if sampler_factory else None
    regions: List[float] = []
    k = warmup
    reps = 1
    while len(regions) < reps:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(steps):
            run_step(k)
            k += 1
        if end_region is not None:
            end_region()          # work that a step left in flight belongs to the region
        ev1.record(stream)
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1) if measures else 0.0
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            HS.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        barrier()
        regions.append(ms)
        if len(regions) == 1 and ms > 0:
            reps = max(1, min(max_reps, int(min_seconds * 1e3 / ms) + 1))
    clocks = sampler.stop() if sampler else {}
    return regions, clocks


def summarize(regions: List[float], steps: int) -> Dict[str, float]:
    per_step = [r / steps for r in regions]
    return {"reps": len(regions), "ms_per_step_median": round(statistics.median(per_step), 4),
            "ms_per_step_min": round(min(per_step), 4), "ms_per_step_max": round(max(per_step), 4),
            "timed_seconds": round(sum(regions) / 1e3, 3)}


def _event_ms(fn: Callable[[], None], stream, iters: int = 5) -> float:
    best = 1e30
    for _ in range(iters):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        fn()
        e1.record(stream)
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return best


def measure_ceilings(pair: PDBenchPair, nbytes: int = 1 << 30, host_bytes: int = 256 << 20) -> dict:
    """Copy-engine bandwidths of this run: device -> peer (or device -> device on one GPU) with one
    ``cudaMemcpyAsync`` of ``nbytes``, pinned host -> device and device -> host with ``host_bytes``.
    Returned GB/s are the maximum-time (slowest rank) figures."""
    K, dev, world = pair.K, pair.dev, pair.world
    out = {"copy_bytes": nbytes}
    ms = 0.0
    if pair.is_sender:
        n = min(nbytes, pair.src.numel(), pair.probe_bytes)
        s = pair.stream
        ms = _event_ms(lambda: K.kvt_memcpy_async(pair.probe_dst_ptr, pair.src.data_ptr(), n, s.cuda_stream), s)
        out["copy_bytes"] = n
    hms_h2d = hms_d2h = 0.0
    if pair.is_sender:
        h = torch.empty(host_bytes, dtype=torch.uint8, pin_memory=True)
        d = pair.src[:host_bytes]
        s = pair.stream
        keep = d.clone()
        with torch.cuda.stream(s):
            hms_d2h = _event_ms(lambda: h.copy_(d, non_blocking=True), s, 3)
            hms_h2d = _event_ms(lambda: d.copy_(h, non_blocking=True), s, 3)
            d.copy_(keep)
        s.synchronize()
    t = torch.tensor([ms, hms_h2d, hms_d2h], dtype=torch.float64, device=dev)
    if world > 1:
        HS.all_reduce(t, op=_dist().ReduceOp.MAX)
    ms, hms_h2d, hms_d2h = (float(x) for x in t)
    gbs = lambda b, m: round(b / m / 1e6, 1) if m > 0 else None
    if world > 1:
        out["peer_copy_GBps"] = gbs(out["copy_bytes"], ms)
        out["what"] = "one cudaMemcpyAsync device -> peer GPU per pair (copy engine over NVLink), slowest pair"
    else:
        out["local_copy_GBps"] = gbs(out["copy_bytes"], ms)
        out["what"] = "one cudaMemcpyAsync device -> device on the one GPU (payload GB/s; HBM reads and writes it)"
    out["pinned_h2d_GBps"] = gbs(host_bytes, hms_h2d)
    out["pinned_d2h_GBps"] = gbs(host_bytes, hms_d2h)
    return out


# ---------------------------------------------------------------------------------------------
# baseline arms
# ---------------------------------------------------------------------------------------------
def memcpy_peer_arm(pair: PDBenchPair, steps: int, warmup: int, sampler_factory=None) -> dict:
    """One ``cudaMemcpyAsync`` per merged IpcBlock of the CPU planner, per layer, from the prefill
    cache into the peer-mapped decode cache of the same (NHD) layout."""
    import numpy as np

    K = pair.K
    per_slot = []
    planned = 0
    if pair.is_sender:
        W = K.WorkerInfo
        info = W()
        info.inst_id, info.worker_id, info.engine_tp_size, info.worker_tp_rank = "x|0|1", 0, 1, 0
        info.block_sizes, info.token_sizes = [pair.src_l.block_bytes], [pair.src_l.token_bytes]
        info.layer_num_blocks, info.num_layers, info.num_kv_heads = pair.src_l.num_blocks, pair.n_layers, KV_HEADS
        for cs in pair.slot_chunks:
            tasks = [(f"r{i}", 0, c.new_tokens, True, [list(c.src_blocks)], [list(c.dst_blocks)]) for i, c in enumerate(cs)]
            blocks = K.plan_ipc_blocks(info, info, int(CacheShape.FLASH), tasks, merge=True)[0][0]
            arr = np.ascontiguousarray(np.array(blocks, dtype=np.uint64).reshape(-1))
            per_slot.append(arr)
        planned = len(per_slot[0]) // 3

    def step(i: int) -> None:
        if not pair.is_sender:
            return
        slot = i % pair.slots
        pair.touched.add(slot)
        arr = per_slot[slot]
        s = pair.stream.cuda_stream
        for layer in range(pair.n_layers):
            K.kvt_memcpy_triples(pair.dst_layer_ptrs[layer], pair.src.data_ptr() + layer * pair.src_l.layer_bytes, arr, s)

    regions, clocks = timed_reps(step, steps, warmup, pair.stream, pair.world, pair.dev, pair.is_sender,
                                 sampler_factory=sampler_factory)
    pair.verify(layers=range(pair.n_layers))
    return {"regions": regions, "clocks": clocks, "copies_per_step": planned * pair.n_layers,
            "api": "CPU planner -> merged IpcBlocks -> one cudaMemcpyAsync per block into the peer cache"}


def nccl_arm(pair: PDBenchPair, steps: int, warmup: int, sampler_factory=None) -> dict:
    """Gather kernel (paged NHD -> contiguous staging), NCCL send / recv of the staging buffer,
    scatter kernel (staging -> paged HND) on the decode GPU.  One GPU: no NCCL hop, the two kernels only."""
    dist = _dist()
    dev = pair.dev
    blocks_per_req = (pair.tokens + BLOCK - 1) // BLOCK
    n_stage = pair.requests * blocks_per_req
    stage_l = AttnLayout(CacheShape.FLASH, n_stage, BLOCK, KV_HEADS, HEAD_DIM, 2)
    stage = torch.empty(pair.n_layers * stage_l.layer_bytes, dtype=torch.uint8, device=dev)
    stage_ptrs = [stage.data_ptr() + i * stage_l.layer_bytes for i in range(pair.n_layers)]
    ident = list(range(n_stage))
    gather = scatter = None
    g_plans, s_plans = [], []
    if pair.is_sender:
        src_ptrs = [pair.src.data_ptr() + i * pair.src_l.layer_bytes for i in range(pair.n_layers)]
        gather = AttnTransfer(pair.src_l, stage_l, src_ptrs, stage_ptrs, dev)
        for cs in pair.slot_chunks:
            k, chunks = 0, []
            for c in cs:
                chunks.append(ReqChunk(c.src_blocks, ident[k:k + blocks_per_req], 0, c.new_tokens))
                k += blocks_per_req
            g_plans.append(gather.plan(chunks, stream=pair.stream))
    if pair.is_receiver:
        dst_ptrs = [pair.dst.data_ptr() + i * pair.dst_l.layer_bytes for i in range(pair.n_layers)]
        scatter = AttnTransfer(stage_l, pair.dst_l, stage_ptrs, dst_ptrs, dev)
        for cs in pair.slot_chunks:
            k, chunks = 0, []
            for c in cs:
                chunks.append(ReqChunk(ident[k:k + blocks_per_req], c.dst_blocks, 0, c.new_tokens))
                k += blocks_per_req
            s_plans.append(scatter.plan(chunks, stream=pair.stream))
    torch.cuda.synchronize()
    peer = (pair.rank + pair.n_pairs) if pair.rank < pair.n_pairs else (pair.rank - pair.n_pairs)

    def step(i: int) -> None:
        slot = i % pair.slots
        pair.touched.add(slot)
        with torch.cuda.stream(pair.stream):
            if pair.is_sender:
                gather.launch(g_plans[slot], 0, pair.n_layers, stream=pair.stream)
                if not pair.loopback:
                    dist.send(stage, peer)
            if pair.is_receiver:
                if not pair.loopback:
                    dist.recv(stage, peer)
                scatter.launch(s_plans[slot], 0, pair.n_layers, stream=pair.stream)

    regions, clocks = timed_reps(step, steps, warmup, pair.stream, pair.world, dev, True, sampler_factory=sampler_factory)
    pair.verify(layers=range(pair.n_layers))
    return {"regions": regions, "clocks": clocks,
            "api": "gather kernel -> torch.distributed (NCCL) send/recv of the staging buffer -> scatter kernel"}


# ---------------------------------------------------------------------------------------------
# store-form probe
# ---------------------------------------------------------------------------------------------
def link_probe(pair: PDBenchPair, seconds_per_case: float = 0.25) -> List[dict]:
    """Kernel-only GB/s per pair of the transfer kernel for every way its tiles can leave:
    tile order (tokens or heads outermost in shared memory), tensor store or one linear bulk store,
    pipeline depth, CTA count, L2 policy.  Same tiles, same peer mapping, same block tables."""
    dist = _dist()
    dev = pair.dev
    rows = []
    cases = []
    for order, form in ((0, 0), (1, 0), (1, 1)):
        for stages in (0, 1, 2, 4):
            for grid in (148, 296, 592):
                cases.append((order, form, stages, grid, 0))
    cases += [(1, 1, 0, 592, 1), (1, 0, 0, 592, 1), (0, 0, 0, 592, 1), (1, 1, 0, 1184, 0), (1, 1, 2, 1184, 0)]
    xfers = {}
    if pair.is_sender:
        src_ptrs = [pair.src.data_ptr() + i * pair.src_l.layer_bytes for i in range(pair.n_layers)]
        for order, form in ((0, 0), (1, 0), (1, 1)):
            xfers[(order, form)] = AttnTransfer(pair.src_l, pair.dst_l, src_ptrs, pair.dst_layer_ptrs, dev,
                                                tile_order=order, store_form=form, dst_remote=not pair.loopback)
    lanes = [pair.stream] + pair.side
    for order, form, stages, grid, hint in cases:
        ms_total, n_steps = 0.0, 0

        def one_step(i, order=order, form=form, stages=stages, grid=grid, hint=hint):
            x = xfers[(order, form)]
            x.tma_stages, x.cache_hint = stages, hint
            plan = pair.plans[i % pair.slots]
            pair._fan_out()
            for layer in range(pair.n_layers):
                x.launch(plan, layer, layer + 1, stream=lanes[layer % len(lanes)], grid=grid)
            pair._fan_in()

        if pair.is_sender:
            for i in range(3):
                one_step(i)
        if pair.world > 1:
            HS.barrier()
        torch.cuda.synchronize()
        if pair.is_sender:
            i = 3
            while ms_total < seconds_per_case * 1e3 and n_steps < 2000:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(pair.stream)
                for _ in range(10):
                    one_step(i)
                    i += 1
                e1.record(pair.stream)
                torch.cuda.synchronize()
                ms_total += e0.elapsed_time(e1)
                n_steps += 10
            st = xfers[(order, form)].check_status()
            assert st == (0, 0), st
        per_step = ms_total / max(n_steps, 1)
        t = torch.tensor([per_step], dtype=torch.float64, device=dev)
        if pair.world > 1:
            HS.all_reduce(t, op=dist.ReduceOp.MAX)
        per_step = float(t.item())
        rows.append({"tile_order": "heads outermost" if order else "tokens outermost",
                     "store": "linear bulk" if form else "tensor", "stages": stages or "auto", "ctas": grid,
                     "l2_evict_first": bool(hint), "ms_per_step": round(per_step, 4),
                     "per_pair_GBps": round(pair.bytes_per_step / per_step / 1e6, 1) if per_step > 0 else 0.0})
    # ---- pull: the decode GPU runs the same kernel and LOADS the tiles over NVLink (plain TMA loads from
    #      peer memory, no multicast), storing into its own cache -----------------------------------------
    if not pair.loopback:
        pair.map_src_on_receiver()
        pull = None
        plans = None
        if pair.is_receiver:
            dst_ptrs = [pair.dst.data_ptr() + i * pair.dst_l.layer_bytes for i in range(pair.n_layers)]
            pull = AttnTransfer(pair.src_l, pair.dst_l, pair.src_peer_ptrs, dst_ptrs, dev, tile_order=1, store_form=1)
            with torch.cuda.stream(pair.stream):
                plans = [pull.plan(cs, stream=pair.stream) for cs in pair.slot_chunks]
            torch.cuda.synchronize()
        for stages, grid in ((0, 592), (2, 592), (4, 296), (0, 1184)):
            ms_total, n_steps = 0.0, 0

            def pull_step(i, stages=stages, grid=grid):
                pull.tma_stages = stages
                pair._fan_out()
                for layer in range(pair.n_layers):
                    pull.launch(plans[i % pair.slots], layer, layer + 1, stream=lanes[layer % len(lanes)], grid=grid)
                pair._fan_in()

            if pair.is_receiver:
                for i in range(3):
                    pull_step(i)
            HS.barrier()
            torch.cuda.synchronize()
            if pair.is_receiver:
                i = 3
                while ms_total < seconds_per_case * 1e3 and n_steps < 2000:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(pair.stream)
                    for _ in range(10):
                        pull_step(i)
                        i += 1
                    e1.record(pair.stream)
                    torch.cuda.synchronize()
                    ms_total += e0.elapsed_time(e1)
                    n_steps += 10
                assert pull.check_status() == (0, 0)
            t = torch.tensor([ms_total / max(n_steps, 1)], dtype=torch.float64, device=dev)
            HS.all_reduce(t, op=dist.ReduceOp.MAX)
            per_step = float(t.item())
            rows.append({"tile_order": "heads outermost", "store": "PULL: TMA loads from the peer, linear local store",
                         "stages": stages or "auto", "ctas": grid, "l2_evict_first": False, "ms_per_step": round(per_step, 4),
                         "per_pair_GBps": round(pair.bytes_per_step / per_step / 1e6, 1) if per_step > 0 else 0.0})
    for s in range(pair.slots):
        pair.touched.add(s)
    return rows
