#!/usr/bin/env python
"""Headline benchmark: prefill->decode KV transfer bandwidth on B200.

Config (BASELINE.json, Llama-3-8B-shaped PD separation): 32 layers, 8 KV heads, head_dim 128,
bf16, block_size 16; the prefill cache is FlashAttention NHD, the decode cache FlashInfer HND;
synthetic N(0,1) KV.  One *step* = the KV of one batch of prompts (default 8192 tokens) leaving
a prefill GPU for its decode GPU, issued layer by layer (32 launches) the way save_kv_layer
does during a forward pass.

N GPUs form N/2 prefill->decode pairs (rank i -> rank i + N/2); with N == 1 the one pair is a
loopback on the same GPU (source and destination caches both local), so the roofline there is
HBM copy bandwidth, not NVLink.  `value` is the aggregate payload GB/s over all pairs.

  python bench.py --gpus 1 --steps 20 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
      --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 3
  python bench.py --impl reference ...      # the reference's own data path, same metric
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
os.environ.setdefault("BLLM_KVTRANS_QUIET_ENV", "1")   # stdout carries exactly one JSON line

METRIC = "p2d_kv_transfer_GBps"
MODEL = "llama-3-8b-kv(32L,8kvh,128d,bf16,block16,NHD->HND)"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "memcpy_peer", "nccl"],
                    help="ours: the fused transfer kernel; reference: the reference's own data path; memcpy_peer: the CPU "
                         "planner's merged IpcBlocks, one cudaMemcpyAsync each, into the peer cache (NHD->NHD); nccl: gather "
                         "kernel -> NCCL send/recv -> scatter kernel.  The last two are library baselines.")
    ap.add_argument("--tokens", type=int, default=8192, help="prompt tokens per request")
    ap.add_argument("--requests", type=int, default=1, help="requests per step")
    ap.add_argument("--slots", type=int, default=4, help="distinct request slots cycled through (each larger than L2)")
    ap.add_argument("--grid", type=int, default=0, help="CTAs of the transfer kernel (0 = tuned default)")
    ap.add_argument("--no-tma", action="store_true")
    ap.add_argument("--streams", type=int, default=8, help="transfer streams the layers alternate over")
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--small", action="store_true", help="tiny case for profiler captures")
    ap.add_argument("--mode", default="p2d", choices=["p2d", "kvstore", "migration", "ttft", "quant", "gdn", "mla", "fanout", "relay", "linkprobe"],
                    help="p2d: prefill->decode transfer (the headline); kvstore: host-DRAM store save/load GB/s; "
                         "migration: decode->decode latency against the number of blocks; fanout (4 or 8 GPUs): replicated "
                         "MLA pages to a decode TP group, unicast against the NVLS relay; linkprobe: the transfer "
                         "kernel's GB/s for every store form, pipeline depth and grid, next to the copy engine's")
    ap.add_argument("--kernels-on", default="decode", choices=["decode", "prefill"],
                    help="kernel-only number between two GPUs: the decode GPU loads over NVLink (pull, what the transport "
                         "does) or the prefill GPU stores (push)")
    ap.add_argument("--ahead", type=int, default=1,
                    help="end-to-end number: steps the engine thread may run ahead of the transfers (0: wait for every "
                         "step's completion record before submitting the next)")
    ap.add_argument("--min-seconds", type=float, default=1.0,
                    help="repeat the timed region of --steps steps until this much device time has been measured")
    ap.add_argument("--prompt-mix", action="store_true",
                    help="ttft mode: prompt lengths uniform in [tokens/8, 4*tokens] (1k-32k by default) instead of fixed")
    ap.add_argument("--graph", action="store_true",
                    help="kernel-only number: replay each step's per-layer launches from a CUDA graph")
    ap.add_argument("--e2e-only", action="store_true")
    ap.add_argument("--layers-per-launch", type=int, default=1,
                    help="kernel-only number: layers moved by one launch (1 = the per-layer flow of save_kv_layer)")
    ap.add_argument("--transport", default="nvlink", choices=["nvlink", "shm", "tcp"],
                    help="p2d mode, end to end through the engine: the NVLink transport (default) or one of the host-staged "
                         "fallbacks (1 GPU, same layout on both sides, end-to-end number only)")
    ap.add_argument("--e2e-path", default="engine", choices=["engine", "ops"],
                    help="end-to-end number through KVTransferClient/Server (engine) or the AttnTransfer op (ops)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU (read-only NVML) while the timed region runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int, period_s: float = 0.002):
        import threading

        self.samples, self.bits, self.max_mhz, self.err = [], 0, None, None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                ids = [x for x in visible.split(",") if x != ""]
                if index < len(ids) and ids[index].isdigit():
                    phys = int(ids[index])
            h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))

            def loop():
                while not self._stop.is_set():
                    try:
                        self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        self.bits |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
                    except Exception as ex:  # keep the benchmark alive if a query is refused
                        self.err = str(ex)
                        return
                    time.sleep(period_s)

            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
        except Exception as ex:
            self.err = f"{type(ex).__name__}: {ex}"

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        reasons = sorted(n for b, n in self.REASONS.items() if self.bits & b)
        out = {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
               "samples": len(self.samples), "reasons": reasons}
        if self.err:
            out["note"] = self.err[:120]
        return out


def reference_arm(args):
    from baseline import reference_bench

    reference_bench.main(args)


def main():
    args = parse_args()
    if args.impl == "reference":
        try:
            reference_arm(args)
        except Exception as ex:  # the reference arm must never take the driver down
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(ex).__name__}: {ex}"[:300]}))
        return

    import torch
    import torch.distributed as dist

    import llumnix_kv_b200
    from benchmarks import hostsync as HS
    from benchmarks.support import PDBenchPair

    K = llumnix_kv_b200.load_ops()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        HS.init()      # barriers and small exchanges go over the host: no rank waits inside a NCCL kernel

    if args.small:
        args.tokens, args.slots, args.layers = 2048, 2, 4

    if args.mode == "quant":
        from benchmarks.support import quant_reshard_bandwidth

        if world in (4, 8) and args.e2e_path == "engine":
            from benchmarks.support import tp_mismatch_fp8_engine

            res = tp_mismatch_fp8_engine(K, rank, world, dev, n_layers=8 if args.small else 80,
                                         min_tokens=512 if args.small else 4096, max_tokens=2048 if args.small else 16384)
            if rank == 0:
                print(json.dumps({"metric": "tp_mismatch_fp8_transfer_GBps", "value": res["aggregate_src_GBps"], "unit": "GB/s",
                                  "n_gpus": args.gpus, "higher_is_better": True, "dtype": "bf16->mxfp8", "config": {
                                      "model": "llama-3-70b-kv (80L, 8 kv heads, 128d, block 16), bf16 NHD -> block-scaled e4m3 HND",
                                      "parallelism": f"prefill TP{world // 2} -> 2 x decode TP{max(world // 4, 1)}",
                                      "seq_len": "uniform 4k-16k", "api": "KVTransferClient (engine, NVLINK transport)"},
                                  "result": res}))
            dist.destroy_process_group()
            return
        if world > 1:
            from benchmarks.support import quant_reshard_nvlink

            res = quant_reshard_nvlink(K, rank, world, dev, tokens=2048 if args.small else args.tokens,
                                       n_layers=8 if args.small else 80)
        else:
            res = quant_reshard_bandwidth(dev, tokens=2048 if args.small else args.tokens, n_layers=8 if args.small else 80)
        if world > 1:
            if rank == 0:
                print(json.dumps({"metric": "tp_mismatch_fp8_transfer_GBps", "unit": "GB/s", "n_gpus": args.gpus,
                                  "dtype": "bf16->mxfp8", "config": {
                                      "model": "llama-3-70b-kv (80L, 8 kv heads, 128d), prefill TP4 ranks -> decode TP2 ranks over "
                                               "NVLink, NHD -> HND", "seq_len": args.tokens}, "result": res}))
            dist.destroy_process_group()
            return
        if rank == 0:
            print(json.dumps({"metric": "tp_mismatch_fp8_transfer_GBps", "unit": "GB/s", "n_gpus": 1, "dtype": "bf16->mxfp8",
                              "config": {"model": "llama-3-70b-kv (80L, 8 kv heads, 128d), prefill TP4 rank -> decode TP2 rank, "
                                                  "NHD -> HND", "seq_len": args.tokens}, "result": res}))
        return
    if args.mode == "kvstore" and world > 1:
        from benchmarks.support import kvstore_concurrent

        res = kvstore_concurrent(K, rank, world, dev, n_requests=32 if args.small else 256,
                                 min_tokens=512 if args.small else 4096, max_tokens=2048 if args.small else 16384,
                                 store_gib=2.0 if args.small else 24.0, n_layers=4 if args.small else 32)
        if rank == 0:
            print(json.dumps({"metric": "kvstore_shared_save_load_GBps", "value": res["save"]["aggregate_GBps"], "unit": "GB/s",
                              "n_gpus": args.gpus, "higher_is_better": True, "dtype": "bf16", "config": {
                                  "model": "llama-3-8b-kv (32L, 8 kv heads, 128d, bf16, block 16)",
                                  "requests": "256 concurrent, 4k-16k tokens, one pinned host-DRAM store shared by all ranks"},
                              "result": res}))
        dist.destroy_process_group()
        return
    if args.mode == "kvstore":
        from benchmarks.support import kvstore_bandwidth

        res = kvstore_bandwidth(dev, n_layers=args.layers, n_blocks=256 if args.small else 1024)
        if rank == 0:
            print(json.dumps({"metric": "kvstore_save_load_GBps", "unit": "GB/s", "n_gpus": 1, "dtype": "bf16",
                              "config": {"model": MODEL, "layers": args.layers, "store": "pinned host DRAM (POSIX shm)"},
                              "result": res}))
        return
    if args.mode in ("gdn", "mla"):
        from benchmarks.support import hybrid_state_bandwidth

        res = hybrid_state_bandwidth(K, rank, world, dev, which=args.mode, tokens=2048 if args.small else 32768,
                                     steps=args.steps if args.steps != 20 else 10, warmup=args.warmup, small=args.small)
        if rank == 0:
            model = ("qwen3-next-like hybrid pages (GDN state 16x128x128 fp32 + conv, attention 2 kv heads x 256, bf16)"
                     if args.mode == "gdn" else "deepseek-v3.2-like MLA (latent+rope 656 B/token, indexer 132 B/token, 64-token blocks)")
            print(json.dumps({"metric": "hybrid_state_transfer_GBps", "unit": "GB/s", "n_gpus": args.gpus,
                              "higher_is_better": True, "config": {"model": model, "seq_len": res["tokens"],
                                                                   "api": "KVTransferClient (engine, NVLINK transport: the walk kernel expands the planner's affine rules on the device)"},
                              "result": res}))
        if world > 1:
            dist.destroy_process_group()
        return
    if args.mode == "fanout":
        from benchmarks.support import mla_fanout_bandwidth

        assert world >= 3, "--mode fanout needs --gpus 4 or 8 (one prefill GPU, a decode TP group on the others)"
        res = mla_fanout_bandwidth(K, rank, world, dev, tokens=4096 if args.small else 32768, n_layers=8 if args.small else 61)
        if rank == 0:
            print(json.dumps({"metric": "replicated_kv_fanout_GBps", "unit": "GB/s", "n_gpus": args.gpus, "higher_is_better": True,
                              "dtype": "bytes", "config": {
                                  "model": "deepseek-v3.2-like MLA latent pages (656 B/token, 64-token blocks), identical on "
                                           "every decode TP rank", "seq_len": res["tokens"],
                                  "parallelism": f"1 prefill GPU -> decode TP{world - 1} group",
                                  "paths": "unicast peer stores per rank vs one peer copy + multimem.st relay through NVSwitch"},
                              "result": res}))
        dist.destroy_process_group()
        return
    if args.mode == "relay":
        from benchmarks.support import relay_bandwidth

        assert world >= 3, "--mode relay needs --gpus 4 or 8 (one prefill worker, a decode instance on the others)"
        res = relay_bandwidth(K, rank, world, dev, tokens=2048 if args.small else 8192, n_layers=8 if args.small else 61)
        if rank == 0:
            print(json.dumps({"metric": "replicated_kv_relay_speedup", "value": res["speedup"], "unit": "x", "n_gpus": args.gpus,
                              "higher_is_better": True, "dtype": "bytes", "config": {
                                  "model": "deepseek-v3.2-like MLA caches (indexer 132 B/token + latent 656 B/token, 64-token "
                                           "blocks), identical on every decode TP rank",
                                  "parallelism": f"1 prefill worker -> decode instance TP{world - 1}",
                                  "api": "KVTransferClient.submit_req_send2(..., fanout=k): the destination worker's pull "
                                         "session relays to its NVLink multicast group"},
                              "result": res}))
        dist.destroy_process_group()
        return
    if args.mode == "ttft":
        from benchmarks.support import ttft_added

        res = ttft_added(K, rank, world, dev, tokens=512 if args.small else args.tokens, iters=max(args.steps, 5),
                         warmup=args.warmup, tiny=args.small, mix=args.prompt_mix)
        if world > 1:
            import torch as _t

            t = _t.tensor([res["colocated_ms_p50"], res["disagg_ms_p50"], res["colocated_ms_p99"], res["disagg_ms_p99"]],
                          dtype=_t.float64, device=dev)
            HS.all_reduce(t, op=dist.ReduceOp.MAX)      # slowest prefill rank
            res.update(colocated_ms_p50=float(t[0]), disagg_ms_p50=float(t[1]), colocated_ms_p99=float(t[2]),
                       disagg_ms_p99=float(t[3]))
            res["added_ttft_p50_pct"] = round(100.0 * (float(t[1]) - float(t[0])) / float(t[0]), 2)
            res["added_ttft_p99_pct"] = round(100.0 * (float(t[3]) - float(t[2])) / float(t[2]), 2)
        if rank == 0:
            print(json.dumps({"metric": "added_ttft_pct_vs_colocated_prefill", "unit": "%", "n_gpus": args.gpus,
                              "higher_is_better": False, "dtype": "bf16", "data": "synthetic tokens, random-init weights",
                              "config": {"model": "llama-3-8b (32L, 4096 hidden, 32q/8kv heads, 14336 ffn)",
                                         "seq_len": res["tokens"], "parallelism": f"{max(world // 2, 1)}P->{max(world // 2, 1)}D tp1",
                                         "kv": "NHD -> HND, pushed per layer through KVTransferClient.record_event"},
                              "result": res}))
        if world > 1:
            dist.destroy_process_group()
        return
    if args.mode == "migration":
        from benchmarks.support import migration_sweep
        from llumnix_kv_b200.ops.layouts import CacheShape

        blocks = 256 if args.small else 4096
        pair = PDBenchPair(K, rank, world, dev, tokens=blocks * 16, requests=1, slots=1, n_layers=args.layers,
                           use_tma=not args.no_tma, grid=args.grid, n_streams=1, src_shape=CacheShape.FLASHINFER,
                           dst_shape=CacheShape.FLASHINFER)
        pair.setup_engine()
        res = migration_sweep(pair)
        pair.touched.add(0)
        pair.verify()
        pair.close_engine()
        if rank == 0:
            print(json.dumps({"metric": "migration_latency_us_vs_blocks", "unit": "us", "n_gpus": args.gpus,
                              "higher_is_better": False, "dtype": "bf16",
                              "config": {"model": MODEL.replace("NHD->HND", "HND->HND"), "layers": args.layers,
                                         "transport": pair.transport_name,
                                         "api": "KVTransferClient.start_req_send (frozen step) + drain"},
                              "result": res}))
        if world > 1:
            dist.destroy_process_group()
        return

    from benchmarks import baselines as BL
    from llumnix_kv_b200.ops.layouts import CacheShape as _CS

    staged = args.transport != "nvlink"
    baseline_arm = args.impl in ("memcpy_peer", "nccl")
    if staged:
        assert world == 1, "--transport shm|tcp measures the host-staged fallbacks on one GPU"
        args.e2e_only, args.e2e_path = True, "engine"
    same_layout = staged or args.impl == "memcpy_peer"      # byte-range paths keep the layout
    pair = PDBenchPair(K, rank, world, dev, tokens=args.tokens, requests=args.requests, slots=args.slots,
                       n_layers=args.layers, use_tma=not args.no_tma, grid=args.grid, n_streams=args.streams,
                       **({"dst_shape": _CS.FLASH} if same_layout else {}))
    pair.layers_per_launch = args.layers_per_launch
    sampler = lambda: ClockSampler(local_rank)
    ceilings = BL.measure_ceilings(pair)
    if args.kernels_on == "decode" and world > 1 and not baseline_arm and args.mode == "p2d":
        pair.use_pull_kernels()
    elif world > 1:
        # the engine region follows the kernel-only region: the prefill GPU stores
        os.environ["BLLM_KVTRANS_NVLINK_PULL"] = "0"

    def roofline(per_pair: float) -> dict:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        out = {"measured_in_run": ceilings}
        if staged:
            roof = ceilings.get("pinned_h2d_GBps") or 0.0
            out.update(peak_GBps_per_pair=roof, what="pinned cudaMemcpyAsync host->device measured in this run "
                                                       "(both hops of the staged path overlap)")
        elif world == 1:
            roof = peaks.get("hbm_gbs", 6650.0) / 2.0  # a copy reads and writes every payload byte
            out.update(peak_GBps_per_pair=roof, what="hbm_copy/2 " + ("of measured" if peaks else "of fallback"),
                       fraction_of_copy_engine_in_run=round(per_pair / ceilings["local_copy_GBps"], 3)
                       if ceilings.get("local_copy_GBps") else None)
        else:
            roof = ceilings.get("peer_copy_GBps") or 0.0
            out.update(peak_GBps_per_pair=roof, what="copy-engine peer copy per direction measured in this run",
                       fraction_of_nominal_900=round(per_pair / 900.0, 3))
        out["fraction"] = round(per_pair / roof, 3) if roof else None
        return out

    if args.mode == "linkprobe":
        rows = BL.link_probe(pair)
        checked = pair.verified_layers()
        if rank == 0:
            best = max(rows, key=lambda r: r["per_pair_GBps"])
            print(json.dumps({"metric": "p2d_store_form_probe_GBps", "unit": "GB/s per pair, kernel-only", "n_gpus": args.gpus,
                              "config": {"model": MODEL, "seq_len": args.tokens, "layers": args.layers,
                                         "transport": pair.transport_name},
                              "measured_in_run": ceilings, "best": best, "layers_verified": checked, "rows": rows}))
        if world > 1:
            dist.destroy_process_group()
        return

    if baseline_arm:
        res = (BL.memcpy_peer_arm if args.impl == "memcpy_peer" else BL.nccl_arm)(pair, args.steps, args.warmup, sampler)
        stat = BL.summarize(res["regions"], args.steps)
        ms_step = stat["ms_per_step_median"]
        value = pair.n_pairs * pair.bytes_per_step / (ms_step * 1e-3) / 1e9 if ms_step > 0 else 0.0
        if rank == 0:
            print(json.dumps({
                "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic N(0,1) KV, random block tables", "impl": args.impl,
                "config": {"model": MODEL.replace("NHD->HND", "NHD->NHD") if same_layout else MODEL,
                           "global_batch": args.requests * pair.n_pairs, "seq_len": args.tokens,
                           "parallelism": f"{pair.n_pairs}P->{pair.n_pairs}D tp1" if world > 1 else "1 GPU loopback pair",
                           "layers": args.layers, "api": res["api"], "transport": pair.transport_name,
                           "l2": f"inputs larger than L2: {pair.slot_bytes >> 20} MiB per step, {args.slots} slots cycled"},
                "per_pair_GBps": round(value / pair.n_pairs, 2), "timing": stat, "roofline": roofline(value / pair.n_pairs),
                "clocks": res["clocks"], "copies_per_step": res.get("copies_per_step"), "gpu_launches": 0,
                "layers_verified": args.layers}))
        if world > 1:
            dist.destroy_process_group()
        return

    if args.graph and not args.e2e_only:
        pair.build_graphs()
    # ---- kernel-only number: descriptors resident on the device, device-timed -----------
    if args.e2e_only:
        dev_regions, clocks = [], {}
    else:
        dev_regions, clocks = BL.timed_reps(pair.step_device, args.steps, args.warmup, pair.stream, world, dev,
                                            pair.kernel_measures, args.min_seconds, sampler_factory=sampler)
    # ---- end to end through the public API: pinned block tables -> H2D, 32 per-layer
    #      launches, completion word + status read back on the host every step ------------
    sync_stat = None
    if args.e2e_path == "engine":
        pair.setup_engine(args.transport)
        # every step waits for its own completion record before the next one is submitted ...
        pair.engine_ahead = 0
        sync_regions, _ = BL.timed_reps(pair.step_engine, args.steps, args.warmup, pair.stream, world, dev,
                                        pair.is_sender, args.min_seconds / 2, end_region=pair.finish_engine)
        sync_stat = BL.summarize(sync_regions, args.steps)
        # ... and the way a serving engine drives it: the next step is submitted while the previous one still
        # transfers; each step reads the completion record of the step before it, the region ends with all read
        pair.engine_ahead = 0 if staged else args.ahead
        e2e_regions, clocks_e2e = BL.timed_reps(pair.step_engine, args.steps, args.warmup, pair.stream, world, dev,
                                                pair.is_sender, args.min_seconds, sampler_factory=sampler,
                                                end_region=pair.finish_engine)
        h2d_bytes, d2h_bytes = pair.engine_h2d_bytes, pair.engine_d2h_bytes
        e2e_api = pair.engine_api
    else:
        e2e_regions, clocks_e2e = BL.timed_reps(pair.step_e2e, args.steps, args.warmup, pair.stream, world, dev,
                                                pair.is_sender, args.min_seconds, sampler_factory=sampler)
        h2d_bytes, d2h_bytes = pair.h2d_bytes_per_step, pair.d2h_bytes_per_step
        e2e_api = "AttnTransfer.plan/launch x layers + completion flag + status read"
    layers_verified = pair.verified_layers()
    post = None
    if args.e2e_path == "engine":
        pair.close_engine()
    if world >= 4 and not staged and not args.small:
        from benchmarks.support import post_checks

        post = post_checks(K, rank, world, dev)     # untimed: TP-mismatch + MXFP8 and hybrid requests through the engine

    n_pairs = pair.n_pairs
    bytes_per_step = pair.bytes_per_step
    dev_stat = BL.summarize(dev_regions, args.steps) if dev_regions else None
    e2e_stat = BL.summarize(e2e_regions, args.steps)
    agg = lambda st: (n_pairs * bytes_per_step / (st["ms_per_step_median"] * 1e-3) / 1e9) if st and st["ms_per_step_median"] > 0 else 0.0
    head_stat = dev_stat if not args.e2e_only else e2e_stat
    value = agg(head_stat)
    if rank == 0:
        out = {
            "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": head_stat["ms_per_step_median"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic N(0,1) KV, random block tables",
            "impl": "ours",
            "config": {"model": MODEL.replace("NHD->HND", "NHD->NHD") if staged else MODEL,
                       "global_batch": args.requests * n_pairs, "seq_len": args.tokens,
                       "parallelism": f"{n_pairs}P->{n_pairs}D tp1" if world > 1 else "1 GPU loopback pair",
                       "layers": args.layers, "l2": f"inputs larger than L2: {pair.slot_bytes >> 20} MiB per step, "
                                                    f"{args.slots} slots cycled",
                       "transport": pair.transport_name,
                       "launch": "cuda graph replay" if args.graph else (
                           "one launch per layer from the host" if args.layers_per_launch == 1 else
                           f"one launch per {args.layers_per_launch} layers from the host"),
                       "scaling_note": "N=1 is a same-GPU loopback bounded by HBM; N>=2 are N/2 one-directional "
                                       "NVLink pairs bounded by the link: compare N=2,4,8 with one another"},
            "per_pair_GBps": round(value / n_pairs, 2),
            "reps": head_stat["reps"], "timing": head_stat,
            "roofline": roofline(value / n_pairs),
            "clocks": clocks or clocks_e2e,
            "e2e": {"value": round(agg(e2e_stat), 2), "unit": "GB/s", "ms_per_step": e2e_stat["ms_per_step_median"],
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes, "api": e2e_api,
                    "timing": e2e_stat, "clocks": clocks_e2e, "steps_in_flight": (0 if staged else args.ahead) + 1,
                    "one_step_at_a_time": None if sync_stat is None else {
                        "value": round(agg(sync_stat), 2), "ms_per_step": sync_stat["ms_per_step_median"],
                        "what": "the same steps, each waiting for its own completion record before the next is submitted"},
                    "fraction_of_kernel_only": round(agg(e2e_stat) / value, 3) if value > 0 else None},
            "layers_verified": layers_verified,
            # kernel-only region: one launch per --layers-per-launch layers; end-to-end region: one per layer plus
            # the plan upload's copy and the completion record; both regions are timed unless --e2e-only
            "gpu_launches": ((0 if args.e2e_only else -(-pair.launches_per_step // args.layers_per_launch) *
                              (dev_stat["reps"] if dev_stat else 0)) +
                             (pair.launches_per_step + 1) * e2e_stat["reps"]) * args.steps,
        }
        if post is not None:
            out["post_checks"] = post
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
