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
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "p2d_kv_transfer_GBps"
MODEL = "llama-3-8b-kv(32L,8kvh,128d,bf16,block16,NHD->HND)"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=8192, help="prompt tokens per request")
    ap.add_argument("--requests", type=int, default=1, help="requests per step")
    ap.add_argument("--slots", type=int, default=4, help="distinct request slots cycled through (each larger than L2)")
    ap.add_argument("--grid", type=int, default=0, help="CTAs of the transfer kernel (0 = tuned default)")
    ap.add_argument("--no-tma", action="store_true")
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--small", action="store_true", help="tiny case for profiler captures")
    ap.add_argument("--e2e-only", action="store_true")
    return ap.parse_args()


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


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
    from llumnix_kv_b200.bench_support import PDBenchPair

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

    if args.small:
        args.tokens, args.slots, args.layers = 2048, 2, 4

    pair = PDBenchPair(K, rank, world, dev, tokens=args.tokens, requests=args.requests, slots=args.slots,
                       n_layers=args.layers, use_tma=not args.no_tma, grid=args.grid)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(run_step, steps, warmup):
        for i in range(warmup):
            run_step(i)
        barrier()
        sampler = ClockSampler(local_rank)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for i in range(steps):
            run_step(warmup + i)
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1) if pair.is_sender else 0.0
        clocks = sampler.stop()
        barrier()
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, clocks

    # ---- kernel-only number: descriptors resident on the device, device-timed -----------
    ms_dev, clocks = (0.0, {}) if args.e2e_only else timed(pair.step_device, args.steps, args.warmup)
    # ---- end to end through the public API: pinned block tables -> H2D, 32 per-layer
    #      launches, completion word + status read back on the host every step ------------
    ms_e2e, clocks_e2e = timed(pair.step_e2e, args.steps, args.warmup)
    pair.verify()

    n_pairs = pair.n_pairs
    bytes_per_step = pair.bytes_per_step
    agg = lambda ms: (n_pairs * bytes_per_step * args.steps / (ms * 1e-3) / 1e9) if ms > 0 else 0.0
    value = agg(ms_dev) if not args.e2e_only else agg(ms_e2e)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    if world == 1:
        roof = peaks.get("hbm_gbs", 6650.0) / 2.0  # a copy reads and writes every payload byte
        roof_name = "hbm_copy/2 " + ("of measured" if peaks else "of fallback")
    else:
        roof = 770.0
        roof_name = "nvlink peer copy per direction (measured 770 GB/s)"
    if rank == 0:
        out = {
            "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round((ms_dev if not args.e2e_only else ms_e2e) / args.steps, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic N(0,1) KV, random block tables",
            "impl": "ours",
            "config": {"model": MODEL, "global_batch": args.requests * n_pairs, "seq_len": args.tokens,
                       "parallelism": f"{n_pairs}P->{n_pairs}D tp1" if world > 1 else "1 GPU loopback pair",
                       "layers": args.layers, "l2": f"inputs larger than L2: {pair.slot_bytes >> 20} MiB per step, "
                                                    f"{args.slots} slots cycled",
                       "transport": pair.transport_name},
            "per_pair_GBps": round(value / n_pairs, 2),
            "roofline": {"peak_GBps_per_pair": roof, "what": roof_name,
                         "fraction": round(value / n_pairs / roof, 3)},
            "clocks": clocks or clocks_e2e,
            "e2e": {"value": round(agg(ms_e2e), 2), "unit": "GB/s", "ms_per_step": round(ms_e2e / args.steps, 4),
                    "h2d_bytes_per_step": pair.h2d_bytes_per_step, "d2h_bytes_per_step": pair.d2h_bytes_per_step,
                    "clocks": clocks_e2e},
            "gpu_launches": pair.launches_per_step * args.steps,
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
