"""Prefill / decode separation in one process, end to end through the HybridConnector.

    python -m llumnix_kv_b200.examples.pd_demo                      # host-memory caches, TCP/SHM transport
    python -m llumnix_kv_b200.examples.pd_demo --device cuda:0      # both engines on one GPU (NVLINK transport)
    python -m llumnix_kv_b200.examples.pd_demo --device cuda:0 --decode-device cuda:1 --decode-shape 5

A prefill engine (``kv_producer``) and a decode engine (``kv_consumer``) are built from the minimal
engine that ships with the package; requests are given to the decode engine with the prefill engine's
RPC address, the decode engine pushes each request to the prefill engine, the prefill engine computes
the prompt and ships every layer's KV into the blocks the decode engine reserved, and the decode
engine continues from there.  ``--store`` adds the host-DRAM prefix store on the prefill side
(backend ``kvt+kvs``): a repeated prompt is then loaded from the store instead of recomputed.
"""
from __future__ import annotations

import argparse
import os
import time

os.environ.setdefault("BLLM_KVTRANS_QUIET_ENV", "1")

from llumnix_kv_b200.engine.config import (CacheConfig, KVTransferConfig, ModelConfig, ParallelConfig, SchedulerConfig,
                                            VllmConfig)
from llumnix_kv_b200.engine.core import MiniEngineCore
from llumnix_kv_b200.engine.types import EngineCoreRequest, SamplingParams


def make_cfg(role: str, name: str, device: str, shape: int, backend: str, tp: int, extra: dict) -> VllmConfig:
    ex = {"backend": backend, "kvt_inst_id": name, "naming_url": "fake://", "rpc_port": 0}
    ex.update(extra)
    return VllmConfig(model_config=ModelConfig(num_layers=4, num_kv_heads=8, head_dim=128),
                      cache_config=CacheConfig(block_size=16, num_gpu_blocks=256, cache_shape=shape),
                      parallel_config=ParallelConfig(tensor_parallel_size=tp),
                      scheduler_config=SchedulerConfig(max_num_batched_tokens=2048),
                      kv_transfer_config=KVTransferConfig(kv_role=role, kv_connector_extra_config=ex),
                      device=device, instance_name=name)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--decode-device", default=None)
    ap.add_argument("--prefill-shape", type=int, default=2, help="cache shape id of the prefill engine (2 = NHD)")
    ap.add_argument("--decode-shape", type=int, default=None, help="cache shape id of the decode engine (5 = HND, GPU only)")
    ap.add_argument("--prefill-tp", type=int, default=1)
    ap.add_argument("--decode-tp", type=int, default=1)
    ap.add_argument("--requests", type=int, default=4)
    ap.add_argument("--prompt", type=int, default=500)
    ap.add_argument("--store", action="store_true", help="prefill engine also keeps prompts in the host-DRAM store")
    args = ap.parse_args()
    ddev = args.decode_device or args.device
    dshape = args.decode_shape if args.decode_shape is not None else args.prefill_shape
    store = f"kvx_demo_{os.getpid()}"
    p = MiniEngineCore(make_cfg("kv_producer", "P", args.device, args.prefill_shape, "kvt+kvs" if args.store else "kvt",
                                args.prefill_tp, {"kvs_name": store, "kvs_slots": 512} if args.store else {}))
    d = MiniEngineCore(make_cfg("kv_consumer", "D", ddev, dshape, "kvt", args.decode_tp, {}))
    try:
        params = {"remote_host": "127.0.0.1", "remote_port": p.proxy.rpc_port()}
        t0 = time.time()
        for i in range(args.requests):
            toks = [(7919 * (i % 2) + 104729 * j) % 31999 + 1 for j in range(args.prompt)]   # every other prompt repeats
            d.add_request(EngineCoreRequest(f"req{i}", toks, SamplingParams(max_tokens=8, extra_args={
                "kv_transfer_params": dict(params)}), None))
        for i in range(args.requests):
            out = d.wait_finished(f"req{i}", 120)
            assert out is not None, f"req{i} did not finish"
            print(f"req{i}: {out.finish_reason.name}, tokens {d.output_tokens(f'req{i}')}")
        print(f"{args.requests} requests in {time.time() - t0:.2f}s")
        for name, e in (("prefill", p), ("decode", d)):
            st = e.connector.get_hybrid_connector_stats(e.cfg.cache_config.num_gpu_blocks)
            print(f"{name}: loads {st.load_done_count} (failed {st.load_failed_count}), saves {st.save_done_count} "
                  f"(failed {st.save_failed_count}) by source {st.save_done_count_by_source}")
    finally:
        d.shutdown()
        p.shutdown()
        if args.store:
            from llumnix_kv_b200 import load_ops

            load_ops().KvStore.unlink(store)


if __name__ == "__main__":
    main()
