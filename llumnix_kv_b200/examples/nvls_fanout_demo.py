"""Replicated KV pages to every rank of a decode TP group through NVSwitch multicast.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        --master-port 29590 -m llumnix_kv_b200.examples.nvls_fanout_demo

Every rank is a TP rank of one decode instance and owns a ``MulticastKVCache`` (its paged cache, in
memory bound to the group's multicast object).  Rank 0 plays the rank that received a request's
pages from a prefill GPU (here it just fills them); one ``fanout`` call replicates them into the same
block ids of every rank, the others wait on the completion word with a bounded device-side wait.
All ranks tear the cache down together.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def main() -> None:
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from llumnix_kv_b200.parallel.nvls import MulticastKVCache

    layers, num_blocks, block_bytes = 4, 256, 64 * 656          # MLA latent + rope pages of 64 tokens
    cache = MulticastKVCache(layers, num_blocks * block_bytes, dist.group.WORLD, dev)
    ok = True
    try:
        block_ids = [17, 3, 200, 42]
        if rank == 0:
            g = torch.Generator(device=dev).manual_seed(1)
            for layer in cache.layers:
                pages = layer.view(num_blocks, block_bytes)
                pages[block_ids] = torch.randint(0, 256, (len(block_ids), block_bytes), dtype=torch.uint8, device=dev, generator=g)
            torch.cuda.synchronize()
            cache.fanout(block_ids, block_bytes, num_blocks, flag_value=1)
        arrived = cache.wait(1, timeout_s=2.0, slots=[0])
        sums = torch.stack([layer.view(num_blocks, block_bytes)[block_ids].to(torch.int64).sum() for layer in cache.layers])
        all_sums = [torch.zeros_like(sums) for _ in range(dist.get_world_size())]
        dist.all_gather(all_sums, sums)
        ok = arrived and all(torch.equal(s, all_sums[0]) for s in all_sums)
        if rank == 0:
            print(f"{dist.get_world_size()} ranks hold the same {len(block_ids)} pages x {layers} layers: {ok}")
    finally:
        cache.close()            # collective: nobody leaves while memory is bound to the multicast object
        dist.destroy_process_group()
    if not ok:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
