"""Workload builder shared by ``bench.py`` and the profiling commands.

``PDBenchPair`` sets up one prefill->decode pair of the Llama-3-8B-shaped config: a source
paged cache in FlashAttention NHD on the prefill GPU, a destination cache in FlashInfer HND
on the decode GPU (peer-mapped through CUDA IPC when the two are different processes), and
random non-contiguous block tables.  ``step_device`` replays a pre-uploaded plan (kernel-only
timing); ``step_e2e`` does what a prefill worker does every engine step: pack the block
tables into pinned memory, upload them, launch one transfer kernel per layer and read the
completion word and status back.
"""
from __future__ import annotations

import ctypes
import random
from typing import List

import torch

from . import hostsync as HS
from llumnix_kv_b200.ops.layouts import AttnLayout, CacheShape
from llumnix_kv_b200.ops.p2d_attn import AttnTransfer, ReqChunk

BLOCK = 16
KV_HEADS = 8
HEAD_DIM = 128


class PDBenchPair:
    def __init__(self, K, rank: int, world: int, dev, tokens: int, requests: int, slots: int, n_layers: int,
                 use_tma: bool, grid: int, n_streams: int = 2, src_shape: CacheShape = CacheShape.FLASH,
                 dst_shape: CacheShape = CacheShape.FLASHINFER):
        import torch.distributed as dist

        self.K, self.rank, self.world, self.dev = K, rank, world, dev
        self.n_pairs = max(world // 2, 1)
        self.loopback = world == 1
        self.is_sender = self.loopback or rank < self.n_pairs
        self.is_receiver = self.loopback or rank >= self.n_pairs
        self.n_layers, self.grid, self.requests, self.slots = n_layers, grid, requests, slots
        blocks_per_req = (tokens + BLOCK - 1) // BLOCK
        self.tokens = tokens
        n_blocks = slots * requests * blocks_per_req + 1
        self.src_l = AttnLayout(src_shape, n_blocks, BLOCK, KV_HEADS, HEAD_DIM, 2)
        self.dst_l = AttnLayout(dst_shape, n_blocks, BLOCK, KV_HEADS, HEAD_DIM, 2)
        self.slot_bytes = requests * blocks_per_req * self.src_l.block_bytes * n_layers
        self.bytes_per_step = requests * tokens * self.src_l.token_bytes * n_layers
        self.launches_per_step = n_layers
        self.stream = torch.cuda.Stream(device=dev)
        # Layers are independent transfers: alternate them over a few streams so that one
        # layer's tail overlaps the next layer's ramp-up.  self.stream brackets all of them.
        self.side = [torch.cuda.Stream(device=dev) for _ in range(max(n_streams - 1, 0))]
        self.ev_begin = torch.cuda.Event()
        self.ev_side = [torch.cuda.Event() for _ in self.side]
        self.touched = set()

        # block tables: a fixed random permutation, identical on every rank (same seed)
        rng = random.Random(1234)
        ids_s = list(range(1, n_blocks))
        ids_d = list(range(1, n_blocks))
        rng.shuffle(ids_s)
        rng.shuffle(ids_d)
        self.slot_chunks: List[List[ReqChunk]] = []
        k = 0
        for _ in range(slots):
            cs = []
            for _ in range(requests):
                cs.append(ReqChunk(ids_s[k:k + blocks_per_req], ids_d[k:k + blocks_per_req], 0, tokens))
                k += blocks_per_req
            self.slot_chunks.append(cs)

        # caches
        self.src = self.dst = None
        if self.is_sender:
            self.src = torch.empty(n_layers * self.src_l.layer_bytes, dtype=torch.uint8, device=dev)
            for i in range(n_layers):
                self._fill_layer(self.src, i, self._pair_id())
        dst_ptrs = None
        # a landing area for the copy-engine ceiling measured inside the run (never read back)
        self.probe_bytes = min(1 << 30, n_layers * self.src_l.layer_bytes)
        self.probe = None
        if self.is_receiver:
            self.dst = torch.zeros(n_layers * self.dst_l.layer_bytes, dtype=torch.uint8, device=dev)
            self.probe = torch.empty(self.probe_bytes, dtype=torch.uint8, device=dev)
        if self.loopback:
            dst_ptrs = [self.dst.data_ptr() + i * self.dst_l.layer_bytes for i in range(n_layers)]
            self.probe_dst_ptr = self.probe.data_ptr()
            self.transport_name = "local HBM (same GPU)"
        else:
            mine = None
            if self.is_receiver:
                h, base, _size = K.kvt_ipc_get_handle(self.dst.data_ptr())
                h2, base2, _size2 = K.kvt_ipc_get_handle(self.probe.data_ptr())
                mine = (h, self.dst.data_ptr() - base, h2, self.probe.data_ptr() - base2)
            infos = [None] * world
            HS.all_gather_object(infos, mine)
            if self.is_sender:
                h, off, h2, off2 = infos[rank + self.n_pairs]
                self.peer_base = K.kvt_ipc_open_handle(h)
                self.probe_dst_ptr = (self.peer_base if h2 == h else K.kvt_ipc_open_handle(h2)) + off2
                dst_ptrs = [self.peer_base + off + i * self.dst_l.layer_bytes for i in range(n_layers)]
            self.transport_name = "NVLink P2P stores into CUDA-IPC mapped peer cache"
        self.dst_layer_ptrs = dst_ptrs
        self.pull = False
        self.kernel_measures = self.is_sender     # the rank that launches (and times) the kernel-only steps

        self.xfer = None
        self.h2d_bytes_per_step = 0
        self.d2h_bytes_per_step = 16
        if self.is_sender:
            src_ptrs = [self.src.data_ptr() + i * self.src_l.layer_bytes for i in range(n_layers)]
            self.xfer = AttnTransfer(self.src_l, self.dst_l, src_ptrs, dst_ptrs, dev, use_tma=use_tma)
            self.use_tma = self.xfer.use_tma
            with torch.cuda.stream(self.stream):
                self.plans = [self.xfer.plan(cs, stream=self.stream) for cs in self.slot_chunks]
            self.h2d_bytes_per_step = self.plans[0].nbytes
            self.pinned = torch.empty(max(self.plans[0].nbytes, 16), dtype=torch.uint8, pin_memory=True)
            self.flag_host, self.flag_dev = K.kvt_host_alloc_mapped(64)
            self.flag = ctypes.c_uint64.from_address(self.flag_host)
            self.flag.value = 0
            self.seq = 0
            self.status_host = torch.zeros(4, dtype=torch.int32, pin_memory=True)
        torch.cuda.synchronize()

    def map_src_on_receiver(self) -> None:
        """Maps the prefill cache into the decode rank's address space (CUDA IPC), for the probe's "pull"
        rows: the decode GPU runs the kernel and loads over NVLink instead of the prefill GPU storing."""
        import torch.distributed as dist

        self.src_peer_ptrs = None
        if self.loopback:
            return
        mine = None
        if self.is_sender:
            h, base, _size = self.K.kvt_ipc_get_handle(self.src.data_ptr())
            mine = (h, self.src.data_ptr() - base)
        infos = [None] * self.world
        HS.all_gather_object(infos, mine)
        if self.is_receiver:
            h, off = infos[self.rank - self.n_pairs]
            base = self.K.kvt_ipc_open_handle(h)
            self.src_peer_ptrs = [base + off + i * self.src_l.layer_bytes for i in range(self.n_layers)]

    def use_pull_kernels(self) -> None:
        """Kernel-only number with the kernels on the DECODE GPU (what the NVLINK transport does between two
        GPUs): the decode rank maps the prefill cache, builds the plans and launches; it is the rank that times."""
        if self.loopback:
            return
        self.map_src_on_receiver()
        self.pull = True
        self.kernel_measures = self.is_receiver
        if self.is_receiver:
            dst_ptrs = [self.dst.data_ptr() + i * self.dst_l.layer_bytes for i in range(self.n_layers)]
            self.xfer = AttnTransfer(self.src_l, self.dst_l, self.src_peer_ptrs, dst_ptrs, self.dev, use_tma=True)
            with torch.cuda.stream(self.stream):
                self.plans = [self.xfer.plan(cs, stream=self.stream) for cs in self.slot_chunks]
            torch.cuda.synchronize()
        self.transport_name = "NVLink: TMA loads by the decode GPU from the CUDA-IPC mapped prefill cache (pull)"

    def _pair_id(self) -> int:
        return self.rank % self.n_pairs if not self.loopback else 0

    def _fill_layer(self, buf: torch.Tensor, layer: int, pair: int) -> None:
        g = torch.Generator(device=self.dev)
        g.manual_seed(977 * pair + layer)
        n = self.src_l.layer_bytes // 2
        view = buf[layer * self.src_l.layer_bytes:(layer + 1) * self.src_l.layer_bytes].view(torch.bfloat16)
        chunk = 1 << 26
        for o in range(0, n, chunk):
            m = min(chunk, n - o)
            view[o:o + m].copy_(torch.randn(m, dtype=torch.float32, device=self.dev, generator=g))

    # ---- steps ------------------------------------------------------------------------
    def step_device(self, i: int) -> None:
        if not self.kernel_measures:
            return
        plan = self.plans[i % self.slots]
        self.touched.add(i % self.slots)
        self._fan_out()
        lanes = [self.stream] + self.side
        step = max(1, int(getattr(self, "layers_per_launch", 1)))
        for k, layer in enumerate(range(0, self.n_layers, step)):
            self.xfer.launch(plan, layer, min(layer + step, self.n_layers), stream=lanes[k % len(lanes)], grid=self.grid)
        self._fan_in()

    def build_graphs(self) -> None:
        """Capture each slot's 32 per-layer launches (with their fan-out over the side streams) into
        a CUDA graph; ``step_device`` then replays it, which takes the host's launch rate out of the
        kernel-only number."""
        self.graphs = []
        if not self.kernel_measures:
            return
        for i in range(self.slots):
            self.step_device(i)                 # warm-up outside capture
        torch.cuda.synchronize()
        for i in range(self.slots):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.stream):
                self._issue_layers(self.plans[i])
            self.graphs.append(g)
        torch.cuda.synchronize()

    def _issue_layers(self, plan) -> None:
        self._fan_out()
        lanes = [self.stream] + self.side
        for layer in range(self.n_layers):
            self.xfer.launch(plan, layer, layer + 1, stream=lanes[layer % len(lanes)], grid=self.grid)
        self._fan_in()

    def _fan_out(self) -> None:
        if self.side:
            self.ev_begin.record(self.stream)
            for s in self.side:
                s.wait_event(self.ev_begin)

    def _fan_in(self) -> None:
        for s, e in zip(self.side, self.ev_side):
            e.record(s)
            self.stream.wait_event(e)

    def step_e2e(self, i: int) -> None:
        if not self.is_sender:
            return
        self.seq += 1
        self.touched.add(i % self.slots)
        with torch.cuda.stream(self.stream):
            plan = self.xfer.plan(self.slot_chunks[i % self.slots], stream=self.stream, pinned=self.pinned)
        self._fan_out()
        lanes = [self.stream] + self.side
        for layer in range(self.n_layers):
            self.xfer.launch(plan, layer, layer + 1, stream=lanes[layer % len(lanes)], grid=self.grid)
        self._fan_in()
        with torch.cuda.stream(self.stream):
            self.K.kvt_launch_set_flag(self.flag_dev, self.seq, self.stream.cuda_stream)
            self.status_host.copy_(self.xfer.status, non_blocking=True)
        self.stream.synchronize()
        if self.flag.value != self.seq or int(self.status_host[0]) != 0:
            raise RuntimeError(f"transfer step {self.seq} failed: flag={self.flag.value} "
                               f"status={self.status_host.tolist()}")

    # ---- the same step through the engine's public API ---------------------------------------
    def setup_engine(self, transport: str = "nvlink") -> None:
        """KVTransferServer on the decode rank, KVTransferClient on the prefill rank, NVLink
        transport (or one of the host-staged ones: "shm", "tcp"); the WorkerInfo string travels the
        way a decode engine hands it to a prefill engine inside a request."""
        from llumnix_kv_b200.kv_transfer_impl import KVTransferClient, KVTransferProtocolType as PT, KVTransferServer

        proto = {"nvlink": PT.NVLINK, "shm": PT.SHM, "tcp": PT.TCP}[transport]
        if transport != "nvlink":
            self.transport_name = {"shm": "host-staged: gather kernel -> pinned POSIX shm -> scatter kernel (SHM transport)",
                                   "tcp": "host-staged: gather kernel -> pinned host -> TCP loopback -> pinned host -> "
                                          "scatter kernel (TCP transport, the reference's one-box path)"}[transport]

        pair = self._pair_id() if self.is_sender else self.rank - self.n_pairs
        self.dst_inst = f"D{pair}|0|1"
        self.srv = self.cli = None
        winfo = None
        if self.is_receiver:
            lb = self.dst_l.layer_bytes
            layers = [self.dst[i * lb:(i + 1) * lb] for i in range(self.n_layers)]
            self.srv = KVTransferServer(self.dst_inst, 1, 0, 0, self.dst_l.block_bytes, self.dst_l.token_bytes, "fake://",
                                        layers, [proto], num_kv_heads=KV_HEADS, cache_shape=int(self.dst_l.shape))
            winfo = self.srv.worker_info()
        if self.world > 1:
            import torch.distributed as dist

            infos = [None] * self.world
            HS.all_gather_object(infos, winfo)
            if self.is_sender:
                winfo = infos[self.rank + self.n_pairs]
        self.winfo = winfo
        if self.is_sender:
            lb = self.src_l.layer_bytes
            layers = [self.src[i * lb:(i + 1) * lb] for i in range(self.n_layers)]
            self.cli = KVTransferClient(f"P{pair}|0|1", 1, 0, 0, self.src_l.block_bytes, self.src_l.token_bytes, "fake://",
                                        layers, [proto], num_kv_heads=KV_HEADS, cache_shape=int(self.src_l.shape))
        self.engine_seq = 0
        self.engine_ahead = 0
        self.engine_h2d_bytes = self.h2d_bytes_per_step
        # the channel's completion record (sequence number, two status words, two GPU timer stamps) lands in
        # mapped host memory behind each batch; the host reads it to report the requests done
        self.engine_d2h_bytes = 32
        self.engine_api = ("KVTransferClient.submit_req_send2/start_send_step/record_event x layers/flush_send_step, "
                           "then wait_inflight(): completion records read on the host")

    def step_engine(self, i: int) -> None:
        """What a prefill worker does in one engine step, through KVTransferClient: submit the
        requests, open the step, mark each layer's KV as written on the forward stream, close
        the step and wait until the engine has reported every request done."""
        if not self.is_sender:
            return
        self.engine_seq += 1
        stepid = 4096 + self.engine_seq
        slot = i % self.slots
        self.touched.add(slot)
        cli = self.cli
        for r, c in enumerate(self.slot_chunks[slot]):
            cli.submit_req_send2(self.dst_inst, 0, f"b{self.engine_seq}.{r}", 0, c.new_tokens, True, list(c.src_blocks),
                                 list(c.dst_blocks), self.winfo, stepid=stepid)
        cli.start_send_step(stepid, 1)
        for layer in range(self.n_layers):
            cli.record_event(layer, self.stream)
        cli.flush_send_step()
        # read completion records on the host: this step's (ahead == 0) or, running one step ahead of the
        # transfers as a serving engine does, the previous step's
        if not cli.wait_inflight(self.engine_ahead, 30.0):
            raise RuntimeError("a transfer step did not complete in 30 s")

    def finish_engine(self) -> None:
        """End of a timed region: every step's completion record has been read."""
        if getattr(self, "cli", None) is None:
            return
        if not self.cli.wait_inflight(0, 30.0):
            raise RuntimeError("transfer steps did not complete in 30 s")
        if self.cli.failed_batches():
            raise RuntimeError(f"{self.cli.failed_batches()} transfer steps failed: a timing that includes them means nothing")

    def close_engine(self) -> None:
        if getattr(self, "srv", None) is not None:
            self.srv.stop()

    # ---- correctness after the timed runs ---------------------------------------------------
    def verify(self, layers=None) -> int:
        """Compares the decode cache with the prefill cache for every slot a step touched: every layer
        (or the given ones), every full block, and the tokens of a partial last block one by one.  The
        decode rank of a pair regenerates the prefill rank's cache from its seed.  Returns the number
        of layers compared; raises on the first difference."""
        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist

            HS.barrier()
        touched = sorted(self.touched)
        if self.world > 1:
            import torch.distributed as dist

            got = [None] * self.world
            HS.all_gather_object(got, touched)
            touched = got[self.rank - self.n_pairs] if self.rank >= self.n_pairs else touched
        if not self.is_receiver:
            return 0
        pair = (self.rank - self.n_pairs) if not self.loopback else 0
        layers = range(self.n_layers) if layers is None else layers
        tmp = None if self.loopback else torch.empty(self.src_l.layer_bytes, dtype=torch.uint8, device=self.dev)
        checked = 0
        for layer in layers:
            if layer >= self.n_layers:
                continue
            if self.loopback:
                src_layer = self.src[layer * self.src_l.layer_bytes:(layer + 1) * self.src_l.layer_bytes]
            else:
                g = torch.Generator(device=self.dev)
                g.manual_seed(977 * pair + layer)
                n = self.src_l.layer_bytes // 2
                v = tmp.view(torch.bfloat16)
                chunk = 1 << 26
                for o in range(0, n, chunk):
                    m = min(chunk, n - o)
                    v[o:o + m].copy_(torch.randn(m, dtype=torch.float32, device=self.dev, generator=g))
                src_layer = tmp
            dst_layer = self.dst[layer * self.dst_l.layer_bytes:(layer + 1) * self.dst_l.layer_bytes]
            sv = self.src_l.view(src_layer, torch.int16)       # [block, kv, slot, head, dim] whatever the layout
            dv = self.dst_l.view(dst_layer, torch.int16)
            for slot in touched:
                for c in self.slot_chunks[slot]:
                    nb_full = c.new_tokens // BLOCK
                    sb = torch.tensor(list(c.src_blocks[:nb_full]), device=self.dev)
                    db = torch.tensor(list(c.dst_blocks[:nb_full]), device=self.dev)
                    if not torch.equal(dv[db], sv[sb]):
                        raise RuntimeError(f"rank {self.rank}: destination cache mismatch in layer {layer}")
                    tail = c.new_tokens - nb_full * BLOCK
                    if tail:
                        s_t = sv[c.src_blocks[nb_full], :, :tail]
                        d_t = dv[c.dst_blocks[nb_full], :, :tail]
                        if not torch.equal(d_t, s_t):
                            raise RuntimeError(f"rank {self.rank}: tail tokens differ in layer {layer}")
            checked += 1
        return checked

    def verified_layers(self, layers=None) -> int:
        """verify() on the decode ranks, the smallest count over them reported on every rank."""
        n = self.verify(layers)
        if self.world > 1:
            import torch.distributed as dist

            t = torch.tensor([n if self.is_receiver else 1 << 30], dtype=torch.int64, device=self.dev)
            HS.all_reduce(t, op=dist.ReduceOp.MIN)
            n = int(t.item())
        return n


# ---------------------------------------------------------------------------------------------
# other headline measurements: host-DRAM store bandwidth, migration latency vs. block count
# ---------------------------------------------------------------------------------------------
def kvstore_bandwidth(dev, n_layers: int = 32, n_blocks: int = 1024, iters: int = 4) -> dict:
    """Save / load GB/s of the pinned host-DRAM store for Llama-3-8B-shaped KV (bf16 pages and
    block-scaled fp8 pages), device-timed on the store's stream, plus the pinned cudaMemcpy
    baseline of the same box."""
    import os

    from llumnix_kv_b200 import load_ops
    from llumnix_kv_b200.kvstore import PinnedKVStore

    res: dict = {}
    for fp8 in (False, True):
        lay = AttnLayout(CacheShape.FLASH, n_blocks + 8, BLOCK, KV_HEADS, HEAD_DIM, 2)
        layers = [lay.alloc(dev, fill="normal", seed=i) for i in range(n_layers)]
        name = f"kvx_bw_{os.getpid()}_{int(fp8)}"
        st = PinnedKVStore(name, lay, layers, 0, 1, n_blocks, create=True, fp8=fp8)
        try:
            keys = st.keys(list(range(BLOCK * n_blocks)), n_blocks)
            new, _full = st.reserve(keys)
            blocks, slots = list(range(1, n_blocks + 1)), [s for _, s in new]
            payload = n_blocks * lay.block_bytes * n_layers
            for what, fn in (("save", st.save_layers), ("load", st.load_layers)):
                ts = []
                for _ in range(iters):
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(st.stream)
                    fn(0, n_layers, blocks, slots)
                    e1.record(st.stream)
                    torch.cuda.synchronize()
                    ts.append(e0.elapsed_time(e1))
                st.check_status()
                ms = min(ts[1:])
                res[f"{what}_{'fp8' if fp8 else 'bf16'}"] = {
                    "ms": round(ms, 3), "engine_GBps": round(payload / ms / 1e6, 1),
                    "pcie_GBps": round(st.slot_bytes * n_blocks / ms / 1e6, 1)}
            st.seal(keys)
        finally:
            st.close()
            load_ops().KvStore.unlink(name)
        del layers
    n = 1 << 30
    h = torch.empty(n, dtype=torch.uint8, pin_memory=True)
    d = torch.empty(n, dtype=torch.uint8, device=dev)
    for what in ("d2h", "h2d"):
        ts = []
        for _ in range(3):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if what == "d2h":
                h.copy_(d, non_blocking=True)
            else:
                d.copy_(h, non_blocking=True)
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        res[f"cudaMemcpy_pinned_{what}_GBps"] = round(n / min(ts) / 1e6, 1)
    return res


def migration_sweep(pair: "PDBenchPair", counts=(1, 4, 16, 64, 256, 1024, 4096), iters: int = 8) -> list:
    """Latency of moving a running request's KV (all layers, one frozen step) between two decode
    caches of the same layout, against the number of blocks, through KVTransferClient.start_req_send.
    ``pair`` must have been built with identical source and destination layouts and
    ``setup_engine()`` called."""
    from llumnix_kv_b200.kv_transfer_impl import ReqMeta

    out = []
    seq = 0
    for n in counts:
        chunk = pair.slot_chunks[0][0]
        if n > len(chunk.src_blocks):
            break
        ts = []
        if pair.is_sender:
            for _ in range(iters):
                seq += 1
                m = ReqMeta()
                m.dst_inst, m.dst_worker, m.reqid = pair.dst_inst, 0, f"mig{seq}"
                m.seen_tokens, m.new_tokens = 0, n * BLOCK
                m.src_block_ids, m.dst_block_ids = [list(chunk.src_blocks[:n])], [list(chunk.dst_blocks[:n])]
                m.dst_worker_info = pair.winfo
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(pair.stream)
                pair.cli.start_req_send([m], stepid=100000 + seq)
                pair.cli.drain()
                e1.record(pair.stream)
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) * 1000.0)
        ts = sorted(ts[2:]) if len(ts) > 2 else ts
        nbytes = n * pair.src_l.block_bytes * pair.n_layers
        med = ts[len(ts) // 2] if ts else 0.0
        out.append({"blocks": n, "bytes": nbytes, "p50_us": round(med, 1), "min_us": round(ts[0], 1) if ts else 0.0,
                    "GBps_at_p50": round(nbytes / med / 1e3, 1) if med > 0 else 0.0})
    return out


def ttft_added(K, rank: int, world: int, dev, tokens: int = 8192, iters: int = 30, warmup: int = 3,
               tiny: bool = False, mix: bool = False) -> dict:
    """Time to first token of a Llama-3-8B-shaped prefill, alone ("colocated") and with every
    layer's KV pushed to the decode GPU while the next layers compute ("disaggregated", until the
    first token is on the host AND the decode side holds the whole KV).  Rank r < world/2 prefills,
    rank r + world/2 is its decode GPU; with one GPU both caches share it."""
    import random

    from llumnix_kv_b200.kv_transfer_impl import KVTransferClient, KVTransferProtocolType as PT, KVTransferServer
    from .llama_prefill import LLAMA3_8B_GEOMETRY, TINY_GEOMETRY, PrefillWorker

    geo = TINY_GEOMETRY if tiny else LLAMA3_8B_GEOMETRY
    n_pairs = max(world // 2, 1)
    sender = world == 1 or rank < n_pairs
    receiver = world == 1 or rank >= n_pairs
    pair = rank % n_pairs
    # ``mix``: every timed request draws its prompt length uniformly from [tokens / 8, 4 * tokens]
    # (1k-32k for the default 8k), the same sequence on every rank
    rng = random.Random(99)
    lengths = [rng.randint(max(16, tokens // 8), tokens * 4) for _ in range(iters)] if mix else [tokens] * iters
    max_tokens = max(lengths + [tokens])
    n_blk = (max_tokens + BLOCK - 1) // BLOCK
    num_blocks = n_blk + 8
    src_ids = rng.sample(range(1, num_blocks), n_blk)
    dst_ids = rng.sample(range(1, num_blocks), n_blk)
    dst_l = AttnLayout(CacheShape.FLASHINFER, num_blocks, BLOCK, geo.num_kv_heads, geo.head_dim, 2)
    srv = cli = worker = None
    winfo = None
    dst_inst = f"D{pair}|0|1"
    if receiver:
        dst = [dst_l.alloc(dev) for _ in range(geo.num_layers)]
        srv = KVTransferServer(dst_inst, 1, 0, 0, dst_l.block_bytes, dst_l.token_bytes, "fake://", dst, [PT.NVLINK],
                               num_kv_heads=geo.num_kv_heads, cache_shape=int(CacheShape.FLASHINFER))
        winfo = srv.worker_info()
    if world > 1:
        import torch.distributed as dist

        infos = [None] * world
        HS.all_gather_object(infos, winfo)
        if sender:
            winfo = infos[rank + n_pairs]
    colo, disagg = [], []
    if sender:
        worker = PrefillWorker(geo, dev, num_blocks, BLOCK, seed=pair)
        cli = KVTransferClient(f"P{pair}|0|1", 1, 0, 0, worker.layout.block_bytes, worker.layout.token_bytes, "fake://",
                               worker.kv_caches, [PT.NVLINK], num_kv_heads=geo.num_kv_heads,
                               cache_shape=int(CacheShape.FLASH))
        all_toks = torch.randint(0, geo.vocab, (max_tokens,), device=dev)
        all_blocks = torch.tensor(src_ids, device=dev)
        stream = torch.cuda.current_stream(dev)

        def run(push: bool, seq: int, n_tok: int = tokens) -> float:
            nb = (n_tok + BLOCK - 1) // BLOCK
            toks, blocks = all_toks[:n_tok], all_blocks[:nb]
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            if push:
                stepid = 9000 + seq
                cli.submit_req_send2(dst_inst, 0, f"t{seq}", 0, n_tok, True, src_ids[:nb], dst_ids[:nb], winfo,
                                     stepid=stepid)
                cli.start_send_step(stepid, 1)
                tok = worker.prefill(toks, blocks, after_layer=lambda i: cli.record_event(i, stream))
                cli.flush_send_step()
                first = int(tok.item())
                cli.drain()
            else:
                first = int(worker.prefill(toks, blocks).item())
            e1.record(stream)
            torch.cuda.synchronize()
            assert 0 <= first < geo.vocab
            return e0.elapsed_time(e1)

        for i in range(warmup):
            run(False, i)
            run(True, i)
        for i in range(iters):
            if mix:
                run(False, 0, lengths[i])      # a new prompt length: let the libraries pick their kernels untimed
            colo.append(run(False, warmup + i, lengths[i]))
            disagg.append(run(True, warmup + i, lengths[i]))
    torch.cuda.synchronize()
    if world > 1:
        import torch.distributed as dist

        HS.barrier()
    ok = True
    if world == 1 and sender:
        # the decode cache must hold what the prefill cache holds, layer 0 and last, all full blocks
        nb = lengths[-1] // BLOCK
        sb, db = torch.tensor(src_ids[:nb], device=dev), torch.tensor(dst_ids[:nb], device=dev)
        for layer in (0, geo.num_layers - 1):
            sv = worker.layout.view(worker.kv_caches[layer], torch.int16)[sb]
            dv = dst_l.view(dst[layer], torch.int16)[db]
            ok = ok and bool(torch.equal(sv, dv))
    if srv is not None:
        srv.stop()

    def pct(v, p):
        s = sorted(v)
        return s[min(len(s) - 1, int(round(p * (len(s) - 1))))] if s else 0.0

    res = {"colocated_ms_p50": round(pct(colo, 0.5), 3), "colocated_ms_p99": round(pct(colo, 0.99), 3),
           "disagg_ms_p50": round(pct(disagg, 0.5), 3), "disagg_ms_p99": round(pct(disagg, 0.99), 3),
           "iters": iters, "tokens": tokens, "kv_bytes": tokens * 2 * geo.num_kv_heads * geo.head_dim * 2 * geo.num_layers,
           "verified": ok}
    if colo:
        res["added_ttft_p50_pct"] = round(100.0 * (res["disagg_ms_p50"] - res["colocated_ms_p50"]) / res["colocated_ms_p50"], 2)
        res["added_ttft_p99_pct"] = round(100.0 * (res["disagg_ms_p99"] - res["colocated_ms_p99"]) / res["colocated_ms_p99"], 2)
    if colo and mix:
        # per request: the same prompt with and without the transfer
        per_req = [100.0 * (d - c) / c for c, d in zip(colo, disagg)]
        res["prompt_tokens_min_max"] = [min(lengths), max(lengths)]
        res["per_request_added_pct_p50"] = round(pct(per_req, 0.5), 2)
        res["per_request_added_pct_p99"] = round(pct(per_req, 0.99), 2)
        res["per_request_added_ms_p50"] = round(pct([d - c for c, d in zip(colo, disagg)], 0.5), 3)
        res["per_request_added_ms_p99"] = round(pct([d - c for c, d in zip(colo, disagg)], 0.99), 3)
        # Poisson arrivals at 70 % utilisation of the colocated prefill, first come first served on the one
        # prefill GPU: the measured service times of the two variants replayed against one arrival trace
        # (time to first token = queueing + service).  The transfer's completion is counted inside the
        # service time, although a real engine would start the next prefill while the last layer drains.
        mean_c = sum(colo) / len(colo)
        arr, t = [], 0.0
        for _ in colo:
            t += rng.expovariate(0.7 / mean_c)
            arr.append(t)

        def replay(service):
            free, out = 0.0, []
            for a, sv in zip(arr, service):
                start = max(a, free)
                free = start + sv
                out.append(free - a)
            return out

        qc, qd = replay(colo), replay(disagg)
        res["poisson_rho_0.7"] = {
            "colocated_ttft_ms_p50": round(pct(qc, 0.5), 2), "colocated_ttft_ms_p99": round(pct(qc, 0.99), 2),
            "disagg_ttft_ms_p50": round(pct(qd, 0.5), 2), "disagg_ttft_ms_p99": round(pct(qd, 0.99), 2),
            "added_p50_pct": round(100.0 * (pct(qd, 0.5) - pct(qc, 0.5)) / pct(qc, 0.5), 2),
            "added_p99_pct": round(100.0 * (pct(qd, 0.99) - pct(qc, 0.99)) / pct(qc, 0.99), 2)}
    return res


def quant_reshard_bandwidth(dev, tokens: int = 8192, n_layers: int = 80, iters: int = 5, n_streams: int = 8) -> dict:
    """Llama-3-70B-shaped TP-mismatch transfer on one GPU (kernel-only): a prefill TP=4 rank (2 of the 8
    KV heads, bf16, NHD) pushes into its half of a decode TP=2 rank's pages (4 heads, HND), as a
    plain copy and as block-scaled fp8 (one UE8M0 scale per 32 values).  GB/s are bf16 source bytes."""
    from llumnix_kv_b200.ops.p2d_attn import MODE_BF16_TO_MXFP8, MODE_COPY, HeadMap

    n_blk = (tokens + BLOCK - 1) // BLOCK
    src_l = AttnLayout(CacheShape.FLASH, n_blk + 1, BLOCK, 2, HEAD_DIM, 2)
    res = {}
    src = [src_l.alloc(dev, fill="normal", seed=i) for i in range(n_layers)]
    import random

    rng = random.Random(5)
    sb, db = rng.sample(range(1, n_blk + 1), n_blk), rng.sample(range(1, n_blk + 1), n_blk)
    for name, mode, dst_l in (
            ("copy_bf16", MODE_COPY, AttnLayout(CacheShape.FLASHINFER, n_blk + 1, BLOCK, 4, HEAD_DIM, 2)),
            ("bf16_to_mxfp8", MODE_BF16_TO_MXFP8, AttnLayout(CacheShape.FLASHINFER, n_blk + 1, BLOCK, 4, HEAD_DIM, 1,
                                                           mx_scaled=True))):
        dst = [dst_l.alloc(dev) for _ in range(n_layers)]
        xfer = AttnTransfer(src_l, dst_l, [t.data_ptr() for t in src], [t.data_ptr() for t in dst], dev,
                            head_map=HeadMap(0, 2, 2), mode=mode)
        streams = [torch.cuda.Stream(dev) for _ in range(n_streams)]
        main = torch.cuda.current_stream(dev)
        plan = xfer.plan([ReqChunk(sb, db, 0, tokens)])
        torch.cuda.synchronize()

        def issue():
            for s in streams:
                s.wait_stream(main)
            for layer in range(n_layers):
                xfer.launch(plan, layer, layer + 1, stream=streams[layer % n_streams])
            for s in streams:
                main.wait_stream(s)

        def timed(fn):
            ts = []
            for _ in range(iters):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(main)
                fn()
                e1.record(main)
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            return min(ts[1:])

        ms_host = timed(issue)
        side = torch.cuda.Stream(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            main_saved, main = main, side        # capture on a side stream, fan out from it
            with torch.cuda.graph(g, stream=side):
                issue()
            main = main_saved
        torch.cuda.synchronize()
        ms_graph = timed(g.replay)
        assert xfer.check_status() == (0, 0)
        nbytes = tokens * 2 * 2 * HEAD_DIM * 2 * n_layers
        res[name] = {"ms_host_launched": round(ms_host, 3), "ms_graph_replay": round(ms_graph, 3),
                     "src_GBps_host_launched": round(nbytes / ms_host / 1e6, 1),
                     "src_GBps_graph_replay": round(nbytes / ms_graph / 1e6, 1), "tma": bool(xfer.use_tma),
                     "dst_bytes": tokens * dst_l.token_bytes // 2 * n_layers}
        del dst
    return res


def hybrid_state_bandwidth(K, rank: int, world: int, dev, which: str = "gdn", tokens: int = 32768, steps: int = 10,
                           warmup: int = 3, small: bool = False) -> dict:
    """Hybrid-attention and MLA caches through the engine (KVTransferClient -> NVLink channel ->
    descriptor copy kernel), rank r -> rank r + world/2 (one GPU: loopback).

    ``gdn``: Qwen3-Next-like pages: 48 layers in a 3:1 GDN:attention pattern = 12 physical cache tensors
    whose pages hold either attention KV (2 KV heads x 256 dims, bf16, kernel blocks of 16 tokens) or one
    request's recurrent state of a GDN layer (conv 3 x 8192 bf16 + 16 heads x 128 x 128 fp32).
    ``mla``: DeepSeek-V3.2-like: 61 layers, two tensors per layer: indexer keys (128 fp8 + scale = 132 B per
    token) and latent + rope (656 B per token), 64-token blocks, identical on every TP rank."""
    import random

    from llumnix_kv_b200.kv_transfer_impl import KVTransferClient, KVTransferProtocolType as PT, KVTransferServer

    n_pairs = max(world // 2, 1)
    sender = world == 1 or rank < n_pairs
    receiver = world == 1 or rank >= n_pairs
    pair = rank % n_pairs
    rng = random.Random(17)
    if which == "gdn":
        n_tensors_per_layer, n_layers, shape = 1, 2 if small else 12, 3
        tok = 2 * 2 * 256 * 2
        conv_rows, dims, ssm = 3, [2048, 2048, 4096], [1, 16, 128, 128]
        state_bytes = conv_rows * sum(dims) * 2 + 16 * 128 * 128 * 4
        ntpb = (state_bytes + tok - 1) // tok
        ntpb = (ntpb + 15) // 16 * 16
        sizes, toks = [ntpb * tok], [tok]
        kw = dict(num_kv_heads=2, num_gdn_layers=3, conv_state_shape=[1, conv_rows, sum(dims)], ssm_state_shape=ssm,
                  gdn_conv_channel_dims=dims, gdn_conv_elem_size=2, gdn_ssm_elem_size=4)
        # attention kernels see 16-token blocks inside the manager's large pages
        import os

        os.environ["BLLM_KVTRANS_ATTN_KERNEL_BLK_SIZE"] = "16"
        n_attn = (tokens + ntpb - 1) // ntpb
        n_blocks = n_attn + 3 + 2
        ids_s, ids_d = rng.sample(range(1, n_blocks), n_attn + 3), rng.sample(range(1, n_blocks), n_attn + 3)
        sb = [[ids_s[0]], [ids_s[1]], [ids_s[2]], ids_s[3:]]
        db = [[ids_d[0]], [ids_d[1]], [ids_d[2]], ids_d[3:]]
    else:
        n_tensors_per_layer, n_layers, shape = 2, 4 if small else 61, 4
        toks, ntpb = [132, 656], 64
        sizes = [t * ntpb for t in toks]
        kw = dict(num_kv_heads=1)
        n_attn = (tokens + ntpb - 1) // ntpb
        n_blocks = n_attn + 2
        sb, db = [rng.sample(range(1, n_blocks), n_attn)], [rng.sample(range(1, n_blocks), n_attn)]

    def alloc(fill):
        out = []
        for layer in range(n_layers):
            ts = []
            for bs in sizes:
                t = torch.empty(bs * n_blocks, dtype=torch.uint8, device=dev)
                if fill:
                    g = torch.Generator(device=dev)
                    g.manual_seed(layer + 1)
                    t.copy_(torch.randint(1, 255, t.shape, dtype=torch.uint8, device=dev, generator=g))
                    t[:bs] = 0
                else:
                    t.zero_()
                ts.append(t)
            out.append(ts)
        return out

    dst_inst = f"D{pair}|0|1"
    srv = cli = None
    winfo = None
    if receiver:
        dst = alloc(False)
        srv = KVTransferServer(dst_inst, 1, 0, 0, list(sizes), list(toks), "fake://", dst, [PT.NVLINK], cache_shape=shape, **kw)
        winfo = srv.worker_info()
    if world > 1:
        import torch.distributed as dist

        infos = [None] * world
        HS.all_gather_object(infos, winfo)
        if sender:
            winfo = infos[rank + n_pairs]
    ms = ms_sync = 0.0
    moved = 0
    ok = True
    if sender:
        src = alloc(True)
        cli = KVTransferClient(f"P{pair}|0|1", 1, 0, 0, list(sizes), list(toks), "fake://", src, [PT.NVLINK],
                               cache_shape=shape, **kw)
        stream = torch.cuda.current_stream(dev)
        W = K.WorkerInfo
        pw, dw = W.from_string(cli.worker_info()), W.from_string(winfo)
        for w_ in (pw, dw):
            for k_, v_ in kw.items():
                setattr(w_, k_, v_)
        per_tensor = K.plan_ipc_blocks(pw, dw, shape, [("x", 0, tokens, True, sb, db)])[0]
        moved = sum(n for blocks in per_tensor for _, _, n in blocks) * n_layers

        def step(i, ahead):
            stepid = 7000 + i
            cli.submit_req_send2(dst_inst, 0, f"h{i}", 0, tokens, True, sb, db, winfo, stepid=stepid)
            cli.start_send_step(stepid, 1)
            for layer in range(n_layers):
                cli.record_event(layer, stream)
            cli.flush_send_step()
            assert cli.wait_inflight(ahead, 30.0)      # completion records read on the host

        def timed(ahead, first):
            for i in range(warmup):
                step(first + i, ahead)
            assert cli.wait_inflight(0, 30.0)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(steps):
                step(first + warmup + i, ahead)
            assert cli.wait_inflight(0, 30.0)
            e1.record(stream)
            torch.cuda.synchronize()
            assert cli.failed_batches() == 0, "transfer steps failed: a timing that includes them means nothing"
            return e0.elapsed_time(e1)

        ms_sync = timed(0, 0)                 # every step waits for its own completion before the next is submitted
        ms = timed(1, 1000)                   # one step ahead of the transfers, as a serving engine runs
    # the decode side compares a sample of the planned byte ranges (the first and last 64 of every tensor,
    # first and last layer) with the prefill side's bytes, regenerated from the same seeds on another GPU
    sample = None
    if sender:
        sample = [blocks[:64] + blocks[-64:] for blocks in per_tensor]
    if world > 1:
        import torch.distributed as dist

        got = [None] * world
        HS.all_gather_object(got, sample)
        if receiver:
            sample = got[rank - n_pairs]
        torch.cuda.synchronize()
        HS.barrier()
    if receiver:
        ref = src if world == 1 else alloc(True)
        for layer in (0, n_layers - 1):
            for t, blocks in enumerate(sample):
                s_, d_ = ref[layer][t], dst[layer][t]
                for s_off, d_off, n in blocks:
                    ok = ok and bool(torch.equal(d_[d_off:d_off + n], s_[s_off:s_off + n]))
    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([ms, float(moved), 0.0 if ok else 1.0, ms_sync], dtype=torch.float64, device=dev)
        HS.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, moved, ok, ms_sync = float(t[0]), int(t[1]), float(t[2]) == 0.0, float(t[3])
        HS.barrier()
    if srv is not None:
        srv.stop()
    gbps = n_pairs * moved * steps / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
    return {"which": which, "tokens": tokens, "layers_or_tensors": n_layers * n_tensors_per_layer,
            "bytes_per_step_per_pair": moved, "ms_per_step": round(ms / max(steps, 1), 4), "GBps": round(gbps, 1),
            "per_pair_GBps": round(gbps / n_pairs, 1), "steps_in_flight": 2,
            "one_step_at_a_time_GBps": round(n_pairs * moved * steps / (ms_sync * 1e-3) / 1e9, 1) if ms_sync > 0 else 0.0,
            "verified": ok}


def quant_reshard_nvlink(K, rank: int, world: int, dev, tokens: int = 8192, n_layers: int = 80, iters: int = 5,
                         n_streams: int = 8) -> dict:
    """The TP-mismatch fp8 transfer across GPUs: ranks [0, world/2) are ranks of a prefill TP=4 group
    (2 KV heads each, bf16, NHD); prefill ranks 2j and 2j+1 both push into decode rank world/2 + j
    (TP=2 rank: 4 heads, HND, block-scaled fp8), each into its half of the heads, over NVLink.  world=8
    is the whole group: GPUs 0-3 -> GPUs 4-5.  Kernel-only, device-timed, max over ranks."""
    import random

    import torch.distributed as dist

    from llumnix_kv_b200.ops.p2d_attn import MODE_BF16_TO_MXFP8, HeadMap, mx_quantize_reference

    n_p = world // 2
    n_d = max(n_p // 2, 1)
    sender = rank < n_p
    receiver = n_p <= rank < n_p + n_d
    n_blk = (tokens + BLOCK - 1) // BLOCK
    src_l = AttnLayout(CacheShape.FLASH, n_blk + 1, BLOCK, 2, HEAD_DIM, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, n_blk + 1, BLOCK, 4, HEAD_DIM, 1, mx_scaled=True)
    rng = random.Random(5)
    sb, db = rng.sample(range(1, n_blk + 1), n_blk), rng.sample(range(1, n_blk + 1), n_blk)
    mine = None
    dst = None
    if receiver:
        dst = torch.zeros(n_layers * dst_l.layer_bytes, dtype=torch.uint8, device=dev)
        h, base, _size = K.kvt_ipc_get_handle(dst.data_ptr())
        mine = (h, dst.data_ptr() - base)
    infos = [None] * world
    HS.all_gather_object(infos, mine)
    ms_host = ms_graph = 0.0
    src = None
    if sender:
        d_rank = n_p + min(rank // 2, n_d - 1)
        h, off = infos[d_rank]
        peer = K.kvt_ipc_open_handle(h)
        dst_ptrs = [peer + off + i * dst_l.layer_bytes for i in range(n_layers)]
        src = [src_l.alloc(dev, fill="normal", seed=1000 * rank + i) for i in range(n_layers)]
        xfer = AttnTransfer(src_l, dst_l, [t.data_ptr() for t in src], dst_ptrs, dev,
                            head_map=HeadMap(0, (rank % 2) * 2, 2), mode=MODE_BF16_TO_MXFP8, dst_remote=True)
        streams = [torch.cuda.Stream(dev) for _ in range(n_streams)]
        holder = {"main": torch.cuda.current_stream(dev)}
        plan = xfer.plan([ReqChunk(sb, db, 0, tokens)])
        torch.cuda.synchronize()

        def issue():
            for s in streams:
                s.wait_stream(holder["main"])
            for layer in range(n_layers):
                xfer.launch(plan, layer, layer + 1, stream=streams[layer % n_streams])
            for s in streams:
                holder["main"].wait_stream(s)

        issue()
        torch.cuda.synchronize()
        side = torch.cuda.Stream(dev)
        g = torch.cuda.CUDAGraph()
        keep = holder["main"]
        holder["main"] = side
        with torch.cuda.graph(g, stream=side):
            issue()
        holder["main"] = keep
        torch.cuda.synchronize()
    HS.barrier()

    def timed(fn):
        best = 1e30
        for _ in range(iters):
            HS.barrier()
            torch.cuda.synchronize()
            ms = 0.0
            if sender:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1)
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            HS.all_reduce(t, op=dist.ReduceOp.MAX)
            best = min(best, float(t.item()))
        return best

    ms_host = timed(issue if sender else (lambda: None))
    ms_graph = timed(g.replay if sender else (lambda: None))
    ok = True
    if sender:
        ok = xfer.check_status() == (0, 0)
    HS.barrier()
    if receiver:
        # regenerate what both feeding prefill ranks hold for layer 0 and compare codes and scales
        for j in range(2):
            p_rank = 2 * (rank - n_p) + j
            if p_rank >= n_p:
                continue
            s0 = src_l.alloc(dev, fill="normal", seed=1000 * p_rank)
            nb = min(tokens // BLOCK, 64)
            x = src_l.view(s0, torch.bfloat16)[torch.tensor(sb[:nb], device=dev)].float()       # [blk, kv, slot, 2 heads, dim]
            codes, exps = mx_quantize_reference(x)
            layer0 = dst[:dst_l.layer_bytes]
            got_c = dst_l.view(layer0, torch.uint8)[torch.tensor(db[:nb], device=dev)][:, :, :, 2 * j:2 * j + 2]
            got_e = dst_l.scale_view(layer0)[torch.tensor(db[:nb], device=dev)][:, :, :, 2 * j:2 * j + 2]
            ok = ok and bool(torch.equal(got_c, codes)) and bool(torch.equal(got_e, exps))
    t = torch.tensor([1.0 if ok else 0.0], device=dev)
    HS.all_reduce(t, op=dist.ReduceOp.MIN)
    src_bytes = tokens * 2 * 2 * HEAD_DIM * 2 * n_layers
    link_bytes = tokens * dst_l.token_bytes // 2 * n_layers
    return {"prefill_ranks": n_p, "decode_ranks": n_d, "src_bytes_per_rank": src_bytes, "link_bytes_per_rank": link_bytes,
            "ms_host_launched": round(ms_host, 3), "ms_graph_replay": round(ms_graph, 3),
            "aggregate_src_GBps_host_launched": round(n_p * src_bytes / ms_host / 1e6, 1) if ms_host > 0 else 0.0,
            "aggregate_src_GBps_graph_replay": round(n_p * src_bytes / ms_graph / 1e6, 1) if ms_graph > 0 else 0.0,
            "link_GBps_into_each_decode_rank_graph_replay":
                round(min(2, n_p) * link_bytes / ms_graph / 1e6, 1) if ms_graph > 0 else 0.0,
            "verified": bool(t.item())}


def mla_fanout_bandwidth(K, rank: int, world: int, dev, tokens: int = 32768, n_layers: int = 61, iters: int = 5,
                         warmup: int = 2, n_streams: int = 4, layer_group: int = 4) -> dict:
    """Replicated MLA latent pages from one prefill GPU (rank 0) to every rank of a decode TP group
    (ranks 1..world-1), two ways, device-timed, max over ranks:

      unicast   the prefill GPU pushes the pages into each decode rank's cache (world-1 copies leave its
                link; what the reference's P<D fan-out does, kvtbackend.py:637-664);
      nvls      the prefill GPU pushes ONE copy, layer by layer, into a landing buffer on decode rank 1;
                that rank waits (bounded) for each layer's flag and replicates the layer into every
                member's cache with ``multimem.st`` through NVSwitch; the last layer carries the
                completion word every member waits for (bounded).  The relay rank receives two copies
                (the push and the echo of its own multicast);
      scatter   the prefill GPU still sends one copy, but scatters the blocks over landing buffers of ALL
                members; every member relays its share the same way and signals in its own completion
                word; everybody waits for all words.  No member receives more than 1 + 1/k copies.
    """
    import random
    import struct

    import torch.distributed as dist

    from llumnix_kv_b200.parallel.nvls import MulticastKVCache

    assert world >= 3, "one prefill rank and a decode group of at least two"
    # the relay arms move ``layer_group`` layers per launch and flag: with one launch per layer and member the
    # prefill GPU's launch rate, not its link, bounds a group of seven
    groups = [(lo, min(lo + layer_group, n_layers)) for lo in range(0, n_layers, layer_group)]
    blk_tokens, tok_bytes = 64, 656
    blk = blk_tokens * tok_bytes                      # 41984 bytes, a multiple of 16
    n_blk = (tokens + blk_tokens - 1) // blk_tokens
    num_blocks = n_blk + n_blk // 4
    layer_bytes = num_blocks * blk
    is_p, r0 = rank == 0, 1
    k = world - 1
    bounds = [n_blk * j // k for j in range(k + 1)]          # member j (rank j + 1) relays blocks [bounds[j], bounds[j + 1])
    share_max = max(bounds[j + 1] - bounds[j] for j in range(k))
    d_group = dist.new_group(list(range(1, world)))
    rng = random.Random(23)
    sb = rng.sample(range(num_blocks), n_blk)
    db = rng.sample(range(num_blocks), n_blk)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    rules = torch.frombuffer(bytearray(struct.pack("<qqqqII", 0, 0, 0, 0, blk, 1)), dtype=torch.uint8).to(dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    counter = torch.zeros(n_layers + 1, dtype=torch.int32, device=dev)

    def gen_layer(layer: int) -> torch.Tensor:
        g = torch.Generator(device=dev)
        g.manual_seed(977 + layer)
        return torch.randint(0, 256, (layer_bytes,), dtype=torch.uint8, device=dev, generator=g)

    # ---- memory -------------------------------------------------------------------------------------------
    cache = plain = landing = flags = src = None
    mine = None
    if is_p:
        src = torch.empty(n_layers * layer_bytes, dtype=torch.uint8, device=dev)
        for layer in range(n_layers):
            src[layer * layer_bytes:(layer + 1) * layer_bytes].copy_(gen_layer(layer))
    else:
        cache = MulticastKVCache(n_layers, layer_bytes, d_group, dev)
        plain = torch.zeros(n_layers * layer_bytes, dtype=torch.uint8, device=dev)
        flags = torch.zeros(n_layers + 8, dtype=torch.int64, device=dev)      # [0, L): per-layer arrival, [L]: unicast done
        mine = {}
        tensors = {"plain": plain, "flags": flags}
        landing = torch.zeros(n_layers * n_blk * blk, dtype=torch.uint8, device=dev) if rank == r0 else \
            torch.zeros(n_layers * share_max * blk, dtype=torch.uint8, device=dev)
        tensors["landing"] = landing
        for name, t in tensors.items():
            h, base, _size = K.kvt_ipc_get_handle(t.data_ptr())
            mine[name] = (h, t.data_ptr() - base)
    infos = [None] * world
    HS.all_gather_object(infos, mine)
    torch.cuda.synchronize()

    main = torch.cuda.current_stream(dev)
    streams = [torch.cuda.Stream(dev) for _ in range(n_streams)]
    if is_p:
        opened = {}

        def peer(r, name):
            h, off = infos[r][name]
            if h not in opened:
                opened[h] = K.kvt_ipc_open_handle(h)
            return opened[h] + off

        src_layers = torch.tensor([src.data_ptr() + i * layer_bytes for i in range(n_layers)], dtype=torch.int64, device=dev)
        uni_layers = {r: torch.tensor([peer(r, "plain") + i * layer_bytes for i in range(n_layers)], dtype=torch.int64,
                                      device=dev) for r in range(1, world)}
        land_layers = torch.tensor([peer(r0, "landing") + i * n_blk * blk for i in range(n_layers)], dtype=torch.int64,
                                   device=dev)
        peer_flags = {r: peer(r, "flags") for r in range(1, world)}
        sb_t, db_t, seq_t = i32(sb), i32(db), i32(list(range(n_blk)))
        share_layers = {r: torch.tensor([peer(r, "landing") + i * ((n_blk if r == r0 else share_max) * blk)
                                         for i in range(n_layers)], dtype=torch.int64, device=dev) for r in range(1, world)}

    def push(dst_layers, dst_stride, dst_nblk, dst_ids, layer, stream, flag=0, value=0, lo=0, hi=None, cnt=None,
             layer_end=None):
        hi = n_blk if hi is None else hi
        K.kvt_launch_p2d_state(src_layers.data_ptr(), dst_layers.data_ptr(), layer, layer + 1 if layer_end is None else layer_end,
                               blk, dst_stride, num_blocks, dst_nblk, sb_t[lo:].data_ptr(), dst_ids.data_ptr(), hi - lo,
                               rules.data_ptr(), 1, status.data_ptr(),
                               (counter if cnt is None else cnt)[layer:].data_ptr() if flag else 0, flag, value, 0, 512,
                               stream.cuda_stream)

    def run_unicast(step: int) -> None:
        if is_p:
            for s in streams:
                s.wait_stream(main)
            k = 0
            for layer in range(n_layers):
                for r in range(1, world):
                    push(uni_layers[r], blk, num_blocks, db_t, layer, streams[k % n_streams])
                    k += 1
            for s in streams:
                main.wait_stream(s)
            for r in range(1, world):
                K.kvt_launch_set_flag(peer_flags[r] + 8 * n_layers, step, main.cuda_stream)
        else:
            K.kvt_launch_wait_flag(flags[n_layers:].data_ptr(), step, int(5e9), status.data_ptr(), main.cuda_stream)

    def run_nvls(step: int) -> None:
        if is_p:
            for s in streams:
                s.wait_stream(main)
            for gi, (lo, hi) in enumerate(groups):
                push(land_layers, blk, n_blk, seq_t, lo, streams[gi % n_streams], peer_flags[r0] + 8 * lo, step, layer_end=hi)
            for s in streams:
                main.wait_stream(s)
        elif rank == r0:
            two = streams[:2]
            for s in two:
                s.wait_stream(main)
            for gi, (lo, hi) in enumerate(groups):
                last = gi == len(groups) - 1
                st = main if last else two[gi % 2]
                if last:
                    for s in two:
                        main.wait_stream(s)
                K.kvt_launch_wait_flag(flags[lo:].data_ptr(), step, int(5e9), status.data_ptr(), st.cuda_stream)
                cache.fanout(db_r0, blk, num_blocks, layers=(lo, hi), flag_value=step if last else 0, stream=st,
                             src_layers=land_src, src_block_ids=seq_r0, src_block_stride=blk, src_num_blocks=n_blk)
            cache.wait(step, timeout_s=5.0, stream=main, slots=[r0 - 1], sync=False)
        else:
            cache.wait(step, timeout_s=5.0, stream=main, slots=[r0 - 1], sync=False)

    def run_scatter(step: int) -> None:
        if is_p:
            for s in streams:
                s.wait_stream(main)
            n = 0
            for lo, hi in groups:
                for j in range(k):
                    r = j + 1
                    push(share_layers[r], blk, n_blk if r == r0 else share_max, seq_t, lo, streams[n % n_streams],
                         peer_flags[r] + 8 * lo, step, lo=bounds[j], hi=bounds[j + 1], cnt=counters_by_member[j], layer_end=hi)
                    n += 1
            for s in streams:
                main.wait_stream(s)
        else:
            j = rank - 1
            two = streams[:2]
            for s in two:
                s.wait_stream(main)
            for gi, (lo, hi) in enumerate(groups):
                last = gi == len(groups) - 1
                st = main if last else two[gi % 2]
                if last:
                    for s in two:
                        main.wait_stream(s)
                K.kvt_launch_wait_flag(flags[lo:].data_ptr(), step, int(5e9), status.data_ptr(), st.cuda_stream)
                cache.fanout(db_mine, blk, num_blocks, layers=(lo, hi), flag_value=step if last else 0, stream=st,
                             src_layers=land_mine, src_block_ids=seq_mine, src_block_stride=blk,
                             src_num_blocks=n_blk if rank == r0 else share_max)
            cache.wait(step, timeout_s=5.0, stream=main, sync=False)

    if is_p:
        counters_by_member = [torch.zeros(n_layers + 1, dtype=torch.int32, device=dev) for _ in range(k)]
    else:
        j = rank - 1
        db_mine, seq_mine = i32(db[bounds[j]:bounds[j + 1]]), i32(list(range(bounds[j + 1] - bounds[j])))
        land_mine = torch.tensor([landing.data_ptr() + i * ((n_blk if rank == r0 else share_max) * blk)
                                  for i in range(n_layers)], dtype=torch.int64, device=dev)
    if rank == r0:
        db_r0, seq_r0 = i32(db), i32(list(range(n_blk)))
        land_src = torch.tensor([landing.data_ptr() + i * n_blk * blk for i in range(n_layers)], dtype=torch.int64, device=dev)

    errors = []

    def timed(fn, first_step: int) -> float:
        best = 1e30
        for it in range(warmup + iters):
            HS.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            try:
                fn(first_step + it)
            except Exception as ex:   # keep every rank in step: the memory is bound to a multicast object
                errors.append(f"rank {rank}: {type(ex).__name__}: {ex}"[:300])
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
            HS.all_reduce(t, op=dist.ReduceOp.MAX)
            if it >= warmup:
                best = min(best, float(t.item()))
        return best

    ms_uni = ms_nvls = ms_scatter = 0.0
    try:
        ms_uni = timed(run_unicast, 1)
        ms_nvls = timed(run_nvls, 1)
        torch.cuda.synchronize()

        def check(name, t):
            for layer in (0, n_layers - 1):
                want = gen_layer(layer).view(num_blocks, blk)[i32(sb).long()]
                got = t[layer * layer_bytes:(layer + 1) * layer_bytes].view(num_blocks, blk)[i32(db).long()]
                if not torch.equal(got, want):
                    errors.append(f"rank {rank}: {name} layer {layer} differs")

        if not is_p:
            check("unicast", plain)
            check("nvls single relay", cache.buffer)
            cache.buffer[:n_layers * layer_bytes].zero_()    # the scatter arm must be seen to deliver too
        ms_scatter = timed(run_scatter, 100)
        torch.cuda.synchronize()
        code = int(status[0].item())
        if code != 0:
            errors.append(f"rank {rank}: kernel status {code} detail {int(status[1].item())}")
        if not is_p:
            if cache.wait_failed():
                errors.append(f"rank {rank}: a bounded wait for a completion word ran out")
            cache.check_status()
            check("nvls scatter", cache.buffer)
    except Exception as ex:   # every rank still takes part in the collective teardown below
        errors.append(f"rank {rank}: {type(ex).__name__}: {ex}")
    all_errors = [None] * world
    HS.all_gather_object(all_errors, errors)
    if cache is not None:
        cache.close()
    HS.barrier()
    bytes_per_copy = n_layers * n_blk * blk
    n_d = world - 1
    flat = [e for es in all_errors for e in es]
    return {"decode_ranks": n_d, "tokens": tokens, "layers": n_layers, "layers_per_launch": layer_group,
            "bytes_per_copy": bytes_per_copy,
            "unicast_ms": round(ms_uni, 4), "nvls_single_relay_ms": round(ms_nvls, 4),
            "nvls_scatter_ms": round(ms_scatter, 4),
            "unicast_delivered_GBps": round(n_d * bytes_per_copy / (ms_uni * 1e-3) / 1e9, 1) if ms_uni > 0 else 0.0,
            "nvls_single_relay_delivered_GBps": round(n_d * bytes_per_copy / (ms_nvls * 1e-3) / 1e9, 1) if ms_nvls > 0 else 0.0,
            "nvls_scatter_delivered_GBps": round(n_d * bytes_per_copy / (ms_scatter * 1e-3) / 1e9, 1) if ms_scatter > 0 else 0.0,
            "speedup_single_relay": round(ms_uni / ms_nvls, 2) if ms_nvls > 0 else 0.0,
            "speedup_scatter": round(ms_uni / ms_scatter, 2) if ms_scatter > 0 else 0.0,
            "prefill_egress_bytes": {"unicast": n_d * bytes_per_copy, "nvls": bytes_per_copy},
            "verified": not flat, "errors": flat[:4]}


def post_checks(K, rank: int, world: int, dev) -> dict:
    """Untimed correctness pass after a multi-GPU benchmark, through KVTransferClient / KVTransferServer over
    NVLink, rank r -> rank r + world/2: (1) a TP-mismatched request with a block-scaled fp8 destination
    (prefill TP=4 rank 1: 2 of 8 heads, bf16, NHD -> decode TP=2 rank 0: 4 heads, e4m3 + UE8M0 scales, HND),
    compared with the PyTorch quantiser oracle on the decode GPU; (2) a hybrid request (GDN state pages +
    attention pages) and an MLA request, compared byte range by byte range with the CPU planner's ranges."""
    import torch.distributed as dist

    from llumnix_kv_b200.kv_transfer_impl import KVTransferClient, KVTransferProtocolType as PT, KVTransferServer
    from llumnix_kv_b200.ops.p2d_attn import MODE_BF16_TO_MXFP8, HeadMap, reference_transfer

    n_pairs = world // 2
    sender, receiver = rank < n_pairs, n_pairs <= rank < 2 * n_pairs
    pair = rank % n_pairs
    out = {}
    n_layers = 2
    src_l = AttnLayout(CacheShape.FLASH, 40, 16, 2, 128, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, 40, 16, 4, 128, 1, mx_scaled=True)
    reqs = [("a", [3, 9, 1], [7, 2, 30], 48), ("b", [5, 6], [11, 4], 21), ("c", [20], [21], 16)]
    inst = f"QD{pair}|0|2"
    srv = None
    winfo = None
    dst = None
    if receiver:
        dst = [dst_l.alloc(dev) for _ in range(n_layers)]
        srv = KVTransferServer(inst, 2, 0, 0, dst_l.block_bytes, dst_l.token_bytes, "fake://", dst, [PT.NVLINK],
                               num_kv_heads=8, cache_shape=5, mx_scaled=True)
        winfo = srv.worker_info()
    infos = [None] * world
    HS.all_gather_object(infos, winfo)
    if sender:
        src = [src_l.alloc(dev, "normal", seed=4000 + 10 * pair + i) for i in range(n_layers)]
        cli = KVTransferClient(f"QP{pair}|0|4", 4, 1, 1, src_l.block_bytes, src_l.token_bytes, "fake://", src, [PT.NVLINK],
                               num_kv_heads=8, cache_shape=2)
        for rid, sb, db, total in reqs:
            cli.submit_req_send2(inst, 0, rid, 0, total, True, sb, db, infos[rank + n_pairs], stepid=1)
        cli.start_send_step(1, 1)
        for layer in range(n_layers):
            cli.record_event(layer)
        cli.flush_send_step()
        cli.drain()
    torch.cuda.synchronize()
    HS.barrier()
    ok = True
    if receiver:
        chunks = [ReqChunk(sb, db, 0, t) for _, sb, db, t in reqs]
        for i in range(n_layers):
            s_i = src_l.alloc(dev, "normal", seed=4000 + 10 * pair + i)
            expect = torch.zeros_like(dst[i])
            reference_transfer(src_l, dst_l, s_i, expect, chunks, HeadMap(0, 2, 2), MODE_BF16_TO_MXFP8)
            ok = ok and bool(torch.equal(dst[i], expect))
        srv.stop()
    t = torch.tensor([0.0 if ok else 1.0], device=dev)
    HS.all_reduce(t, op=dist.ReduceOp.MAX)
    out["tp4_to_tp2_mxfp8_through_engine"] = bool(t.item() == 0.0)
    for which in ("gdn", "mla"):
        res = hybrid_state_bandwidth(K, rank, world, dev, which=which, tokens=2048, steps=1, warmup=1, small=True)
        out[f"{which}_through_engine"] = bool(res["verified"])
    return out


def relay_bandwidth(K, rank: int, world: int, dev, tokens: int = 8192, n_layers: int = 61, requests_per_worker: int = 1,
                    steps: int = 6, warmup: int = 2) -> dict:
    """Replicated MLA-like caches (indexer 132 B/token + latent 656 B/token, 64-token blocks, the same bytes
    on every tensor-parallel decode rank) from ONE prefill worker (rank 0) to a decode instance of
    k = world - 1 workers, through KVTransferClient both ways:

      unicast   the prefill worker submits every request to each of the k decode workers
                (what the reference's P<D fan-out does, blade_kvt/hybrid_connector/kvtbackend.py:637-664):
                k copies cross its link;
      relay     the prefill worker submits every request once, with fanout=k, to one decode worker (round
                robin over the group); that worker's pull session loads the bytes and stores what it wrote to
                the group's NVLink multicast mapping: one copy crosses the prefill worker's link.
      multicast the prefill GPU is itself bound to the group's multicast object (a member of the same symmetric
                allocation, with memory that only absorbs the echo) and a second client is given its mapping of
                it: the same fanout=k submissions leave as multicast stores from the prefill GPU; one copy
                crosses its link and one arrives at every decode worker.

    A step moves k * requests_per_worker requests of ``tokens`` tokens.  Timed on the prefill rank (the steps
    end when their completion records have been read), one step in flight ahead; every decode rank verifies
    every request in every layer afterwards."""
    import tempfile

    import torch.distributed as dist

    from llumnix_kv_b200.kv_transfer_impl import KVTransferClient, KVTransferProtocolType as PT, KVTransferServer
    from llumnix_kv_b200.parallel.nvls import MulticastKVCache

    assert world >= 3
    k = world - 1
    toks, ntpb = [132, 656], 64
    sizes = [t * ntpb for t in toks]
    n_req = k * requests_per_worker
    blocks_per_req = (tokens + ntpb - 1) // ntpb
    n_blocks = n_req * blocks_per_req + 2
    d_group = dist.group.WORLD          # the prefill GPU joins the multicast group for the third arm
    tmp = [tempfile.mkdtemp() if rank == 0 else None]
    HS.all_gather_object(got := [None] * world, tmp[0])
    naming = f"file:{got[0]}"
    rng = random.Random(29)
    ids_s, ids_d = rng.sample(range(1, n_blocks), n_req * blocks_per_req), rng.sample(range(1, n_blocks), n_req * blocks_per_req)
    reqs = [(i, ids_s[i * blocks_per_req:(i + 1) * blocks_per_req], ids_d[i * blocks_per_req:(i + 1) * blocks_per_req])
            for i in range(n_req)]

    def src_tensor(layer: int, t: int) -> torch.Tensor:
        g = torch.Generator(device=dev)
        g.manual_seed(31 * layer + t + 1)
        return torch.randint(1, 255, (sizes[t] * n_blocks,), dtype=torch.uint8, device=dev, generator=g)

    inst = f"DR|0|{k}"
    caches, srv, cli = [], None, None
    caches = [MulticastKVCache(n_layers, sizes[t] * n_blocks, d_group, dev) for t in range(2)]
    mc_mine = [[caches[t].mc_ptr + layer * caches[t].layer_bytes for t in range(2)] for layer in range(n_layers)]
    if rank > 0:
        layers = [[caches[t].layers[layer] for t in range(2)] for layer in range(n_layers)]
        srv = KVTransferServer(inst, k, rank - 1, rank - 1, list(sizes), list(toks), naming, layers, [PT.NVLINK], cache_shape=4,
                               num_kv_heads=1, mc_layers=mc_mine, mc_size=world)
    HS.barrier()
    bytes_per_req = sum(toks) * tokens * n_layers
    result = {"decode_workers": k, "requests_per_step": n_req, "tokens_per_request": tokens, "layers": n_layers,
              "bytes_per_request": bytes_per_req}
    seq = [0]
    if rank == 0:
        src = [[src_tensor(layer, t) for t in range(2)] for layer in range(n_layers)]
        cli = KVTransferClient("PR|0|1", 1, 0, 0, list(sizes), list(toks), naming, src, [PT.NVLINK], cache_shape=4, num_kv_heads=1)
        cli_mc = KVTransferClient("PM|0|1", 1, 0, 0, list(sizes), list(toks), naming, src, [PT.NVLINK], cache_shape=4, num_kv_heads=1,
                                  mc_layers=mc_mine, mc_size=world)
        stream = torch.cuda.current_stream(dev)

        def step(cli, relay: bool, ahead: int):
            seq[0] += 1
            stepid = 9000 + seq[0]
            for i, sb, db in reqs:
                if relay:
                    cli.submit_req_send2(inst, i % k, f"q{seq[0]}.{i}", 0, tokens, True, [sb], [db], None, stepid=stepid, fanout=k)
                else:
                    for w in range(k):
                        cli.submit_req_send2(inst, w, f"q{seq[0]}.{i}", 0, tokens, True, [sb], [db], None, stepid=stepid)
            cli.start_send_step(stepid, 1)
            for layer in range(n_layers):
                cli.record_event(layer, stream)
            cli.flush_send_step()
            assert cli.wait_inflight(ahead, 60.0)

        def timed(cli, relay: bool) -> float:
            for _ in range(warmup):
                step(cli, relay, 1)
            assert cli.wait_inflight(0, 60.0)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                step(cli, relay, 1)
            assert cli.wait_inflight(0, 60.0)
            e1.record(stream)
            torch.cuda.synchronize()
            assert cli.failed_batches() == 0, "transfer steps failed"
            return e0.elapsed_time(e1) / steps

    def verify(tag: str) -> bool:
        ok = True
        if rank > 0:
            torch.cuda.synchronize()
            for layer in range(n_layers):
                for t in range(2):
                    ref, have = src_tensor(layer, t), caches[t].layers[layer]
                    for _, sb, db in reqs:
                        s_idx = torch.tensor(sb, device=dev, dtype=torch.int64)
                        d_idx = torch.tensor(db, device=dev, dtype=torch.int64)
                        full = tokens // ntpb
                        a = ref.view(n_blocks, sizes[t])[s_idx[:full]]
                        b = have.view(n_blocks, sizes[t])[d_idx[:full]]
                        ok = ok and bool(torch.equal(a, b))
                        rest = tokens - full * ntpb
                        if rest:
                            n = rest * toks[t]
                            ok = ok and bool(torch.equal(ref.view(n_blocks, sizes[t])[sb[full], :n],
                                                         have.view(n_blocks, sizes[t])[db[full], :n]))
            for c in caches:
                c.buffer.zero_()
            torch.cuda.synchronize()
        t_ok = torch.tensor([1.0 if ok else 0.0])
        HS.all_reduce(t_ok, op=dist.ReduceOp.MIN)
        return bool(t_ok.item())

    for name, relay in (("unicast", False), ("relay", True), ("multicast", True)):
        ms = timed(cli_mc if name == "multicast" else cli, relay) if rank == 0 else 0.0
        HS.barrier()
        t_ms = torch.tensor([ms], dtype=torch.float64)
        HS.all_reduce(t_ms, op=dist.ReduceOp.MAX)
        ms = float(t_ms.item())
        verified = verify(name)
        HS.barrier()
        copies = 1 if relay else k
        result[name] = {"ms_per_step": round(ms, 3), "verified": verified, "speedup_over_unicast": 0.0,
                        "prefill_egress_bytes_per_step": copies * n_req * bytes_per_req,
                        "prefill_egress_GBps": round(copies * n_req * bytes_per_req / ms / 1e6, 1) if ms > 0 else 0.0,
                        "delivered_GBps": round(k * n_req * bytes_per_req / ms / 1e6, 1) if ms > 0 else 0.0}
    for name in ("relay", "multicast"):
        if result[name]["ms_per_step"] > 0:
            result[name]["speedup_over_unicast"] = round(result["unicast"]["ms_per_step"] / result[name]["ms_per_step"], 2)
    result["speedup"] = max(result["relay"]["speedup_over_unicast"], result["multicast"]["speedup_over_unicast"])
    if srv is not None:
        srv.stop()
    HS.barrier()
    for c in caches:
        c.close()
    HS.barrier()
    return result


def tp_mismatch_fp8_engine(K, rank: int, world: int, dev, n_layers: int = 80, steps: int = 16, warmup: int = 4,
                           min_tokens: int = 4096, max_tokens: int = 16384) -> dict:
    """Llama-3-70B-shaped KV (80 layers, 8 KV heads, head_dim 128, block 16) with a TP mismatch, through
    KVTransferClient: the first world/2 ranks are the tensor-parallel workers of ONE prefill instance
    (TP = world/2: 4 on eight GPUs, each holding 8/TP heads in bf16, NHD); the other ranks form TWO decode
    instances of TP = world/4 (2 on eight GPUs, each worker holding 8/TP heads as block-scaled e4m3 with one
    scale per 32 values, HND).  Every step sends one request of a random prompt length (uniform
    ``min_tokens``..``max_tokens``) to the decode instances in turn; the heads are resharded and quantised
    inside the transfer kernel.  Timed on the prefill ranks, one step in flight ahead, max over ranks; the
    decode workers compare the last request they received with the quantiser's oracle."""

    import torch.distributed as dist

    from llumnix_kv_b200.kv_transfer_impl import KVTransferClient, KVTransferProtocolType as PT, KVTransferServer
    from llumnix_kv_b200.ops.p2d_attn import mx_quantize_reference

    assert world in (4, 8), "prefill TP world/2 against two decode instances of TP world/4"
    n_p = world // 2
    d_tp = max(n_p // 2, 1)
    p_heads, d_heads = 8 // n_p, 8 // d_tp
    group = n_p // d_tp                         # prefill ranks that feed one decode worker
    sender = rank < n_p
    inst_of = lambda r: (r - n_p) // d_tp       # decode rank -> instance 0 / 1
    rng = random.Random(41)
    lengths = [rng.randint(min_tokens, max_tokens) for _ in range(warmup + steps)]
    max_blk = (max_tokens + BLOCK - 1) // BLOCK
    pool = max_blk + 8
    src_l = AttnLayout(CacheShape.FLASH, pool, BLOCK, p_heads, HEAD_DIM, 2)
    dst_l = AttnLayout(CacheShape.FLASHINFER, pool, BLOCK, d_heads, HEAD_DIM, 1, mx_scaled=True)
    tables = []
    for n_tok in lengths:
        nb = (n_tok + BLOCK - 1) // BLOCK
        tables.append((rng.sample(range(1, pool), nb), rng.sample(range(1, pool), nb)))
    srv = cli = None
    winfo = None
    dst = src = None
    if not sender:
        dst = [dst_l.alloc(dev) for _ in range(n_layers)]
        srv = KVTransferServer(f"D70{inst_of(rank)}|0|{d_tp}", d_tp, (rank - n_p) % d_tp, (rank - n_p) % d_tp, dst_l.block_bytes,
                               dst_l.token_bytes, "fake://", dst, [PT.NVLINK], num_kv_heads=8, cache_shape=5, mx_scaled=True)
        winfo = srv.worker_info()
    infos = [None] * world
    HS.all_gather_object(infos, winfo)
    HS.barrier()
    ms = 0.0
    moved = sum(lengths[warmup:]) * src_l.token_bytes * n_layers        # source bytes this prefill rank sends in the timed steps
    if sender:
        src = [src_l.alloc(dev, fill="normal", seed=1000 * rank + i) for i in range(n_layers)]
        cli = KVTransferClient(f"P70|0|{n_p}", n_p, rank, rank, src_l.block_bytes, src_l.token_bytes, "fake://", src, [PT.NVLINK],
                               num_kv_heads=8, cache_shape=2)
        stream = torch.cuda.current_stream(dev)
        d_local = rank // group                 # decode tp rank this prefill rank feeds

        def step(i: int):
            inst = i % 2
            d_rank = n_p + inst * d_tp + d_local
            sb, db = tables[i]
            stepid = 5000 + i
            cli.submit_req_send2(f"D70{inst}|0|{d_tp}", d_local, f"m{i}", 0, lengths[i], True, sb, db, infos[d_rank], stepid=stepid)
            cli.start_send_step(stepid, 1)
            for layer in range(n_layers):
                cli.record_event(layer, stream)
            cli.flush_send_step()
            assert cli.wait_inflight(1, 60.0)

        for i in range(warmup):
            step(i)
        assert cli.wait_inflight(0, 60.0)
    HS.barrier()
    torch.cuda.synchronize()
    if sender:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(warmup, warmup + steps):
            step(i)
        assert cli.wait_inflight(0, 60.0)
        e1.record(stream)
        torch.cuda.synchronize()
        assert cli.failed_batches() == 0, "transfer steps failed"
        ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], dtype=torch.float64)
    HS.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    HS.barrier()
    ok = True
    if not sender:
        torch.cuda.synchronize()
        inst = inst_of(rank)
        last = max(i for i in range(warmup + steps) if i % 2 == inst)
        sb, db = tables[last]
        nb = min(lengths[last] // BLOCK, 48)
        d_local = (rank - n_p) % d_tp
        for layer in (0, n_layers - 1):
            for j in range(group):
                p_rank = d_local * group + j
                s0 = src_l.alloc(dev, fill="normal", seed=1000 * p_rank + layer)
                x = src_l.view(s0, torch.bfloat16)[torch.tensor(sb[:nb], device=dev)].float()
                codes, exps = mx_quantize_reference(x)
                # both views are [block, kv, slot, head, ...] whatever the memory order
                got_c = dst_l.view(dst[layer], torch.uint8)[torch.tensor(db[:nb], device=dev)][:, :, :, j * p_heads:(j + 1) * p_heads]
                got_e = dst_l.scale_view(dst[layer])[torch.tensor(db[:nb], device=dev)][:, :, :, j * p_heads:(j + 1) * p_heads]
                ok = ok and bool(torch.equal(got_c, codes)) and bool(torch.equal(got_e, exps))
    t = torch.tensor([1.0 if ok else 0.0])
    HS.all_reduce(t, op=dist.ReduceOp.MIN)
    if srv is not None:
        srv.stop()
    HS.barrier()
    agg = n_p * moved / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
    return {"prefill_tp": n_p, "decode_instances": 2, "decode_tp": d_tp, "layers": n_layers, "steps": steps,
            "prompt_tokens_min_max": [min(lengths[warmup:]), max(lengths[warmup:])],
            "src_bytes_per_prefill_rank": moved, "ms_total": round(ms, 3), "ms_per_step": round(ms / max(steps, 1), 3),
            "aggregate_src_GBps": round(agg, 1), "src_GBps_per_prefill_rank": round(agg / n_p, 1),
            "link_GBps_per_prefill_rank": round(agg / n_p * dst_l.token_bytes / d_heads * p_heads / src_l.token_bytes, 1),
            "steps_in_flight": 2, "verified": bool(t.item())}


def kvstore_concurrent(K, rank: int, world: int, dev, n_requests: int = 256, min_tokens: int = 4096, max_tokens: int = 16384,
                       store_gib: float = 24.0, n_layers: int = 32) -> dict:
    """256 requests of 4k-16k tokens (Llama-3-8B KV shape, bf16) saved to and loaded from ONE pinned host-DRAM
    store that every rank of the box attaches to.  The requests are dealt round robin to the ranks; every rank
    saves its requests back to back (reserve -> gather kernel on the store's stream -> seal), all ranks at the
    same time, then loads back the requests of its NEIGHBOUR rank that are still resident (the store holds
    ``store_gib`` GiB and evicts least recently used blocks), which shows the sharing between ranks.  Device-timed
    per rank on the store's stream, aggregate = all bytes / slowest rank's time; the loaded blocks are compared
    with what the saving rank held."""
    import os

    import torch.distributed as dist

    from llumnix_kv_b200 import load_ops
    from llumnix_kv_b200.kvstore import PinnedKVStore

    rng = random.Random(53)
    lengths = [rng.randint(min_tokens, max_tokens) for _ in range(n_requests)]
    max_blk = (max_tokens + BLOCK - 1) // BLOCK
    lay = AttnLayout(CacheShape.FLASH, 2 * max_blk + 1, BLOCK, KV_HEADS, HEAD_DIM, 2)
    slot_bytes = lay.block_bytes * n_layers
    n_slots = int(store_gib * (1 << 30) // slot_bytes)
    name = "kvx_shared_bench"
    names = [None] * world
    HS.all_gather_object(names, f"{name}_{os.getpid()}" if rank == 0 else None)
    name = names[0]

    def fill(owner: int):
        return [lay.alloc(dev, fill="normal", seed=100 * owner + i) for i in range(n_layers)]

    layers = fill(rank)
    st = None
    if rank == 0:
        st = PinnedKVStore(name, lay, layers, 0, 1, n_slots, create=True)
    HS.barrier()
    if rank != 0:
        st = PinnedKVStore(name, lay, layers, 0, 1, n_slots, create=False)
    HS.barrier()
    mine = [i for i in range(n_requests) if i % world == rank]
    theirs = [i for i in range(n_requests) if i % world == (rank + 1) % world]

    # ---- the ceiling of this box for that traffic: every rank copies 1 GiB between its GPU and pinned host
    #      memory at the same time (the GPUs share PCIe switches and the host's memory) ------------------------
    def concurrent_copy(d2h: bool) -> float:
        n = 1 << 30
        h = torch.empty(n, dtype=torch.uint8, pin_memory=True)
        d = torch.empty(n, dtype=torch.uint8, device=dev)
        best = 1e30
        for _ in range(3):
            torch.cuda.synchronize()
            HS.barrier()
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            c0.record()
            if d2h:
                h.copy_(d, non_blocking=True)
            else:
                d.copy_(h, non_blocking=True)
            c1.record()
            torch.cuda.synchronize()
            t_c = torch.tensor([c0.elapsed_time(c1)], dtype=torch.float64)
            HS.all_reduce(t_c, op=dist.ReduceOp.MAX)
            best = min(best, float(t_c.item()))
        del h, d
        return world * n / best / 1e6

    ceil_d2h, ceil_h2d = concurrent_copy(True), concurrent_copy(False)

    def tokens_of(i: int):
        return list(range(i * 100000, i * 100000 + lengths[i]))

    def blocks_of(i: int, base: int):
        nb = lengths[i] // BLOCK            # whole blocks are what a store keeps
        return list(range(base, base + nb))

    # ---- save: all ranks at once -------------------------------------------------------------------
    saved_bytes = 0
    torch.cuda.synchronize()
    HS.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(st.stream)
    pending = []
    for i in mine:
        blocks = blocks_of(i, 1)
        keys = st.keys(tokens_of(i), len(blocks))
        new, _full = st.reserve(keys)
        if new:
            ev = st.save_layers(0, n_layers, [blocks[j] for j, _ in new], [s for _, s in new])
            pending.append((ev, [keys[j] for j, _ in new]))
            saved_bytes += len(new) * slot_bytes
        while len(pending) > 2:             # seal a request once its gather has finished; two in flight
            ev, ks = pending.pop(0)
            ev.synchronize()
            st.seal(ks)
    for ev, ks in pending:
        ev.synchronize()
        st.seal(ks)
    e1.record(st.stream)
    torch.cuda.synchronize()
    save_ms = e0.elapsed_time(e1)
    st.check_status()
    HS.barrier()
    # ---- load what the neighbour saved and is still resident --------------------------------------
    ref = fill((rank + 1) % world)
    loaded_bytes, hits, asked, ok = 0, 0, 0, True
    torch.cuda.synchronize()
    HS.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(st.stream)
    last = None
    inflight = []                           # (event, pinned keys): two requests in flight, into alternating halves of the cache
    started = 0
    for i in reversed(theirs):
        blocks = blocks_of(i, 1)
        keys = st.keys(tokens_of(i), len(blocks))
        asked += len(keys)
        slots = st.pin(keys)                # leading resident blocks, protected from eviction while they are read
        if not slots:
            continue
        base = 1 if started % 2 == 0 else max_blk + 1      # the load before the previous one has been waited for
        started += 1
        dst_blocks = list(range(base, base + len(slots)))
        ev = st.load_layers(0, n_layers, dst_blocks, slots)
        hits += len(slots)
        loaded_bytes += len(slots) * slot_bytes
        inflight.append((ev, keys[:len(slots)], base))
        last = (dst_blocks, blocks)
        while len(inflight) > 1:            # the older one has landed: its pins can go
            ev0, ks0, _ = inflight.pop(0)
            ev0.synchronize()
            st.unpin(ks0)
    for ev0, ks0, _ in inflight:
        ev0.synchronize()
        st.unpin(ks0)
    e1.record(st.stream)
    torch.cuda.synchronize()
    load_ms = e0.elapsed_time(e1)
    if last is not None:                    # the request loaded last is still in the cache: compare it, outside the timing
        dst_blocks, blocks = last
        for layer in (0, n_layers // 2, n_layers - 1):
            a = lay.view(layers[layer], torch.int16)[torch.tensor(dst_blocks, device=dev)]
            b = lay.view(ref[layer], torch.int16)[torch.tensor(blocks[:len(dst_blocks)], device=dev)]
            ok = ok and bool(torch.equal(a, b))
    st.check_status()
    stats = st.stats()
    t = torch.tensor([save_ms, load_ms, float(saved_bytes), float(loaded_bytes), float(hits), float(asked), 0.0 if ok else 1.0],
                     dtype=torch.float64)
    tmax = t.clone()
    HS.all_reduce(tmax, op=dist.ReduceOp.MAX)
    tsum = t.clone()
    HS.all_reduce(tsum, op=dist.ReduceOp.SUM)
    HS.barrier()
    st.close()
    HS.barrier()
    if rank == 0:
        load_ops().KvStore.unlink(name)
    return {"requests": n_requests, "ranks": world, "prompt_tokens_min_max": [min(lengths), max(lengths)],
            "store_GiB": store_gib, "slot_bytes": slot_bytes, "slots": n_slots,
            "save": {"bytes": int(tsum[2]), "ms_slowest_rank": round(float(tmax[0]), 1),
                     "aggregate_GBps": round(float(tsum[2]) / float(tmax[0]) / 1e6, 1) if tmax[0] > 0 else 0.0},
            "load_from_neighbour_rank": {"bytes": int(tsum[3]), "ms_slowest_rank": round(float(tmax[1]), 1),
                                         "aggregate_GBps": round(float(tsum[3]) / float(tmax[1]) / 1e6, 1) if tmax[1] > 0 else 0.0,
                                         "blocks_resident_of_asked": [int(tsum[4]), int(tsum[5])]},
            "concurrent_pinned_cudaMemcpy_GBps": {"d2h_all_ranks": round(ceil_d2h, 1), "h2d_all_ranks": round(ceil_h2d, 1)},
            "evictions": int(stats.get("evictions", 0)), "verified": float(tmax[6]) == 0.0}
