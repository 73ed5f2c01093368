"""Python face of the fused P->D transfer kernel (csrc/kernels/kvt_p2d_attn.cu).

``AttnTransfer`` binds a source cache (all layers of one rank) to a destination cache that
may live on the same GPU, on a peer GPU (NVLink) or in mapped pinned host memory, and
issues one kernel per layer (or one for a layer range).  It plays the role of the
reference's channel ``register_data`` / ``send_data(layer)`` pair
(kvtransfer/include/channel.h:59-83) with the ParseBlock step folded into the kernel.

``reference_transfer`` is the plain-PyTorch fp32/byte oracle the GPU tests compare with.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Sequence, Tuple

import torch

from .layouts import MX_GROUP, AttnLayout

MODE_COPY = 0
MODE_BF16_TO_MXFP8 = 1
MODE_MXFP8_TO_BF16 = 2
REQ_PAD_TAIL = 1


def _ops():
    from llumnix_kv_b200 import kvtransfer_ops

    return kvtransfer_ops


@dataclasses.dataclass
class ReqChunk:
    """Tokens ``[seen, seen+new)`` of one request, with its block tables on both sides."""

    src_blocks: Sequence[int]
    dst_blocks: Sequence[int]
    seen_tokens: int
    new_tokens: int
    pad_tail: bool = False

    def as_tuple(self):
        return (list(self.src_blocks), list(self.dst_blocks), int(self.seen_tokens), int(self.new_tokens),
                REQ_PAD_TAIL if self.pad_tail else 0)


@dataclasses.dataclass
class HeadMap:
    """Which source heads land where on the destination rank (TP-mismatch resharding).

    P==D: (0, 0, H).  P>D with ``group_n`` prefill ranks per decode rank: (0, group_off*H_p, H_p).
    P<D: (group_off*H_d, 0, H_d).  Mirrors the group_off placement of
    kvtransfer/src/parse_block_common.cpp:81-129 and parse_block_flashinfer.cpp:34-68.
    """

    src_head0: int
    dst_head0: int
    n_heads: int


class DevicePlan:
    """A step's requests packed for the kernel and uploaded with one copy."""

    def __init__(self, chunks: Sequence[ReqChunk], tile_tokens: int, dst_ntpb: int, device, stream=None,
                 pinned: Optional[torch.Tensor] = None):
        K = _ops()
        blob, self.n_reqs, self.total_tiles, pool_off = K.kvt_pack_plan([c.as_tuple() for c in chunks],
                                                                       tile_tokens, dst_ntpb)
        self.nbytes = len(blob)
        self.pool_offset = pool_off
        n = max(self.nbytes, 16)
        if pinned is None or pinned.numel() < n:
            pinned = torch.empty(n, dtype=torch.uint8, pin_memory=torch.cuda.is_available())
        self.pinned = pinned
        if self.nbytes:
            pinned[: self.nbytes].copy_(torch.frombuffer(bytearray(blob), dtype=torch.uint8))
        self.dev = torch.empty(n, dtype=torch.uint8, device=device)
        if stream is None:
            self.dev.copy_(pinned[:n], non_blocking=True)
        else:
            with torch.cuda.stream(stream):
                self.dev.copy_(pinned[:n], non_blocking=True)

    @property
    def reqs_ptr(self) -> int:
        return self.dev.data_ptr()

    @property
    def block_ids_ptr(self) -> int:
        return self.dev.data_ptr() + self.pool_offset


class AttnTransfer:
    """Source cache -> destination cache binding for one (prefill rank, decode rank) pair."""

    def __init__(self, src_layout: AttnLayout, dst_layout: AttnLayout, src_ptrs: Sequence[int],
                 dst_ptrs: Sequence[int], device, head_map: Optional[HeadMap] = None, mode: int = MODE_COPY,
                 tile_tokens: Optional[int] = None, use_tma: bool = True, simt_tile: int = 0,
                 dst_remote: bool = False, tile_order: Optional[int] = None, store_form: Optional[int] = None,
                 tma_stages: int = 0, cache_hint: int = 0):
        K = _ops()
        assert len(src_ptrs) == len(dst_ptrs)
        self.K = K
        self.device = torch.device(device)
        self.src_layout, self.dst_layout = src_layout, dst_layout
        self.src_kvt, self.dst_kvt = src_layout.to_kvt(), dst_layout.to_kvt()
        self.num_layers = len(src_ptrs)
        self.mode = mode
        self.simt_tile = simt_tile      # 2: a CTA per tile (mapped host memory on the other side), else a warp per tile
        self.dst_remote = dst_remote    # the destination pointers are another GPU's memory (peer-mapped)
        self.head_map = head_map or HeadMap(0, 0, min(src_layout.num_heads, dst_layout.num_heads))
        import math

        self.tile_tokens = tile_tokens or math.gcd(src_layout.ntpb, dst_layout.ntpb)
        self.src_layers = torch.tensor(list(src_ptrs), dtype=torch.int64, device=self.device)
        self.dst_layers = torch.tensor(list(dst_ptrs), dtype=torch.int64, device=self.device)
        # status[0] error code, status[1] detail, status[2] done counter (kept apart from flags)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.src_maps = self.dst_maps = None
        self.use_tma = False
        # TMA tiles sit in shared memory in the destination's own order (heads outermost for an HND page), and
        # leave as ONE linear bulk store when that makes the tile a contiguous run of the destination; both can be
        # forced (tile_order 0 / 1, store_form 0 / 1) for measurements.
        hm = self.head_map
        if tile_order is None:
            tile_order = 1 if self.dst_kvt.token_stride < self.dst_kvt.head_stride else 0
        flat_ok = K.kvt_tile_is_flat(self.dst_kvt, hm.n_heads, self.tile_tokens, tile_order)
        if store_form is None:
            store_form = 1 if flat_ok else 0
        if store_form and not flat_ok:
            raise ValueError("store_form=1 needs tiles that are contiguous in the destination layout")
        self.tile_order, self.store_form, self.tma_stages, self.cache_hint = tile_order, store_form, tma_stages, cache_hint
        if use_tma and mode == MODE_COPY:
            try:
                sm = b"".join(K.kvt_encode_tensor_map(p, self.src_kvt, hm.n_heads, self.tile_tokens, tile_order)
                              for p in src_ptrs)
                dm = b"".join(K.kvt_encode_tensor_map(p, self.dst_kvt, hm.n_heads, self.tile_tokens, tile_order)
                              for p in dst_ptrs)
                self.src_maps = torch.frombuffer(bytearray(sm), dtype=torch.uint8).to(self.device)
                self.dst_maps = torch.frombuffer(bytearray(dm), dtype=torch.uint8).to(self.device)
                assert self.src_maps.data_ptr() % 64 == 0 and self.dst_maps.data_ptr() % 64 == 0
                self.use_tma = True
            except RuntimeError:
                self.use_tma = False

    def plan(self, chunks: Sequence[ReqChunk], stream=None, pinned=None) -> DevicePlan:
        return DevicePlan(chunks, self.tile_tokens, self.dst_layout.ntpb, self.device, stream, pinned)

    def launch(self, plan: DevicePlan, layer_begin: int = 0, layer_end: Optional[int] = None, stream=None,
               grid: int = 0, threads: int = 0, flag_ptr: int = 0, flag_value: int = 0,
               use_tma: Optional[bool] = None) -> None:
        if plan.n_reqs == 0:
            return
        if layer_end is None:
            layer_end = self.num_layers
        s = stream.cuda_stream if stream is not None else torch.cuda.current_stream(self.device).cuda_stream
        tma = self.use_tma if use_tma is None else (use_tma and self.use_tma)
        hm = self.head_map
        self.K.kvt_launch_p2d_attn(
            self.src_layers.data_ptr(), self.dst_layers.data_ptr(),
            self.src_maps.data_ptr() if tma else 0, self.dst_maps.data_ptr() if tma else 0,
            self.src_kvt, self.dst_kvt, layer_begin, layer_end, plan.reqs_ptr, plan.n_reqs, plan.total_tiles,
            plan.block_ids_ptr, self.tile_tokens, hm.src_head0, hm.dst_head0, hm.n_heads, self.mode,
            self.status.data_ptr(), self.status.data_ptr() + 8 if flag_ptr else 0, flag_ptr, flag_value,
            grid, threads, 1 if tma else 0, s, self.simt_tile, 1 if self.dst_remote else 0, self.tile_order,
            self.store_form, self.tma_stages, self.cache_hint)

    def check_status(self) -> Tuple[int, int]:
        st = self.status[:2].tolist()
        return st[0], st[1]


# ---------------------------------------------------------------------------------------
# PyTorch oracle
# ---------------------------------------------------------------------------------------
def mx_quantize_reference(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 reference of the in-kernel block-scaled quantiser.

    ``x``: [..., D] float32 (values exactly representable in bf16).  Returns
    (uint8 e4m3 codes [..., D], uint8 UE8M0 exponents [..., D/32]).
    """
    shp = x.shape
    g = x.reshape(*shp[:-1], shp[-1] // MX_GROUP, MX_GROUP).float()
    amax = g.abs().amax(dim=-1)
    ratio = amax * torch.tensor(1.0 / 448.0, dtype=torch.float32, device=x.device)
    bits = ratio.view(torch.int32)
    e = (bits >> 23) & 0xFF
    mant = bits & 0x7FFFFF
    e = torch.where((mant != 0) & (e != 0), e + 1, e)
    e = torch.where(e == 0, torch.ones_like(e), e)
    e = e.clamp(1, 254)
    e = torch.where(amax > 0, e, torch.full_like(e, 127))
    inv = ((254 - e) << 23).to(torch.int32).view(torch.float32)
    q = (g * inv.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).reshape(shp), e.to(torch.uint8)


def mx_dequantize_reference(codes: torch.Tensor, exps: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`mx_quantize_reference`; returns bf16."""
    shp = codes.shape
    v = codes.view(torch.float8_e4m3fn).float().reshape(*shp[:-1], shp[-1] // MX_GROUP, MX_GROUP)
    s = (exps.to(torch.int32) << 23).view(torch.float32)
    return (v * s.unsqueeze(-1)).reshape(shp).to(torch.bfloat16)


def reference_transfer(src_layout: AttnLayout, dst_layout: AttnLayout, src: torch.Tensor, dst: torch.Tensor,
                       chunks: Sequence[ReqChunk], head_map: Optional[HeadMap] = None,
                       mode: int = MODE_COPY) -> None:
    """Apply the transfer to ``dst`` (flat uint8 layer tensor) in plain PyTorch, token by token."""
    hm = head_map or HeadMap(0, 0, min(src_layout.num_heads, dst_layout.num_heads))
    hs = slice(hm.src_head0, hm.src_head0 + hm.n_heads)
    hd = slice(hm.dst_head0, hm.dst_head0 + hm.n_heads)
    if mode == MODE_COPY:
        sv = src_layout.view(src, torch.uint8 if src_layout.elem_bytes == 1 else torch.int16)
        dv = dst_layout.view(dst, torch.uint8 if dst_layout.elem_bytes == 1 else torch.int16)
    elif mode == MODE_BF16_TO_MXFP8:
        sv = src_layout.view(src, torch.bfloat16)
        dv = dst_layout.view(dst, torch.uint8)
        dsc = dst_layout.scale_view(dst)
    else:
        sv = src_layout.view(src, torch.uint8)
        ssc = src_layout.scale_view(src)
        dv = dst_layout.view(dst, torch.bfloat16)
    for c in chunks:
        end = c.seen_tokens + c.new_tokens
        for t in range(c.seen_tokens, end):
            sb, ss = c.src_blocks[t // src_layout.ntpb], t % src_layout.ntpb
            db, ds = c.dst_blocks[t // dst_layout.ntpb], t % dst_layout.ntpb
            if mode == MODE_COPY:
                dv[db, :, ds, hd, :] = sv[sb, :, ss, hs, :]
            elif mode == MODE_BF16_TO_MXFP8:
                q, e = mx_quantize_reference(sv[sb, :, ss, hs, :].float())
                dv[db, :, ds, hd, :] = q
                dsc[db, :, ds, hd, :] = e
            else:
                dv[db, :, ds, hd, :] = mx_dequantize_reference(sv[sb, :, ss, hs, :], ssc[sb, :, ss, hs, :])
        if c.pad_tail and end % dst_layout.ntpb:
            pad_end = (end + dst_layout.ntpb - 1) // dst_layout.ntpb * dst_layout.ntpb
            for t in range(end, pad_end):
                db, ds = c.dst_blocks[t // dst_layout.ntpb], t % dst_layout.ntpb
                dv[db, :, ds, hd, :] = 0
