"""Paged KV-cache layouts as byte-stride descriptors.

Every cache shape the reference enumerates (kvtransfer/include/envcfg.h:25-52; prose in
kvtransfer/docs/cache_transfer_spec.md:400-478) is an affine map
``(block, kv, slot, head) -> byte offset``.  The transfer kernels take that map
(``KvtLayout``) for the source and the destination independently, which is what makes a
cross-layout transfer (FlashAttention NHD on prefill, FlashInfer HND on decode) a
parameter instead of a new code path.
"""
from __future__ import annotations

import dataclasses
import enum
from typing import Optional, Tuple

import torch


class CacheShape(enum.IntEnum):
    """Cache-shape ids; values match BLLM_KVTRANS_CACHE_SHAPE of the reference."""

    RAGGED_FLASH = 1          # [blocks, slots, 2, heads, dim]
    FLASH = 2                 # [2, blocks, slots, heads, dim]            (NHD)
    QWEN3_NEXT_FLASH = 3      # stride order [blocks, 2, slots, heads, dim] (hybrid, NHD)
    DPSK_V32_SPARSE_MLA = 4   # two 3-D tensors per layer [blocks, slots, width]
    FLASHINFER = 5            # [blocks, 2, heads, slots, dim]            (HND)
    TURBOQUANT = 6
    QWEN3_NEXT_FLASHINFER = 7  # hybrid with HND attention pages
    KIMI_K3_MLA = 8


MX_GROUP = 32  # values per UE8M0 scale in block-scaled fp8 pages


@dataclasses.dataclass(frozen=True)
class AttnLayout:
    """Python mirror of ``KvtLayout`` plus what is needed to allocate and view the tensor."""

    shape: CacheShape
    num_blocks: int
    ntpb: int               # token slots per block
    num_heads: int          # heads on this rank
    head_dim: int
    elem_bytes: int         # 2 for bf16/fp16, 1 for fp8
    kv_count: int = 2
    mx_scaled: bool = False  # block-scaled fp8 page: payload followed by UE8M0 scales
    block_stride_override: int = 0  # bytes between blocks when pages are embedded in larger records (0 = dense)

    # ---- derived byte strides -------------------------------------------------------
    @property
    def head_bytes(self) -> int:
        return self.head_dim * self.elem_bytes

    @property
    def payload_block_bytes(self) -> int:
        return self.kv_count * self.ntpb * self.num_heads * self.head_bytes

    @property
    def scale_row_bytes(self) -> int:
        return self.head_dim // MX_GROUP if self.mx_scaled else 0

    @property
    def scale_block_bytes(self) -> int:
        return self.kv_count * self.ntpb * self.num_heads * self.scale_row_bytes

    @property
    def block_bytes(self) -> int:
        """Bytes of one block of one layer (what WorkerInfo.block_sizes carries)."""
        return self.payload_block_bytes + self.scale_block_bytes

    @property
    def token_bytes(self) -> int:
        return self.block_bytes // self.ntpb

    @property
    def layer_bytes(self) -> int:
        return (self.block_stride_override or self.block_bytes) * self.num_blocks

    def strides(self) -> Tuple[int, int, int, int]:
        """(block, kv, token, head) byte strides of the payload."""
        T, H, hb, B = self.ntpb, self.num_heads, self.head_bytes, self.num_blocks
        if self.block_stride_override:
            assert self.shape != CacheShape.FLASH, "K and V planes of this shape are not block-major"
            dense = dataclasses.replace(self, block_stride_override=0).strides()
            return (self.block_stride_override,) + dense[1:]
        if self.kv_count == 1:
            # single-tensor caches (MLA latent, indexer keys): [blocks, slots, width]
            return (self.block_bytes, 0, H * hb, hb)
        if self.shape == CacheShape.FLASH:
            assert not self.mx_scaled, "block-scaled pages need K and V inside one block"
            return (T * H * hb, B * T * H * hb, H * hb, hb)
        if self.shape == CacheShape.RAGGED_FLASH:
            assert not self.mx_scaled
            return (T * 2 * H * hb, H * hb, 2 * H * hb, hb)
        if self.shape in (CacheShape.QWEN3_NEXT_FLASH, CacheShape.TURBOQUANT):
            return (self.block_bytes, T * H * hb, H * hb, hb)
        if self.shape in (CacheShape.FLASHINFER, CacheShape.QWEN3_NEXT_FLASHINFER):
            return (self.block_bytes, H * T * hb, hb, T * hb)
        raise ValueError(f"no attention stride rule for {self.shape!r}")

    def scale_strides(self) -> Tuple[int, int, int, int]:
        """(base, kv, token, head) byte offsets/strides of the scale region inside a block."""
        if not self.mx_scaled:
            return (0, 0, 0, 0)
        T, H, sb = self.ntpb, self.num_heads, self.scale_row_bytes
        base = self.payload_block_bytes
        if self.kv_count == 1:
            return (base, 0, H * sb, sb)
        if self.shape in (CacheShape.FLASHINFER, CacheShape.QWEN3_NEXT_FLASHINFER):
            return (base, H * T * sb, sb, T * sb)
        return (base, T * H * sb, H * sb, sb)

    def to_kvt(self):
        from llumnix_kv_b200 import kvtransfer_ops as K

        l = K.KvtLayout()
        l.block_stride, l.kv_stride, l.token_stride, l.head_stride = self.strides()
        l.scale_base, l.scale_kv_stride, l.scale_token_stride, l.scale_head_stride = self.scale_strides()
        l.ntpb = self.ntpb
        l.num_heads = self.num_heads
        l.head_bytes = self.head_bytes
        l.num_blocks = self.num_blocks
        l.kv_count = self.kv_count
        return l

    # ---- allocation and views ---------------------------------------------------------
    def alloc(self, device, fill: Optional[str] = None, seed: int = 0) -> torch.Tensor:
        """One layer's cache as a flat uint8 tensor (layout applied through views)."""
        t = torch.zeros(self.layer_bytes, dtype=torch.uint8, device=device)
        if fill == "normal":
            g = torch.Generator(device=device)
            g.manual_seed(seed)
            dt = torch.bfloat16 if self.elem_bytes == 2 else torch.uint8
            if dt == torch.uint8:
                t.copy_(torch.randint(0, 255, (self.layer_bytes,), dtype=torch.uint8, device=device, generator=g))
            else:
                v = torch.randn(self.layer_bytes // 2, dtype=torch.float32, device=device, generator=g)
                t.view(torch.bfloat16).copy_(v.to(torch.bfloat16))
        return t

    def view(self, flat: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        """Canonical strided view ``[block, kv, slot, head, dim]`` of a flat uint8 layer tensor."""
        es = torch.empty((), dtype=dtype).element_size()
        assert es == self.elem_bytes
        bs, ks, ts, hs = self.strides()
        typed = flat.view(dtype)
        return torch.as_strided(
            typed,
            (self.num_blocks, self.kv_count, self.ntpb, self.num_heads, self.head_dim),
            (bs // es, ks // es, ts // es, hs // es, 1),
        )

    def scale_view(self, flat: torch.Tensor) -> torch.Tensor:
        """``[block, kv, slot, head, dim/32]`` uint8 view of the UE8M0 scales."""
        assert self.mx_scaled
        base, ks, ts, hs = self.scale_strides()
        return torch.as_strided(
            flat,
            (self.num_blocks, self.kv_count, self.ntpb, self.num_heads, self.scale_row_bytes),
            (self.strides()[0], ks, ts, hs, 1),
            storage_offset=flat.storage_offset() + base,
        )


def mla_layout(num_blocks: int, ntpb: int, width_bytes: int, mx_scaled: bool = False) -> AttnLayout:
    """Single-tensor cache (MLA latent+rope or indexer keys): one 'head' of ``width_bytes``."""
    return AttnLayout(CacheShape.DPSK_V32_SPARSE_MLA, num_blocks, ntpb, 1, width_bytes, 1, kv_count=1,
                      mx_scaled=mx_scaled)
