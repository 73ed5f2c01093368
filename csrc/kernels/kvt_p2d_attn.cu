// kvt_p2d_attn: the fused P->D paged-KV transfer kernel for sm_100a.
//
// One launch walks the block tables of every request scheduled in a step (the job of the
// reference's CPU ParseBlock generators, kvtransfer/src/parse_block_flash.cpp:10-130,
// parse_block_flashinfer.cpp:15-72, parse_block_ragged.cpp:29-217), converts between cache
// layouts (FlashAttention NHD, FlashInfer HND, ragged, MLA single-tensor), re-shards heads for
// TP-mismatched prefill/decode ranks (group_off placement of parse_block_common.cpp:81-129),
// optionally quantises bf16 -> block-scaled e4m3 (the reference only has an unscaled cast,
// kvtransfer/src/copy_kernels.cu:287-481) and stores straight into the destination cache,
// which may be local memory, a peer GPU's memory mapped over NVLink, or mapped pinned host
// memory.  No staging buffer and no library copy is involved.
//
// Work unit ("tile"): tile_tokens consecutive token slots of one request for one of K / V in
// one layer, all transferred heads.  Full tiles move with TMA: one elected thread issues a
// cp.async.bulk.tensor load of the {head_bytes, heads, tokens} box into shared memory and a
// cp.async.bulk.tensor store of the same box through a destination map whose strides encode
// the destination layout, so the NHD<->HND permutation is done by the copy engine and the SM
// issues two instructions per 8-32 KiB.  Ragged edges (a chunk that starts or ends inside a
// block), the fp8 paths and layouts TMA cannot describe run on a 16-byte-vector SIMT path in
// the same launch.  TMA loads never use cluster multicast.
//
// Every wait is bounded; on a bad block id or a timeout the kernel records a status word and
// skips the access instead of faulting.
#include <atomic>

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "kvt_kernels.h"

namespace {

constexpr int kMaxStages = 8;
constexpr int kMaxDevices = 64;
constexpr uint32_t kSmemBudget = 200 * 1024;     // bytes of dynamic shared memory we ask for at most
constexpr long long kWaitCycles = 4000000000LL;  // ~2 s at 2 GHz: bound of an mbarrier wait
constexpr uint32_t kStagePayload = 4096;         // quantiser staging per warp: e4m3 payload of a tile ...
constexpr uint32_t kStageScales = 256;           // ... and its scale bytes
constexpr uint32_t kStagePerWarp = kStagePayload + kStageScales;

struct TileInfo {
  uint32_t req;        // request index
  uint32_t tok_lo;     // first absolute token slot of the tile
  uint32_t copy_lo;    // [copy_lo, copy_hi) are copied
  uint32_t copy_hi;
  uint32_t zero_hi;    // [copy_hi', zero_hi) are zero-filled on the destination (tail pad)
  uint32_t sblk, dblk; // physical block ids
  uint32_t s_slot0, d_slot0;
  bool ok;
};

__device__ __forceinline__ void set_status(uint32_t* status, uint32_t code, uint32_t detail) {
  if (status != nullptr) {
    if (atomicCAS(status, 0u, code) == 0u) status[1] = detail;
  }
}

// Largest r with reqs[r].first_tile <= t.
__device__ __forceinline__ uint32_t find_req(const KvtReqDesc* __restrict__ reqs, uint32_t n, uint32_t t) {
  uint32_t lo = 0, hi = n;
  while (hi - lo > 1) {
    uint32_t mid = (lo + hi) >> 1;
    if (__ldg(&reqs[mid].first_tile) <= t) lo = mid; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ TileInfo decode_tile(const KvtAttnLaunch& p, uint32_t tile) {
  TileInfo ti;
  const uint32_t r = find_req(p.reqs, p.n_reqs, tile);
  const KvtReqDesc rd = p.reqs[r];
  const uint32_t tt = p.tile_tokens;
  const uint32_t local = tile - rd.first_tile;
  const uint32_t tok_lo = (rd.seen_tokens / tt + local) * tt;
  const uint32_t tok_hi = tok_lo + tt;
  const uint32_t end_tok = rd.seen_tokens + rd.new_tokens;
  uint32_t end_pad = end_tok;
  if (rd.flags & KVT_REQ_PAD_TAIL) {
    end_pad = (end_tok + p.dst.ntpb - 1) / p.dst.ntpb * p.dst.ntpb;
  }
  ti.req = r;
  ti.tok_lo = tok_lo;
  ti.copy_lo = max(rd.seen_tokens, tok_lo);
  ti.copy_hi = max(ti.copy_lo, min(end_tok, tok_hi));
  ti.zero_hi = max(ti.copy_hi, min(end_pad, tok_hi));
  const uint32_t sbi = tok_lo / p.src.ntpb;
  const uint32_t dbi = tok_lo / p.dst.ntpb;
  ti.s_slot0 = tok_lo - sbi * p.src.ntpb;
  ti.d_slot0 = tok_lo - dbi * p.dst.ntpb;
  ti.ok = true;
  ti.sblk = 0;
  ti.dblk = 0;
  const bool need_src = ti.copy_hi > ti.copy_lo;
  if (need_src) {
    if (sbi >= rd.n_src_blocks) {
      ti.ok = false;
    } else {
      ti.sblk = __ldg(&p.block_ids[rd.src_blk_off + sbi]);
      if (ti.sblk >= p.src.num_blocks) ti.ok = false;
    }
  }
  if (dbi >= rd.n_dst_blocks) {
    ti.ok = false;
  } else {
    ti.dblk = __ldg(&p.block_ids[rd.dst_blk_off + dbi]);
    if (ti.dblk >= p.dst.num_blocks) ti.ok = false;
  }
  return ti;
}

__device__ __forceinline__ bool tile_is_full(const KvtAttnLaunch& p, const TileInfo& ti) {
  return ti.copy_lo == ti.tok_lo && ti.copy_hi == ti.tok_lo + p.tile_tokens;
}

// ---- PTX wrappers -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* ptr) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(ptr));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ void tma_load_5d(uint32_t smem_dst, const void* map, uint32_t bar, int c0, int c1,
                                            int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
      ::"r"(smem_dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_store_5d(const void* map, uint32_t smem_src, int c0, int c1, int c2, int c3,
                                             int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.global.shared::cta.bulk_group"
      " [%0, {%2, %3, %4, %5, %6}], [%1];"
      ::"l"(map), "r"(smem_src), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}
__device__ __forceinline__ void bulk_store_flat(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void tma_load_5d_hint(uint32_t smem_dst, const void* map, uint32_t bar, int c0, int c1,
                                                 int c2, int c3, int c4, uint64_t pol) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3, %4, %5, %6}], [%7], %8;"
      ::"r"(smem_dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar), "l"(pol)
      : "memory");
}
__device__ __forceinline__ void tma_store_5d_hint(const void* map, uint32_t smem_src, int c0, int c1, int c2, int c3,
                                                  int c4, uint64_t pol) {
  asm volatile(
      "cp.async.bulk.tensor.5d.global.shared::cta.bulk_group.L2::cache_hint"
      " [%0, {%2, %3, %4, %5, %6}], [%1], %7;"
      ::"l"(map), "r"(smem_src), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "l"(pol)
      : "memory");
}
__device__ __forceinline__ void bulk_store_flat_hint(void* gdst, uint32_t smem_src, uint32_t bytes, uint64_t pol) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;" ::"l"(gdst),
               "r"(smem_src), "r"(bytes), "l"(pol)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ int4 ld_nc_16(const void* p) {
  int4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_16(void* p, int4 v) {
  asm volatile("st.global.v4.s32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// ---- block-scaled fp8 helpers -----------------------------------------------------------
// Scale of a 32-value group: the smallest power of two s with amax / s <= 448 (e4m3 max), stored
// as a biased UE8M0 exponent byte.  amax == 0 maps to exponent 127 (scale 1).
__device__ __forceinline__ uint32_t ue8m0_from_amax(float amax) {
  if (!(amax > 0.f)) return 127u;
  const float ratio = amax * (1.0f / 448.0f);
  const uint32_t bits = __float_as_uint(ratio);
  int e = static_cast<int>((bits >> 23) & 0xffu);
  const uint32_t mant = bits & 0x7fffffu;
  if (e == 0) {  // subnormal ratio: the smallest normal power of two is already large enough
    return 1u;
  }
  if (mant != 0u) e += 1;  // round the scale up so the largest value does not saturate
  if (e > 254) e = 254;
  if (e < 1) e = 1;
  return static_cast<uint32_t>(e);
}
__device__ __forceinline__ float scale_from_ue8m0(uint32_t e) { return __uint_as_float(e << 23); }

__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// ---- SIMT tile movers ---------------------------------------------------------------------
// Rows are enumerated in destination order so that consecutive threads write consecutive
// destination addresses (NVLink and PCIe like long contiguous write runs).
struct RowIter {
  uint32_t ntok, nh;
  bool token_inner;
  __device__ __forceinline__ void decode(uint32_t row, uint32_t& t, uint32_t& h) const {
    if (token_inner) {
      h = row / ntok;
      t = row - h * ntok;
    } else {
      t = row / nh;
      h = row - t * nh;
    }
  }
};

__device__ __forceinline__ void simt_copy_tile(const KvtAttnLaunch& p, const TileInfo& ti, uint32_t kv,
                                       const char* __restrict__ src, char* __restrict__ dst, uint32_t tid,
                                       uint32_t nthr) {
  const uint32_t cpr = p.src.head_bytes >> 4;  // 16-byte chunks per row
  RowIter it;
  it.ntok = ti.copy_hi - ti.copy_lo;
  it.nh = p.n_heads;
  it.token_inner = p.dst.token_stride < p.dst.head_stride;
  const uint32_t chunks = it.ntok * it.nh * cpr;
  const int64_t s_base = (int64_t)ti.sblk * p.src.block_stride + (int64_t)kv * p.src.kv_stride +
                         (int64_t)(ti.s_slot0 + (ti.copy_lo - ti.tok_lo)) * p.src.token_stride +
                         (int64_t)p.src_head0 * p.src.head_stride;
  const int64_t d_base = (int64_t)ti.dblk * p.dst.block_stride + (int64_t)kv * p.dst.kv_stride +
                         (int64_t)(ti.d_slot0 + (ti.copy_lo - ti.tok_lo)) * p.dst.token_stride +
                         (int64_t)p.dst_head0 * p.dst.head_stride;
  constexpr int U = 4;
  for (uint32_t base = tid; base < chunks; base += nthr * U) {
    int4 v[U];
    int64_t doff[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t i = base + u * nthr;
      doff[u] = -1;
      if (i < chunks) {
        const uint32_t row = i / cpr;
        const uint32_t c = i - row * cpr;
        uint32_t t, h;
        it.decode(row, t, h);
        v[u] = ld_nc_16(src + s_base + (int64_t)t * p.src.token_stride + (int64_t)h * p.src.head_stride + (c << 4));
        doff[u] = d_base + (int64_t)t * p.dst.token_stride + (int64_t)h * p.dst.head_stride + (c << 4);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (doff[u] >= 0) st_16(dst + doff[u], v[u]);
    }
  }
}

// bf16 source rows -> e4m3 rows + UE8M0 scales.  One thread converts 16 values (32 B in,
// 16 B out); two neighbouring lanes form one 32-value scale group.
// With `stage` (a warp's own shared-memory buffer, warp-per-tile mode) a full tile bound for an HND
// destination is quantised into shared memory and leaves as one bulk copy per head (payload) plus one
// per head (scales): the async-copy engine writes NVLink packets of 256 bytes where the warp's own
// 16-byte stores leave as 128-byte ones (measured 615 GB/s of link for those against 705 for bulk stores).
__device__ __forceinline__ void simt_quant_tile(const KvtAttnLaunch& p, const TileInfo& ti, uint32_t kv,
                                       const char* __restrict__ src, char* __restrict__ dst, uint32_t tid,
                                       uint32_t nthr, unsigned char* stage) {
  const uint32_t cpr = p.src.head_bytes >> 5;  // 32-byte source chunks per row (even: head_dim % 32 == 0)
  RowIter it;
  it.ntok = ti.copy_hi - ti.copy_lo;
  it.nh = p.n_heads;
  it.token_inner = p.dst.token_stride < p.dst.head_stride;
  const uint32_t chunks = it.ntok * it.nh * cpr;
  const uint32_t slot_s = ti.s_slot0 + (ti.copy_lo - ti.tok_lo);
  const uint32_t slot_d = ti.d_slot0 + (ti.copy_lo - ti.tok_lo);
  const int64_t s_base = (int64_t)ti.sblk * p.src.block_stride + (int64_t)kv * p.src.kv_stride +
                         (int64_t)slot_s * p.src.token_stride + (int64_t)p.src_head0 * p.src.head_stride;
  const int64_t d_blk = (int64_t)ti.dblk * p.dst.block_stride;
  const int64_t d_base = d_blk + (int64_t)kv * p.dst.kv_stride + (int64_t)slot_d * p.dst.token_stride +
                         (int64_t)p.dst_head0 * p.dst.head_stride;
  const int64_t sc_base = d_blk + p.dst.scale_base + (int64_t)kv * p.dst.scale_kv_stride +
                          (int64_t)slot_d * p.dst.scale_token_stride +
                          (int64_t)p.dst_head0 * p.dst.scale_head_stride;
  // rows of a multiple of 128 values, scale rows 4-byte aligned: scales leave as 32-bit words
  const bool wide_scales = (cpr & 7u) == 0u &&
                           (((uint64_t)sc_base | (uint64_t)p.dst.scale_token_stride | (uint64_t)p.dst.scale_head_stride |
                             (uint64_t)p.dst.block_stride | reinterpret_cast<uintptr_t>(dst)) & 3u) == 0u;
  const uint32_t run_bytes = it.ntok * p.dst.head_bytes;          // one head's rows of the tile, contiguous in HND
  const uint32_t sc_run = it.ntok * (cpr >> 1);
  const bool staged = stage != nullptr && wide_scales && it.token_inner && nthr == 32u &&
                      p.dst.token_stride == (int64_t)p.dst.head_bytes && p.dst.scale_token_stride == (int64_t)(cpr >> 1) &&
                      chunks * 16u <= kStagePayload && (chunks >> 1) <= kStageScales &&
                      ((run_bytes | sc_run | (uint32_t)p.dst.head_stride | (uint32_t)p.dst.scale_head_stride) & 15u) == 0u &&
                      ((reinterpret_cast<uintptr_t>(dst + d_base) | reinterpret_cast<uintptr_t>(dst + sc_base)) & 15u) == 0u;
  if (staged) {
    // the bulk stores of this warp's previous tile must have read the buffer before it is refilled
    if (tid == 0) bulk_wait_read<0>();
    __syncwarp();
  }
  // Two rounds in flight per thread: the loads of both are issued before either is converted.
  const uint32_t rounds = (chunks + nthr - 1) / nthr;
  for (uint32_t rnd = 0; rnd < rounds; rnd += 2) {
    uint32_t w[2][8];
    uint32_t t[2] = {0, 0}, h[2] = {0, 0}, c[2] = {0, 0};
    bool active[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const uint32_t i = (rnd + u) * nthr + tid;
      active[u] = (rnd + u) < rounds && i < chunks;
#pragma unroll
      for (int k = 0; k < 8; ++k) w[u][k] = 0;
      if (active[u]) {
        const uint32_t row = i / cpr;
        c[u] = i - row * cpr;
        it.decode(row, t[u], h[u]);
        const char* sp = src + s_base + (int64_t)t[u] * p.src.token_stride + (int64_t)h[u] * p.src.head_stride + (c[u] << 5);
        const int4 a = ld_nc_16(sp);
        const int4 b = ld_nc_16(sp + 16);
        w[u][0] = a.x; w[u][1] = a.y; w[u][2] = a.z; w[u][3] = a.w;
        w[u][4] = b.x; w[u][5] = b.y; w[u][6] = b.z; w[u][7] = b.w;
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float amax = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        amax = fmaxf(amax, fabsf(bf16lo(w[u][k])));
        amax = fmaxf(amax, fabsf(bf16hi(w[u][k])));
      }
      // the partner lane holds the other half of the 32-value group (all lanes take part in the shuffle)
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      const uint32_t e = ue8m0_from_amax(amax);
      const float inv = __uint_as_float((254u - e) << 23);  // 1 / 2^(e-127)
      if (active[u]) {
        int4 q;
        q.x = pack_e4m3x4(bf16lo(w[u][0]) * inv, bf16hi(w[u][0]) * inv, bf16lo(w[u][1]) * inv, bf16hi(w[u][1]) * inv);
        q.y = pack_e4m3x4(bf16lo(w[u][2]) * inv, bf16hi(w[u][2]) * inv, bf16lo(w[u][3]) * inv, bf16hi(w[u][3]) * inv);
        q.z = pack_e4m3x4(bf16lo(w[u][4]) * inv, bf16hi(w[u][4]) * inv, bf16lo(w[u][5]) * inv, bf16hi(w[u][5]) * inv);
        q.w = pack_e4m3x4(bf16lo(w[u][6]) * inv, bf16hi(w[u][6]) * inv, bf16lo(w[u][7]) * inv, bf16hi(w[u][7]) * inv);
        if (staged) {
          // chunk i of the tile in destination order sits at byte 16 i of the buffer: rows of a head are adjacent
          *reinterpret_cast<int4*>(stage + (((rnd + u) * nthr + tid) << 4)) = q;
        } else {
          st_16(dst + d_base + (int64_t)t[u] * p.dst.token_stride + (int64_t)h[u] * p.dst.head_stride + (c[u] << 4), q);
        }
      }
      if (wide_scales) {
        // eight neighbouring lanes hold 128 values of one row = four scales: one 4-byte store instead of
        // four 1-byte stores (over NVLink every store is a packet of its own, whatever its size)
        const uint32_t lane = tid & 31u;
        const uint32_t e1 = __shfl_sync(0xffffffffu, e, (lane & ~7u) + 2u);
        const uint32_t e2 = __shfl_sync(0xffffffffu, e, (lane & ~7u) + 4u);
        const uint32_t e3 = __shfl_sync(0xffffffffu, e, (lane & ~7u) + 6u);
        if (active[u] && (lane & 7u) == 0u) {
          const uint32_t packed = e | (e1 << 8) | (e2 << 16) | (e3 << 24);
          if (staged) {
            // chunk i of the tile (destination order) owns scale byte i / 2; lanes with lane % 8 == 0 hold a
            // multiple of eight, so the word is 4-byte aligned whatever the row length
            *reinterpret_cast<uint32_t*>(stage + kStagePayload + (((rnd + u) * nthr + tid) >> 1)) = packed;
          } else {
            *reinterpret_cast<uint32_t*>(dst + sc_base + (int64_t)t[u] * p.dst.scale_token_stride +
                                         (int64_t)h[u] * p.dst.scale_head_stride + (c[u] >> 1)) = packed;
          }
        }
      } else if (active[u] && (c[u] & 1u) == 0u) {
        dst[sc_base + (int64_t)t[u] * p.dst.scale_token_stride + (int64_t)h[u] * p.dst.scale_head_stride +
            (c[u] >> 1)] = static_cast<char>(e);
      }
    }
  }
  if (staged) {
    __syncwarp();
    fence_proxy_async();          // the buffer was written through the generic proxy, the copies read it through the async one
    if (tid == 0) {
      for (uint32_t h = 0; h < it.nh; ++h) {
        bulk_store_flat(dst + d_base + (int64_t)h * p.dst.head_stride, smem_u32(stage + h * run_bytes), run_bytes);
        bulk_store_flat(dst + sc_base + (int64_t)h * p.dst.scale_head_stride, smem_u32(stage + kStagePayload + h * sc_run),
                        sc_run);
      }
      bulk_commit();
    }
    __syncwarp();
  }
}

// e4m3 rows + UE8M0 scales -> bf16 rows.  One thread expands 16 values (16 B in, 32 B out).
__device__ __forceinline__ void simt_dequant_tile(const KvtAttnLaunch& p, const TileInfo& ti, uint32_t kv,
                                       const char* __restrict__ src, char* __restrict__ dst, uint32_t tid,
                                       uint32_t nthr) {
  const uint32_t cpr = p.src.head_bytes >> 4;
  RowIter it;
  it.ntok = ti.copy_hi - ti.copy_lo;
  it.nh = p.n_heads;
  it.token_inner = p.dst.token_stride < p.dst.head_stride;
  const uint32_t chunks = it.ntok * it.nh * cpr;
  const uint32_t slot_s = ti.s_slot0 + (ti.copy_lo - ti.tok_lo);
  const uint32_t slot_d = ti.d_slot0 + (ti.copy_lo - ti.tok_lo);
  const int64_t s_blk = (int64_t)ti.sblk * p.src.block_stride;
  const int64_t s_base = s_blk + (int64_t)kv * p.src.kv_stride + (int64_t)slot_s * p.src.token_stride +
                         (int64_t)p.src_head0 * p.src.head_stride;
  const int64_t sc_base = s_blk + p.src.scale_base + (int64_t)kv * p.src.scale_kv_stride +
                          (int64_t)slot_s * p.src.scale_token_stride +
                          (int64_t)p.src_head0 * p.src.scale_head_stride;
  const int64_t d_base = (int64_t)ti.dblk * p.dst.block_stride + (int64_t)kv * p.dst.kv_stride +
                         (int64_t)slot_d * p.dst.token_stride + (int64_t)p.dst_head0 * p.dst.head_stride;
  for (uint32_t i = tid; i < chunks; i += nthr) {
    const uint32_t row = i / cpr;
    const uint32_t c = i - row * cpr;
    uint32_t t, h;
    it.decode(row, t, h);
    const int4 q = ld_nc_16(src + s_base + (int64_t)t * p.src.token_stride + (int64_t)h * p.src.head_stride + (c << 4));
    const uint32_t e = static_cast<uint8_t>(
        src[sc_base + (int64_t)t * p.src.scale_token_stride + (int64_t)h * p.src.scale_head_stride + (c >> 1)]);
    const float s = scale_from_ue8m0(e);
    const uint32_t qw[4] = {(uint32_t)q.x, (uint32_t)q.y, (uint32_t)q.z, (uint32_t)q.w};
    uint32_t o[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __half2_raw h01 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(qw[k] & 0xffffu), __NV_E4M3);
      const __half2_raw h23 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(qw[k] >> 16), __NV_E4M3);
      const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01));
      const float2 f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
      const __nv_bfloat162 b01 = __floats2bfloat162_rn(f01.x * s, f01.y * s);
      const __nv_bfloat162 b23 = __floats2bfloat162_rn(f23.x * s, f23.y * s);
      o[2 * k] = *reinterpret_cast<const uint32_t*>(&b01);
      o[2 * k + 1] = *reinterpret_cast<const uint32_t*>(&b23);
    }
    char* dp = dst + d_base + (int64_t)t * p.dst.token_stride + (int64_t)h * p.dst.head_stride + (c << 5);
    st_16(dp, make_int4(o[0], o[1], o[2], o[3]));
    st_16(dp + 16, make_int4(o[4], o[5], o[6], o[7]));
  }
}

// Zero destination slots [copy_hi, zero_hi) of a tile (tail pad of the last block).
__device__ __forceinline__ void simt_zero_tail(const KvtAttnLaunch& p, const TileInfo& ti, uint32_t kv,
                                               char* __restrict__ dst, uint32_t tid, uint32_t nthr) {
  const uint32_t ntok = ti.zero_hi - ti.copy_hi;
  if (ntok == 0) return;
  const uint32_t cpr = p.dst.head_bytes >> 4;
  RowIter it;
  it.ntok = ntok;
  it.nh = p.n_heads;
  it.token_inner = p.dst.token_stride < p.dst.head_stride;
  const uint32_t chunks = ntok * it.nh * cpr;
  const int64_t d_base = (int64_t)ti.dblk * p.dst.block_stride + (int64_t)kv * p.dst.kv_stride +
                         (int64_t)(ti.d_slot0 + (ti.copy_hi - ti.tok_lo)) * p.dst.token_stride +
                         (int64_t)p.dst_head0 * p.dst.head_stride;
  for (uint32_t i = tid; i < chunks; i += nthr) {
    const uint32_t row = i / cpr;
    const uint32_t c = i - row * cpr;
    uint32_t t, h;
    it.decode(row, t, h);
    st_16(dst + d_base + (int64_t)t * p.dst.token_stride + (int64_t)h * p.dst.head_stride + (c << 4),
          make_int4(0, 0, 0, 0));
  }
}

// Who owns a tile.  GROUP = 1: a warp (many tiles in flight per SM, nobody waits at tile boundaries;
// best for long launches into device memory).  GROUP = 4: four warps share a tile, so that a
// launch with few tiles still spreads over every SM and a whole tile is in flight at once (short
// launches: one layer of a request).  GROUP = 0: the whole CTA (longer contiguous write runs, which
// is what a PCIe destination prefers).  The owners of a CTA take consecutive tiles and the launcher
// sizes the grid to the tiles, so that every resident CTA is full of busy warps: a CTA keeps its
// registers until its last warp exits, and half-empty CTAs of one launch would keep the CTAs of
// launches on other streams off the SM.
template <int MODE, bool USE_TMA, int GROUP>
__device__ __forceinline__ void simt_pass(const KvtAttnLaunch& p, uint64_t total, uint32_t per_layer,
                                          unsigned char* stage_base) {
  constexpr uint32_t kGroupThreads = GROUP > 0 ? 32u * GROUP : 0u;
  const uint32_t tid = GROUP > 0 ? (threadIdx.x % kGroupThreads) : threadIdx.x;
  const uint32_t nthr = GROUP > 0 ? kGroupThreads : blockDim.x;
  const uint32_t owners = GROUP > 0 ? (blockDim.x / kGroupThreads) : 1u;
  const uint32_t me = GROUP > 0 ? (threadIdx.x / kGroupThreads) : 0u;
  if (me >= owners) return;   // a block size that is not a multiple of the group: the odd warps sit out
  unsigned char* stage = (GROUP == 1 && MODE == KVT_MODE_BF16_TO_MXFP8 && stage_base != nullptr)
                             ? stage_base + (size_t)me * kStagePerWarp : nullptr;
  for (uint64_t w = (uint64_t)blockIdx.x * owners + me; w < total; w += (uint64_t)gridDim.x * owners) {
    const uint32_t layer = (uint32_t)(w / per_layer);
    const uint32_t rem = (uint32_t)(w - (uint64_t)layer * per_layer);
    const uint32_t kv = rem / p.total_tiles;
    const uint32_t tile = rem - kv * p.total_tiles;
    const TileInfo ti = decode_tile(p, tile);
    if (!ti.ok) {
      if (tid == 0) set_status(p.status, KVT_ERR_BLOCK_RANGE, tile);
      continue;
    }
    const char* src = reinterpret_cast<const char*>(p.src_layers[p.layer_begin + layer]);
    char* dst = reinterpret_cast<char*>(p.dst_layers[p.layer_begin + layer]);
    if (ti.copy_hi > ti.copy_lo) {
      if constexpr (MODE == KVT_MODE_COPY) {
        if (!(USE_TMA && tile_is_full(p, ti))) simt_copy_tile(p, ti, kv, src, dst, tid, nthr);
      } else if constexpr (MODE == KVT_MODE_BF16_TO_MXFP8) {
        simt_quant_tile(p, ti, kv, src, dst, tid, nthr, stage);
      } else {
        simt_dequant_tile(p, ti, kv, src, dst, tid, nthr);
      }
    }
    if (ti.zero_hi > ti.copy_hi) simt_zero_tail(p, ti, kv, dst, tid, nthr);
  }
  if (stage != nullptr) {
    // the bulk stores of the last tile must be complete before this CTA reports the launch done
    if (tid == 0) bulk_wait_all();
    __syncwarp();
    fence_proxy_async();
  }
}

// ---- the kernel ---------------------------------------------------------------------------
template <int MODE, bool USE_TMA>
__global__ void __launch_bounds__(512, 2) kvt_p2d_attn_kernel(const __grid_constant__ KvtAttnLaunch p,
                                                            const uint32_t n_stages, const uint32_t tile_bytes,
                                                            const uint32_t warp_tiles) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t n_layers = p.layer_end - p.layer_begin;
  const uint32_t per_layer = p.total_tiles * p.src.kv_count;
  const uint64_t total = (uint64_t)n_layers * per_layer;

  // Work index w -> (layer, kv, tile).  Consecutive CTAs take consecutive tiles of one layer.
  if constexpr (USE_TMA) {
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)n_stages * tile_bytes);
    if (threadIdx.x == 0) {
      for (uint32_t s = 0; s < n_stages; ++s) mbar_init(smem_u32(&bars[s]), 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      fence_proxy_async();
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // Producer warp.  All 32 lanes decode tiles in parallel (the block-table walk is a chain
      // of dependent loads, so doing it on one thread would serialise ~1 us per tile); lane 0
      // runs the software pipeline: at most n_stages-1 loads in flight, one store behind.
      const uint32_t lane = threadIdx.x;
      // dmap == nullptr: the tile is one contiguous run of the destination, stored by an untiled bulk copy to `flat`
      struct Slot { const void* dmap; char* flat; int c1, c2, c3, c4; };
      Slot slots[kMaxStages];
      uint32_t issued = 0, stored = 0;
      bool failed = false;
      const bool token_inner = p.tile_order != 0u;
      const bool flat_store = p.store_form != 0u;
      const bool hinted = p.cache_hint != 0u;
      const uint64_t pol = hinted ? policy_evict_first() : 0ull;
      auto consume_one = [&]() {
        const uint32_t s = stored % n_stages;
        const uint32_t bar = smem_u32(&bars[s]);
        const uint32_t parity = (stored / n_stages) & 1u;
        const long long t0 = clock64();
        while (!mbar_try_wait(bar, parity)) {
          if (clock64() - t0 > kWaitCycles) {
            failed = true;
            break;
          }
        }
        if (failed) {
          set_status(p.status, KVT_ERR_TMA_TIMEOUT, stored);
          return;
        }
        const uint32_t sm = smem_u32(smem + (size_t)s * tile_bytes);
        if (slots[s].dmap == nullptr) {
          if (hinted) bulk_store_flat_hint(slots[s].flat, sm, tile_bytes, pol);
          else bulk_store_flat(slots[s].flat, sm, tile_bytes);
        } else if (hinted) {
          tma_store_5d_hint(slots[s].dmap, sm, 0, slots[s].c1, slots[s].c2, slots[s].c3, slots[s].c4, pol);
        } else {
          tma_store_5d(slots[s].dmap, sm, 0, slots[s].c1, slots[s].c2, slots[s].c3, slots[s].c4);
        }
        bulk_commit();
        ++stored;
      };
      for (uint64_t batch = 0;; batch += 32) {
        const uint64_t w = blockIdx.x + (batch + lane) * (uint64_t)gridDim.x;
        bool full = false;
        TileInfo ti;
        ti.sblk = ti.dblk = ti.s_slot0 = ti.d_slot0 = 0;
        uint32_t layer = 0, kv = 0;
        if (w < total) {
          layer = (uint32_t)(w / per_layer);
          const uint32_t rem = (uint32_t)(w - (uint64_t)layer * per_layer);
          kv = rem / p.total_tiles;
          ti = decode_tile(p, rem - kv * p.total_tiles);
          full = ti.ok && tile_is_full(p, ti);  // bad tiles are reported by the SIMT pass
        }
        const unsigned any = __ballot_sync(0xffffffffu, w < total);
        unsigned fullmask = __ballot_sync(0xffffffffu, full);
        if (any == 0u) break;
        while (fullmask != 0u) {
          const int j = __ffs(fullmask) - 1;
          fullmask &= fullmask - 1u;
          const uint32_t j_sblk = __shfl_sync(0xffffffffu, ti.sblk, j);
          const uint32_t j_dblk = __shfl_sync(0xffffffffu, ti.dblk, j);
          const uint32_t j_ss = __shfl_sync(0xffffffffu, ti.s_slot0, j);
          const uint32_t j_ds = __shfl_sync(0xffffffffu, ti.d_slot0, j);
          const uint32_t j_layer = __shfl_sync(0xffffffffu, layer, j);
          const uint32_t j_kv = __shfl_sync(0xffffffffu, kv, j);
          if (lane == 0 && !failed) {
            if (n_stages == 1) {
              if (issued > stored) consume_one();
              if (!failed) bulk_wait_read<0>();
            } else if (issued - stored == n_stages - 1) {
              consume_one();
              // the stage refilled below was last read by the store issued one step earlier
              if (!failed) bulk_wait_read<1>();
            }
            if (!failed) {
              const uint32_t s = issued % n_stages;
              const uint32_t bar = smem_u32(&bars[s]);
              const CUtensorMap* smap = reinterpret_cast<const CUtensorMap*>(p.src_maps) + (p.layer_begin + j_layer);
              const CUtensorMap* dmap = reinterpret_cast<const CUtensorMap*>(p.dst_maps) + (p.layer_begin + j_layer);
              mbar_expect_tx(bar, tile_bytes);
              // coordinate order of the maps: {row, head, slot, block, kv}, or {row, slot, head, block, kv} when the
              // tile is kept token-inner (heads outermost in shared memory, the order of an HND destination)
              const int s1 = token_inner ? (int)j_ss : (int)p.src_head0;
              const int s2 = token_inner ? (int)p.src_head0 : (int)j_ss;
              if (hinted) {
                tma_load_5d_hint(smem_u32(smem + (size_t)s * tile_bytes), smap, bar, 0, s1, s2, (int)j_sblk, (int)j_kv, pol);
              } else {
                tma_load_5d(smem_u32(smem + (size_t)s * tile_bytes), smap, bar, 0, s1, s2, (int)j_sblk, (int)j_kv);
              }
              slots[s].dmap = flat_store ? nullptr : dmap;
              slots[s].flat = reinterpret_cast<char*>(p.dst_layers[p.layer_begin + j_layer]) +
                              (int64_t)j_dblk * p.dst.block_stride + (int64_t)j_kv * p.dst.kv_stride +
                              (int64_t)j_ds * p.dst.token_stride + (int64_t)p.dst_head0 * p.dst.head_stride;
              slots[s].c1 = token_inner ? (int)j_ds : (int)p.dst_head0;
              slots[s].c2 = token_inner ? (int)p.dst_head0 : (int)j_ds;
              slots[s].c3 = (int)j_dblk;
              slots[s].c4 = (int)j_kv;
              ++issued;
            }
          }
        }
      }
      if (lane == 0) {
        while (!failed && stored < issued) consume_one();
        bulk_wait_all();
        fence_proxy_async();
      }
      __syncwarp();
    }
  }

  // SIMT pass: everything the TMA pass does not take.
  // without TMA tiles a non-zero tile_bytes says that every warp owns a staging buffer of that size
  unsigned char* stage_base = (!USE_TMA && tile_bytes == kStagePerWarp) ? smem : nullptr;
  if (warp_tiles == 1u) {
    simt_pass<MODE, USE_TMA, 1>(p, total, per_layer, stage_base);
  } else if (warp_tiles == 4u) {
    simt_pass<MODE, USE_TMA, 4>(p, total, per_layer, nullptr);
  } else {
    simt_pass<MODE, USE_TMA, 0>(p, total, per_layer, nullptr);
  }

  // Completion: the last CTA to finish publishes the flag after a system-scope fence, so a
  // reader on the destination GPU or on the host that sees the flag also sees the data.
  if (p.flag != nullptr && p.done_counter != nullptr) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t prev = atomicAdd(p.done_counter, 1u);
      if (prev == gridDim.x - 1) {
        *p.done_counter = 0;  // re-arm for the next launch on this stream
        __threadfence_system();
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p.flag), "l"(p.flag_value) : "memory");
      }
    }
  }
}

struct DriverApi {
  CUresult (*encode_tiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                           const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                           CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
  bool tried = false;
};
DriverApi g_driver;

bool load_driver_api() {
  if (g_driver.tried) return g_driver.encode_tiled != nullptr;
  g_driver.tried = true;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess) {
    g_driver.encode_tiled = reinterpret_cast<decltype(g_driver.encode_tiled)>(fn);
  }
  return g_driver.encode_tiled != nullptr;
}

template <int MODE, bool USE_TMA>
cudaError_t launch_impl(const KvtAttnLaunch& a, int grid, int threads, uint32_t stages, uint32_t tile_bytes,
                        size_t smem, cudaStream_t stream) {
  // BLLM_KVTRANS_SIMT_TILE overrides KvtAttnLaunch::simt_tile: 1 = a warp per tile, 4 = four warps per
  // tile (lower latency of a lone short launch, lower throughput of overlapped ones), 2 = a CTA per tile.
  static const int env_simt = [] {
    const char* v = getenv("BLLM_KVTRANS_SIMT_TILE");
    return v != nullptr ? atoi(v) : 0;
  }();
  const int choice = env_simt != 0 ? env_simt : (int)a.simt_tile;
  uint32_t warp_tiles;
  const uint64_t total = (uint64_t)(a.layer_end - a.layer_begin) * a.total_tiles * a.src.kv_count;
  const uint32_t warps = (uint32_t)(threads / 32);
  if (choice == 2) {
    warp_tiles = 0u;
  } else if (choice == 1 || (choice == 4 && threads % 128 == 0)) {
    warp_tiles = (uint32_t)choice;
  } else {
    // Measured with 80 one-layer launches of 1024 tiles on 8 streams: a warp per tile moves 2884 GB/s
    // through the quantiser, four warps per tile 2046 (every warp of the four walks the block table).
    warp_tiles = 1u;
  }
  if (!USE_TMA && warp_tiles != 0u) {
    const uint64_t owners = warps / warp_tiles;
    const uint64_t need = (total + owners - 1) / owners;
    if ((uint64_t)grid > need) grid = (int)need;
  }
  if (MODE == KVT_MODE_BF16_TO_MXFP8 && !USE_TMA && warp_tiles == 1u) {
    // BLLM_KVTRANS_QUANT_STAGE: 0 = direct 16-byte stores always, 1 = staged bulk stores always; unset =
    // staged for a remote destination (668 against 614 GB/s of link), direct for a local one (2842
    // against 2494 GB/s of source).
    static const int stage_env = [] {
      const char* v = getenv("BLLM_KVTRANS_QUANT_STAGE");
      return v == nullptr ? -1 : atoi(v);
    }();
    if (stage_env > 0 || (stage_env < 0 && a.dst_remote != 0)) {
      tile_bytes = kStagePerWarp;
      smem = (size_t)warps * kStagePerWarp;
    }
  }
  auto kern = kvt_p2d_attn_kernel<MODE, USE_TMA>;
  if (smem > 48 * 1024) {
    // the opt-in is per device and sticky: ask once per device (and again only for a larger size)
    static std::atomic<size_t> granted[kMaxDevices];
    int dev = 0;
    cudaGetDevice(&dev);
    std::atomic<size_t>* slot = dev >= 0 && dev < kMaxDevices ? &granted[dev] : nullptr;
    if (slot == nullptr || slot->load(std::memory_order_relaxed) < smem) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      if (slot != nullptr) slot->store(smem, std::memory_order_relaxed);
    }
  }
  kern<<<grid, threads, smem, stream>>>(a, stages, tile_bytes, warp_tiles);
  return cudaGetLastError();
}

}  // namespace

extern "C" uint32_t kvt_req_tiles(uint32_t seen, uint32_t new_tokens, uint32_t tile_tokens, uint32_t flags,
                                  uint32_t dst_ntpb) {
  if (tile_tokens == 0) return 0;
  uint64_t end_tok = (uint64_t)seen + new_tokens;
  if ((flags & KVT_REQ_PAD_TAIL) && dst_ntpb > 0) end_tok = (end_tok + dst_ntpb - 1) / dst_ntpb * dst_ntpb;
  if (end_tok <= seen && new_tokens == 0) return 0;
  const uint64_t first = seen / tile_tokens;
  const uint64_t last = (end_tok + tile_tokens - 1) / tile_tokens;
  return (uint32_t)(last - first);
}

extern "C" int kvt_encode_tensor_map(void* out, uint64_t base, const KvtLayout* l, uint32_t box_heads,
                                     uint32_t box_tokens) {
  return kvt_encode_tensor_map_ordered(out, base, l, box_heads, box_tokens, 0);
}

extern "C" int kvt_tile_is_flat(const KvtLayout* l, uint32_t n_heads, uint32_t tile_tokens, uint32_t token_inner) {
  const int64_t hb = l->head_bytes;
  if (token_inner) {
    // heads outermost: rows of a head adjacent, heads adjacent (HND pages)
    return l->token_stride == hb && (n_heads == 1 || l->head_stride == (int64_t)tile_tokens * hb) ? 1 : 0;
  }
  // tokens outermost: heads of a token adjacent, tokens adjacent (NHD pages, all heads moved)
  return l->head_stride == hb && (tile_tokens == 1 || l->token_stride == (int64_t)n_heads * hb) ? 1 : 0;
}

extern "C" int kvt_encode_tensor_map_ordered(void* out, uint64_t base, const KvtLayout* l, uint32_t box_heads,
                                             uint32_t box_tokens, uint32_t token_inner) {
  if (!load_driver_api()) return -1;
  if (l->head_bytes % 16 != 0 || (base & 15) != 0) return -2;
  if (l->head_bytes / 4 > 256 || box_heads > 256 || box_tokens > 256) return -3;
  if (box_heads == 0 || box_tokens == 0 || box_heads > l->num_heads || box_tokens > l->ntpb) return -3;
  const int64_t strides[4] = {l->head_stride, l->token_stride, l->block_stride,
                              l->kv_count > 1 ? l->kv_stride : l->block_stride * (int64_t)l->num_blocks};
  for (int i = 0; i < 4; ++i) {
    if (strides[i] <= 0 || (strides[i] % 16) != 0 || strides[i] >= (1ll << 40)) return -4;
  }
  cuuint64_t gdim[5] = {l->head_bytes / 4, l->num_heads, l->ntpb, l->num_blocks, l->kv_count ? l->kv_count : 1};
  cuuint64_t gstr[4] = {(cuuint64_t)strides[0], (cuuint64_t)strides[1], (cuuint64_t)strides[2],
                        (cuuint64_t)strides[3]};
  cuuint32_t box[5] = {l->head_bytes / 4, box_heads, box_tokens, 1, 1};
  if (token_inner) {   // the slot dimension before the head dimension: a tile lands as [head][slot][row]
    gdim[1] = l->ntpb;
    gdim[2] = l->num_heads;
    gstr[0] = (cuuint64_t)strides[1];
    gstr[1] = (cuuint64_t)strides[0];
    box[1] = box_tokens;
    box[2] = box_heads;
  }
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = g_driver.encode_tiled(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_UINT32, 5,
                                     reinterpret_cast<void*>(base), gdim, gstr, box, estr,
                                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return (int)r;
}

extern "C" int kvt_launch_p2d_attn(const KvtAttnLaunch* args, int grid_ctas, int threads, int use_tma,
                                   void* stream_) {
  const KvtAttnLaunch& a = *args;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (a.n_reqs == 0 || a.total_tiles == 0 || a.layer_end <= a.layer_begin) return (int)cudaSuccess;
  if (a.tile_tokens == 0 || a.src.ntpb % a.tile_tokens != 0 || a.dst.ntpb % a.tile_tokens != 0)
    return (int)cudaErrorInvalidValue;
  if (a.src.kv_count != a.dst.kv_count || a.n_heads == 0) return (int)cudaErrorInvalidValue;
  if (a.src_head0 + a.n_heads > a.src.num_heads || a.dst_head0 + a.n_heads > a.dst.num_heads)
    return (int)cudaErrorInvalidValue;
  if (a.mode == KVT_MODE_COPY) {
    if (a.src.head_bytes != a.dst.head_bytes || a.src.head_bytes % 16 != 0) return (int)cudaErrorInvalidValue;
  } else if (a.mode == KVT_MODE_BF16_TO_MXFP8) {
    if (a.src.head_bytes != 2 * a.dst.head_bytes || a.src.head_bytes % 64 != 0) return (int)cudaErrorInvalidValue;
  } else if (a.mode == KVT_MODE_MXFP8_TO_BF16) {
    if (2 * a.src.head_bytes != a.dst.head_bytes || a.dst.head_bytes % 64 != 0) return (int)cudaErrorInvalidValue;
  } else {
    return (int)cudaErrorInvalidValue;
  }
  int dev = 0;
  cudaGetDevice(&dev);
  static std::atomic<int> sm_cache[kMaxDevices];
  int sms = dev >= 0 && dev < kMaxDevices ? sm_cache[dev].load(std::memory_order_relaxed) : 0;
  if (sms == 0) {
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (dev >= 0 && dev < kMaxDevices) sm_cache[dev].store(sms, std::memory_order_relaxed);
  }
  // Default: four CTAs per SM.  Many small CTAs, each with one tile in flight, measured faster
  // than one deep software pipeline per SM, and they let launches on different streams share SMs.
  int grid = grid_ctas > 0 ? grid_ctas : 4 * sms;
  const uint64_t total = (uint64_t)(a.layer_end - a.layer_begin) * a.total_tiles * a.src.kv_count;
  if ((uint64_t)grid > total) grid = (int)total;
  if (threads <= 0) threads = use_tma ? 128 : 512;
  if (threads > 512) threads = 512;
  threads = (threads + 31) / 32 * 32;
  const bool tma = use_tma && a.mode == KVT_MODE_COPY && a.src_maps != nullptr && a.dst_maps != nullptr;
  if (tma) {
    const uint32_t tile_bytes = a.src.head_bytes * a.n_heads * a.tile_tokens;
    if (tile_bytes % 128 != 0 || tile_bytes > kSmemBudget) return (int)cudaErrorInvalidValue;
    // the shared-memory budget of an SM is split among the CTAs meant to live on it together
    const uint32_t ctas_per_sm = sms > 0 ? (uint32_t)((grid + sms - 1) / sms) : 1u;
    uint32_t stages = kSmemBudget / (ctas_per_sm > 0 ? ctas_per_sm : 1u) / tile_bytes;
    if (stages > (uint32_t)kMaxStages) stages = kMaxStages;
    if (stages < 1) stages = 1;
    // BLLM_KVTRANS_TMA_STAGES caps the pipeline depth: fewer stages = less shared memory per
    // CTA, so that CTAs of launches on different streams can share an SM.
    static const int env_stages = [] {
      const char* v = getenv("BLLM_KVTRANS_TMA_STAGES");
      return v != nullptr ? atoi(v) : 0;
    }();
    if (env_stages > 0 && stages > (uint32_t)env_stages) stages = (uint32_t)env_stages;
    if (a.tma_stages > 0 && stages > a.tma_stages) stages = a.tma_stages;
    if (a.store_form != 0u && !kvt_tile_is_flat(&a.dst, a.n_heads, a.tile_tokens, a.tile_order)) return (int)cudaErrorInvalidValue;
    const uint64_t per_cta = (total + grid - 1) / grid;
    if (stages > per_cta + 1) stages = (uint32_t)per_cta + 1;
    if (stages < 1) stages = 1;
    const size_t smem = (size_t)stages * tile_bytes + kMaxStages * sizeof(uint64_t);
    return (int)launch_impl<KVT_MODE_COPY, true>(a, grid, threads, stages, tile_bytes, smem, stream);
  }
  switch (a.mode) {
    case KVT_MODE_COPY:
      return (int)launch_impl<KVT_MODE_COPY, false>(a, grid, threads, 0, 0, 0, stream);
    case KVT_MODE_BF16_TO_MXFP8:
      return (int)launch_impl<KVT_MODE_BF16_TO_MXFP8, false>(a, grid, threads, 0, 0, 0, stream);
    default:
      return (int)launch_impl<KVT_MODE_MXFP8_TO_BF16, false>(a, grid, threads, 0, 0, 0, stream);
  }
}
