// Unit decode of the block-table walk, shared by the device kernel (kvt_walk.cu) and the host routine
// that expands ops into byte ranges (plan/walk_plan.cpp): the CPU tests of the expansion exercise the
// very arithmetic the kernel runs.
#pragma once
#include <stdint.h>

#include "kvt_kernels.h"

#if defined(__CUDACC__)
#define KVT_HD __host__ __device__ __forceinline__
#else
#define KVT_HD inline
#endif

// The pieces of one unit: n pieces of len bytes, piece j at src_off + j * src_step / dst_off + j * dst_step.
struct KvtWalkPieces {
  int64_t src_off;
  int64_t dst_off;
  int64_t src_step;
  int64_t dst_step;
  uint32_t len;
  uint32_t n;       // 0: nothing to do (a segment past the end of a short piece)
  uint32_t error;   // 1: a block index fell outside its table
};

// local_unit counts within the op: ((slot * inner_total + inner_index) * segs + segment) for bulk ops,
// (slot * inner_total + inner_index) for the others.
KVT_HD KvtWalkPieces kvt_walk_unit(const KvtWalkOp& op, const uint32_t* pool, uint64_t local_unit) {
  KvtWalkPieces out;
  out.src_off = out.dst_off = out.src_step = out.dst_step = 0;
  out.len = 0;
  out.n = 0;
  out.error = 0;
  uint32_t seg = 0;
  uint32_t inner_idx;
  uint64_t slot;
  if ((local_unit >> 32) == 0) {
    // the usual case: 32-bit divisions (a 64-bit one costs several times as much on the device)
    uint32_t u = (uint32_t)local_unit;
    if (op.flags & KVT_WALK_BULK) {
      seg = u % op.segs;
      u /= op.segs;
    }
    inner_idx = u % op.inner_total;
    slot = (uint64_t)(op.pos_lo / op.run) + u / op.inner_total;
  } else {
    if (op.flags & KVT_WALK_BULK) {
      seg = (uint32_t)(local_unit % op.segs);
      local_unit /= op.segs;
    }
    inner_idx = (uint32_t)(local_unit % op.inner_total);
    slot = op.pos_lo / op.run + local_unit / op.inner_total;
  }
  const uint64_t lo = slot * op.run, hi = lo + op.run;
  const uint32_t p0 = (uint32_t)(lo > op.pos_lo ? lo : op.pos_lo);
  const uint32_t p1 = (uint32_t)(hi < op.pos_hi ? hi : op.pos_hi);
  if (p1 <= p0) return out;
  int64_t s_in = 0, d_in = 0;
  for (int k = (int)op.n_inner - 1; k >= 0; --k) {
    const uint32_t c = op.inner[k].count;
    const uint32_t i = inner_idx % c;
    inner_idx /= c;
    s_in += (int64_t)i * op.inner[k].src_stride;
    d_in += (int64_t)i * op.inner[k].dst_stride;
  }
  const bool zero = (op.flags & KVT_WALK_ZERO) != 0;
  if (!zero) {
    const uint32_t bi = p0 / op.src_per_block;
    if (bi >= op.n_src) {
      out.error = 1;
      return out;
    }
    const uint32_t q = p0 - bi * op.src_per_block;
    out.src_off = (int64_t)pool[op.src_tbl + bi] * op.src_block_stride + (int64_t)(q / op.src_per_kb) * op.src_kb_stride +
                  (int64_t)(q % op.src_per_kb) * op.src_pos_stride + op.src_add + s_in;
  }
  {
    const uint32_t bi = p0 / op.dst_per_block;
    if (bi >= op.n_dst) {
      out.error = 1;
      return out;
    }
    const uint32_t q = p0 - bi * op.dst_per_block;
    out.dst_off = (int64_t)pool[op.dst_tbl + bi] * op.dst_block_stride + (int64_t)(q / op.dst_per_kb) * op.dst_kb_stride +
                  (int64_t)(q % op.dst_per_kb) * op.dst_pos_stride + op.dst_add + d_in;
  }
  const uint32_t n = p1 - p0;
  if (op.flags & KVT_WALK_CONTIG) {
    uint64_t piece = (uint64_t)n * op.len;
    if (op.flags & KVT_WALK_BULK) {
      // the piece in op.segs segments of (nearly) one size, each a multiple of 16 bytes and at most KVT_WALK_SEG:
      // a 41984-byte page is six segments of about 7 KiB, not five of 8 KiB and a 1 KiB tail that would hold a
      // pipeline stage for a fraction of the bytes
      uint64_t seg_len;
      if ((piece >> 32) == 0) seg_len = (((uint32_t)piece + op.segs - 1) / op.segs + 15u) & ~15u;
      else seg_len = ((piece + op.segs - 1) / op.segs + 15u) & ~(uint64_t)15u;
      const uint64_t off = (uint64_t)seg * seg_len;
      if (off >= piece) return out;
      out.src_off += (int64_t)off;
      out.dst_off += (int64_t)off;
      piece = piece - off < seg_len ? piece - off : seg_len;
    }
    out.len = (uint32_t)piece;
    out.n = 1;
  } else {
    out.len = op.len;
    out.n = n;
    out.src_step = op.src_pos_stride;
    out.dst_step = op.dst_pos_stride;
  }
  return out;
}

// Units of an op in its class.
KVT_HD uint64_t kvt_walk_units(const KvtWalkOp& op) {
  if (op.pos_hi <= op.pos_lo) return 0;
  const uint64_t slots = ((uint64_t)op.pos_hi + op.run - 1) / op.run - op.pos_lo / op.run;
  return slots * op.inner_total * ((op.flags & KVT_WALK_BULK) ? op.segs : 1u);
}
