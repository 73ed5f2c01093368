// Host side of the block-table walk: completing the ops the planner recorded (unit bookkeeping, class,
// order) and expanding them into byte ranges with the kernel's own unit decode.
#include <algorithm>
#include <numeric>
#include <stdexcept>

#include "kernels/kvt_walk.h"
#include "plan/planner.h"

namespace {

bool aligned16(int64_t v) { return (v & 15) == 0; }

bool finalize_one(KvtWalkOp& op) {
  if (op.src_per_kb == 0 || op.dst_per_kb == 0 || op.src_per_block == 0 || op.dst_per_block == 0) return false;
  if (op.src_per_block % op.src_per_kb != 0 || op.dst_per_block % op.dst_per_kb != 0) return false;
  if (op.n_inner > KVT_WALK_MAX_INNER || op.len == 0) return false;
  const bool zero = (op.flags & KVT_WALK_ZERO) != 0;
  op.run = zero ? op.dst_per_kb : std::gcd(op.src_per_kb, op.dst_per_kb);
  if (op.run == 0) return false;
  uint64_t total = 1;
  for (uint32_t k = 0; k < op.n_inner; ++k) {
    if (op.inner[k].count == 0) return false;
    total *= op.inner[k].count;
  }
  if (total > 0xffffffffull) return false;
  op.inner_total = static_cast<uint32_t>(total);
  op.flags &= ~(KVT_WALK_BULK | KVT_WALK_CONTIG);
  const bool contig = op.run == 1 || (op.dst_pos_stride == static_cast<int64_t>(op.len) &&
                                      (zero || op.src_pos_stride == static_cast<int64_t>(op.len)));
  if (contig) op.flags |= KVT_WALK_CONTIG;
  op.segs = 1;
  const uint64_t piece = contig ? static_cast<uint64_t>(op.run) * op.len : op.len;
  if (piece > 0xffffffffull) return false;
  // Bulk asks whole 16-byte words of every row, not only of the unit: an op whose rows are not (132-byte indexer
  // keys: the 64-row page is 8448 bytes, a multiple of 16) would qualify unit by unit, but measured on the MLA
  // shape it is better left to the SIMT warps, which otherwise idle beside the one warp that drives the bulk
  // pipeline (2317 against 2152 GB/s end to end with those pages moved to the pipeline).
  bool al = aligned16(op.len) && aligned16(op.src_block_stride) && aligned16(op.dst_block_stride) &&
            aligned16(op.src_kb_stride) && aligned16(op.dst_kb_stride) && aligned16(op.src_pos_stride) &&
            aligned16(op.dst_pos_stride) && aligned16(op.src_add) && aligned16(op.dst_add);
  for (uint32_t k = 0; k < op.n_inner; ++k) al = al && aligned16(op.inner[k].src_stride) && aligned16(op.inner[k].dst_stride);
  if (contig && !zero && al && piece >= 2048) {
    op.flags |= KVT_WALK_BULK;
    op.segs = static_cast<uint32_t>((piece + KVT_WALK_SEG - 1) / KVT_WALK_SEG);
  }
  return true;
}

}  // namespace

extern "C" int kvt_walk_finalize(KvtWalkOp* ops, uint32_t n_ops, KvtWalkCounts* counts) {
  for (uint32_t i = 0; i < n_ops; ++i)
    if (!finalize_one(ops[i])) return -1;
  auto cls = [](const KvtWalkOp& o) { return (o.flags & KVT_WALK_ZERO) ? 2 : ((o.flags & KVT_WALK_BULK) ? 0 : 1); };
  std::stable_sort(ops, ops + n_ops, [&](const KvtWalkOp& a, const KvtWalkOp& b) { return cls(a) < cls(b); });
  KvtWalkCounts c{};
  for (uint32_t i = 0; i < n_ops; ++i) {
    const int k = cls(ops[i]);
    uint64_t& acc = k == 0 ? c.bulk_units : (k == 1 ? c.simt_units : c.zero_units);
    (k == 0 ? c.n_bulk : (k == 1 ? c.n_simt : c.n_zero)) += 1;
    ops[i].first_unit = acc;
    acc += kvt_walk_units(ops[i]);
  }
  *counts = c;
  return static_cast<int>(c.n_bulk);
}

namespace kvx {

void WalkPlan::finalize(uint32_t src_num_blocks, uint32_t dst_num_blocks) {
  n_bulk = n_simt = n_zero = 0;
  bulk_units = simt_units = zero_units = 0;
  if (ops.empty()) return;
  // every table entry an op can reach must name a block of its cache: the kernel then needs no per-piece check
  // of the block id, only of the index into the table
  for (const KvtWalkOp& op : ops) {
    if (!(op.flags & KVT_WALK_ZERO)) {
      if (static_cast<size_t>(op.src_tbl) + op.n_src > pool.size()) throw std::out_of_range("walk op: source table beyond the pool");
      for (uint32_t i = 0; i < op.n_src; ++i)
        if (pool[op.src_tbl + i] >= src_num_blocks) throw std::out_of_range("walk op: source block id beyond the cache");
    }
    if (static_cast<size_t>(op.dst_tbl) + op.n_dst > pool.size()) throw std::out_of_range("walk op: destination table beyond the pool");
    for (uint32_t i = 0; i < op.n_dst; ++i)
      if (pool[op.dst_tbl + i] >= dst_num_blocks) throw std::out_of_range("walk op: destination block id beyond the cache");
  }
  KvtWalkCounts c{};
  if (kvt_walk_finalize(ops.data(), static_cast<uint32_t>(ops.size()), &c) < 0)
    throw std::invalid_argument("walk op with unusable geometry");
  n_bulk = c.n_bulk;
  n_simt = c.n_simt;
  n_zero = c.n_zero;
  bulk_units = c.bulk_units;
  simt_units = c.simt_units;
  zero_units = c.zero_units;
}

std::vector<WalkPiece> expand_walk_plan(const WalkPlan& plan, const std::vector<uint64_t>& src_caps,
                                        const std::vector<uint64_t>& dst_caps) {
  std::vector<WalkPiece> out;
  for (const KvtWalkOp& op : plan.ops) {
    const uint64_t units = kvt_walk_units(op);
    const bool zero = (op.flags & KVT_WALK_ZERO) != 0;
    if (op.tensor >= src_caps.size() || op.tensor >= dst_caps.size()) throw std::out_of_range("walk op: tensor index");
    for (uint64_t u = 0; u < units; ++u) {
      const KvtWalkPieces p = kvt_walk_unit(op, plan.pool.data(), u);
      if (p.error != 0) throw std::out_of_range("walk op: block index beyond the request's table");
      for (uint32_t j = 0; j < p.n; ++j) {
        const int64_t s = p.src_off + static_cast<int64_t>(j) * p.src_step, d = p.dst_off + static_cast<int64_t>(j) * p.dst_step;
        if (d < 0 || static_cast<uint64_t>(d) + p.len > dst_caps[op.tensor] ||
            (!zero && (s < 0 || static_cast<uint64_t>(s) + p.len > src_caps[op.tensor])))
          throw std::out_of_range("walk op: piece beyond the tensor");
        out.push_back(WalkPiece{op.tensor, zero, zero ? 0 : static_cast<uint64_t>(s), static_cast<uint64_t>(d), p.len});
      }
    }
  }
  return out;
}

}  // namespace kvx
