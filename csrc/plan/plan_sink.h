// Internal to the planner's translation units: the output side of the walkers.
#pragma once
#include <initializer_list>
#include <limits>
#include <stdexcept>

#include "plan/planner.h"

namespace kvx {
namespace plan_detail {

// Output of the walkers for one cache tensor: a bounds-checked appender of byte ranges, or a recorder of
// walk ops (PlanOut::walk) for the device.
struct Sink {
  std::vector<IpcBlock>* out;   // byte-range mode
  PlanOut* po;                  // op mode when po->walk != nullptr
  size_t src_cap;
  size_t dst_cap;
  size_t src_scale;  // 2 when lengths are fp8 bytes of a bf16 source
  size_t tensor;

  bool ops() const { return po != nullptr && po->walk != nullptr; }

  void put(size_t s, size_t d, size_t len) {
    const bool scale_bad = src_scale == 0 || len > std::numeric_limits<size_t>::max() / src_scale;
    const size_t eff = scale_bad ? std::numeric_limits<size_t>::max() : len * src_scale;
    const bool src_bad = len == 0 || scale_bad || s > src_cap || eff > src_cap - s;
    const bool dst_bad = len == 0 || d > dst_cap || len > dst_cap - d;
    if (src_bad || dst_bad) {
      LOG(ERROR) << "KVT GPU buffer range validation failed,copy_path=parse_block_generation,layer_idx=0"
                 << ",tensor_idx=" << tensor << ",block_idx=" << out->size()
                 << ",offset_kind=" << (src_bad ? "src" : "dst") << ",src_offset=" << s << ",dst_offset=" << d
                 << ",length=" << len << ",length_scale=" << (src_bad ? src_scale : 1)
                 << ",effective_length=" << (src_bad ? eff : len)
                 << ",capacity=" << (src_bad ? src_cap : dst_cap);
      throw std::out_of_range("KVT GPU buffer range validation failed");
    }
    out->emplace_back(s, d, len);
  }

  // ---- op mode -------------------------------------------------------------------------------------
  // Pool offset of a block table of the request being planned (copied into the pool the first time).
  uint32_t table(const std::vector<uint32_t>& v) {
    for (const auto& t : po->tables)
      if (t.first == v.data()) return t.second;
    const uint32_t off = static_cast<uint32_t>(po->walk->pool.size());
    po->walk->pool.insert(po->walk->pool.end(), v.begin(), v.end());
    po->tables.emplace_back(v.data(), off);
    return off;
  }

  struct Side {
    const std::vector<uint32_t>* blocks;
    uint32_t per_block, per_kb;
    size_t block_stride, kb_stride, pos_stride, add;
  };
  struct Loop {
    uint32_t count;
    size_t src_stride, dst_stride;
  };

  // One op over positions [lo, hi); `src == nullptr` makes it a zero fill of the destination pieces.
  void op(const Side* src, const Side& dst, uint32_t lo, uint32_t hi, size_t len, std::initializer_list<Loop> loops) {
    if (hi <= lo || len == 0) return;
    RTASSERT(!po->walk->ops.empty() || po->walk->pool.size() < (1u << 31));
    RTASSERT(src_scale == 1);   // the unscaled cast belongs to the host-staged transports
    KvtWalkOp o{};
    if (src != nullptr) {
      o.src_tbl = table(*src->blocks);
      o.n_src = static_cast<uint32_t>(src->blocks->size());
      o.src_per_block = src->per_block;
      o.src_per_kb = src->per_kb;
      o.src_block_stride = static_cast<int64_t>(src->block_stride);
      o.src_kb_stride = static_cast<int64_t>(src->kb_stride);
      o.src_pos_stride = static_cast<int64_t>(src->pos_stride);
      o.src_add = static_cast<int64_t>(src->add);
    } else {
      o.flags |= KVT_WALK_ZERO;
      o.src_per_block = o.src_per_kb = 1;
    }
    o.dst_tbl = table(*dst.blocks);
    o.n_dst = static_cast<uint32_t>(dst.blocks->size());
    o.dst_per_block = dst.per_block;
    o.dst_per_kb = dst.per_kb;
    o.dst_block_stride = static_cast<int64_t>(dst.block_stride);
    o.dst_kb_stride = static_cast<int64_t>(dst.kb_stride);
    o.dst_pos_stride = static_cast<int64_t>(dst.pos_stride);
    o.dst_add = static_cast<int64_t>(dst.add);
    o.pos_lo = lo;
    o.pos_hi = hi;
    RTASSERT(len <= 0xffffffffull);
    o.len = static_cast<uint32_t>(len);
    o.tensor = static_cast<uint32_t>(tensor);
    RTASSERT(loops.size() <= KVT_WALK_MAX_INNER);
    size_t per_pos = len;
    for (const Loop& l : loops) {
      if (l.count == 0) return;
      if (l.count == 1) continue;
      o.inner[o.n_inner].count = l.count;
      o.inner[o.n_inner].src_stride = static_cast<int64_t>(l.src_stride);
      o.inner[o.n_inner].dst_stride = static_cast<int64_t>(l.dst_stride);
      ++o.n_inner;
      per_pos *= l.count;
    }
    po->walk->bytes += static_cast<uint64_t>(hi - lo) * per_pos;
    po->walk->ops.push_back(o);
  }
};

inline size_t layer_capacity(const WorkerInfo& w, size_t t, const char* side) {
  if (t >= w.block_sizes.size() || w.layer_num_blocks == 0) {
    LOG(ERROR) << "KVT parse block capacity metadata mismatch,side=" << side << ",cache_idx=" << t
               << ",block_size_count=" << w.block_sizes.size() << ",layer_num_blocks=" << w.layer_num_blocks;
    throw std::out_of_range("KVT parse block capacity metadata mismatch");
  }
  const size_t bs = w.block_sizes[t];
  if (bs > std::numeric_limits<size_t>::max() / w.layer_num_blocks) {
    throw std::overflow_error("KVT parse block capacity overflow");
  }
  return bs * w.layer_num_blocks;
}

inline Sink make_sink(const PlanEnv& env, PlanOut& po, size_t t) {
  std::vector<IpcBlock>* v = nullptr;
  if (po.blocks != nullptr) {
    if (po.blocks->size() <= t) po.blocks->resize(t + 1);
    v = &(*po.blocks)[t];
  }
  return Sink{v, &po, layer_capacity(*env.src, t, "source"), layer_capacity(*env.dst, t, "destination"),
              env.cast_bf16_to_fp8 ? size_t{2} : size_t{1}, t};
}

inline size_t at(const std::vector<uint32_t>& v, size_t i) {
  if (i >= v.size()) throw std::out_of_range("block index beyond the request's block table");
  return v[i];
}

inline const std::vector<uint32_t>& group(const BlockIds& ids, size_t g) {
  if (g >= ids.size()) throw std::out_of_range("block group beyond the request's groups");
  return ids[g];
}

// Pages [first, first + count) of one block group, one piece per page and inner iteration.
inline void page_op(Sink& k, const std::vector<uint32_t>& sb, const std::vector<uint32_t>& db, size_t s_bs, size_t d_bs,
             size_t s_add, size_t d_add, size_t len, std::initializer_list<Sink::Loop> loops) {
  const Sink::Side s{&sb, 1, 1, s_bs, 0, 0, s_add}, d{&db, 1, 1, d_bs, 0, 0, d_add};
  k.op(&s, d, 0, static_cast<uint32_t>(sb.size()), len, loops);
}

}  // namespace plan_detail
}  // namespace kvx
