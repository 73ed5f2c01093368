#include "plan/device_plan.h"

#include <cstring>
#include <numeric>

namespace kvx {

static int heads_of(const WorkerInfo& w) {
  if (w.num_kv_heads > 0 && static_cast<uint32_t>(w.num_kv_heads) >= w.engine_tp_size)
    return w.num_kv_heads / static_cast<int>(w.engine_tp_size);
  return w.num_kv_heads > 0 ? 1 : 0;
}

bool attn_layout_from_worker(const WorkerInfo& w, int shape, bool mx, uint32_t head_bytes_hint, KvtLayout* out) {
  if (w.token_sizes.size() != 1 || w.block_sizes.size() != 1) return false;
  if (shape != RAGGED_FLASH_CACHE_SHAPE && shape != FLASH_CACHE_SHAPE && shape != FLASHINFER_CACHE_SHAPE) return false;
  const size_t tok = w.token_sizes[0], bs = w.block_sizes[0];
  if (tok == 0 || bs % tok != 0) return false;
  const uint32_t T = static_cast<uint32_t>(bs / tok);
  // token bytes = 2 * heads * (head_bytes [+ head_bytes/32 scale bytes])
  uint32_t H = 0, hb = 0;
  const int ext_heads = w.ext_int("heads", 0);
  const int known_heads = ext_heads > 0 ? ext_heads : heads_of(w);
  if (head_bytes_hint > 0) {
    hb = head_bytes_hint;
    const size_t per_head = mx ? hb + hb / 32 : hb;
    if (tok % (2 * per_head) != 0) return false;
    H = static_cast<uint32_t>(tok / (2 * per_head));
  } else if (known_heads > 0) {
    H = static_cast<uint32_t>(known_heads);
    if (tok % (2 * H) != 0) return false;
    const size_t per_head = tok / (2 * H);
    hb = static_cast<uint32_t>(mx ? per_head * 32 / 33 : per_head);
    if (mx && hb + hb / 32 != per_head) return false;
  } else {
    return false;
  }
  if (H == 0 || hb == 0 || hb % 16 != 0) return false;
  KvtLayout l{};
  l.ntpb = T;
  l.num_heads = H;
  l.head_bytes = hb;
  l.num_blocks = w.layer_num_blocks;
  l.kv_count = 2;
  const int64_t Tl = T, Hl = H, hbl = hb, B = w.layer_num_blocks;
  const int64_t sb = mx ? hb / 32 : 0;
  const int64_t payload = 2 * Tl * Hl * hbl;
  switch (shape) {
    case FLASH_CACHE_SHAPE:
      if (mx) return false;  // K and V live in different halves of the tensor: no per-block scale region
      l.block_stride = Tl * Hl * hbl;
      l.kv_stride = B * Tl * Hl * hbl;
      l.token_stride = Hl * hbl;
      l.head_stride = hbl;
      break;
    case RAGGED_FLASH_CACHE_SHAPE:
      if (mx) return false;
      l.block_stride = Tl * 2 * Hl * hbl;
      l.kv_stride = Hl * hbl;
      l.token_stride = 2 * Hl * hbl;
      l.head_stride = hbl;
      break;
    default:  // FLASHINFER HND
      l.block_stride = static_cast<int64_t>(bs);
      l.kv_stride = Hl * Tl * hbl;
      l.token_stride = hbl;
      l.head_stride = Tl * hbl;
      if (mx) {
        l.scale_base = payload;
        l.scale_kv_stride = Hl * Tl * sb;
        l.scale_token_stride = sb;
        l.scale_head_stride = Tl * sb;
      }
      break;
  }
  *out = l;
  return true;
}

bool device_attn_params(const PlanEnv& env, TPKind kind, int src_shape, int dst_shape, bool dst_mx,
                        DeviceAttnParams* out, std::string* why) {
  auto fail = [&](const char* msg) {
    if (why != nullptr) *why = msg;
    return false;
  };
  DeviceAttnParams p{};
  if (!attn_layout_from_worker(*env.src, src_shape, false, 0, &p.src)) return fail("source layout not describable");
  const uint32_t dst_hb = dst_mx ? p.src.head_bytes / 2 : p.src.head_bytes;
  if (!attn_layout_from_worker(*env.dst, dst_shape, dst_mx, dst_hb, &p.dst)) return fail("destination layout not describable");
  p.mode = dst_mx ? KVT_MODE_BF16_TO_MXFP8 : KVT_MODE_COPY;
  p.tile_tokens = std::gcd(p.src.ntpb, p.dst.ntpb);
  p.skip = false;
  const uint32_t Hs = p.src.num_heads, Hd = p.dst.num_heads;
  switch (kind) {
    case TPKind::PEQD:
      if (Hs != Hd) {
        // replicated cache sent by rank 0 only (same token size although TP differs)
        return fail("head counts differ for an equal-TP pair");
      }
      p.src_head0 = p.dst_head0 = 0;
      p.n_heads = Hs;
      break;
    case TPKind::PGTD: {
      if (!env.valid_ranks[env.src->worker_tp_rank]) {
        p.skip = true;
        break;
      }
      const uint32_t g_n = static_cast<uint32_t>(env.valid_ranks.count()) / env.dst->engine_tp_size;
      if (g_n == 0 || Hd != Hs * g_n) return fail("P>D head counts do not tile the destination");
      p.src_head0 = 0;
      p.dst_head0 = (env.kvt_tp_rank % g_n) * Hs;
      p.n_heads = Hs;
      break;
    }
    case TPKind::PLTD: {
      if (Hd == 0 || Hs % Hd != 0) return fail("P<D head counts do not tile the source");
      const uint32_t g_n = Hs / Hd;  // distinct head slices of this prefill rank
      const uint32_t fan = env.dst->engine_tp_size / env.src->engine_tp_size;
      if (fan == 0 || fan % g_n != 0) return fail("P<D fan-out does not match the head split");
      const uint32_t replicas = fan / g_n;
      const uint32_t g_off = ((env.dst->worker_tp_rank % fan) / replicas) % g_n;
      p.src_head0 = g_off * Hd;
      p.dst_head0 = 0;
      p.n_heads = Hd;
      break;
    }
    default:
      return fail("unknown TP relation");
  }
  *out = p;
  return true;
}

PackedPlan pack_device_plan(const std::vector<const ReqSendTask*>& tasks, size_t group, uint32_t tile_tokens,
                            uint32_t dst_ntpb, bool pad_tail) {
  PackedPlan pp;
  std::vector<KvtReqDesc> descs;
  std::vector<uint32_t> pool;
  for (const ReqSendTask* t : tasks) {
    if (group >= t->src_blocks().size() || group >= t->dst_blocks().size())
      throw std::out_of_range("block group beyond the request's groups");
    const auto& sb = t->src_blocks()[group];
    const auto& db = t->dst_blocks()[group];
    KvtReqDesc d{};
    d.seen_tokens = t->seen_tokens;
    d.new_tokens = t->new_tokens;
    d.flags = (pad_tail && t->reach_last_token) ? KVT_REQ_PAD_TAIL : 0u;
    const uint32_t n = kvt_req_tiles(d.seen_tokens, d.new_tokens, tile_tokens, d.flags, dst_ntpb);
    if (n == 0) continue;
    d.src_blk_off = static_cast<uint32_t>(pool.size());
    pool.insert(pool.end(), sb.begin(), sb.end());
    d.dst_blk_off = static_cast<uint32_t>(pool.size());
    pool.insert(pool.end(), db.begin(), db.end());
    d.n_src_blocks = static_cast<uint32_t>(sb.size());
    d.n_dst_blocks = static_cast<uint32_t>(db.size());
    d.first_tile = pp.total_tiles;
    pp.total_tiles += n;
    descs.push_back(d);
  }
  pp.n_reqs = static_cast<uint32_t>(descs.size());
  pp.pool_offset = descs.size() * sizeof(KvtReqDesc);
  pp.blob.resize(pp.pool_offset + pool.size() * sizeof(uint32_t));
  if (!descs.empty()) memcpy(pp.blob.data(), descs.data(), pp.pool_offset);
  if (!pool.empty()) memcpy(pp.blob.data() + pp.pool_offset, pool.data(), pool.size() * sizeof(uint32_t));
  return pp;
}

}  // namespace kvx
