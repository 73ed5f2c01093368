// Planner for cache shape 8 (Kimi-K3 style): leading KDA linear-attention state groups followed
// by one rank-replicated MLA group whose real bytes sit at the start of KDA-sized physical pages.
// Offset rules: kvtransfer/src/parse_block_kda.cpp:8-330 and parse_block_kimi_k3.cpp:9-235.
#include <algorithm>
#include <stdexcept>

#include "plan/plan_sink.h"
#include "plan/planner.h"

namespace kvx {

namespace {

using namespace plan_detail;
using Out = Sink;

Out open_out(const PlanEnv& e, PlanOut& out) {
  RTASSERT(!e.src->block_sizes.empty() && !e.dst->block_sizes.empty());
  return make_sink(e, out, 0);
}

size_t page_stride(const WorkerInfo& w) { return w.kda_page_stride != 0 ? w.kda_page_stride : w.block_sizes.at(0); }

struct KdaGeom {
  size_t state_len;   // conv taps kept per channel
  size_t channels;    // q + k + v channels on this rank
  size_t conv_bytes;
  size_t rec_bytes;
  size_t elem;
};

KdaGeom kda_geom(const WorkerInfo& w) {
  RTASSERT(w.conv_state_shape.size() >= 3 && w.ssm_state_shape.size() >= 4);
  KdaGeom g;
  g.elem = w.gdn_conv_elem_size;
  // "SD" keeps [state_len, channels] rows; "DS" (conv dim first) keeps [channels, state_len].
  g.state_len = w.kda_conv_dim_first ? w.conv_state_shape[2] : w.conv_state_shape[1];
  g.channels = w.kda_conv_dim_first ? w.conv_state_shape[1] : w.conv_state_shape[2];
  size_t sum = 0;
  for (size_t d : w.gdn_conv_channel_dims) sum += d;
  RTASSERT(sum == g.channels);
  g.conv_bytes = g.state_len * g.channels * g.elem;
  g.rec_bytes = w.ssm_state_shape[1] * w.ssm_state_shape[2] * w.ssm_state_shape[3] * w.gdn_ssm_elem_size;
  return g;
}

// One KDA page, P>D: this prefill rank's q/k/v components interleave into the merged page.
void kda_page_merge(Out& o, size_t p0, size_t d0, uint32_t g_n, uint32_t g_off, const WorkerInfo& src,
                    const KdaGeom& g) {
  if (src.kda_conv_dim_first) {
    size_t pre = 0;
    for (size_t dim : src.gdn_conv_channel_dims) {
      const size_t comp = dim * g.state_len * g.elem;
      o.put(p0 + pre, d0 + g_n * pre + g_off * comp, comp);
      pre += comp;
    }
  } else {
    const size_t p_row = g.channels * g.elem, d_row = g_n * p_row;
    for (size_t s = 0; s < g.state_len; ++s) {
      size_t pre = 0;
      for (size_t dim : src.gdn_conv_channel_dims) {
        const size_t comp = dim * g.elem;
        o.put(p0 + s * p_row + pre, d0 + s * d_row + g_n * pre + g_off * comp, comp);
        pre += comp;
      }
    }
  }
  o.put(p0 + g.conv_bytes, d0 + g_n * g.conv_bytes + g_off * g.rec_bytes, g.rec_bytes);
}

// One KDA page, P<D: decode rank g_off takes its share of each component and of the recurrent state.
void kda_page_split(Out& o, size_t p0, size_t d0, uint32_t g_n, uint32_t g_off, const WorkerInfo& src,
                    const KdaGeom& g) {
  const size_t d_rec = g.rec_bytes / g_n;
  size_t d_conv = 0;
  if (src.kda_conv_dim_first) {
    size_t p_pre = 0, d_pre = 0;
    for (size_t dim : src.gdn_conv_channel_dims) {
      const size_t comp = (dim / g_n) * g.state_len * g.elem;
      o.put(p0 + p_pre + g_off * comp, d0 + d_pre, comp);
      p_pre += g_n * comp;
      d_pre += comp;
    }
    d_conv = d_pre;
  } else {
    const size_t p_row = g.channels * g.elem, d_row = p_row / g_n;
    for (size_t s = 0; s < g.state_len; ++s) {
      size_t p_pre = 0, d_pre = 0;
      for (size_t dim : src.gdn_conv_channel_dims) {
        const size_t comp = (dim / g_n) * g.elem;
        o.put(p0 + s * p_row + p_pre + g_off * comp, d0 + s * d_row + d_pre, comp);
        p_pre += g_n * comp;
        d_pre += comp;
      }
    }
    d_conv = g.conv_bytes / g_n;
  }
  o.put(p0 + g.conv_bytes + g_off * d_rec, d0 + d_conv, d_rec);
}

enum class Rel { EQ, GT, LT };

// The two page rules above as walk ops over all pages of a group: one op per q / k / v component
// (with a row loop when the rows come first) and one for the recurrent state.
void kda_pages_ops(Out& o, const std::vector<uint32_t>& sb, const std::vector<uint32_t>& db, size_t p_stride,
                   size_t d_stride, uint32_t g_n, uint32_t g_off, const WorkerInfo& src, const KdaGeom& g, bool merge) {
  const uint32_t rows = static_cast<uint32_t>(g.state_len);
  if (merge) {
    size_t pre = 0;
    if (src.kda_conv_dim_first) {
      for (size_t dim : src.gdn_conv_channel_dims) {
        const size_t comp = dim * g.state_len * g.elem;
        page_op(o, sb, db, p_stride, d_stride, pre, g_n * pre + g_off * comp, comp, {});
        pre += comp;
      }
    } else {
      const size_t p_row = g.channels * g.elem, d_row = g_n * p_row;
      for (size_t dim : src.gdn_conv_channel_dims) {
        const size_t comp = dim * g.elem;
        page_op(o, sb, db, p_stride, d_stride, pre, g_n * pre + g_off * comp, comp, {{rows, p_row, d_row}});
        pre += comp;
      }
    }
    page_op(o, sb, db, p_stride, d_stride, g.conv_bytes, g_n * g.conv_bytes + g_off * g.rec_bytes, g.rec_bytes, {});
    return;
  }
  const size_t d_rec = g.rec_bytes / g_n;
  size_t p_pre = 0, d_pre = 0, d_conv = 0;
  if (src.kda_conv_dim_first) {
    for (size_t dim : src.gdn_conv_channel_dims) {
      const size_t comp = (dim / g_n) * g.state_len * g.elem;
      page_op(o, sb, db, p_stride, d_stride, p_pre + g_off * comp, d_pre, comp, {});
      p_pre += g_n * comp;
      d_pre += comp;
    }
    d_conv = d_pre;
  } else {
    const size_t p_row = g.channels * g.elem, d_row = p_row / g_n;
    for (size_t dim : src.gdn_conv_channel_dims) {
      const size_t comp = (dim / g_n) * g.elem;
      page_op(o, sb, db, p_stride, d_stride, p_pre + g_off * comp, d_pre, comp, {{rows, p_row, d_row}});
      p_pre += g_n * comp;
      d_pre += comp;
    }
    d_conv = g.conv_bytes / g_n;
  }
  page_op(o, sb, db, p_stride, d_stride, g.conv_bytes + g_off * d_rec, d_conv, d_rec, {});
}

// KDA state pages leave once, with the request's last chunk.
void kda_groups(const PlanEnv& e, const ReqSendTask& t, PlanOut& out, Rel rel) {
  Out o = open_out(e, out);
  const WorkerInfo& src = *e.src;
  const WorkerInfo& dst = *e.dst;
  RTASSERT(src.num_gdn_layers <= t.src_blocks().size() && src.num_gdn_layers <= t.dst_blocks().size());
  for (size_t g = 0; g < src.num_gdn_layers; ++g) RTASSERT(t.src_blocks()[g].size() == t.dst_blocks()[g].size());
  if (!t.reach_last_token) return;
  const size_t p_stride = page_stride(src), d_stride = page_stride(dst);
  uint32_t g_n = 1, g_off = 0;
  if (rel == Rel::GT) {
    g_n = src.engine_tp_size / dst.engine_tp_size;
    g_off = src.worker_tp_rank % g_n;
  } else if (rel == Rel::LT) {
    g_n = dst.engine_tp_size / src.engine_tp_size;
    g_off = dst.worker_tp_rank % g_n;
  }
  const KdaGeom geom = rel == Rel::EQ ? KdaGeom{} : kda_geom(src);
  for (size_t g = 0; g < src.num_gdn_layers; ++g) {
    const auto& sb = t.src_blocks()[g];
    const auto& db = t.dst_blocks()[g];
    if (o.ops()) {
      if (rel == Rel::EQ) page_op(o, sb, db, p_stride, d_stride, 0, 0, p_stride, {});
      else kda_pages_ops(o, sb, db, p_stride, d_stride, g_n, g_off, src, geom, rel == Rel::GT);
      continue;
    }
    for (size_t i = 0; i < sb.size(); ++i) {
      const size_t p0 = sb[i] * p_stride, d0 = db[i] * d_stride;
      if (rel == Rel::EQ) o.put(p0, d0, p_stride);
      else if (rel == Rel::GT) kda_page_merge(o, p0, d0, g_n, g_off, src, geom);
      else kda_page_split(o, p0, d0, g_n, g_off, src, geom);
    }
  }
}

// The MLA group is identical on every TP rank; representative ranks send it.  Equal TP moves
// manager blocks whole; otherwise kernel-block pages move once complete (block-aligned policy).
void mla_prefix(const PlanEnv& e, const ReqSendTask& t, PlanOut& out) {
  const WorkerInfo& src = *e.src;
  const WorkerInfo& dst = *e.dst;
  if (!e.valid_ranks.test(src.worker_tp_rank)) return;
  Out o = open_out(e, out);
  const size_t grp = src.num_gdn_layers;
  RTASSERT(grp < t.src_blocks().size() && grp < t.dst_blocks().size());
  const auto& sb = t.src_blocks()[grp];
  const auto& db = t.dst_blocks()[grp];
  const uint32_t s_ntpb = static_cast<uint32_t>(src.block_sizes.at(0) / src.token_sizes.at(0));
  const uint32_t d_ntpb = static_cast<uint32_t>(dst.block_sizes.at(0) / dst.token_sizes.at(0));
  const uint32_t kb = src.attn_kernel_blk_ntpb;
  RTASSERT(kb > 0 && src.hybrid_attn_token_size > 0);
  const size_t tok = src.hybrid_attn_token_size;
  const size_t kpage = static_cast<size_t>(kb) * tok;
  const size_t p_stride = page_stride(src), d_stride = page_stride(dst);
  if (o.ops()) {
    if (src.engine_tp_size == dst.engine_tp_size) {
      const uint32_t first = t.seen_tokens / s_ntpb;
      const uint32_t end = t.reach_last_token ? static_cast<uint32_t>(sb.size()) : t.end_tokens() / s_ntpb;
      const Sink::Side s{&sb, 1, 1, p_stride, 0, 0, 0}, d{&db, 1, 1, d_stride, 0, 0, 0};
      o.op(&s, d, first, end, static_cast<size_t>(s_ntpb) * tok, {});
      return;
    }
    // positions are kernel-block pages: a page moves once the chunk reaches its end, or with the last chunk
    RTASSERT(s_ntpb % kb == 0 && d_ntpb % kb == 0);
    const uint32_t end_tok = t.seen_tokens + t.new_tokens;
    const uint32_t lo = t.seen_tokens / kb;
    const uint32_t hi = t.new_tokens == 0 ? lo : (t.reach_last_token ? (end_tok + kb - 1) / kb : end_tok / kb);
    const Sink::Side s{&sb, s_ntpb / kb, s_ntpb / kb, p_stride, 0, kpage, 0}, d{&db, d_ntpb / kb, d_ntpb / kb, d_stride, 0, kpage, 0};
    o.op(&s, d, lo, hi, kpage, {});
    if (!e.pad_last_attn_block || !t.reach_last_token) return;
    const size_t cap_tok = db.size() * static_cast<size_t>(d_ntpb);
    if (end_tok >= cap_tok) return;
    const Sink::Side dz{&db, d_ntpb, d_ntpb, d_stride, 0, tok, 0};
    o.op(nullptr, dz, end_tok, static_cast<uint32_t>(cap_tok), tok, {});
    return;
  }
  if (src.engine_tp_size == dst.engine_tp_size) {
    const size_t first = t.seen_tokens / s_ntpb;
    const size_t end = t.reach_last_token ? sb.size() : t.end_tokens() / s_ntpb;
    for (size_t b = first; b < end; ++b) {
      RTASSERT(b < db.size());
      o.put(static_cast<size_t>(sb[b]) * p_stride, static_cast<size_t>(db[b]) * d_stride,
            static_cast<size_t>(s_ntpb) * tok);
    }
    return;
  }
  uint32_t pos = t.seen_tokens, left = t.new_tokens;
  while (left > 0) {
    const uint32_t i = pos % kb;
    const uint32_t run = std::min(kb - i, left);
    if (run == kb || t.reach_last_token || i + run == kb) {
      const uint32_t sbi = pos / s_ntpb, dbi = pos / d_ntpb;
      RTASSERT(sbi < sb.size() && dbi < db.size());
      o.put(static_cast<size_t>(sb[sbi]) * p_stride + static_cast<size_t>((pos % s_ntpb) / kb) * kpage,
            static_cast<size_t>(db[dbi]) * d_stride + static_cast<size_t>((pos % d_ntpb) / kb) * kpage, kpage);
    }
    pos += run;
    left -= run;
  }
  if (!e.pad_last_attn_block || !t.reach_last_token) return;
  const size_t total = static_cast<size_t>(t.seen_tokens) + t.new_tokens;
  const size_t cap_tokens = db.size() * static_cast<size_t>(d_ntpb);
  if (total >= cap_tokens) return;
  RTASSERT(!sb.empty());
  const size_t zero_src = static_cast<size_t>(sb[0]) * p_stride;
  for (size_t p = total; p < cap_tokens;) {
    const size_t i = p % d_ntpb;
    const size_t run = std::min(static_cast<size_t>(d_ntpb) - i, cap_tokens - p);
    size_t d_off = static_cast<size_t>(db[p / d_ntpb]) * d_stride + i * tok;
    size_t len = run * tok;
    while (len > 0) {
      const size_t seg = std::min(len, p_stride);
      o.put(zero_src, d_off, seg);
      d_off += seg;
      len -= seg;
    }
    p += run;
  }
}

}  // namespace

void kda_k3_eq(const PlanEnv& e, const ReqSendTask& t, PlanOut& out) {
  mla_prefix(e, t, out);
  kda_groups(e, t, out, Rel::EQ);
}
void kda_k3_gt(const PlanEnv& e, const ReqSendTask& t, PlanOut& out) {
  mla_prefix(e, t, out);
  kda_groups(e, t, out, Rel::GT);
}
void kda_k3_lt(const PlanEnv& e, const ReqSendTask& t, PlanOut& out) {
  mla_prefix(e, t, out);
  kda_groups(e, t, out, Rel::LT);
}

}  // namespace kvx
