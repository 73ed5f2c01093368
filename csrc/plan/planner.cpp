#include "plan/planner.h"
#include "plan/plan_sink.h"

#include <algorithm>
#include <limits>
#include <stdexcept>

namespace kvx {

RankSet compute_valid_ranks_pd(uint32_t p_tp, uint32_t d_tp, int num_kv_heads) {
  RankSet out;
  const uint32_t heads = num_kv_heads > 0 ? static_cast<uint32_t>(num_kv_heads) : 0;
  auto all = [&] {
    for (uint32_t i = 0; i < p_tp; ++i) out.set(i);
    return out;
  };
  // Fan-out (P<D): every prefill rank serves distinct decode ranks, replicated or not.
  if (p_tp < d_tp) {
    RTASSERT(d_tp % p_tp == 0);
    if (heads > p_tp && heads < d_tp) {
      RTASSERT(heads % p_tp == 0);
      RTASSERT(d_tp % heads == 0);
    }
    return all();
  }
  // Unknown head count, or at least one head per prefill rank: nobody is a replica.
  if (heads == 0 || heads >= p_tp) return all();
  // Heads replicated across prefill ranks.  If decode TP does not exceed the head count, one
  // representative per head; otherwise one representative per decode rank's subgroup.
  if (d_tp <= heads) {
    RTASSERT(p_tp % heads == 0);
    const uint32_t stride = p_tp / heads;
    for (uint32_t h = 0; h < heads; ++h) out.set(h * stride);
    return out;
  }
  RTASSERT(d_tp % heads == 0);
  RTASSERT(p_tp % d_tp == 0);
  const uint32_t per_d = p_tp / d_tp;
  for (uint32_t d = 0; d < d_tp; ++d) out.set(d * per_d);
  return out;
}

namespace {

using namespace plan_detail;

// ---- generic walkers -----------------------------------------------------------------------

// Contiguous runs of whole tokens; both sides store a token as `tok` contiguous bytes.
void walk_runs(Sink& k, size_t s_bs, size_t d_bs, size_t tok, uint32_t s_ntpb, uint32_t d_ntpb,
               const std::vector<uint32_t>& sb, const std::vector<uint32_t>& db, uint32_t seen, uint32_t n,
               size_t s_add = 0, size_t d_add = 0) {
  if (k.ops()) {
    const Sink::Side s{&sb, s_ntpb, s_ntpb, s_bs, 0, tok, s_add}, d{&db, d_ntpb, d_ntpb, d_bs, 0, tok, d_add};
    k.op(&s, d, seen, seen + n, tok, {});
    return;
  }
  uint32_t pos = seen, left = n;
  while (left > 0) {
    const uint32_t si = pos % s_ntpb, di = pos % d_ntpb;
    const uint32_t run = std::min({s_ntpb - si, d_ntpb - di, left});
    k.put(at(sb, pos / s_ntpb) * s_bs + si * tok + s_add, at(db, pos / d_ntpb) * d_bs + di * tok + d_add,
          static_cast<size_t>(run) * tok);
    pos += run;
    left -= run;
  }
}

// One piece per token between a "small" side (token stride sm_tok, the piece starts the token)
// and a "big" side (token stride bg_tok, the piece sits at slot g_off inside the token).
// src_is_small selects the direction (P>D: small is the source; P<D: small is the destination).
void walk_slices(Sink& k, size_t sm_tok, size_t piece, size_t bg_tok, uint32_t ntpb, size_t g_off,
                 const std::vector<uint32_t>& sm_blocks, const std::vector<uint32_t>& bg_blocks, uint32_t seen,
                 uint32_t n, bool src_is_small, size_t sm_add = 0, size_t bg_add = 0) {
  const size_t sm_bs = sm_tok * ntpb, bg_bs = bg_tok * ntpb;
  if (k.ops()) {
    const Sink::Side sm{&sm_blocks, ntpb, ntpb, sm_bs, 0, sm_tok, sm_add};
    const Sink::Side bg{&bg_blocks, ntpb, ntpb, bg_bs, 0, bg_tok, g_off * piece + bg_add};
    if (src_is_small) k.op(&sm, bg, seen, seen + n, piece, {}); else k.op(&bg, sm, seen, seen + n, piece, {});
    return;
  }
  for (uint32_t pos = seen; pos < seen + n; ++pos) {
    const uint32_t b = pos / ntpb, i = pos % ntpb;
    const size_t sm = at(sm_blocks, b) * sm_bs + i * sm_tok + sm_add;
    const size_t bg = at(bg_blocks, b) * bg_bs + i * bg_tok + g_off * piece + bg_add;
    if (src_is_small) k.put(sm, bg, piece); else k.put(bg, sm, piece);
  }
}

// HND pages, optionally sub-divided into kernel blocks of kb tokens:
//   block = [kernel blocks][K|V][head][token in kernel block][head_dim].
// The small side holds `heads` heads; the big side holds g_n groups of them, this one at g_off.
void walk_hnd(Sink& k, size_t sm_tok, size_t bg_tok, size_t sm_bs, size_t bg_bs, uint32_t sm_ntpb, uint32_t bg_ntpb,
              uint32_t sm_kb, uint32_t bg_kb, int heads, uint32_t g_n, uint32_t g_off,
              const std::vector<uint32_t>& sm_blocks, const std::vector<uint32_t>& bg_blocks, uint32_t seen,
              uint32_t n, bool src_is_small) {
  RTASSERT(heads > 0);
  RTASSERT(sm_tok % (2 * static_cast<size_t>(heads)) == 0);
  const size_t hd = sm_tok / 2 / static_cast<size_t>(heads);
  const size_t sm_kbs = sm_kb * sm_tok, bg_kbs = bg_kb * bg_tok;
  const size_t sm_head = sm_kb * hd, bg_head = bg_kb * hd;
  const size_t group_bytes = static_cast<size_t>(heads) * bg_head;
  RTASSERT(group_bytes * g_n == bg_kbs / 2);
  if (k.ops()) {
    RTASSERT(sm_ntpb % sm_kb == 0 && bg_ntpb % bg_kb == 0);
    const Sink::Side sm{&sm_blocks, sm_ntpb, sm_kb, sm_bs, sm_kbs, hd, 0};
    const Sink::Side bg{&bg_blocks, bg_ntpb, bg_kb, bg_bs, bg_kbs, hd, g_off * group_bytes};
    const uint32_t nh = static_cast<uint32_t>(heads);
    if (src_is_small) k.op(&sm, bg, seen, seen + n, hd, {{nh, sm_head, bg_head}, {2, sm_kbs / 2, bg_kbs / 2}});
    else k.op(&bg, sm, seen, seen + n, hd, {{nh, bg_head, sm_head}, {2, bg_kbs / 2, sm_kbs / 2}});
    return;
  }
  uint32_t pos = seen, left = n;
  while (left > 0) {
    const uint32_t sbi = pos / sm_ntpb, bbi = pos / bg_ntpb;
    const uint32_t s_kbi = (pos - sbi * sm_ntpb) / sm_kb, b_kbi = (pos - bbi * bg_ntpb) / bg_kb;
    const uint32_t s_i = pos % sm_kb, b_i = pos % bg_kb;
    const uint32_t run = std::min({sm_kb - s_i, bg_kb - b_i, left});
    const size_t s_base = at(sm_blocks, sbi) * sm_bs + s_kbi * sm_kbs;
    const size_t b_base = at(bg_blocks, bbi) * bg_bs + b_kbi * bg_kbs + g_off * group_bytes;
    const size_t len = static_cast<size_t>(run) * hd;
    for (int h = 0; h < heads; ++h) {
      const size_t sk = s_base + h * sm_head + s_i * hd;
      const size_t bk = b_base + h * bg_head + b_i * hd;
      if (src_is_small) {
        k.put(sk, bk, len);
        k.put(sk + sm_kbs / 2, bk + bg_kbs / 2, len);
      } else {
        k.put(bk, sk, len);
        k.put(bk + bg_kbs / 2, sk + sm_kbs / 2, len);
      }
    }
    pos += run;
    left -= run;
  }
}

// NHD pages of hybrid models: block = [kernel block x pack][K|V][token][head*dim]; `pack`
// consecutive attention layers share one physical page, interleaved per kernel block.
void walk_nhd_hybrid(Sink& k, uint32_t sm_ntpb, uint32_t bg_ntpb, size_t sm_tok, size_t bg_tok, size_t sm_bs,
                     size_t bg_bs, uint32_t sm_kb, uint32_t bg_kb, uint32_t pack, uint32_t g_off,
                     const std::vector<uint32_t>& sm_blocks, const std::vector<uint32_t>& bg_blocks, uint32_t seen,
                     uint32_t n, bool src_is_small) {
  if (pack == 0) pack = 1;
  const size_t sm_kbs = sm_kb * sm_tok, bg_kbs = bg_kb * bg_tok;
  const size_t sm_step = sm_tok / 2, bg_step = bg_tok / 2;
  const uint32_t sm_layer_ntpb = sm_ntpb / pack, bg_layer_ntpb = bg_ntpb / pack;
  RTASSERT(sm_layer_ntpb * pack == sm_ntpb && bg_layer_ntpb * pack == bg_ntpb);
  if (k.ops()) {
    RTASSERT(sm_layer_ntpb % sm_kb == 0 && bg_layer_ntpb % bg_kb == 0);
    const Sink::Side sm{&sm_blocks, sm_layer_ntpb, sm_kb, sm_bs, pack * sm_kbs, sm_step, 0};
    const Sink::Side bg{&bg_blocks, bg_layer_ntpb, bg_kb, bg_bs, pack * bg_kbs, bg_step, g_off * sm_step};
    if (src_is_small) k.op(&sm, bg, seen, seen + n, sm_step, {{pack, sm_kbs, bg_kbs}, {2, sm_kbs / 2, bg_kbs / 2}});
    else k.op(&bg, sm, seen, seen + n, sm_step, {{pack, bg_kbs, sm_kbs}, {2, bg_kbs / 2, sm_kbs / 2}});
    return;
  }
  uint32_t pos = seen, left = n;
  while (left > 0) {
    const uint32_t sbi = pos / sm_layer_ntpb, bbi = pos / bg_layer_ntpb;
    const uint32_t s_kbi = (pos % sm_layer_ntpb) / sm_kb, b_kbi = (pos % bg_layer_ntpb) / bg_kb;
    const uint32_t s_i = pos % sm_kb, b_i = pos % bg_kb;
    const uint32_t run = std::min({sm_kb - s_i, bg_kb - b_i, left});
    const size_t s_blk = at(sm_blocks, sbi) * sm_bs + static_cast<size_t>(s_kbi) * pack * sm_kbs;
    const size_t b_blk = at(bg_blocks, bbi) * bg_bs + static_cast<size_t>(b_kbi) * pack * bg_kbs;
    for (uint32_t sub = 0; sub < pack; ++sub) {
      for (uint32_t j = 0; j < run; ++j) {
        const size_t sk = s_blk + sub * sm_kbs + (s_i + j) * sm_step;
        const size_t bk = b_blk + sub * bg_kbs + (b_i + j) * bg_step + g_off * sm_step;
        if (src_is_small) {
          k.put(sk, bk, sm_step);
          k.put(sk + sm_kbs / 2, bk + bg_kbs / 2, sm_step);
        } else {
          k.put(bk, sk, sm_step);
          k.put(bk + bg_kbs / 2, sk + sm_kbs / 2, sm_step);
        }
      }
    }
    pos += run;
    left -= run;
  }
}

// Block-aligned policy: a page moves whole, and only once the chunk reaches its end (or the
// request ends); a chunk that stops inside a page leaves it to the next step.  On the last
// chunk every remaining allocated page (speculative-decode look-ahead) goes too.
void walk_aligned_pages(Sink& k, size_t bs, const ReqSendTask& task, const std::vector<uint32_t>& sb,
                        const std::vector<uint32_t>& db, uint32_t ntpb) {
  if (k.ops()) {
    // the pages the loop below sends: every page the chunk reaches the end of; with the last chunk also the
    // page it stops in and every allocated page after it
    const uint32_t end = task.seen_tokens + task.new_tokens;
    uint32_t lo = task.seen_tokens / ntpb, hi = end / ntpb;
    if (task.new_tokens == 0) lo = hi = (task.seen_tokens + ntpb - 1) / ntpb;
    if (task.reach_last_token) {
      RTASSERT(sb.size() == db.size());
      hi = std::max<uint32_t>((end + ntpb - 1) / ntpb, static_cast<uint32_t>(sb.size()));
    }
    const Sink::Side s{&sb, 1, 1, bs, 0, 0, 0}, d{&db, 1, 1, bs, 0, 0, 0};
    k.op(&s, d, lo, hi, bs, {});
    return;
  }
  uint32_t pos = task.seen_tokens, left = task.new_tokens;
  while (left > 0) {
    const uint32_t b = pos / ntpb, i = pos % ntpb;
    const uint32_t run = std::min(ntpb - i, left);
    const bool closes_page = i + run == ntpb;
    const bool send = run == ntpb || task.reach_last_token || (i != 0 && closes_page);
    if (send) k.put(at(sb, b) * bs, at(db, b) * bs, bs);
    pos += run;
    left -= run;
  }
  if (task.reach_last_token) {
    RTASSERT(sb.size() == db.size());
    for (size_t b = (pos + ntpb - 1) / ntpb; b < sb.size(); ++b) k.put(sb[b] * bs, db[b] * bs, bs);
  }
}

// Destination run [d_off, d_off+len) filled from the start of the request's first source block,
// which the engine keeps all-zero; no piece reads past that block.
void zero_fill(Sink& k, size_t zero_src, size_t d_off, size_t len, size_t max_seg) {
  for (size_t done = 0; done < len;) {
    const size_t seg = std::min(max_seg, len - done);
    k.put(zero_src, d_off + done, seg);
    done += seg;
  }
}

// ---- recurrent state pages (GDN / PLE) -----------------------------------------------------
struct StateGeom {
  size_t rows, row_bytes, conv_bytes, ssm_bytes, elem;
  const std::vector<size_t>* channel_dims;
};

StateGeom gdn_geom(const WorkerInfo& w) {
  RTASSERT(w.conv_state_shape.size() >= 3 && w.ssm_state_shape.size() >= 4 && !w.gdn_conv_channel_dims.empty());
  StateGeom g;
  g.elem = w.gdn_conv_elem_size;
  g.rows = w.conv_state_shape[1];
  g.row_bytes = w.conv_state_shape[2] * g.elem;
  g.conv_bytes = g.rows * g.row_bytes;
  g.ssm_bytes = w.ssm_state_shape[1] * w.ssm_state_shape[2] * w.ssm_state_shape[3] * w.gdn_ssm_elem_size;
  g.channel_dims = &w.gdn_conv_channel_dims;
  return g;
}

void gdn_equal(Sink& k, size_t bs, size_t n_groups, const BlockIds& sb, const BlockIds& db) {
  for (size_t g = 0; g < n_groups; ++g) {
    const auto& s = group(sb, g);
    const auto& d = group(db, g);
    RTASSERT(s.size() == d.size());
    if (k.ops()) {
      page_op(k, s, d, bs, bs, 0, 0, bs, {});
      continue;
    }
    for (size_t i = 0; i < s.size(); ++i) k.put(s[i] * bs, d[i] * bs, bs);
  }
}

// P>D: g_n prefill ranks interleave their conv channel segments (q | k | v) inside each row of
// the decode page and append their SSM slices after the merged conv region.
void gdn_merge(Sink& k, size_t p_bs, size_t d_bs, size_t n_groups, uint32_t g_n, uint32_t g_off,
               const WorkerInfo& src, const BlockIds& sb, const BlockIds& db) {
  const StateGeom g = gdn_geom(src);
  for (size_t grp = 0; grp < n_groups; ++grp) {
    const auto& s = group(sb, grp);
    const auto& d = group(db, grp);
    if (k.ops()) {
      RTASSERT(d.size() >= s.size());
      size_t pre = 0;
      for (size_t dim : *g.channel_dims) {
        const size_t seg = dim * g.elem;
        page_op(k, s, d, p_bs, d_bs, pre, g_n * pre + g_off * seg, seg,
                {{static_cast<uint32_t>(g.rows), g.row_bytes, g_n * g.row_bytes}});
        pre += seg;
      }
      RTASSERT(pre == g.row_bytes);
      page_op(k, s, d, p_bs, d_bs, g.conv_bytes, g_n * g.conv_bytes + g_off * g.ssm_bytes, g.ssm_bytes, {});
      continue;
    }
    for (size_t i = 0; i < s.size(); ++i) {
      const size_t p0 = s[i] * p_bs, d0 = at(d, i) * d_bs;
      for (size_t r = 0; r < g.rows; ++r) {
        size_t pre = 0;
        for (size_t dim : *g.channel_dims) {
          const size_t seg = dim * g.elem;
          k.put(p0 + r * g.row_bytes + pre, d0 + r * g_n * g.row_bytes + g_n * pre + g_off * seg, seg);
          pre += seg;
        }
        RTASSERT(pre == g.row_bytes);
      }
      k.put(p0 + g.conv_bytes, d0 + g_n * g.conv_bytes + g_off * g.ssm_bytes, g.ssm_bytes);
    }
  }
}

// P<D: the mirror image; decode rank g_off takes its slice of every channel segment and of the SSM state.
void gdn_split(Sink& k, size_t p_bs, size_t d_bs, size_t n_groups, uint32_t g_n, uint32_t g_off,
               const WorkerInfo& src, const BlockIds& sb, const BlockIds& db) {
  const StateGeom g = gdn_geom(src);
  RTASSERT(g.row_bytes % g_n == 0 && g.ssm_bytes % g_n == 0);
  const size_t d_row = g.row_bytes / g_n, d_ssm = g.ssm_bytes / g_n;
  for (size_t grp = 0; grp < n_groups; ++grp) {
    const auto& s = group(sb, grp);
    const auto& d = group(db, grp);
    if (k.ops()) {
      RTASSERT(d.size() >= s.size());
      size_t p_pre = 0, d_pre = 0;
      for (size_t dim : *g.channel_dims) {
        const size_t p_seg = dim * g.elem;
        RTASSERT(p_seg % g_n == 0);
        const size_t d_seg = p_seg / g_n;
        page_op(k, s, d, p_bs, d_bs, p_pre + g_off * d_seg, d_pre, d_seg, {{static_cast<uint32_t>(g.rows), g.row_bytes, d_row}});
        p_pre += p_seg;
        d_pre += d_seg;
      }
      page_op(k, s, d, p_bs, d_bs, g.conv_bytes + g_off * d_ssm, g.rows * d_row, d_ssm, {});
      continue;
    }
    for (size_t i = 0; i < s.size(); ++i) {
      const size_t p0 = s[i] * p_bs, d0 = at(d, i) * d_bs;
      for (size_t r = 0; r < g.rows; ++r) {
        size_t p_pre = 0, d_pre = 0;
        for (size_t dim : *g.channel_dims) {
          const size_t p_seg = dim * g.elem;
          RTASSERT(p_seg % g_n == 0);
          const size_t d_seg = p_seg / g_n;
          k.put(p0 + r * g.row_bytes + p_pre + g_off * d_seg, d0 + r * d_row + d_pre, d_seg);
          p_pre += p_seg;
          d_pre += d_seg;
        }
      }
      k.put(p0 + g.conv_bytes + g_off * d_ssm, d0 + g.rows * d_row, d_ssm);
    }
  }
}

// PLE short-conv state is replicated across TP ranks: P==D copies pages, P>D lets only the
// first rank of each group send the real state bytes, P<D sends them to every decode rank.
void ple_pages(Sink& k, size_t p_bs, size_t d_bs, const WorkerInfo& src, const BlockIds& sb, const BlockIds& db,
               bool whole_page, bool skip) {
  if (src.num_ple_layers == 0 || skip) return;
  size_t len = p_bs;
  if (!whole_page) {
    RTASSERT(src.ple_conv_state_shape.size() == 3);
    len = src.ple_conv_state_shape[1] * src.ple_conv_state_shape[2] * src.ple_conv_elem_size;
    RTASSERT(len <= p_bs && len <= d_bs);
  }
  for (size_t i = 0; i < src.num_ple_layers; ++i) {
    const auto& s = group(sb, src.ple_block_group + i);
    const auto& d = group(db, src.ple_block_group + i);
    RTASSERT(s.size() == d.size());
    if (k.ops()) {
      page_op(k, s, d, p_bs, d_bs, 0, 0, len, {});
      continue;
    }
    for (size_t j = 0; j < s.size(); ++j) k.put(s[j] * p_bs, d[j] * d_bs, len);
  }
}

int heads_per_rank(const WorkerInfo& w) {
  if (w.num_kv_heads > 0 && static_cast<uint32_t>(w.num_kv_heads) >= w.engine_tp_size)
    return w.num_kv_heads / static_cast<int>(w.engine_tp_size);
  return std::max(1, w.num_kv_heads);
}

struct One {  // the single-tensor sizes most shapes use
  size_t p_tok, d_tok, p_bs, d_bs;
  uint32_t p_ntpb, d_ntpb;
};
One single_tensor(const PlanEnv& e) {
  RTASSERT(e.src->token_sizes.size() == 1 && e.dst->token_sizes.size() == 1);
  RTASSERT(e.src->block_sizes.size() == 1 && e.dst->block_sizes.size() == 1);
  One o{e.src->token_sizes[0], e.dst->token_sizes[0], e.src->block_sizes[0], e.dst->block_sizes[0], 0, 0};
  o.p_ntpb = static_cast<uint32_t>(o.p_bs / o.p_tok);
  o.d_ntpb = static_cast<uint32_t>(o.d_bs / o.d_tok);
  RTASSERT(o.p_ntpb * o.p_tok == o.p_bs && o.d_ntpb * o.d_tok == o.d_bs);
  return o;
}

// ---- shape 1: ragged [block, slot, 2, head, dim] ------------------------------------------------
void ragged_eq(const PlanEnv& e, const ReqSendTask& t, PlanOut& out) {
  const One o = single_tensor(e);
  RTASSERT(o.p_tok == o.d_tok && o.p_bs == o.d_bs);
  Sink k = make_sink(e, out, 0);
  walk_runs(k, o.p_bs, o.d_bs, o.p_tok, o.p_ntpb, o.d_ntpb, group(t.src_blocks(), 0), group(t.dst_blocks(), 0),
            t.seen_tokens, t.new_tokens);
}

// Same token size on both sides although P TP > D TP: the cache is replicated (MLA); rank 0 sends.
void ragged_gt_replicated(const PlanEnv& e, const ReqSendTask& t, PlanOut& out) {
  if (e.src->worker_tp_rank != 0) return;
  ragged_eq(e, t, out);
}

void ragged_sliced(const PlanEnv& e, const ReqSendTask& t, PlanOut& out, bool p_gt_d) {
  const One o = single_tensor(e);
  const size_t sm_tok = p_gt_d ? o.p_tok : o.d_tok, bg_tok = p_gt_d ? o.d_tok : o.p_tok;
  const uint32_t sm_tp = p_gt_d ? e.dst->engine_tp_size : e.kvt_tp_size;
  const uint32_t bg_tp = p_gt_d ? e.kvt_tp_size : e.dst->engine_tp_size;
  RTASSERT(bg_tp > sm_tp && bg_tp % sm_tp == 0);
  const uint32_t g_n = bg_tp / sm_tp;
  const uint32_t rank = p_gt_d ? e.src->worker_tp_rank : e.dst->worker_tp_rank;
  const uint32_t g_off = rank % g_n;
  RTASSERT(bg_tok == sm_tok * g_n && sm_tok % 2 == 0);
  const size_t sm_k = sm_tok / 2, bg_k = bg_tok / 2;
  const uint32_t ntpb = p_gt_d ? o.p_ntpb : o.d_ntpb;
  RTASSERT(o.p_ntpb == o.d_ntpb);
  const auto& sm_blocks = group(p_gt_d ? t.src_blocks() : t.dst_blocks(), 0);
  const auto& bg_blocks = group(p_gt_d ? t.dst_blocks() : t.src_blocks(), 0);
  Sink k = make_sink(e, out, 0);
  walk_slices(k, sm_tok, sm_k, bg_tok, ntpb, g_off, sm_blocks, bg_blocks, t.seen_tokens, t.new_tokens, p_gt_d);
  walk_slices(k, sm_tok, sm_k, bg_tok, ntpb, g_off, sm_blocks, bg_blocks, t.seen_tokens, t.new_tokens, p_gt_d,
              sm_k, bg_k);
}
void ragged_gt(const PlanEnv& e, const ReqSendTask& t, PlanOut& o) { ragged_sliced(e, t, o, true); }
void ragged_lt(const PlanEnv& e, const ReqSendTask& t, PlanOut& o) { ragged_sliced(e, t, o, false); }

// ---- shape 2: FlashAttention NHD [2, block, slot, head, dim] --------------------------------------
void flash_eq(const PlanEnv& e, const ReqSendTask& t, PlanOut& out) {
  const One o = single_tensor(e);
  RTASSERT(o.p_tok == o.d_tok && o.p_bs == o.d_bs);
  const size_t k_tok = o.p_tok / 2, k_bs = o.p_bs / 2;
  const size_t s_v = k_bs * e.src->layer_num_blocks, d_v = k_bs * e.dst->layer_num_blocks;
  Sink k = make_sink(e, out, 0);
  const auto& sb = group(t.src_blocks(), 0);
  const auto& db = group(t.dst_blocks(), 0);
  walk_runs(k, k_bs, k_bs, k_tok, o.p_ntpb, o.d_ntpb, sb, db, t.seen_tokens, t.new_tokens);
  walk_runs(k, k_bs, k_bs, k_tok, o.p_ntpb, o.d_ntpb, sb, db, t.seen_tokens, t.new_tokens, s_v, d_v);
}

void flash_sliced(const PlanEnv& e, const ReqSendTask& t, PlanOut& out, bool p_gt_d) {
  const One o = single_tensor(e);
  uint32_t g_n, g_off;
  if (p_gt_d) {
    if (!e.valid_ranks[e.src->worker_tp_rank]) return;
    g_n = static_cast<uint32_t>(e.valid_ranks.count()) / e.dst->engine_tp_size;
    RTASSERT(g_n > 0);
    g_off = e.kvt_tp_rank % g_n;
  } else {
    g_n = e.dst->engine_tp_size / e.kvt_tp_size;
    RTASSERT(g_n > 0);
    g_off = e.dst->worker_tp_rank % g_n;
  }
  const size_t sm_tok = p_gt_d ? o.p_tok : o.d_tok, bg_tok = p_gt_d ? o.d_tok : o.p_tok;
  RTASSERT(o.p_ntpb == o.d_ntpb && sm_tok % 2 == 0);
  const size_t sm_k = sm_tok / 2, bg_k = bg_tok / 2;
  // With the unscaled bf16->fp8 cast the destination sizes and the piece length are fp8 bytes.
  const size_t piece = e.cast_bf16_to_fp8 && p_gt_d ? sm_k / 2 : sm_k;
  RTASSERT(e.cast_bf16_to_fp8 || bg_k == sm_k * g_n);
  const uint32_t ntpb = o.p_ntpb;
  const size_t p_v = ntpb * (o.p_tok / 2) * e.src->layer_num_blocks;
  const size_t d_v = ntpb * (o.d_tok / 2) * e.dst->layer_num_blocks;
  const auto& sm_blocks = group(p_gt_d ? t.src_blocks() : t.dst_blocks(), 0);
  const auto& bg_blocks = group(p_gt_d ? t.dst_blocks() : t.src_blocks(), 0);
  Sink k = make_sink(e, out, 0);
  walk_slices(k, sm_k, piece, bg_k, ntpb, g_off, sm_blocks, bg_blocks, t.seen_tokens, t.new_tokens, p_gt_d);
  walk_slices(k, sm_k, piece, bg_k, ntpb, g_off, sm_blocks, bg_blocks, t.seen_tokens, t.new_tokens, p_gt_d,
              p_gt_d ? p_v : d_v, p_gt_d ? d_v : p_v);
}
void flash_gt(const PlanEnv& e, const ReqSendTask& t, PlanOut& o) { flash_sliced(e, t, o, true); }
// The reference has no P<D planner for this shape; the mirror rule is provided because the
// fused kernel supports the fan-out and needs an oracle.
void flash_lt(const PlanEnv& e, const ReqSendTask& t, PlanOut& o) { flash_sliced(e, t, o, false); }

// ---- shape 5: FlashInfer HND [block, 2, head, slot, dim] -----------------------------------------
void hnd_eq(const PlanEnv& e, const ReqSendTask& t, PlanOut& out) {
  const One o = single_tensor(e);
  RTASSERT(o.p_ntpb == o.d_ntpb);
  Sink k = make_sink(e, out, 0);
  walk_hnd(k, o.p_tok, o.d_tok, o.p_bs, o.d_bs, o.p_ntpb, o.d_ntpb, o.p_ntpb, o.d_ntpb, heads_per_rank(*e.src), 1, 0,
           group(t.src_blocks(), 0), group(t.dst_blocks(), 0), t.seen_tokens, t.new_tokens, true);
}

void hnd_gt(const PlanEnv& e, const ReqSendTask& t, PlanOut& out) {
  if (!e.valid_ranks[e.src->worker_tp_rank]) return;
  const One o = single_tensor(e);
  RTASSERT(o.p_ntpb == o.d_ntpb);
  const uint32_t g_n = static_cast<uint32_t>(e.valid_ranks.count()) / e.dst->engine_tp_size;
  RTASSERT(g_n > 0);
  Sink k = make_sink(e, out, 0);
  walk_hnd(k, o.p_tok, o.d_tok, o.p_bs, o.d_bs, o.p_ntpb, o.d_ntpb, o.p_ntpb, o.d_ntpb, heads_per_rank(*e.src), g_n,
           e.kvt_tp_rank % g_n, group(t.src_blocks(), 0), group(t.dst_blocks(), 0), t.seen_tokens, t.new_tokens,
           true);
}

void hnd_lt(const PlanEnv& e, const ReqSendTask& t, PlanOut& out) {
  const One o = single_tensor(e);
  RTASSERT(o.p_ntpb == o.d_ntpb && o.p_tok % o.d_tok == 0);
  const uint32_t g_n = static_cast<uint32_t>(o.p_tok / o.d_tok);
  const uint32_t replicas = std::max(1u, e.dst->engine_tp_size / (e.src->engine_tp_size * g_n));
  const uint32_t g_off = (e.dst->worker_tp_rank / replicas) % g_n;
  const int d_heads = std::max(1, heads_per_rank(*e.src) / static_cast<int>(g_n));
  Sink k = make_sink(e, out, 0);
  walk_hnd(k, o.d_tok, o.p_tok, o.d_bs, o.p_bs, o.d_ntpb, o.p_ntpb, o.d_ntpb, o.p_ntpb, d_heads, g_n, g_off,
           group(t.dst_blocks(), 0), group(t.src_blocks(), 0), t.seen_tokens, t.new_tokens, false);
}

// ---- shape 4: several single-tensor caches per layer (sparse MLA: indexer keys + latent) ------------
void multi_eq(const PlanEnv& e, const ReqSendTask& t, PlanOut& out) {
  if (!e.valid_ranks[e.src->worker_tp_rank]) return;
  RTASSERT(e.src->token_sizes == e.dst->token_sizes && e.src->block_sizes == e.dst->block_sizes);
  for (size_t i = 0; i < e.src->token_sizes.size(); ++i) {
    Sink k = make_sink(e, out, i);
    const size_t bs = e.src->block_sizes[i], tok = e.src->token_sizes[i];
    const uint32_t ntpb = static_cast<uint32_t>(bs / tok);
    walk_runs(k, bs, bs, tok, ntpb, ntpb, group(t.src_blocks(), 0), group(t.dst_blocks(), 0), t.seen_tokens,
              t.new_tokens);
  }
}

void multi_sliced(const PlanEnv& e, const ReqSendTask& t, PlanOut& out, bool p_gt_d) {
  const WorkerInfo& sm = p_gt_d ? *e.src : *e.dst;
  const WorkerInfo& bg = p_gt_d ? *e.dst : *e.src;
  const uint32_t sm_tp = p_gt_d ? e.dst->engine_tp_size : e.kvt_tp_size;
  const uint32_t bg_tp = p_gt_d ? e.kvt_tp_size : e.dst->engine_tp_size;
  RTASSERT(bg_tp > sm_tp && bg_tp % sm_tp == 0);
  const uint32_t g_n = bg_tp / sm_tp;
  const uint32_t g_off = (p_gt_d ? e.src->worker_tp_rank : e.dst->worker_tp_rank) % g_n;
  RTASSERT(sm.token_sizes.size() == bg.token_sizes.size());
  for (size_t i = 0; i < sm.token_sizes.size(); ++i) {
    const size_t sm_tok = sm.token_sizes[i], bg_tok = bg.token_sizes[i];
    RTASSERT(bg_tok == sm_tok * g_n && sm_tok % 2 == 0);
    const uint32_t ntpb = static_cast<uint32_t>(sm.block_sizes[i] / sm_tok);
    RTASSERT(ntpb * bg_tok == bg.block_sizes[i]);
    const auto& sm_blocks = group(p_gt_d ? t.src_blocks() : t.dst_blocks(), 0);
    const auto& bg_blocks = group(p_gt_d ? t.dst_blocks() : t.src_blocks(), 0);
    Sink k = make_sink(e, out, i);
    walk_slices(k, sm_tok, sm_tok / 2, bg_tok, ntpb, g_off, sm_blocks, bg_blocks, t.seen_tokens, t.new_tokens, p_gt_d);
    walk_slices(k, sm_tok, sm_tok / 2, bg_tok, ntpb, g_off, sm_blocks, bg_blocks, t.seen_tokens, t.new_tokens, p_gt_d,
                sm_tok / 2, bg_tok / 2);
  }
}

void multi_gt(const PlanEnv& e, const ReqSendTask& t, PlanOut& out) {
  if (e.src->token_sizes == e.dst->token_sizes) {  // replicated latent cache: rank 0 sends everything
    if (e.src->worker_tp_rank != 0) return;
    RTASSERT(e.src->block_sizes == e.dst->block_sizes);
    for (size_t i = 0; i < e.src->token_sizes.size(); ++i) {
      Sink k = make_sink(e, out, i);
      const size_t bs = e.src->block_sizes[i], tok = e.src->token_sizes[i];
      const uint32_t ntpb = static_cast<uint32_t>(bs / tok);
      walk_runs(k, bs, bs, tok, ntpb, ntpb, group(t.src_blocks(), 0), group(t.dst_blocks(), 0), t.seen_tokens,
                t.new_tokens);
    }
    return;
  }
  multi_sliced(e, t, out, true);
}
void multi_lt(const PlanEnv& e, const ReqSendTask& t, PlanOut& out) {
  if (e.src->token_sizes == e.dst->token_sizes) {  // replicated cache fans out unchanged
    multi_eq(e, t, out);
    return;
  }
  multi_sliced(e, t, out, false);
}

// ---- shapes 3 / 6 / 7: hybrid pages (GDN groups | indexer? | attention | PLE?) ---------------------
struct HybridView {
  One o;
  size_t n_gdn;
  size_t attn_group;  // index of the attention block group
  bool has_indexer;
  uint32_t pack;
};
HybridView hybrid_view(const PlanEnv& e) {
  HybridView v;
  v.o = single_tensor(e);
  v.n_gdn = e.src->num_gdn_layers;
  v.has_indexer = e.src->indexer_blk_ntpb > 0;
  RTASSERT((e.src->indexer_blk_ntpb > 0) == (e.dst->indexer_blk_ntpb > 0));
  v.attn_group = v.n_gdn + (v.has_indexer ? 1 : 0);
  v.pack = e.src->attn_pack_size == 0 ? 1u : e.src->attn_pack_size;
  RTASSERT(v.pack == (e.dst->attn_pack_size == 0 ? 1u : e.dst->attn_pack_size));
  return v;
}

void hybrid_indexer_tokens(Sink& k, const PlanEnv& e, const HybridView& v, const ReqSendTask& t) {
  const size_t tok = e.src->hybrid_indexer_token_size;
  RTASSERT(tok > 0);
  walk_runs(k, v.o.p_bs, v.o.d_bs, tok, e.src->indexer_blk_ntpb, e.dst->indexer_blk_ntpb,
            group(t.src_blocks(), v.n_gdn), group(t.dst_blocks(), v.n_gdn), t.seen_tokens, t.new_tokens);
}

void hybrid_eq(const PlanEnv& e, const ReqSendTask& t, PlanOut& out, bool hnd) {
  const HybridView v = hybrid_view(e);
  RTASSERT(v.o.p_tok == v.o.d_tok && v.o.p_bs == v.o.d_bs);
  RTASSERT(e.src->indexer_blk_ntpb == e.dst->indexer_blk_ntpb);
  Sink k = make_sink(e, out, 0);
  if (v.has_indexer) {
    walk_aligned_pages(k, v.o.p_bs, t, group(t.src_blocks(), v.n_gdn), group(t.dst_blocks(), v.n_gdn),
                       e.src->indexer_blk_ntpb);
  }
  const uint32_t attn_ntpb = hnd ? v.o.p_ntpb : v.o.p_ntpb / v.pack;
  walk_aligned_pages(k, v.o.p_bs, t, group(t.src_blocks(), v.attn_group), group(t.dst_blocks(), v.attn_group),
                     attn_ntpb);
  if (t.reach_last_token) {
    gdn_equal(k, v.o.p_bs, v.n_gdn, t.src_blocks(), t.dst_blocks());
    ple_pages(k, v.o.p_bs, v.o.d_bs, *e.src, t.src_blocks(), t.dst_blocks(), true, false);
  }
}

void hybrid_gt(const PlanEnv& e, const ReqSendTask& t, PlanOut& out, bool hnd) {
  const HybridView v = hybrid_view(e);
  const uint32_t p_tp = e.src->engine_tp_size, d_tp = e.dst->engine_tp_size;
  RTASSERT(p_tp > d_tp && p_tp % d_tp == 0);
  const uint32_t gdn_n = p_tp / d_tp, gdn_off = e.src->worker_tp_rank % gdn_n;
  const uint32_t attn_n = static_cast<uint32_t>(e.valid_ranks.count()) / d_tp;
  const uint32_t attn_off = attn_n > 0 ? e.kvt_tp_rank % attn_n : 0;
  Sink k = make_sink(e, out, 0);
  if (t.reach_last_token) {
    gdn_merge(k, v.o.p_bs, v.o.d_bs, v.n_gdn, gdn_n, gdn_off, *e.src, t.src_blocks(), t.dst_blocks());
    ple_pages(k, v.o.p_bs, v.o.d_bs, *e.src, t.src_blocks(), t.dst_blocks(), false, gdn_off != 0);
  }
  if (v.has_indexer && e.src->worker_tp_rank % gdn_n == 0) hybrid_indexer_tokens(k, e, v, t);
  if (!e.valid_ranks[e.src->worker_tp_rank]) return;
  const auto& sb = group(t.src_blocks(), v.attn_group);
  const auto& db = group(t.dst_blocks(), v.attn_group);
  const uint32_t s_kb = e.src->attn_kernel_blk_ntpb, d_kb = e.dst->attn_kernel_blk_ntpb;
  const uint32_t total = t.seen_tokens + t.new_tokens;
  const bool pad = e.pad_last_attn_block && t.reach_last_token && total > 0;
  const size_t zero_src = pad ? at(sb, 0) * v.o.p_bs : 0;
  if (hnd) {
    const int heads = std::max(1, e.src->num_kv_heads / static_cast<int>(p_tp));
    walk_hnd(k, v.o.p_tok, v.o.d_tok, v.o.p_bs, v.o.d_bs, v.o.p_ntpb, v.o.d_ntpb, s_kb, d_kb, heads, attn_n, attn_off,
             sb, db, t.seen_tokens, t.new_tokens, true);
    const uint32_t filled = total % v.o.d_ntpb;
    if (pad && filled != 0 && k.ops()) {
      const size_t hd = v.o.p_tok / 2 / static_cast<size_t>(heads);
      const size_t d_head = static_cast<size_t>(v.o.d_ntpb) * hd;
      const size_t d_kv = static_cast<size_t>(v.o.d_ntpb) * v.o.d_tok / 2;
      const Sink::Side d{&db, v.o.d_ntpb, v.o.d_ntpb, v.o.d_bs, 0, hd, attn_off * heads * d_head};
      k.op(nullptr, d, total, total + (v.o.d_ntpb - filled), hd, {{static_cast<uint32_t>(heads), 0, d_head}, {2, 0, d_kv}});
    } else if (pad && filled != 0) {
      // one zero run per head and K/V: slots [filled, d_ntpb) of the last destination block
      const size_t hd = v.o.p_tok / 2 / static_cast<size_t>(heads);
      const size_t d_head = static_cast<size_t>(v.o.d_ntpb) * hd;
      const size_t d_kv = static_cast<size_t>(v.o.d_ntpb) * v.o.d_tok / 2;
      const size_t base = at(db, total / v.o.d_ntpb) * v.o.d_bs + attn_off * heads * d_head;
      const size_t len = static_cast<size_t>(v.o.d_ntpb - filled) * hd;
      for (int h = 0; h < heads; ++h) {
        const size_t dk = base + h * d_head + filled * hd;
        zero_fill(k, zero_src, dk, len, v.o.p_bs);
        zero_fill(k, zero_src, dk + d_kv, len, v.o.p_bs);
      }
    }
    return;
  }
  RTASSERT(v.o.d_tok == v.o.p_tok * attn_n);
  walk_nhd_hybrid(k, v.o.p_ntpb, v.o.d_ntpb, v.o.p_tok, v.o.d_tok, v.o.p_bs, v.o.d_bs, s_kb, d_kb, v.pack, attn_off, sb,
                  db, t.seen_tokens, t.new_tokens, true);
  const uint32_t d_layer_ntpb = v.o.d_ntpb / v.pack;
  const uint32_t filled = total % d_layer_ntpb;
  if (pad && filled != 0 && k.ops()) {
    const size_t d_kbs = d_kb * v.o.d_tok, p_step = v.o.p_tok / 2, d_step = v.o.d_tok / 2;
    RTASSERT(d_layer_ntpb % d_kb == 0);
    const Sink::Side d{&db, d_layer_ntpb, d_kb, v.o.d_bs, v.pack * d_kbs, d_step, attn_off * p_step};
    k.op(nullptr, d, total, total + (d_layer_ntpb - filled), p_step, {{v.pack, 0, d_kbs}, {2, 0, d_kbs / 2}});
  } else if (pad && filled != 0) {
    const size_t d_kbs = d_kb * v.o.d_tok, p_step = v.o.p_tok / 2, d_step = v.o.d_tok / 2;
    uint32_t to_fill = d_layer_ntpb - filled, d_pos = total, s_pos = 0;
    while (to_fill > 0) {
      const uint32_t dbi = d_pos / d_layer_ntpb;
      const uint32_t d_kbi = (d_pos % d_layer_ntpb) / d_kb;
      const uint32_t d_i = d_pos % d_kb, s_i = s_pos % s_kb;
      const uint32_t run = std::min({s_kb - s_i, d_kb - d_i, to_fill});
      const size_t d_blk = at(db, dbi) * v.o.d_bs + static_cast<size_t>(d_kbi) * v.pack * d_kbs;
      for (uint32_t sub = 0; sub < v.pack; ++sub) {
        for (uint32_t j = 0; j < run; ++j) {
          const size_t dk = d_blk + sub * d_kbs + (d_i + j) * d_step + attn_off * p_step;
          zero_fill(k, zero_src, dk, p_step, v.o.p_bs);
          zero_fill(k, zero_src, dk + d_kbs / 2, p_step, v.o.p_bs);
        }
      }
      s_pos += run;
      d_pos += run;
      to_fill -= run;
    }
  }
}

void hybrid_lt(const PlanEnv& e, const ReqSendTask& t, PlanOut& out, bool hnd) {
  const HybridView v = hybrid_view(e);
  const uint32_t p_tp = e.src->engine_tp_size, d_tp = e.dst->engine_tp_size;
  RTASSERT(p_tp < d_tp && d_tp % p_tp == 0);
  const uint32_t gdn_n = d_tp / p_tp, gdn_off = e.dst->worker_tp_rank % gdn_n;
  Sink k = make_sink(e, out, 0);
  const auto& sb = group(t.src_blocks(), v.attn_group);
  const auto& db = group(t.dst_blocks(), v.attn_group);
  if (v.o.p_tok == v.o.d_tok) {
    // attention heads fully replicated on both sides: pages go unchanged, block aligned
    RTASSERT(v.o.p_bs == v.o.d_bs);
    if (v.has_indexer) {
      walk_aligned_pages(k, v.o.p_bs, t, group(t.src_blocks(), v.n_gdn), group(t.dst_blocks(), v.n_gdn),
                         e.src->indexer_blk_ntpb);
    }
    walk_aligned_pages(k, v.o.p_bs, t, sb, db, hnd ? v.o.p_ntpb : v.o.p_ntpb / v.pack);
  } else {
    RTASSERT(v.o.p_tok > v.o.d_tok && v.o.p_tok % v.o.d_tok == 0);
    const uint32_t attn_n = static_cast<uint32_t>(v.o.p_tok / v.o.d_tok);
    RTASSERT(d_tp % (p_tp * attn_n) == 0);
    const uint32_t replicas = d_tp / (p_tp * attn_n);
    const uint32_t attn_off = (e.dst->worker_tp_rank / replicas) % attn_n;
    if (v.has_indexer) hybrid_indexer_tokens(k, e, v, t);
    const uint32_t s_kb = e.src->attn_kernel_blk_ntpb, d_kb = e.dst->attn_kernel_blk_ntpb;
    const uint32_t total = t.seen_tokens + t.new_tokens;
    const bool pad = e.pad_last_attn_block && t.reach_last_token;
    if (hnd) {
      const int d_heads = static_cast<uint32_t>(std::max(0, e.src->num_kv_heads)) >= d_tp
                              ? e.src->num_kv_heads / static_cast<int>(d_tp) : 1;
      walk_hnd(k, v.o.d_tok, v.o.p_tok, v.o.d_bs, v.o.p_bs, v.o.d_ntpb, v.o.p_ntpb, d_kb, s_kb, d_heads, attn_n,
               attn_off, db, sb, t.seen_tokens, t.new_tokens, false);
      const uint32_t end = static_cast<uint32_t>(db.size()) * v.o.d_ntpb;
      if (pad && total < end && k.ops()) {
        const size_t hd = v.o.d_tok / 2 / static_cast<size_t>(d_heads);
        const size_t d_head = static_cast<size_t>(v.o.d_ntpb) * hd;
        const Sink::Side d{&db, v.o.d_ntpb, v.o.d_ntpb, v.o.d_bs, 0, hd, 0};
        k.op(nullptr, d, total, end, hd, {{static_cast<uint32_t>(d_heads), 0, d_head}, {2, 0, v.o.d_bs / 2}});
      } else if (pad && total < end) {
        const size_t hd = v.o.d_tok / 2 / static_cast<size_t>(d_heads);
        const size_t d_head = static_cast<size_t>(v.o.d_ntpb) * hd;
        const size_t zero_src = at(sb, 0) * v.o.p_bs;
        for (uint32_t pos = total; pos < end;) {
          const uint32_t i = pos % v.o.d_ntpb;
          const uint32_t run = std::min(v.o.d_ntpb - i, end - pos);
          const size_t d0 = at(db, pos / v.o.d_ntpb) * v.o.d_bs;
          for (int h = 0; h < d_heads; ++h) {
            const size_t dk = d0 + h * d_head + i * hd;
            zero_fill(k, zero_src, dk, static_cast<size_t>(run) * hd, v.o.p_bs);
            zero_fill(k, zero_src, dk + v.o.d_bs / 2, static_cast<size_t>(run) * hd, v.o.p_bs);
          }
          pos += run;
        }
      }
    } else {
      walk_nhd_hybrid(k, v.o.d_ntpb, v.o.p_ntpb, v.o.d_tok, v.o.p_tok, v.o.d_bs, v.o.p_bs, d_kb, s_kb, v.pack, attn_off,
                      db, sb, t.seen_tokens, t.new_tokens, false);
      const uint32_t d_layer_ntpb = v.o.d_ntpb / v.pack;
      const uint32_t end = static_cast<uint32_t>(db.size()) * d_layer_ntpb;
      if (pad && total < end && k.ops()) {
        const size_t d_kbs = d_kb * v.o.d_tok, d_step = v.o.d_tok / 2;
        RTASSERT(d_layer_ntpb % d_kb == 0);
        const Sink::Side d{&db, d_layer_ntpb, d_kb, v.o.d_bs, v.pack * d_kbs, d_step, 0};
        k.op(nullptr, d, total, end, d_step, {{v.pack, 0, d_kbs}, {2, 0, d_kbs / 2}});
      } else if (pad && total < end) {
        const size_t d_kbs = d_kb * v.o.d_tok, d_step = v.o.d_tok / 2;
        const size_t zero_src = at(sb, 0) * v.o.p_bs;
        for (uint32_t pos = total; pos < end;) {
          const uint32_t d_i = pos % d_kb;
          const uint32_t run = std::min(d_kb - d_i, end - pos);
          const size_t d0 = at(db, pos / d_layer_ntpb) * v.o.d_bs +
                            static_cast<size_t>((pos % d_layer_ntpb) / d_kb) * v.pack * d_kbs;
          for (uint32_t sub = 0; sub < v.pack; ++sub) {
            const size_t dk = d0 + sub * d_kbs + d_i * d_step;
            zero_fill(k, zero_src, dk, static_cast<size_t>(run) * d_step, v.o.p_bs);
            zero_fill(k, zero_src, dk + d_kbs / 2, static_cast<size_t>(run) * d_step, v.o.p_bs);
          }
          pos += run;
        }
      }
    }
  }
  if (t.reach_last_token) {
    gdn_split(k, v.o.p_bs, v.o.d_bs, v.n_gdn, gdn_n, gdn_off, *e.src, t.src_blocks(), t.dst_blocks());
    ple_pages(k, v.o.p_bs, v.o.d_bs, *e.src, t.src_blocks(), t.dst_blocks(), false, false);
  }
}

void hyb_nhd_eq(const PlanEnv& e, const ReqSendTask& t, PlanOut& o) { hybrid_eq(e, t, o, false); }
void hyb_nhd_gt(const PlanEnv& e, const ReqSendTask& t, PlanOut& o) { hybrid_gt(e, t, o, false); }
void hyb_nhd_lt(const PlanEnv& e, const ReqSendTask& t, PlanOut& o) { hybrid_lt(e, t, o, false); }
void hyb_hnd_eq(const PlanEnv& e, const ReqSendTask& t, PlanOut& o) { hybrid_eq(e, t, o, true); }
void hyb_hnd_gt(const PlanEnv& e, const ReqSendTask& t, PlanOut& o) { hybrid_gt(e, t, o, true); }
void hyb_hnd_lt(const PlanEnv& e, const ReqSendTask& t, PlanOut& o) { hybrid_lt(e, t, o, true); }

}  // namespace

// Defined in kda_planner.cpp (shape 8: KDA state pages + replicated MLA prefix).
void kda_k3_eq(const PlanEnv&, const ReqSendTask&, PlanOut&);
void kda_k3_gt(const PlanEnv&, const ReqSendTask&, PlanOut&);
void kda_k3_lt(const PlanEnv&, const ReqSendTask&, PlanOut&);

PlannerChoice bind_planner(PlanEnv& env) {
  RTASSERT(env.src != nullptr && env.dst != nullptr);
  const WorkerInfo& src = *env.src;
  const WorkerInfo& dst = *env.dst;
  env.valid_ranks = compute_valid_ranks_pd(src.engine_tp_size, dst.engine_tp_size, src.num_kv_heads);
  env.kvt_tp_size = static_cast<uint32_t>(env.valid_ranks.count());
  uint32_t below = 0;
  for (uint32_t i = 0; i < src.worker_tp_rank && i < MAX_TP_SIZE; ++i) below += env.valid_ranks[i] ? 1 : 0;
  env.kvt_tp_rank = below;
  const int shape = env.cache_shape;
  // Shapes that carry recurrent state group by the engine TP (state is sharded by it); the
  // others compare the effective attention TP with the destination TP.
  const bool by_engine_tp = shape == QWEN3_NEXT_FLASH_CACHE_SHAPE || shape == QWEN3_NEXT_FLASHINFER_CACHE_SHAPE ||
                            shape == KIMI_K3_MLA_CACHE_SHAPE;
  const uint32_t p_tp = by_engine_tp ? src.engine_tp_size : env.kvt_tp_size;
  const uint32_t d_tp = dst.engine_tp_size;
  const int rel = p_tp == d_tp ? 0 : (p_tp > d_tp ? 1 : -1);
  auto pick = [&](PlanFn eq, PlanFn gt, PlanFn lt, const char* name) -> PlannerChoice {
    if (rel == 0) return {eq, TPKind::PEQD, name};
    if (rel > 0 && gt != nullptr) return {gt, TPKind::PGTD, name};
    if (rel < 0 && lt != nullptr) return {lt, TPKind::PLTD, name};
    throw std::runtime_error("unsupported cache_shape");
  };
  switch (shape) {
    case RAGGED_FLASH_CACHE_SHAPE:
      if (rel > 0 && src.token_sizes == dst.token_sizes) return {ragged_gt_replicated, TPKind::PEQD, "ragged"};
      return pick(ragged_eq, ragged_gt, ragged_lt, "ragged");
    case FLASH_CACHE_SHAPE:
      return pick(flash_eq, flash_gt, flash_lt, "flash");
    case FLASHINFER_CACHE_SHAPE:
      return pick(hnd_eq, hnd_gt, hnd_lt, "flashinfer");
    case DPSK_V32_SPARSE_MLA_SHAPE: {
      PlannerChoice c = pick(multi_eq, multi_gt, multi_lt, "dpsk_v32");
      c.kind = TPKind::PEQD;  // pieces are whole-token runs in every relation
      return c;
    }
    case QWEN3_NEXT_FLASH_CACHE_SHAPE:
      return pick(hyb_nhd_eq, hyb_nhd_gt, hyb_nhd_lt, "qwen3_next");
    case TURBOQUANT_CACHE_SHAPE:
      return pick(hyb_nhd_eq, hyb_nhd_gt, nullptr, "turboquant");
    case QWEN3_NEXT_FLASHINFER_CACHE_SHAPE:
      return pick(hyb_hnd_eq, hyb_hnd_gt, hyb_hnd_lt, "qwen3_next_flashinfer");
    case KIMI_K3_MLA_CACHE_SHAPE:
      return pick(kda_k3_eq, kda_k3_gt, kda_k3_lt, "kimi_k3");
    default:
      throw std::runtime_error("unsupported cache_shape");
  }
}

MergeStats merge_interval(std::vector<IpcBlock>& v) {
  if (v.empty()) return {0, 0, 0, 0};
  std::sort(v.begin(), v.end(), [](const IpcBlock& a, const IpcBlock& b) { return a.src_offset < b.src_offset; });
  size_t w = 0;
  for (size_t i = 1; i < v.size(); ++i) {
    IpcBlock& cur = v[w];
    const IpcBlock& nx = v[i];
    if (cur.src_offset + cur.length == nx.src_offset && cur.dst_offset + cur.length == nx.dst_offset) {
      cur.length += nx.length;
    } else {
      v[++w] = nx;
    }
  }
  v.erase(v.begin() + static_cast<std::ptrdiff_t>(w) + 1, v.end());
  MergeStats st{std::numeric_limits<size_t>::max(), 0, 0, v.size()};
  for (const auto& b : v) {
    st.min_len = std::min(st.min_len, b.length);
    st.max_len = std::max(st.max_len, b.length);
    st.total_len += b.length;
  }
  return st;
}

void validate_ipc_block_bounds(const std::vector<IpcBlock>& blocks, size_t capacity, IpcBlockOffset kind,
                               const char* copy_path, size_t layer_idx, size_t tensor_idx, size_t length_scale) {
  for (size_t i = 0; i < blocks.size(); ++i) {
    const IpcBlock& b = blocks[i];
    const size_t off = kind == IpcBlockOffset::SOURCE ? b.src_offset : b.dst_offset;
    const bool overflow = length_scale == 0 || b.length > std::numeric_limits<size_t>::max() / length_scale;
    const size_t eff = overflow ? std::numeric_limits<size_t>::max() : b.length * length_scale;
    if (b.length == 0 || overflow || off > capacity || eff > capacity - off) {
      LOG(ERROR) << "KVT GPU buffer range validation failed,copy_path=" << copy_path << ",layer_idx=" << layer_idx
                 << ",tensor_idx=" << tensor_idx << ",block_idx=" << i
                 << ",offset_kind=" << (kind == IpcBlockOffset::SOURCE ? "src" : "dst") << ",offset=" << off
                 << ",length=" << b.length << ",length_scale=" << length_scale << ",capacity=" << capacity;
      throw std::out_of_range("KVT GPU buffer range validation failed");
    }
  }
}

}  // namespace kvx
