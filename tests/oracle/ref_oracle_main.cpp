// Test-only driver around the reference's ParseBlock functions, compiled at test time from the
// reference checkout when one is present.  Reads one scenario from stdin, prints the IpcBlocks.
// This file contains no reference code: it only calls the functions declared in the
// reference's parse_block_common.h.
#include <bitset>
#include <iostream>
#include <map>
#include <string>
#include <vector>

#include "parse_block_common.h"
#include "parse_block_turboquant.h"

using namespace blade_llm;

static std::vector<size_t> read_vec(std::istream& in) {
  size_t n;
  in >> n;
  std::vector<size_t> v(n);
  for (auto& x : v) in >> x;
  return v;
}

static WorkerInfo read_worker(std::istream& in) {
  WorkerInfo w;
  in >> w.inst_id >> w.worker_id >> w.engine_tp_size >> w.worker_tp_rank;
  w.block_sizes = read_vec(in);
  w.token_sizes = read_vec(in);
  in >> w.layer_num_blocks >> w.attn_kernel_blk_ntpb >> w.indexer_blk_ntpb >> w.attn_pack_size >> w.kda_page_stride;
  in >> w.num_kv_heads >> w.num_gdn_layers >> w.hybrid_indexer_token_size >> w.gdn_conv_elem_size >>
      w.gdn_ssm_elem_size;
  w.conv_state_shape = read_vec(in);
  w.ssm_state_shape = read_vec(in);
  w.gdn_conv_channel_dims = read_vec(in);
  in >> w.num_ple_layers >> w.ple_block_group >> w.ple_conv_elem_size;
  w.ple_conv_state_shape = read_vec(in);
  int dim_first;
  in >> dim_first >> w.hybrid_attn_token_size;
  w.kda_conv_dim_first = dim_first != 0;
  return w;
}

static BlockIds read_blocks(std::istream& in) {
  size_t g;
  in >> g;
  BlockIds ids(g);
  for (auto& grp : ids) {
    size_t n;
    in >> n;
    grp.resize(n);
    for (auto& b : grp) in >> b;
  }
  return ids;
}

int main() {
  static const std::map<std::string, ParseBlockFunc> fns = {
      {"ragged_eq", parse_block_send_p_eq_d},
      {"ragged_gt", parse_block_send_p_gt_d},
      {"ragged_gt_dpsk", parse_block_send_p_gt_d_dpsk},
      {"ragged_lt", parse_block_send_p_lt_d},
      {"flash_eq", vllm_parse_block_send_p_eq_d},
      {"flash_gt", vllm_parse_block_send_p_gt_d},
      {"hnd_eq", vllm_parse_flashinfer_block_send_p_eq_d},
      {"hnd_gt", vllm_parse_flashinfer_block_send_p_gt_d},
      {"multi_eq", vllm_parse_block_send_multi_tensor_p_eq_d},
      {"multi_gt", vllm_parse_block_send_multi_tensor_p_gt_d},
      {"multi_lt", vllm_parse_block_send_multi_tensor_p_lt_d},
      {"hyb_nhd_eq", vllm_parse_hybrid_block_send_p_eq_d_block_aligned},
      {"hyb_nhd_gt", vllm_parse_hybrid_block_send_p_gt_d},
      {"hyb_nhd_lt", vllm_parse_hybrid_block_send_p_lt_d},
      {"hyb_hnd_eq", vllm_parse_qwen3_next_flashinfer_block_send_p_eq_d},
      {"hyb_hnd_gt", vllm_parse_qwen3_next_flashinfer_block_send_p_gt_d},
      {"hyb_hnd_lt", vllm_parse_qwen3_next_flashinfer_block_send_p_lt_d},
      {"k3_eq", parse_kimi_k3_mla_block_send_p_eq_d},
      {"k3_gt", parse_kimi_k3_mla_block_send_p_gt_d},
      {"k3_lt", parse_kimi_k3_mla_block_send_p_lt_d},
      {"tq_eq", turboquant_parse_block_send_p_eq_d},
      {"tq_gt", turboquant_parse_block_send_p_gt_d},
  };
  std::string fn;
  std::string bits;
  uint32_t kvt_tp_size, kvt_tp_rank;
  std::cin >> fn >> bits >> kvt_tp_size >> kvt_tp_rank;
  auto it = fns.find(fn);
  if (it == fns.end()) {
    std::cerr << "unknown fn " << fn << "\n";
    return 2;
  }
  std::bitset<MAX_TP_SIZE> valid(bits);
  WorkerInfo src = read_worker(std::cin);
  WorkerInfo dst = read_worker(std::cin);
  size_t n_tasks;
  std::cin >> n_tasks;
  std::vector<std::vector<IpcBlock>> out;
  try {
    for (size_t i = 0; i < n_tasks; ++i) {
      std::string reqid;
      uint32_t seen, ntok;
      int last;
      std::cin >> reqid >> seen >> ntok >> last;
      BlockIds sb = read_blocks(std::cin);
      BlockIds db = read_blocks(std::cin);
      auto info = std::make_shared<RequestInfo>(dst.inst_id, dst.worker_id, reqid, sb, db);
      ReqSendTask task(info, seen, ntok, last != 0);
      it->second(&src, &dst, valid, kvt_tp_size, kvt_tp_rank, &task, out);
    }
  } catch (const std::exception& ex) {
    std::cout << "EXC " << ex.what() << "\n";
    return 0;
  }
  for (size_t t = 0; t < out.size(); ++t) {
    std::cout << "T " << t << " " << out[t].size() << "\n";
    for (const auto& b : out[t]) std::cout << b.src_offset << " " << b.dst_offset << " " << b.length << "\n";
  }
  return 0;
}
