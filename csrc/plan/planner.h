// Transfer planner: turns one request chunk into the list of byte ranges to move.
//
// Two consumers use it.  Host-driven transports (TCP, shared memory, pinned store) ship the
// IpcBlock list itself; it is also the CPU oracle every device kernel is tested against.  The
// NVLink transport instead asks `device_attn_params()` for the (layout, head window, mode)
// that the fused kernel needs and lets the kernel do the same walk on the GPU.
//
// The offset rules are those of the reference's ParseBlock family (kvtransfer/src/
// parse_block_*.cpp; summarised in kvtransfer/docs/cache_transfer_spec.md:200-478).  They are
// written here as a handful of generic walkers (token runs, per-token slices, per-head HND
// runs, block-aligned pages, strided state rows) combined per cache shape, instead of one
// function per shape and TP relation.
#pragma once
#include <bitset>
#include <vector>

#include "core/envcfg.h"
#include "core/types.h"

namespace kvx {

using RankSet = std::bitset<MAX_TP_SIZE>;

// Which prefill ranks carry unique KV heads for a given decode TP (GQA replication aware).
// Truth table: kvtransfer/src/tx_stub.cpp:18-81.
RankSet compute_valid_ranks_pd(uint32_t p_tp, uint32_t d_tp, int num_kv_heads);

struct PlanEnv {
  const WorkerInfo* src{nullptr};
  const WorkerInfo* dst{nullptr};
  RankSet valid_ranks;
  uint32_t kvt_tp_size{0};   // effective prefill TP after valid_ranks filtering
  uint32_t kvt_tp_rank{0};   // index of src rank inside valid_ranks
  int cache_shape{RAGGED_FLASH_CACHE_SHAPE};
  bool cast_bf16_to_fp8{false};   // unscaled cast of the staged path (lengths are fp8 bytes)
  bool pad_last_attn_block{true};
};

using PlanFn = void (*)(const PlanEnv&, const ReqSendTask&, std::vector<std::vector<IpcBlock>>&);

struct PlannerChoice {
  PlanFn fn{nullptr};
  TPKind kind{TPKind::UNKNOWN};
  const char* name{""};
};

// Fills env.valid_ranks / kvt_tp_size / kvt_tp_rank from src and dst and picks the planner for
// (cache shape, TP relation).  Throws std::runtime_error for unsupported combinations.
PlannerChoice bind_planner(PlanEnv& env);

// Plan one chunk; appends to send_blocks[tensor].  Every range is bounds-checked against the
// registered tensor capacities before it is appended (std::out_of_range otherwise).
inline void plan_request(const PlannerChoice& c, const PlanEnv& env, const ReqSendTask& task,
                         std::vector<std::vector<IpcBlock>>& send_blocks) {
  c.fn(env, task, send_blocks);
}

// Sort by source offset and coalesce ranges adjacent on both sides.
// Returns (min_len, max_len, total_len, count) of the merged list.
struct MergeStats {
  size_t min_len, max_len, total_len, count;
};
MergeStats merge_interval(std::vector<IpcBlock>& blocks);

enum class IpcBlockOffset { SOURCE, DESTINATION };
void validate_ipc_block_bounds(const std::vector<IpcBlock>& blocks, size_t capacity, IpcBlockOffset kind,
                               const char* copy_path, size_t layer_idx, size_t tensor_idx, size_t length_scale = 1);

}  // namespace kvx
