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
#include "kernels/kvt_kernels.h"

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

// Where a planner function writes: byte ranges per cache tensor (the CPU product: host transports, oracle)
// or walk ops (the device product: a handful of affine rules per request that the walk kernel expands
// while it copies, kernels/kvt_kernels.h).  One planner serves both, so the TP relations, group offsets and
// chunk policies of every cache shape exist once.
struct WalkPlan {
  std::vector<KvtWalkOp> ops;
  std::vector<uint32_t> pool;          // block tables referenced by the ops
  // after finalize(): ops = [n_bulk through the TMA engine][n_simt through the SIMT warps][n_zero zero fills, which
  // a second launch writes after the copies]
  uint32_t n_bulk = 0, n_simt = 0, n_zero = 0;
  uint64_t bulk_units = 0, simt_units = 0, zero_units = 0;
  uint64_t bytes = 0;                  // payload bytes of one layer (all tensors)
  void clear() {
    ops.clear();
    pool.clear();
    n_bulk = n_simt = n_zero = 0;
    bulk_units = simt_units = zero_units = bytes = 0;
  }
  // Orders the ops by class, fills their unit bookkeeping and checks every table entry against the block
  // counts of the two caches (std::out_of_range otherwise).
  void finalize(uint32_t src_num_blocks, uint32_t dst_num_blocks);
  bool empty() const { return ops.empty(); }
};

struct PlanOut {
  std::vector<std::vector<IpcBlock>>* blocks{nullptr};   // exactly one of the two is set
  WalkPlan* walk{nullptr};
  // block tables of the request being planned that are already in walk->pool: (data pointer, pool offset)
  std::vector<std::pair<const uint32_t*, uint32_t>> tables;
};

using PlanFn = void (*)(const PlanEnv&, const ReqSendTask&, PlanOut&);

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
  PlanOut out;
  out.blocks = &send_blocks;
  c.fn(env, task, out);
}

// The same chunk as walk ops, appended to `plan` (call plan.finalize() after the last request).
inline void plan_request_ops(const PlannerChoice& c, const PlanEnv& env, const ReqSendTask& task, WalkPlan& plan) {
  PlanOut out;
  out.walk = &plan;
  c.fn(env, task, out);
}

// Host expansion of walk ops into byte ranges, with the kernel's own unit decode: what the device walk
// moves, as data.  Every piece is checked against the tensors' capacities (std::out_of_range).
struct WalkPiece {
  uint32_t tensor;
  bool zero;        // destination bytes are zero-filled; src_offset is unused
  uint64_t src_offset, dst_offset, length;
};
std::vector<WalkPiece> expand_walk_plan(const WalkPlan& plan, const std::vector<uint64_t>& src_caps,
                                        const std::vector<uint64_t>& dst_caps);

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
