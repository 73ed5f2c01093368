// Bridge from the engine's WorkerInfo / PlanEnv world to the fused transfer kernel's
// parameters: cache layouts as byte strides, the head window of a TP-mismatched pair, the
// dtype path and the packed per-request descriptors.
#pragma once
#include <string>
#include <vector>

#include "kernels/kvt_kernels.h"
#include "plan/planner.h"

namespace kvx {

// Byte-stride layout of cache tensor 0 of a worker for an attention cache shape (ids 1, 2, 5).
// `mx_scaled`: the pages are block-scaled e4m3 (payload + one UE8M0 scale per 32 values).
// `head_bytes_hint`: payload bytes of one (token, head) row when it cannot be derived
// (0 = derive from token size and num_kv_heads).  Returns false for shapes the fused kernel
// does not describe (hybrid pages, multi-tensor) - those use the descriptor-driven path.
bool attn_layout_from_worker(const WorkerInfo& w, int cache_shape, bool mx_scaled, uint32_t head_bytes_hint,
                             KvtLayout* out);

struct DeviceAttnParams {
  KvtLayout src, dst;
  uint32_t src_head0, dst_head0, n_heads;
  uint32_t mode;          // KvtMode
  uint32_t tile_tokens;
  bool skip;              // this prefill rank holds only replicas: nothing to send
};

// Fills the parameters for one (src worker, dst worker) pair; returns false when the fused
// kernel cannot serve this pair (caller falls back to IpcBlock descriptors).
bool device_attn_params(const PlanEnv& env, TPKind kind, int src_shape, int dst_shape, bool dst_mx,
                        DeviceAttnParams* out, std::string* why);

// Packs request chunks into [KvtReqDesc x n][uint32 block ids]; returns total tiles.
struct PackedPlan {
  std::vector<char> blob;
  uint32_t n_reqs{0};
  uint32_t total_tiles{0};
  size_t pool_offset{0};
};
PackedPlan pack_device_plan(const std::vector<const ReqSendTask*>& tasks, size_t group, uint32_t tile_tokens,
                            uint32_t dst_ntpb, bool pad_tail);

}  // namespace kvx
