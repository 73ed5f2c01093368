// Decode side of a pull transfer.  One session serves one prefill worker's channel: it maps that worker's
// cache tensors and layer events, owns a BatchEngine on the decode GPU whose source is the mapped prefill
// cache and whose destination is this worker's own cache, and executes the channel's messages in order:
//
//   plan    the batch's request descriptors / walk ops and block tables -> a plan slot on this GPU
//   layers  make a transfer stream wait for the prefill GPU's layer event (a CUDA IPC event: ordered on the
//           device, nobody's host waits for the forward pass) and launch the layer's kernel(s) behind it
//   flush   enqueue the completion record; when it arrives the session answers PULL_DONE on the connection
//
// Loads over NVLink by the TMA engine run at the copy engine's rate, which stores issued by an SM do not
// reach; and the prefill GPU spends no SM on the transfer.  Only plain (non-multicast) loads are used.
#pragma once
#include <memory>
#include <mutex>
#include <string>

#include "core/context.h"
#include "transport/batch_engine.h"
#include "transport/peer_memory.h"

namespace kvx {

constexpr uint32_t PULL_KIND_ATTN = 0, PULL_KIND_WALK = 1;

// Fixed-size head of a PULL_PLAN_REQ body; the plan blob follows.
struct PullPlanHead {
  uint32_t kind;
  uint32_t n_ops;            // walk
  uint32_t pool_len;         // walk
  uint32_t n_reqs;           // attn
  uint32_t total_tiles;      // attn
  uint32_t fanout;           // walk: replicate what the ops wrote to the destination's multicast group
  uint64_t pool_offset;      // attn
  uint64_t blob_bytes;
  KvtWalkCounts walk;
  DeviceAttnParams attn;
};

inline uint32_t pull_protocol_version() {
  return static_cast<uint32_t>(sizeof(PullPlanHead) ^ (sizeof(KvtWalkOp) << 12) ^ (sizeof(KvtReqDesc) << 24)) ^ 0x20250001u;
}

class PullSession : public std::enable_shared_from_this<PullSession> {
 public:
  // `fd` is the connection PULL_DONE frames are written to, under `write_mu`.
  PullSession(Context* ctx, int fd, std::shared_ptr<std::mutex> write_mu);
  ~PullSession();
  // Returns a wire status.  body: what follows the RPC header of PULL_OPEN_REQ.
  uint32_t open(const char* body, size_t len);
  void on_plan(uint64_t seq, const char* body, size_t len);
  void on_layers(uint64_t seq, const char* body, size_t len);
  void on_flush(uint64_t seq, const char* body, size_t len);
  void close();   // the connection went away

 private:
  void send_done(uint64_t seq, uint32_t status, uint32_t detail, uint64_t t0, uint64_t t1);
  Context* ctx_;
  int fd_;
  std::shared_ptr<std::mutex> write_mu_;
  std::atomic<bool> closed_{false};
  PeerMapping src_map_;
  PeerEvents ev_info_;
  std::vector<void*> events_;
  std::unique_ptr<BatchEngine> eng_;
  // the batch being assembled
  uint64_t cur_seq_{0};
  bool have_batch_{false};
  PullPlanHead head_{};
  PackedPlan attn_plan_;
  std::string error_;          // a message of this batch failed: reported with its PULL_DONE
  std::atomic<int> pending_{0};
};

}  // namespace kvx
