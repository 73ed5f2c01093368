// Common value types of the engine: WorkerInfo (the string every worker advertises),
// request / task records, IpcBlock, transfer-protocol flags and the always-on assert macros.
//
// WorkerInfo keeps the comma-separated wire form of the reference (11-14 fields with its
// back-compat rules, kvtransfer/src/common.cpp:50-145).  This engine appends one optional
// trailing field "x:k=v;k=v" carrying what a Blackwell-native transfer needs to know about
// the destination: its cache-shape id (so NHD->HND conversion is possible), device ordinal,
// process id, host id, the control port of its server and whether its pages are block-scaled
// fp8.  A reader that does not know the field can drop any trailing token that starts "x:".
#pragma once
#include <atomic>
#include <cstdint>
#include <map>
#include <memory>
#include <optional>
#include <ostream>
#include <stdexcept>
#include <string>
#include <vector>

#include "core/log.h"

namespace kvx {

constexpr size_t MAX_INSTANCE_NAME_LEN = 256;
constexpr size_t MAX_ADDRESS_LEN = 64;
constexpr uint32_t INVALID_INST_WORKER_ID = 0xffffffffu;

class RtAssertError : public std::logic_error {
 public:
  using std::logic_error::logic_error;
};

[[noreturn]] void rtassert_fail(const char* file, int line, const char* expr, const std::string& detail);

// Release-active checks (role of RTASSERT/RTCHECK, kvtransfer/include/common.h:38-82): they
// throw instead of aborting so that a Python caller sees an exception.
#define RTASSERT(cond)                                                   \
  do {                                                                   \
    if (!(cond)) ::kvx::rtassert_fail(__FILE__, __LINE__, #cond, "");   \
  } while (0)
#define RTCHECK(cond) RTASSERT(cond)
#define RTASSERT_EQ(a, b)                                                                          \
  do {                                                                                             \
    if (!((a) == (b))) {                                                                           \
      std::ostringstream _ss;                                                                      \
      _ss << (a) << " vs " << (b);                                                                 \
      ::kvx::rtassert_fail(__FILE__, __LINE__, #a " == " #b, _ss.str());                          \
    }                                                                                              \
  } while (0)

typedef std::string InstanceId;
typedef uint32_t WorkerId;
typedef std::string RequestId;
// Outer index = KV-cache group (hybrid models have several), inner = block ids of the request.
using BlockIds = std::vector<std::vector<uint32_t>>;

struct TransferProtocol {
  // Bit flags; serialised into WorkerInfo as a u8 mask.  1 and 2 are the reference's values
  // (kvtransfer/include/protocol.h:13-16); NVLINK and SHM are additions of this engine.
  enum Kind : uint8_t { UNKNOWN = 0, RDMA_DIRECT = 1, TCP = 2, NVLINK = 4, SHM = 8 };
  Kind type{UNKNOWN};
  TransferProtocol() = default;
  explicit TransferProtocol(Kind k) : type(k) {}
  std::string to_string() const;
  static TransferProtocol from_string(const std::string& s);
  bool operator==(const TransferProtocol& o) const { return type == o.type; }
};

struct WorkerInfo {
  InstanceId inst_id;
  WorkerId worker_id{INVALID_INST_WORKER_ID};
  uint32_t engine_tp_size{0};
  uint32_t worker_tp_rank{0};
  std::vector<size_t> block_sizes;
  std::vector<size_t> token_sizes;
  uint32_t layer_num_blocks{1};
  uint32_t num_layers{1};
  uint8_t transfer_protocols{0};
  uint32_t attn_kernel_blk_ntpb{0};
  uint32_t indexer_blk_ntpb{0};
  uint32_t attn_pack_size{1};
  uint64_t kda_page_stride{0};
  std::string addr;
  // "x:" extension (serialised when non-empty)
  std::map<std::string, std::string> ext;

  // local-only, not serialised
  int num_kv_heads{-1};
  uint32_t num_gdn_layers{3};
  uint32_t hybrid_indexer_token_size{0};
  uint32_t gdn_conv_elem_size{1};
  uint32_t gdn_ssm_elem_size{1};
  std::vector<size_t> conv_state_shape;
  std::vector<size_t> ssm_state_shape;
  std::vector<size_t> gdn_conv_channel_dims;
  uint32_t num_ple_layers{0};
  uint32_t ple_block_group{0};
  uint32_t ple_conv_elem_size{1};
  std::vector<size_t> ple_conv_state_shape;
  std::vector<size_t> ple_conv_channel_dims;
  bool kda_conv_dim_first{false};
  uint32_t hybrid_attn_token_size{0};

  WorkerInfo() = default;
  WorkerInfo(InstanceId id, WorkerId wid) : inst_id(std::move(id)), worker_id(wid), engine_tp_size(1),
                                            block_sizes({16 * 1024}), token_sizes({1024}) {}
  WorkerInfo(InstanceId id, WorkerId wid, uint32_t tp, uint32_t rank, std::vector<size_t> bsz,
             std::vector<size_t> tsz, uint32_t nblocks, uint32_t nlayers, uint32_t protocols)
      : inst_id(std::move(id)), worker_id(wid), engine_tp_size(tp), worker_tp_rank(rank),
        block_sizes(std::move(bsz)), token_sizes(std::move(tsz)), layer_num_blocks(nblocks), num_layers(nlayers),
        transfer_protocols(static_cast<uint8_t>(protocols)) {}

  static WorkerInfo from_string(const std::string& src);
  [[nodiscard]] std::string to_string() const;

  // ext accessors
  int ext_int(const std::string& key, int def) const;
  std::string ext_str(const std::string& key, const std::string& def = "") const;
  int cache_shape_or(int def) const { return ext_int("shape", def); }
};

struct IpcBlock {
  size_t src_offset;
  size_t dst_offset;
  size_t length;
  IpcBlock(size_t s, size_t d, size_t l) : src_offset(s), dst_offset(d), length(l) {}
  bool operator==(const IpcBlock& o) const {
    return src_offset == o.src_offset && dst_offset == o.dst_offset && length == o.length;
  }
};
static_assert(sizeof(IpcBlock) == 24, "IpcBlock is memcpy'd onto the wire as 3 x size_t");

inline std::ostream& operator<<(std::ostream& os, const IpcBlock& b) {
  return os << "IpcBlock(src=" << b.src_offset << ",dst=" << b.dst_offset << ",len=" << b.length << ")";
}

enum class TPKind { PEQD, PLTD, PGTD, UNKNOWN };

enum class ReqState : int { INPROCESS = 0, OK = 1, FAILED = 2 };

// Immutable description of one request's transfer target; shared by all chunks of the request.
class RequestInfo {
 public:
  const InstanceId dst_inst_id;
  const WorkerId dst_worker_id;
  const std::optional<WorkerInfo> dst_worker_info;
  const RequestId req_id;
  const BlockIds src_blocks;
  const BlockIds dst_blocks;
  // Members of the destination's multicast group that this one transfer serves (1: only dst_worker_id).  With k > 1
  // the destination worker relays the bytes to its whole group and the send-done report counts k times, one for
  // each worker that a sender without the relay would have served.  Set before the first chunk is queued.
  uint32_t replicas{1};

  RequestInfo(InstanceId dst_inst, WorkerId dst_worker, std::optional<WorkerInfo> dst_info, RequestId rid,
              BlockIds src, BlockIds dst)
      : dst_inst_id(std::move(dst_inst)), dst_worker_id(dst_worker), dst_worker_info(std::move(dst_info)),
        req_id(std::move(rid)), src_blocks(std::move(src)), dst_blocks(std::move(dst)) {}
  RequestInfo(InstanceId dst_inst, WorkerId dst_worker, RequestId rid, BlockIds src, BlockIds dst)
      : RequestInfo(std::move(dst_inst), dst_worker, std::nullopt, std::move(rid), std::move(src), std::move(dst)) {}
  RequestInfo(const RequestInfo&) = delete;

  ReqState state() const noexcept { return state_.load(std::memory_order_acquire); }
  void set_state(ReqState s) const noexcept { state_.store(s, std::memory_order_release); }

 private:
  mutable std::atomic<ReqState> state_{ReqState::INPROCESS};
};

// One chunk [seen, seen+new) of a request scheduled in one step.
class ReqSendTask {
  std::shared_ptr<RequestInfo> req_;

 public:
  uint32_t seen_tokens{0};
  uint32_t new_tokens{0};
  bool reach_last_token{false};

  ReqSendTask(std::shared_ptr<RequestInfo> req, uint32_t seen, uint32_t new_toks, bool last)
      : req_(std::move(req)), seen_tokens(seen), new_tokens(new_toks), reach_last_token(last) {}

  void set_state(ReqState s) const noexcept { req_->set_state(s); }
  ReqState state() const noexcept { return req_->state(); }
  const RequestId& req_id() const noexcept { return req_->req_id; }
  const BlockIds& dst_blocks() const noexcept { return req_->dst_blocks; }
  const BlockIds& src_blocks() const noexcept { return req_->src_blocks; }
  const InstanceId& dst_inst_id() const noexcept { return req_->dst_inst_id; }
  WorkerId dst_worker_id() const noexcept { return req_->dst_worker_id; }
  uint32_t end_tokens() const noexcept { return seen_tokens + new_tokens; }
  const RequestInfo& req() const noexcept { return *req_; }
  const std::shared_ptr<RequestInfo>& req_ptr() const noexcept { return req_; }
  bool operator==(const ReqSendTask& o) const {
    return req_ == o.req_ && seen_tokens == o.seen_tokens && new_tokens == o.new_tokens &&
           reach_last_token == o.reach_last_token;
  }
};

std::string block_ids_to_string(const BlockIds& ids);

// Engine-level exception surfaced to Python as KVTransferError.
enum class ErrorKind { INVALID_OPERATION, TRANSPORT, NAMING, CUDA, TIMEOUT };
class KVTransferException : public std::runtime_error {
 public:
  KVTransferException(ErrorKind k, const std::string& msg) : std::runtime_error(msg), kind(k) {}
  const ErrorKind kind;
};

uint64_t new_id();  // process-wide monotone id, starts at 20181218 like the reference's id generator

}  // namespace kvx
