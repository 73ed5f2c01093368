// Transport interface of the send path.
//
// A send stub drives a channel through one batch as
//   connect(dst) -> register_tasks(...) | register_data(...) -> send_data(layer) x L -> flush()
// exactly like the reference's IChannel (kvtransfer/include/channel.h:59-83), with two
// additions for device transports: register_tasks() hands over the *requests* so that the
// block-table walk can run inside the transfer kernel instead of on the CPU, and
// device_ordered() says that send_data(layer) only needs the layer's event to be recorded,
// not completed (the channel orders its own stream after the event).
#pragma once
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "core/context.h"
#include "core/step.h"
#include "plan/planner.h"

namespace kvx {

class IChannel {
 public:
  virtual void connect(const WorkerInfo& dst_info) = 0;
  // Device-planned path.  Return false to make the stub fall back to register_data().
  virtual bool register_tasks(const PlanEnv& env, const std::vector<const ReqSendTask*>& tasks) {
    (void)env; (void)tasks;
    return false;
  }
  // Host-planned path: per cache tensor, the byte ranges to move.  The channel takes the data.
  virtual void register_data(std::vector<std::vector<IpcBlock>>& data, TPKind kind) = 0;
  virtual bool device_ordered() const { return false; }
  // May be asynchronous; flush() blocks until every send_data of the batch has landed.
  virtual void send_data(size_t layer_index, Step* step) = 0;
  // Every layer of [begin, end) at once, for steps whose data is already complete.  Return
  // false to be driven layer by layer through send_data().
  virtual bool send_layers(size_t layer_begin, size_t layer_end, Step* step) {
    (void)layer_begin; (void)layer_end; (void)step;
    return false;
  }
  // Layers [layer_begin, layer_end) are all ready (device ordered: all recorded).  Sends the first one
  // or, when one launch can carry several, the first few; returns how many it took (>= 1).
  virtual size_t send_range(size_t layer_begin, size_t layer_end, Step* step) {
    (void)layer_end;
    send_data(layer_begin, step);
    return 1;
  }
  // `out` receives key=value metrics of the batch.
  virtual void flush(std::string& out) = 0;
  // Device transports complete a batch without a host wait: flush_async() enqueues a completion record
  // behind the batch and returns its ticket at once; poll_completion() says whether that record has
  // arrived (DONE: `out` receives the metrics; FAILED: `out` says why).  Tickets complete in order.
  virtual bool async_flush() const { return false; }
  virtual uint64_t flush_async() { return 0; }
  virtual PollResult poll_completion(uint64_t ticket, std::string& out) {
    (void)ticket; (void)out;
    return PollResult::DONE;
  }
  virtual bool is_active() { return true; }
  // Can the destination relay a request to its NVLink multicast group (RequestInfo::replicas > 1)?
  virtual bool relays_to_group() const { return false; }
  virtual void close() {}
  virtual const char* name() const = 0;
  virtual ~IChannel() = default;
};

using Channel = std::shared_ptr<IChannel>;   // a batch still completing keeps its channel alive

class IChannelFactory {
 public:
  virtual ~IChannelFactory() = default;
  virtual Channel create(const WorkerInfo& dst_info) = 0;
};

// Picks the best protocol both sides support: NVLINK (same host, GPU caches) > SHM (same host)
// > TCP.  A fixed protocol can be forced (tests, BLLM_KVTRANS protocol lists).
class ChannelFactory : public IChannelFactory {
 public:
  ChannelFactory(Context* ctx, std::optional<TransferProtocol> proto) : ctx_(ctx), proto_(proto) {}
  Channel create(const WorkerInfo& dst_info) override;

 private:
  Context* const ctx_;
  const std::optional<TransferProtocol> proto_;
};

Channel make_tcp_channel(Context* ctx, bool use_shm);
Channel make_nvlink_channel(Context* ctx);

// Receiving side.
class ITransferServer {
 public:
  virtual void start_server(Context* ctx) = 0;
  virtual int port() const = 0;
  virtual void stop() = 0;
  virtual ~ITransferServer() = default;
};
std::unique_ptr<ITransferServer> create_transfer_server();

// Where a channel finds the destination's server: WorkerInfo.addr and ext "port"
// (fallback BLLM_KVTRANS_PORT_BASE + worker_id).
int server_port_of(const WorkerInfo& w);

}  // namespace kvx
