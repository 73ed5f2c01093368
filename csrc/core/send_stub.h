// Per-destination sender.  One stub serves one (instance, worker) target: it resolves the
// destination's WorkerInfo, keeps the channel to it, turns a batch of request chunks into a
// transfer (device-planned or host-planned), paces it layer by layer against the step's
// readiness counters and reports finished requests to the scheduler over the send-done RPC.
// Behaviour follows KvSendStub of the reference (kvtransfer/src/tx_stub.cpp:158-263,275-415):
// a failure anywhere in a batch marks every request of the batch FAILED and drops the channel
// so the next batch reconnects.
#pragma once
#include <memory>
#include <mutex>
#include <optional>
#include <vector>

#include "core/step.h"
#include "core/types.h"
#include "naming/naming.h"
#include "transport/channel.h"

namespace kvx {

struct BatchSendTask {
  BatchSendTask() = default;
  explicit BatchSendTask(std::shared_ptr<Step> s, uint32_t substep = 0) : step(std::move(s)), substepid(substep) {}
  std::shared_ptr<Step> step;
  std::vector<ReqSendTask> tasks;
  uint32_t substepid = 0;      // for logs
  Timepoint send_ts = SteadyClock::now();
  InflightCounter* inflight = nullptr;   // released once when the batch has been finished (sent or failed)
};

class ISendStub {
 public:
  ISendStub(InstanceId dstid, WorkerId dstworkerid) : dstid_(std::move(dstid)), dstworkerid_(dstworkerid) {}
  const InstanceId& dstid() const noexcept { return dstid_; }
  WorkerId dstworkerid() const noexcept { return dstworkerid_; }
  virtual void send_batch(BatchSendTask batch) = 0;
  // False while batches of this stub are still completing on a device (the stub must stay alive).
  virtual bool idle() const { return true; }
  virtual ~ISendStub() = default;

 protected:
  const InstanceId dstid_;
  const WorkerId dstworkerid_;
};
using SendStub = std::unique_ptr<ISendStub>;

class ISendStubFactory {
 public:
  virtual SendStub create_stub(const InstanceId& dst, WorkerId dst_worker, uint32_t start_layer, uint32_t num_layers,
                               std::optional<TransferProtocol> proto, const std::optional<WorkerInfo>& dst_info) = 0;
  virtual ~ISendStubFactory() = default;
};

// Sends "these requests finished (ok / failed)" to the scheduler.  Wire format of the
// reference's C++ stubs (kvtransfer/src/tx_stub.cpp:324-386): SEND_DONE_REQ 0x20181219,
// worker_tp_rank | HAS_VER2, n, then per request plen, code, rlen, reqid; optionally the same
// body again under SAVE_DONE2_REQ 0x20181223.  One reconnect-and-retry on a stale socket.
class SendDoneNotifier {
 public:
  // `addr` ("ip:port") overrides BLLM_KVTRANS_SEND_DONE_ADDR; empty = use the environment.
  explicit SendDoneNotifier(uint32_t worker_tp_rank, std::string addr = "") : rank_(worker_tp_rank), addr_(std::move(addr)) {}
  void notify(const std::vector<const ReqSendTask*>& reqs);
  static std::vector<char> encode(uint32_t worker_tp_rank, const std::vector<const ReqSendTask*>& reqs, int head_kind,
                                  int* resp_size);

 private:
  void round_trip(const std::vector<char>& buf, int resp_size);
  std::mutex mu_;   // the sender thread and the completion poller both report finished requests
  uint32_t rank_;
  std::string addr_;
  FdGuard sock_;
};

class KvSendStub : public ISendStub {
 public:
  KvSendStub(InstanceId dstid, WorkerId dstworkerid, const WorkerInfo& src_info, uint32_t start_layer,
             uint32_t num_layers, std::unique_ptr<IChannelFactory> channel_factory,
             std::shared_ptr<INamingWorkerClient> naming, int cache_shape, std::string send_done_addr = "");
  ~KvSendStub() override;
  void send_batch(BatchSendTask batch) noexcept override;
  bool idle() const override;
  // Turns the end-to-end check on (transport/verify.h): every batch whose transfer byte ranges can describe
  // is verified against the destination's cache before its requests are reported; a mismatch fails the batch.
  void enable_check(Context* ctx);

 private:
  struct Impl;
  std::unique_ptr<Impl> impl_;
};

class KvSendStubFactory : public ISendStubFactory {
 public:
  KvSendStubFactory(Context* ctx, std::shared_ptr<INamingClient> naming);
  SendStub create_stub(const InstanceId& dst, WorkerId dst_worker, uint32_t start_layer, uint32_t num_layers,
                       std::optional<TransferProtocol> proto, const std::optional<WorkerInfo>& dst_info) override;

 private:
  Context* ctx_;
  std::shared_ptr<INamingClient> naming_;
  std::shared_ptr<INamingWorkerClient> naming_worker_;
};

}  // namespace kvx
