// Per-process description of one worker: who it is (WorkerInfo), where its cache tensors
// live, how to wait for a layer's KV to be produced, and which transports are usable.
// Role of kvtransfer/include/context.h:32-85 with one addition: device_id < 0 means the cache
// tensors are plain host memory (CPU plumbing without a GPU).
#pragma once
#include <memory>
#include <vector>

#include "core/completion.h"
#include "core/types.h"

namespace kvx {

struct LayerInfo {
  size_t token_size;
  size_t block_size;
  uint64_t layer_addr;
  LayerInfo(size_t t, size_t b, uint64_t a) : token_size(t), block_size(b), layer_addr(a) {}
};

// Waits until the KV of `layer` has been produced on the device.
class ICudaBarrier {
 public:
  virtual void wait(uint32_t layer) = 0;
  // Raw cudaEvent_t of the layer (nullptr when the barrier is not event based); lets a device
  // transport order its stream after the layer without a host wait.
  virtual void* event(uint32_t layer) { (void)layer; return nullptr; }
  virtual ~ICudaBarrier() = default;
};

class NoCudaBarrier : public ICudaBarrier {
 public:
  void wait(uint32_t) override {}
};

class CudaEventBarrier : public ICudaBarrier {
 public:
  explicit CudaEventBarrier(std::vector<uint64_t> events) : events_(std::move(events)) {}
  void wait(uint32_t layer) override;
  void* event(uint32_t layer) override {
    return layer < events_.size() ? reinterpret_cast<void*>(events_[layer]) : nullptr;
  }

 private:
  std::vector<uint64_t> events_;
};

class Context {
 public:
  const InstanceId inst_name;
  const WorkerId worker_id;

  Context(const InstanceId& inst, WorkerId worker);
  Context(const Context&) = delete;

  void set_tp(uint32_t tp_size, uint32_t worker_tp_rank);
  void set_block_params(std::vector<size_t> block_sizes, std::vector<size_t> token_sizes,
                        uint32_t layer_num_blocks, uint32_t indexer_blk_ntpb = 0);
  void set_layer_info(int device_id, const std::vector<std::vector<LayerInfo>>& all_layer_infos);
  void set_cuda_barrier(std::unique_ptr<ICudaBarrier> barrier);
  void set_protocols(uint8_t mask) { worker_info_.transfer_protocols = mask; }

  WorkerInfo* worker_info_mutable() { return &worker_info_; }
  const WorkerInfo& worker_info() const { return worker_info_; }
  ICudaBarrier* cuda_barrier() { return barrier_.get(); }
  const std::vector<std::vector<LayerInfo>>& all_layer_infos() const { return layer_infos_; }
  const std::vector<std::vector<uint64_t>>& layer_data_address() const { return layer_addrs_; }
  // NVLink multicast addresses of the same tensors, when this worker's cache is a member of a multicast group
  // (a tensor-parallel decode group whose caches live in one symmetric allocation); empty otherwise.
  const std::vector<std::vector<uint64_t>>& multicast_address() const { return mc_addrs_; }
  void set_multicast_address(std::vector<std::vector<uint64_t>> a) { mc_addrs_ = std::move(a); }
  int device_id() const { return device_id_; }
  uint32_t num_layers() const { return worker_info_.num_layers; }
  uint32_t layer_num_blocks() const { return worker_info_.layer_num_blocks; }
  const std::vector<size_t>& block_sizes() const { return worker_info_.block_sizes; }
  bool supports(TransferProtocol::Kind k) const { return (worker_info_.transfer_protocols & k) != 0; }
  // Bytes of cache tensor `t` of any layer (block size x blocks): the bound every offset is checked against.
  size_t tensor_capacity(size_t t) const;
  InflightCounter& inflight() { return inflight_; }

 private:
  int device_id_{-1};
  WorkerInfo worker_info_;
  std::vector<std::vector<LayerInfo>> layer_infos_;
  std::vector<std::vector<uint64_t>> layer_addrs_;
  std::vector<std::vector<uint64_t>> mc_addrs_;
  std::unique_ptr<ICudaBarrier> barrier_;
  InflightCounter inflight_;
};

}  // namespace kvx
