#include "core/context.h"

#include <cuda_runtime.h>

#include "core/envcfg.h"

namespace kvx {

void CudaEventBarrier::wait(uint32_t layer) {
  RTASSERT(layer < events_.size());
  cudaError_t e = cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(events_[layer]));
  if (e != cudaSuccess) {
    throw KVTransferException(ErrorKind::CUDA, std::string("cudaEventSynchronize: ") + cudaGetErrorString(e));
  }
}

Context::Context(const InstanceId& inst, WorkerId worker)
    : inst_name(inst), worker_id(worker), worker_info_(inst, worker), barrier_(std::make_unique<NoCudaBarrier>()) {}

void Context::set_tp(uint32_t tp_size, uint32_t worker_tp_rank) {
  // engine TP; the per-destination effective TP (after valid_ranks filtering) is computed by the
  // send stub once the destination is known.
  worker_info_.engine_tp_size = tp_size;
  worker_info_.worker_tp_rank = worker_tp_rank;
}

void Context::set_block_params(std::vector<size_t> block_sizes, std::vector<size_t> token_sizes,
                               uint32_t layer_num_blocks, uint32_t indexer_blk_ntpb) {
  RTASSERT(block_sizes.size() == token_sizes.size());
  RTASSERT(!block_sizes.empty());
  for (size_t i = 0; i < block_sizes.size(); ++i) {
    RTASSERT(token_sizes[i] > 0);
    RTASSERT(block_sizes[i] % token_sizes[i] == 0);
  }
  worker_info_.block_sizes = std::move(block_sizes);
  worker_info_.token_sizes = std::move(token_sizes);
  worker_info_.layer_num_blocks = layer_num_blocks;
  const int forced = env_attn_kernel_blk_size();
  if (forced == -1) {
    // With attn_pack_size > 1 the registered tensor is a physical page holding that many
    // per-layer attention blocks back to back; tokens per kernel block is per packed block.
    const uint32_t pack = worker_info_.attn_pack_size == 0 ? 1u : worker_info_.attn_pack_size;
    const size_t ntpb = worker_info_.block_sizes[0] / worker_info_.token_sizes[0];
    RTASSERT(ntpb % pack == 0);
    worker_info_.attn_kernel_blk_ntpb = static_cast<uint32_t>(ntpb / pack);
  } else {
    worker_info_.attn_kernel_blk_ntpb = static_cast<uint32_t>(forced);
  }
  worker_info_.indexer_blk_ntpb = indexer_blk_ntpb;  // 0: model has no indexer cache
}

void Context::set_layer_info(int device_id, const std::vector<std::vector<LayerInfo>>& all) {
  device_id_ = device_id;
  worker_info_.num_layers = static_cast<uint32_t>(all.size());
  layer_infos_ = all;
  layer_addrs_.clear();
  for (const auto& layer : all) {
    std::vector<uint64_t> addrs;
    for (const auto& li : layer) addrs.push_back(li.layer_addr);
    layer_addrs_.push_back(std::move(addrs));
  }
}

void Context::set_cuda_barrier(std::unique_ptr<ICudaBarrier> barrier) {
  if (barrier == nullptr) throw std::runtime_error("cuda barrier can't be null;");
  barrier_ = std::move(barrier);
}

size_t Context::tensor_capacity(size_t t) const {
  RTASSERT(t < worker_info_.block_sizes.size());
  return worker_info_.block_sizes[t] * static_cast<size_t>(worker_info_.layer_num_blocks);
}

}  // namespace kvx
