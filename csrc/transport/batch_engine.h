// Device side of a transfer between two paged caches that one GPU can address: the machinery that is the
// same whether the prefill GPU pushes (kernels run where the source cache lives and store into the peer) or
// the decode GPU pulls (kernels run where the destination cache lives and load from the peer).
//
// A batch is one engine step's requests for one destination.  It runs in one of a few plan slots (device +
// pinned plan buffer, status block, completion record, a small stream), allocated once when the engine is
// made, so that the step path neither allocates nor frees:
//
//   begin(bytes)        take the next slot (waits, bounded, for the batch that last used it), return its buffers
//   upload(bytes)       plan -> device on the slot's stream; transfer streams join it when the batch first uses them
//   launch_attn / launch_walk / stage()   enqueue the layer's kernel(s) behind an event of the forward pass
//   flush_async()       join the streams the batch used, enqueue its completion record, return the ticket
//   poll(ticket)        has the record arrived (mapped host memory; no stream is synchronised)
//
// Completion records arrive in ticket order.  The bookkeeping that poll() shares with the sender's thread is
// locked; everything else belongs to the one thread that drives the engine.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "core/completion.h"
#include "kernels/kvt_kernels.h"
#include "plan/device_plan.h"
#include "plan/planner.h"
#include "transport/device_stage.h"

namespace kvx {

struct BatchEngineConfig {
  int device = 0;
  int n_streams = 8;
  size_t plan_capacity = 2u << 20;   // bytes per slot
  bool stamps = false;               // GPU timer stamps around every batch (DeviceUs in the metrics)
  bool dst_remote = false;           // the destination is another GPU's memory (quantiser staging, see kvt_kernels.h)
  int grid_ctas = 0;                 // 0: four CTAs per SM scaled by the SM-usage knob
};

class BatchEngine {
 public:
  struct SlotView {
    char* h_plan;         // pinned host staging of the plan
    char* d_plan;         // its place on the device
    uint32_t* d_status;   // 64-byte status block of the batch
    uint64_t seq;         // ticket of the batch
  };
  struct Done {
    uint32_t status{0}, detail{0};
    uint64_t t_start_ns{0}, t_end_ns{0};
    std::string metrics;
  };

  // src_ptrs / dst_ptrs: base address of every cache tensor, [layer][tensor], as THIS device addresses them.
  BatchEngine(const BatchEngineConfig& cfg, std::vector<std::vector<uint64_t>> src_ptrs,
              std::vector<std::vector<uint64_t>> dst_ptrs, std::vector<uint64_t> src_caps, std::vector<uint64_t> dst_caps);
  ~BatchEngine();
  BatchEngine(const BatchEngine&) = delete;

  SlotView begin(size_t bytes);
  void upload(size_t bytes);
  SlotView current();
  bool in_batch() const { return batch_slot_ >= 0; }
  // Transfer stream `i` of the current batch (joined to the plan upload at first use).
  DeviceStage& stage(size_t i);
  size_t n_stages() const { return stages_.size(); }
  size_t next_stage() { return range_rr_++ % stages_.size(); }

  // The fused attention kernel over layers [lo, hi) of the current batch.  `params` may change between
  // batches only in its head window; a layout change re-encodes the tensor maps.
  void launch_attn(const DeviceAttnParams& params, const PackedPlan& plan, size_t lo, size_t hi, size_t stage_idx,
                   void* wait_event);
  // The walk kernel (copies, then zero fills) over layers [lo, hi).
  void launch_walk(const KvtWalkCounts& counts, size_t n_ops, size_t pool_len, size_t lo, size_t hi, size_t stage_idx,
                   void* wait_event);
  // Multicast addresses of the destination tensors ([layer][tensor], as dst_ptrs): set once when the destination
  // cache is a member of an NVLink multicast group.
  void set_multicast(std::vector<std::vector<uint64_t>> mc_ptrs);
  bool has_multicast() const { return !mc_ptrs_.empty(); }
  // Behind launch_walk on the same stage: store what those ops wrote into this GPU's cache to every member
  // of the group (multimem stores through NVSwitch).
  void launch_walk_fanout(const KvtWalkCounts& counts, size_t n_ops, size_t pool_len, size_t lo, size_t hi, size_t stage_idx);
  // The sender's form, on an engine whose "destination" is the multicast mapping itself: the ops' source pieces
  // go from this GPU's cache straight to every member of the group (behind `wait_event` of the forward pass).
  void launch_walk_multicast(const KvtWalkCounts& counts, size_t n_ops, size_t pool_len, size_t lo, size_t hi, size_t stage_idx,
                             void* wait_event);

  uint64_t flush_async(std::string metrics, bool drop_record = false);
  // DONE: `out` holds the record; FAILED: the ticket is unknown or was never flushed.
  PollResult poll(uint64_t ticket, Done* out);
  // Blocks (bounded by the completion timeout) until the ticket's record has arrived; false on timeout.
  bool wait(uint64_t ticket, Done* out);
  void close();
  bool use_tma() const { return use_tma_; }
  int device() const { return cfg_.device; }

 private:
  static constexpr size_t kSlots = 4;
  struct Slot {
    cudaStream_t stream{nullptr};
    cudaEvent_t plan_event{nullptr};
    cudaEvent_t done_event{nullptr};
    char* d_plan{nullptr};
    char* h_plan{nullptr};
    uint32_t* d_status{nullptr};
    KvtCompletion* h_rec{nullptr};
    KvtCompletion* d_rec{nullptr};
    uint64_t seq{0};
    bool pending{false};
    std::string metrics;
  };
  template <typename T>
  struct DevArray {
    T* p{nullptr};
    size_t n{0};
    ~DevArray();
    void upload(const std::vector<T>& v);
  };
  struct alignas(64) TensorMapBytes {
    char b[128];
  };

  void alloc_slots(size_t cap);
  void free_slots();
  void wait_slot(Slot& sl);
  static bool record_arrived(const Slot& sl);
  Done take_record(Slot& sl);
  Slot& cur();
  void begin_batch() { stage_used_.assign(stages_.size(), 0); }
  void ensure_attn_arrays(const DeviceAttnParams& p);
  void ensure_walk_arrays();
  int grid() const;

  BatchEngineConfig cfg_;
  std::vector<std::vector<uint64_t>> src_ptrs_, dst_ptrs_;
  std::vector<uint64_t> src_caps_, dst_caps_;
  std::vector<std::unique_ptr<DeviceStage>> stages_;
  std::vector<char> stage_used_;
  std::vector<Slot> slots_;
  size_t plan_cap_{0}, slot_rr_{0}, range_rr_{0};
  int batch_slot_{-1};
  uint64_t next_seq_{0};
  char* d_plan_all_{nullptr};
  char* h_plan_all_{nullptr};
  char* d_status_all_{nullptr};
  char* h_rec_all_{nullptr};
  cudaEvent_t last_done_event_{nullptr};
  std::mutex slot_mu_;
  std::map<uint64_t, Done> finished_;
  // attention path
  bool attn_ready_{false}, use_tma_{false};
  uint32_t tile_order_{0}, store_form_{0};
  KvtLayout map_src_{}, map_dst_{};
  uint32_t map_heads_{0}, map_tile_{0};
  DevArray<uint64_t> d_src_layers_, d_dst_layers_;
  DevArray<TensorMapBytes> d_src_maps_, d_dst_maps_;
  // walk path
  DevArray<uint64_t> d_walk_src_, d_walk_dst_;
  std::vector<std::vector<uint64_t>> mc_ptrs_;
  DevArray<uint64_t> d_walk_mc_;
};

}  // namespace kvx
