// Mapping another worker's cache tensors (and layer events) into this process.
//
// A worker describes its device memory with a PeerMemInfo (wire.h): address, allocation base and CUDA IPC
// handle of every layer tensor.  PeerMapping turns one into addresses this process can use: the owner's own
// pointers when it lives in this process (after enabling peer access between the two GPUs), IPC mappings
// otherwise.  IPC mappings are shared process-wide, reference counted and closed with their last user; the
// key is the handle itself, which names one allocation of one process, so a peer that restarted (even with a
// recycled pid and the same addresses) is never written or read through a stale mapping.  This is the role
// the MEM_HANDLES_REQ exchange of the reference's RDMA channel plays with rkeys
// (kvtransfer/src/rdma_channel.cpp:77-99, 298-316).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "core/context.h"
#include "transport/wire.h"

namespace kvx {

// What this worker exports about its own cache tensors (IPC handles are looked up once per tensor).
PeerMemInfo export_peer_mem_info(Context* ctx);

class PeerMapping {
 public:
  PeerMapping() = default;
  ~PeerMapping() { release(); }
  PeerMapping(const PeerMapping&) = delete;
  // Maps every tensor of `info` for use from `local_device`.  Throws KVTransferException when the owner is on
  // another host, has no handle for a tensor, or the GPUs cannot reach each other.
  void map(const PeerMemInfo& info, int local_device);
  void release();
  const std::vector<std::vector<uint64_t>>& ptrs() const { return ptrs_; }   // [layer][tensor]
  bool same_process() const { return same_process_; }
  int peer_device() const { return peer_device_; }

 private:
  std::vector<std::vector<uint64_t>> ptrs_;
  std::vector<std::string> keys_;      // IPC mappings this object holds a reference to
  std::vector<uint64_t> locals_;
  bool same_process_{false};
  int peer_device_{-1};
};

size_t ipc_mappings_open();   // process-wide count (tests)

// Layer events of a forward pass, shared with the process that pulls: raw pointers for a consumer in the
// same process, CUDA IPC event handles otherwise (the events must have been created interprocess).
struct PeerEvents {
  struct One {
    uint64_t raw{0};
    char handle[64]{};
    uint8_t has_handle{0};
  };
  int32_t pid{0};
  std::vector<One> events;
  std::string serialize() const;
  static bool parse(const char* p, size_t len, PeerEvents* out);
};
PeerEvents export_peer_events(Context* ctx);
// Opens the events for this process; empty when one of them cannot be opened.
std::vector<void*> open_peer_events(const PeerEvents& ev);
void close_peer_events(const PeerEvents& ev, std::vector<void*>& opened);

}  // namespace kvx
