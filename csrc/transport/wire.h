// Wire format of the host-driven transports (TCP and shared memory).
//
// Every message on a connection is one frame: [u32 payload_len][payload].  The payload of a
// data message is byte-identical to the reference's TCP message (kvtransfer/src/
// tcp_channel.cpp:433-447, 477-588):
//   [magic 'KVCa' u32][reqid u64][layer_idx size_t][num_tensors size_t]
//   { [n_blocks size_t][IpcBlock x n][blob_bytes size_t][blob] } x num_tensors
// The blob is the concatenation of the blocks' bytes in list order; the receiver scatters it
// by dst_offset.  With the shared-memory transport the blob travels through a POSIX shm
// segment instead and the frame carries [SHM magic][reqid][segment offset][same header].
// Control messages share the RPC header (magic u32, reqid u64; kvtransfer/include/protocol/
// barex_protocol.h:47-61).
#pragma once
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "core/types.h"

namespace kvx {

constexpr uint32_t KV_CACHE_DATA_MAGIC = 0x4B564361;   // 'KVCa'
constexpr uint32_t KV_CACHE_SHM_MAGIC = 0x4B565368;    // 'KVSh': blob lives in the attached shm segment
constexpr uint32_t SHM_ATTACH_REQ = 0x4B565341;        // 'KVSA': [name_len u32][name][bytes u64]
constexpr uint32_t MEM_HANDLES_REQ = 0x20181218;       // peer-memory handles of every layer tensor
constexpr uint32_t PING_REQ = 0x4B565069;              // 'KVPi'
// Pull transfers: the decode GPU runs the transfer kernels and loads the prefill cache over NVLink.  The
// prefill side opens a session on the decode worker's server (its own memory handles and layer-event handles
// travel in the request), then drives it with one-way messages; the server answers each flushed batch with
// PULL_DONE when the batch's completion record has arrived.
constexpr uint32_t PULL_OPEN_REQ = 0x4B56504F;         // 'KVPO': [version u32][src caps][PeerMemInfo][PeerEvents] -> [status u32]
constexpr uint32_t PULL_PLAN_REQ = 0x4B565050;         // 'KVPP': a batch's plan (reqid = batch sequence number)
constexpr uint32_t PULL_LAYERS_REQ = 0x4B56504C;       // 'KVPL': layers [lo, hi) of the batch are recorded: enqueue them
constexpr uint32_t PULL_FLUSH_REQ = 0x4B565046;        // 'KVPF': the batch is complete: enqueue its completion record
constexpr uint32_t PULL_DONE = 0x4B565044;             // 'KVPD': [status u32][detail u32][t_start u64][t_end u64]
// End-to-end check of a finished batch (transport/verify.h): the ranges a batch wrote, answered with the
// checksum of what the destination's cache holds there.
constexpr uint32_t CHECK_REQ = 0x4B56436B;             // 'KVCk'
constexpr uint32_t CHECK_ATTN_REQ = 0x4B56436C;        // 'KVCl': the row form, for transfers that change the layout
constexpr size_t RPC_HEADER = sizeof(uint32_t) + sizeof(uint64_t);

enum WireStatus : uint32_t { WIRE_OK = 0, WIRE_BAD_REQUEST = 400, WIRE_INTERNAL = 500 };

inline void put_rpc_header(char* p, uint32_t magic, uint64_t reqid) {
  memcpy(p, &magic, 4);
  memcpy(p + 4, &reqid, 8);
}
inline void get_rpc_header(const char* p, uint32_t* magic, uint64_t* reqid) {
  memcpy(magic, p, 4);
  memcpy(reqid, p + 4, 8);
}

template <typename T>
inline void put(std::string& s, const T& v) {
  s.append(reinterpret_cast<const char*>(&v), sizeof(T));
}
template <typename T>
inline bool take(const char*& p, const char* end, T* v) {
  if (static_cast<size_t>(end - p) < sizeof(T)) return false;
  memcpy(v, p, sizeof(T));
  p += sizeof(T);
  return true;
}

// One frame on a socket; returns false on error / timeout / peer close.
bool send_frame(int fd, const void* payload, size_t len, int timeout_ms);
bool send_frame2(int fd, const void* head, size_t head_len, const void* body, size_t body_len, int timeout_ms);
// Reads the length prefix then the payload into `buf` (resized).  `pinned_hint` lets the caller
// supply a preallocated buffer via the alloc callback.
bool recv_frame(int fd, std::string& buf, int timeout_ms);

// What a server tells a device transport about its memory: where each layer tensor is, and
// how another process can map it.
struct PeerTensor {
  uint64_t ptr;          // address in the owner's process
  uint64_t alloc_base;   // base of the CUDA allocation containing it (IPC handles name allocations)
  char ipc_handle[64];
  uint8_t has_handle;
};
struct PeerMemInfo {
  int32_t pid{0};
  int32_t device{-1};
  uint64_t host_id{0};
  uint32_t num_layers{0};
  uint32_t num_tensors{0};
  std::vector<PeerTensor> tensors;  // [layer][tensor] row-major
  std::string serialize() const;
  static bool parse(const char* p, size_t len, PeerMemInfo* out);
};

uint64_t this_host_id();  // stable id of this machine (boot id hash)

}  // namespace kvx
