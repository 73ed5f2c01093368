#include "transport/peer_memory.h"

#include <cuda_runtime.h>
#include <unistd.h>

#include <map>
#include <mutex>

#include "kernels/kvt_kernels.h"
#include "transport/device_stage.h"

namespace kvx {

namespace {

struct IpcCache {
  struct Mapping {
    uint64_t local = 0;
    uint32_t refs = 0;
  };
  std::mutex mu;
  std::map<std::string, Mapping> mapped;   // 64 handle bytes -> local address
  uint64_t acquire(const char* handle64) {
    std::lock_guard<std::mutex> g(mu);
    const std::string key(handle64, 64);
    auto it = mapped.find(key);
    if (it == mapped.end()) {
      uint64_t local = 0;
      cuda_check(kvt_ipc_open_handle(handle64, &local), "cudaIpcOpenMemHandle");
      it = mapped.emplace(key, Mapping{local, 0}).first;
    }
    ++it->second.refs;
    return it->second.local;
  }
  void release(const std::string& key) {
    std::lock_guard<std::mutex> g(mu);
    auto it = mapped.find(key);
    if (it == mapped.end()) return;
    if (--it->second.refs == 0) {
      kvt_ipc_close(it->second.local);
      mapped.erase(it);
    }
  }
};
IpcCache& ipc_cache() {
  static IpcCache& c = *new IpcCache;   // never destroyed: channels may close while the process exits
  return c;
}

}  // namespace

size_t ipc_mappings_open() {
  IpcCache& c = ipc_cache();
  std::lock_guard<std::mutex> g(c.mu);
  return c.mapped.size();
}

PeerMemInfo export_peer_mem_info(Context* ctx) {
  PeerMemInfo info;
  info.pid = static_cast<int32_t>(getpid());
  info.device = ctx->device_id();
  info.host_id = this_host_id();
  const auto& addrs = ctx->layer_data_address();
  info.num_layers = static_cast<uint32_t>(addrs.size());
  info.num_tensors = addrs.empty() ? 0 : static_cast<uint32_t>(addrs[0].size());
  if (ctx->device_id() < 0) return info;
  cudaSetDevice(ctx->device_id());
  for (const auto& layer : addrs) {
    for (uint64_t ptr : layer) {
      PeerTensor t{};
      t.ptr = ptr;
      t.alloc_base = ptr;
      uint64_t base = 0, size = 0;
      if (kvt_ipc_get_handle(ptr, t.ipc_handle, &base, &size) == 0) {
        t.has_handle = 1;
        t.alloc_base = base;
      } else {
        cudaGetLastError();
        t.has_handle = 0;
      }
      info.tensors.push_back(t);
    }
  }
  return info;
}

void PeerMapping::map(const PeerMemInfo& info, int local_device) {
  release();
  if (info.host_id != this_host_id()) throw KVTransferException(ErrorKind::TRANSPORT, "peer memory is on another host");
  same_process_ = info.pid == static_cast<int32_t>(getpid());
  peer_device_ = info.device;
  cuda_check(cudaSetDevice(local_device), "cudaSetDevice");
  if (info.device != local_device && same_process_) {
    if (!kvt_can_access_peer(local_device, info.device))
      throw KVTransferException(ErrorKind::TRANSPORT, "no peer access between the two GPUs");
    cuda_check(kvt_enable_peer_access(local_device, info.device), "cudaDeviceEnablePeerAccess");
  }
  ptrs_.assign(info.num_layers, std::vector<uint64_t>(info.num_tensors, 0));
  for (uint32_t l = 0; l < info.num_layers; ++l) {
    for (uint32_t t = 0; t < info.num_tensors; ++t) {
      const PeerTensor& pt = info.tensors[static_cast<size_t>(l) * info.num_tensors + t];
      if (same_process_) {
        ptrs_[l][t] = pt.ptr;
        continue;
      }
      if (!pt.has_handle) throw KVTransferException(ErrorKind::TRANSPORT, "peer tensor has no IPC handle");
      const std::string key(pt.ipc_handle, 64);
      uint64_t local = 0;
      for (size_t k = 0; k < keys_.size() && local == 0; ++k)
        if (keys_[k] == key) local = locals_[k];
      if (local == 0) {      // one reference per allocation and mapping object
        local = ipc_cache().acquire(pt.ipc_handle);
        keys_.push_back(key);
        locals_.push_back(local);
      }
      ptrs_[l][t] = local + (pt.ptr - pt.alloc_base);
    }
  }
}

void PeerMapping::release() {
  for (const std::string& key : keys_) ipc_cache().release(key);
  keys_.clear();
  locals_.clear();
  ptrs_.clear();
}

std::string PeerEvents::serialize() const {
  std::string s;
  put(s, pid);
  put(s, static_cast<uint32_t>(events.size()));
  for (const One& e : events) {
    put(s, e.raw);
    s.append(e.handle, 64);
    put(s, e.has_handle);
  }
  return s;
}

bool PeerEvents::parse(const char* p, size_t len, PeerEvents* out) {
  const char* end = p + len;
  uint32_t n = 0;
  if (!take(p, end, &out->pid) || !take(p, end, &n) || n > (1u << 16)) return false;
  out->events.resize(n);
  for (One& e : out->events) {
    if (!take(p, end, &e.raw) || static_cast<size_t>(end - p) < 65) return false;
    memcpy(e.handle, p, 64);
    p += 64;
    e.has_handle = static_cast<uint8_t>(*p++);
  }
  return true;
}

PeerEvents export_peer_events(Context* ctx) {
  PeerEvents out;
  out.pid = static_cast<int32_t>(getpid());
  ICudaBarrier* b = ctx->cuda_barrier();
  if (b == nullptr || ctx->device_id() < 0) return out;
  cudaSetDevice(ctx->device_id());
  for (uint32_t l = 0; l < ctx->num_layers(); ++l) {
    PeerEvents::One e;
    void* ev = b->event(l);
    if (ev == nullptr) return PeerEvents{out.pid, {}};
    e.raw = reinterpret_cast<uint64_t>(ev);
    cudaIpcEventHandle_t h;
    static_assert(sizeof(h) == 64, "IPC event handle is 64 bytes on the wire");
    if (cudaIpcGetEventHandle(&h, static_cast<cudaEvent_t>(ev)) == cudaSuccess) {
      memcpy(e.handle, &h, 64);
      e.has_handle = 1;
    } else {
      cudaGetLastError();    // the event was not created for interprocess use
    }
    out.events.push_back(e);
  }
  return out;
}

std::vector<void*> open_peer_events(const PeerEvents& ev) {
  std::vector<void*> out;
  const bool same = ev.pid == static_cast<int32_t>(getpid());
  for (const PeerEvents::One& e : ev.events) {
    if (same) {
      out.push_back(reinterpret_cast<void*>(e.raw));
      continue;
    }
    cudaEvent_t opened = nullptr;
    cudaIpcEventHandle_t h;
    memcpy(&h, e.handle, 64);
    if (!e.has_handle || cudaIpcOpenEventHandle(&opened, h) != cudaSuccess) {
      cudaGetLastError();
      for (void* o : out) cudaEventDestroy(static_cast<cudaEvent_t>(o));
      return {};
    }
    out.push_back(opened);
  }
  return out;
}

void close_peer_events(const PeerEvents& ev, std::vector<void*>& opened) {
  if (ev.pid != static_cast<int32_t>(getpid()))
    for (void* o : opened) cudaEventDestroy(static_cast<cudaEvent_t>(o));
  opened.clear();
}

}  // namespace kvx
