#include "topo/topology.h"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <sstream>

#include "kernels/kvt_kernels.h"

namespace kvx {

namespace {

// Read-only NVML access through dlopen (the library is absent on machines without a driver).
struct Nvml {
  void* lib{nullptr};
  int (*init)(){nullptr};
  int (*get_handle_by_uuid)(const char*, void**){nullptr};
  int (*get_handle_by_index)(unsigned, void**){nullptr};
  int (*get_nvlink_state)(void*, unsigned, int*){nullptr};
  bool ok{false};
  Nvml() {
    lib = dlopen("libnvidia-ml.so.1", RTLD_NOW | RTLD_LOCAL);
    if (lib == nullptr) return;
    init = reinterpret_cast<int (*)()>(dlsym(lib, "nvmlInit_v2"));
    get_handle_by_index = reinterpret_cast<int (*)(unsigned, void**)>(dlsym(lib, "nvmlDeviceGetHandleByIndex_v2"));
    get_handle_by_uuid = reinterpret_cast<int (*)(const char*, void**)>(dlsym(lib, "nvmlDeviceGetHandleByUUID"));
    get_nvlink_state = reinterpret_cast<int (*)(void*, unsigned, int*)>(dlsym(lib, "nvmlDeviceGetNvLinkState"));
    ok = init != nullptr && get_nvlink_state != nullptr && init() == 0;
  }
};

std::string uuid_string(const cudaUUID_t& u) {
  static const char* hex = "0123456789abcdef";
  std::string s = "GPU-";
  for (int i = 0; i < 16; ++i) {
    if (i == 4 || i == 6 || i == 8 || i == 10) s.push_back('-');
    const unsigned char c = static_cast<unsigned char>(u.bytes[i]);
    s.push_back(hex[c >> 4]);
    s.push_back(hex[c & 15]);
  }
  return s;
}

}  // namespace

Topology discover_topology() {
  Topology t;
  const int n = kvt_device_count();
  if (n <= 0) return t;
  static Nvml nvml;
  typedef int (*attr_fn)(int*, int, int);
  attr_fn cu_attr = nullptr;
  {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuDeviceGetAttribute", &fn, cudaEnableDefault, &q) == cudaSuccess)
      cu_attr = reinterpret_cast<attr_fn>(fn);
    else
      cudaGetLastError();
  }
  for (int i = 0; i < n; ++i) {
    GpuInfo g;
    g.index = i;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, i) == cudaSuccess) {
      g.name = prop.name;
      g.sm_count = prop.multiProcessorCount;
      g.total_mem = prop.totalGlobalMem;
      g.uuid = uuid_string(prop.uuid);
    } else {
      cudaGetLastError();
    }
    if (cu_attr != nullptr) {
      int v = 0;
      const int CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED_ = 132;
      if (cu_attr(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED_, i) == 0) g.multicast_supported = v;
    }
    if (nvml.ok) {
      void* h = nullptr;
      int rc = -1;
      if (nvml.get_handle_by_uuid != nullptr && !g.uuid.empty()) rc = nvml.get_handle_by_uuid(g.uuid.c_str(), &h);
      if (rc != 0 && nvml.get_handle_by_index != nullptr) rc = nvml.get_handle_by_index(static_cast<unsigned>(i), &h);
      if (rc == 0) {
        int up = 0;
        for (unsigned link = 0; link < 18; ++link) {
          int active = 0;
          if (nvml.get_nvlink_state(h, link, &active) == 0 && active == 1) ++up;
        }
        g.nvlink_links_up = up;
      }
    }
    t.gpus.push_back(g);
  }
  for (int i = 0; i < n; ++i) {
    for (int j = 0; j < n; ++j) {
      if (i == j) continue;
      PeerLink l;
      l.src = i;
      l.dst = j;
      l.access = kvt_can_access_peer(i, j);
      l.perf_rank = kvt_p2p_attribute(i, j, 0);
      l.native_atomics = kvt_p2p_attribute(i, j, 2) > 0 ? 1 : 0;
      t.links.push_back(l);
    }
  }
  return t;
}

std::string Topology::to_json() const {
  std::ostringstream ss;
  ss << "{\"gpus\":[";
  for (size_t i = 0; i < gpus.size(); ++i) {
    const GpuInfo& g = gpus[i];
    if (i) ss << ',';
    ss << "{\"index\":" << g.index << ",\"name\":\"" << g.name << "\",\"sm_count\":" << g.sm_count
       << ",\"total_mem\":" << g.total_mem << ",\"multicast_supported\":" << g.multicast_supported
       << ",\"nvlink_links_up\":" << g.nvlink_links_up << ",\"uuid\":\"" << g.uuid << "\"}";
  }
  ss << "],\"links\":[";
  for (size_t i = 0; i < links.size(); ++i) {
    const PeerLink& l = links[i];
    if (i) ss << ',';
    ss << "{\"src\":" << l.src << ",\"dst\":" << l.dst << ",\"access\":" << l.access << ",\"perf_rank\":" << l.perf_rank
       << ",\"native_atomics\":" << l.native_atomics << "}";
  }
  ss << "]}";
  return ss.str();
}

}  // namespace kvx
