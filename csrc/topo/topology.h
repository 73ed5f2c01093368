// NVLink / NVSwitch topology discovery.
//
// The reference discovers which RDMA NIC is closest to each GPU (blade_kvt/nic_affinity.py:24-52,
// read by choose_nic in kvtransfer/src/barex_protocol.cpp:262-302).  On an NVSwitch box the
// question becomes which GPUs can store into each other's memory and how well: peer access,
// the CUDA P2P performance rank, native atomics over the link, NVLS (multicast) support and,
// when NVML is present, how many NVLink links are up.  Everything here only *reads* state.
#pragma once
#include <string>
#include <vector>

namespace kvx {

struct GpuInfo {
  int index{0};
  std::string name;
  int sm_count{0};
  size_t total_mem{0};
  int multicast_supported{-1};   // NVLS capable (-1 unknown)
  int nvlink_links_up{-1};       // from NVML (-1 unknown)
  std::string uuid;
};

struct PeerLink {
  int src{0}, dst{0};
  int access{0};
  int perf_rank{-1};
  int native_atomics{0};
};

struct Topology {
  std::vector<GpuInfo> gpus;
  std::vector<PeerLink> links;
  std::string to_json() const;
};

Topology discover_topology();

}  // namespace kvx
