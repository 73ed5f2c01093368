#include "transport/copy_policy.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <map>
#include <memory>
#include <mutex>
#include <vector>

#include "core/envcfg.h"
#include "core/log.h"
#include "kernels/kvt_kernels.h"

namespace kvx {

namespace {

constexpr size_t kScratch = 32u << 20;
const size_t kRepCount[CopyPolicy::kCountBuckets] = {4, 32, 256, 2048};
const size_t kRepSize[CopyPolicy::kSizeBuckets] = {4u << 10, 64u << 10, 1u << 20, 4u << 20};

struct Scratch {
  void* dev{nullptr};
  void* host{nullptr};
  void* host_dev{nullptr};
  uint64_t* d_triples{nullptr};
  uint64_t* h_triples{nullptr};
  uint32_t* d_status{nullptr};
  cudaStream_t stream{nullptr};
  cudaEvent_t e0{nullptr}, e1{nullptr};
  bool ok{false};

  Scratch() {
    const size_t tb = 2048 * 3 * sizeof(uint64_t);
    ok = cudaMalloc(&dev, kScratch) == cudaSuccess &&
         cudaHostAlloc(&host, kScratch, cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess &&
         cudaHostGetDevicePointer(&host_dev, host, 0) == cudaSuccess &&
         cudaMalloc(reinterpret_cast<void**>(&d_triples), tb) == cudaSuccess &&
         cudaHostAlloc(reinterpret_cast<void**>(&h_triples), tb, cudaHostAllocDefault) == cudaSuccess &&
         cudaMalloc(reinterpret_cast<void**>(&d_status), 16) == cudaSuccess &&
         cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) == cudaSuccess &&
         cudaEventCreate(&e0) == cudaSuccess && cudaEventCreate(&e1) == cudaSuccess;
    if (ok) ok = cudaMemsetAsync(d_status, 0, 16, stream) == cudaSuccess &&
                 cudaMemsetAsync(dev, 0, kScratch, stream) == cudaSuccess;
  }
  ~Scratch() {
    if (stream != nullptr) cudaStreamSynchronize(stream);
    if (e0 != nullptr) cudaEventDestroy(e0);
    if (e1 != nullptr) cudaEventDestroy(e1);
    if (stream != nullptr) cudaStreamDestroy(stream);
    if (d_status != nullptr) cudaFree(d_status);
    if (h_triples != nullptr) cudaFreeHost(h_triples);
    if (d_triples != nullptr) cudaFree(d_triples);
    if (host != nullptr) cudaFreeHost(host);
    if (dev != nullptr) cudaFree(dev);
  }
};

// One timed pass; returns microseconds, or a negative value when a CUDA call failed.
float time_pass(Scratch& s, int device, CopyDir dir, CopyPath path, size_t n, size_t len) {
  const uint64_t src = dir == CopyDir::D2H ? reinterpret_cast<uint64_t>(s.dev) : reinterpret_cast<uint64_t>(s.host_dev);
  const uint64_t dst = dir == CopyDir::D2H ? reinterpret_cast<uint64_t>(s.host_dev) : reinterpret_cast<uint64_t>(s.dev);
  if (cudaEventRecord(s.e0, s.stream) != cudaSuccess) return -1.f;
  if (path == CopyPath::KERNEL) {
    for (size_t i = 0; i < n; i++) {
      s.h_triples[3 * i] = i * len;
      s.h_triples[3 * i + 1] = i * len;
      s.h_triples[3 * i + 2] = len;
    }
    if (cudaMemcpyAsync(s.d_triples, s.h_triples, n * 24, cudaMemcpyHostToDevice, s.stream) != cudaSuccess) return -1.f;
    const int grid = std::max(1, static_cast<int>(0.5 * kvt_sm_count(device) * env_kernel_copy_sm_usage()));   // as DeviceStage::enqueue
    if (kvt_launch_copy_blocks(src, dst, s.d_triples, static_cast<uint32_t>(n), kScratch, kScratch, s.d_status, grid,
                               s.stream) != 0)
      return -1.f;
  } else {
    for (size_t i = 0; i < n; i++) {
      if (cudaMemcpyAsync(reinterpret_cast<void*>(dst + i * len), reinterpret_cast<const void*>(src + i * len), len,
                          cudaMemcpyDefault, s.stream) != cudaSuccess)
        return -1.f;
    }
  }
  if (cudaEventRecord(s.e1, s.stream) != cudaSuccess || cudaEventSynchronize(s.e1) != cudaSuccess) return -1.f;
  float ms = 0.f;
  if (cudaEventElapsedTime(&ms, s.e0, s.e1) != cudaSuccess) return -1.f;
  return ms * 1000.f;
}

}  // namespace

int CopyPolicy::count_bucket(size_t n) { return n <= 4 ? 0 : n <= 32 ? 1 : n <= 512 ? 2 : 3; }
int CopyPolicy::size_bucket(size_t len) { return len <= (16u << 10) ? 0 : len <= (256u << 10) ? 1 : len <= (2u << 20) ? 2 : 3; }

CopyPath CopyPolicy::choose(CopyDir dir, size_t n, size_t total_bytes, size_t min_len) const {
  if (n == 0) return CopyPath::KERNEL;
  if (static_rule_) {
    return n <= static_max_blocks_ && min_len >= static_threshold_ ? CopyPath::MEMCPY : CopyPath::KERNEL;
  }
  return table_[static_cast<int>(dir)][count_bucket(n)][size_bucket(total_bytes / n)];
}

CopyPolicy CopyPolicy::fixed(const std::string& mode) {
  CopyPolicy p;
  p.static_rule_ = mode == "static";
  if (!p.static_rule_) {
    const CopyPath path = mode == "memcpy" ? CopyPath::MEMCPY : CopyPath::KERNEL;
    for (auto& d : p.table_)
      for (auto& c : d)
        for (auto& e : c) e = path;
  }
  return p;
}

void CopyPolicy::measure(int device) {
  int prev = -1;
  cudaGetDevice(&prev);
  if (cudaSetDevice(device) != cudaSuccess) return;
  {
    Scratch s;
    bool ok = s.ok;
    for (int d = 0; ok && d < 2; d++) {
      for (int c = 0; ok && c < kCountBuckets; c++) {
        for (int z = 0; ok && z < kSizeBuckets; z++) {
          const size_t len = kRepSize[z];
          const size_t n = std::max<size_t>(1, std::min(kRepCount[c], kScratch / len));
          float best[2] = {-1.f, -1.f};
          for (int path = 0; ok && path < 2; path++) {
            for (int it = 0; it < 3; it++) {   // the first pass warms up and is not counted
              const float us = time_pass(s, device, static_cast<CopyDir>(d), static_cast<CopyPath>(path), n, len);
              if (us < 0.f) {
                ok = false;
                break;
              }
              if (it > 0 && (best[path] < 0.f || us < best[path])) best[path] = us;
            }
          }
          if (!ok) break;
          us_[d][c][z][0] = best[0];
          us_[d][c][z][1] = best[1];
          // the kernel keeps the list in one launch and checks bounds on the device: the copy
          // engines must win clearly to be chosen
          table_[d][c][z] = best[1] < 0.95f * best[0] ? CopyPath::MEMCPY : CopyPath::KERNEL;
        }
      }
    }
    if (ok) {
      measured_ = true;
      static_rule_ = false;
    } else {
      cudaGetLastError();
      LOG(WARNING) << "copy policy: measurement failed on device " << device << ", using the static rule";
    }
  }
  if (prev >= 0) cudaSetDevice(prev);
}

std::string CopyPolicy::describe() const {
  std::string out;
  if (static_rule_) {
    out = "static: memcpy when n<=" + std::to_string(static_max_blocks_) + " and every len>=" +
          std::to_string(static_threshold_) + "\n";
    return out;
  }
  const char* names[2] = {"d2h", "h2d"};
  for (int d = 0; d < 2; d++) {
    out += names[d];
    out += ":";
    for (int c = 0; c < kCountBuckets; c++) {
      out += " ";
      for (int z = 0; z < kSizeBuckets; z++) out += table_[d][c][z] == CopyPath::MEMCPY ? 'M' : 'K';
    }
    if (measured_) {
      out += "  us(kernel/memcpy):";
      char buf[64];
      for (int c = 0; c < kCountBuckets; c++)
        for (int z = 0; z < kSizeBuckets; z++) {
          snprintf(buf, sizeof(buf), " %.0f/%.0f", us_[d][c][z][0], us_[d][c][z][1]);
          out += buf;
        }
    }
    out += "\n";
  }
  return out;
}

namespace {
// never destroyed: server and sender threads may ask for a policy while the process exits
std::mutex& g_policy_mu = *new std::mutex;
std::map<int, std::unique_ptr<CopyPolicy>>& g_policies = *new std::map<int, std::unique_ptr<CopyPolicy>>;
}  // namespace

void CopyPolicy::reset_for_test() {
  // policies handed out earlier stay alive: a DeviceStage may still hold a reference
  static std::vector<std::unique_ptr<CopyPolicy>>& retired = *new std::vector<std::unique_ptr<CopyPolicy>>;
  std::lock_guard<std::mutex> g(g_policy_mu);
  for (auto& kv : g_policies) retired.push_back(std::move(kv.second));
  g_policies.clear();
}

const CopyPolicy& CopyPolicy::get(int device) {
  auto& policies = g_policies;
  std::lock_guard<std::mutex> g(g_policy_mu);
  auto it = policies.find(device);
  if (it != policies.end()) return *it->second;
  auto p = std::make_unique<CopyPolicy>();
  const int forced = env_copy_path();   // 0 auto, 1 kernel, 2 memcpy
  if (forced == 1 || forced == 2) {
    *p = fixed(forced == 1 ? "kernel" : "memcpy");
  } else {
    p->static_max_blocks_ = env_copy_memcpy_max_blocks();
    p->static_threshold_ = env_copy_memcpy_threshold_bytes();
    if (env_copy_profile_enable()) p->measure(device);
  }
  LOG(INFO) << "copy policy of device " << device << ":\n" << p->describe();
  return *policies.emplace(device, std::move(p)).first->second;
}

}  // namespace kvx
