#include "transport/device_stage.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <cstring>

#include "core/envcfg.h"
#include "core/types.h"
#include "kernels/kvt_kernels.h"
#include "transport/copy_policy.h"

namespace kvx {

namespace {
std::atomic<uint64_t> g_memcpy_lists{0}, g_kernel_lists{0};
}

void copy_path_counters(uint64_t* memcpy_lists, uint64_t* kernel_lists) {
  *memcpy_lists = g_memcpy_lists.load();
  *kernel_lists = g_kernel_lists.load();
}

void cuda_check(int err, const char* what) {
  if (err != 0) {
    throw KVTransferException(ErrorKind::CUDA, std::string(what) + ": " +
                                                   cudaGetErrorString(static_cast<cudaError_t>(err)));
  }
}

PinnedBuffer::~PinnedBuffer() { release(); }

void PinnedBuffer::release() {
  if (host_ == nullptr) return;
  if (pinned_) cudaFreeHost(host_); else free(host_);
  host_ = nullptr;
  dev_ = 0;
  cap_ = 0;
}

char* PinnedBuffer::reserve(size_t bytes, bool pinned) {
  if (bytes <= cap_ && pinned == pinned_ && host_ != nullptr) return host_;
  release();
  size_t cap = std::max<size_t>(bytes, 4096);
  cap = (cap + (cap >> 2) + 4095) & ~size_t{4095};
  pinned_ = pinned;
  if (pinned) {
    void* h = nullptr;
    cuda_check(cudaHostAlloc(&h, cap, cudaHostAllocMapped | cudaHostAllocPortable), "cudaHostAlloc");
    void* d = nullptr;
    cuda_check(cudaHostGetDevicePointer(&d, h, 0), "cudaHostGetDevicePointer");
    host_ = static_cast<char*>(h);
    dev_ = reinterpret_cast<uint64_t>(d);
  } else {
    host_ = static_cast<char*>(malloc(cap));
    if (host_ == nullptr) throw std::bad_alloc();
  }
  cap_ = cap;
  return host_;
}

DeviceStage::DeviceStage(int device) : device_(device) {
  cuda_check(cudaSetDevice(device_), "cudaSetDevice");
  cudaStream_t s;
  cuda_check(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreate");
  stream_ = s;
  void* st = nullptr;
  cuda_check(cudaMalloc(&st, 16), "cudaMalloc(status)");
  d_status_ = static_cast<uint32_t*>(st);
  cuda_check(cudaMemsetAsync(d_status_, 0, 16, s), "cudaMemsetAsync");
  h_status_.reserve(16, true);
}

DeviceStage::~DeviceStage() {
  cudaSetDevice(device_);
  if (stream_ != nullptr) {
    cudaStreamSynchronize(static_cast<cudaStream_t>(stream_));
    cudaStreamDestroy(static_cast<cudaStream_t>(stream_));
  }
  if (done_event_ != nullptr) cudaEventDestroy(static_cast<cudaEvent_t>(done_event_));
  if (d_triples_ != nullptr) cudaFree(d_triples_);
  if (d_status_ != nullptr) cudaFree(d_status_);
}

void* DeviceStage::record_done() {
  if (done_event_ == nullptr) {
    cudaEvent_t e;
    cuda_check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
    done_event_ = e;
  }
  cuda_check(cudaEventRecord(static_cast<cudaEvent_t>(done_event_), static_cast<cudaStream_t>(stream_)), "cudaEventRecord");
  return done_event_;
}

void DeviceStage::wait_event(void* event) {
  if (event == nullptr) return;
  cuda_check(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream_), static_cast<cudaEvent_t>(event), 0),
             "cudaStreamWaitEvent");
}

void DeviceStage::enqueue(uint64_t src_base, uint64_t dst_base, const std::vector<Triple>& triples, uint64_t src_cap,
                          uint64_t dst_cap, int grid_ctas, int host_side, bool cast_bf16_e4m3) {
  if (triples.empty()) return;
  cuda_check(cudaSetDevice(device_), "cudaSetDevice");
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const size_t n = triples.size();
  if (host_side != HOST_NONE && !cast_bf16_e4m3) {
    size_t total = 0, min_len = SIZE_MAX;
    for (const Triple& t : triples) {
      total += t.len;
      min_len = std::min<size_t>(min_len, t.len);
    }
    const CopyDir dir = host_side == HOST_SRC ? CopyDir::H2D : CopyDir::D2H;
    if (CopyPolicy::get(device_).choose(dir, n, total, min_len) == CopyPath::MEMCPY) {
      for (size_t i = 0; i < n; i++) {
        const Triple& t = triples[i];
        if (t.src_off > src_cap || t.len > src_cap - t.src_off || t.dst_off > dst_cap || t.len > dst_cap - t.dst_off) {
          throw KVTransferException(ErrorKind::CUDA, "copy descriptor " + std::to_string(i) + " is out of bounds");
        }
        cuda_check(cudaMemcpyAsync(reinterpret_cast<void*>(dst_base + t.dst_off),
                                   reinterpret_cast<const void*>(src_base + t.src_off), t.len, cudaMemcpyDefault, s),
                   "cudaMemcpyAsync(block)");
      }
      memcpy_lists_++;
      g_memcpy_lists++;
      return;
    }
  }
  kernel_lists_++;
  g_kernel_lists++;
  // Descriptors of all launches since the last sync stay resident: the pinned staging must not
  // be overwritten while an upload is in flight, so grow-and-sync when it would not fit.
  if (used_ + n > d_cap_) {
    if (used_ > 0) sync();
    if (n > d_cap_) {
      if (d_triples_ != nullptr) cuda_check(cudaFree(d_triples_), "cudaFree");
      d_cap_ = std::max<size_t>(n + n / 2, 4096);
      void* p = nullptr;
      cuda_check(cudaMalloc(&p, d_cap_ * sizeof(Triple)), "cudaMalloc(triples)");
      d_triples_ = static_cast<uint64_t*>(p);
      h_triples_.reserve(d_cap_ * sizeof(Triple), true);
    }
  }
  static_assert(sizeof(Triple) == 24, "triples are 3 x u64");
  char* h = h_triples_.data() + used_ * sizeof(Triple);
  memcpy(h, triples.data(), n * sizeof(Triple));
  uint64_t* d = d_triples_ + used_ * 3;
  cuda_check(cudaMemcpyAsync(d, h, n * sizeof(Triple), cudaMemcpyHostToDevice, s), "cudaMemcpyAsync(triples)");
  const size_t max_per_launch = env_kernel_copy_max_block_num();
  int grid = grid_ctas;
  if (grid <= 0) {
    const double usage = env_kernel_copy_sm_usage();
    // a copy with a host end is PCIe-bound: half a CTA per SM keeps the link full (measured 33 GB/s through the
    // SHM transport against 28 with two per SM) and leaves the SMs to the forward pass
    grid = std::max(1, static_cast<int>((host_side != HOST_NONE ? 0.5 : 2.0) * kvt_sm_count(device_) * usage));
  }
  for (size_t off = 0; off < n; off += max_per_launch) {
    const uint32_t cnt = static_cast<uint32_t>(std::min(max_per_launch, n - off));
    if (cast_bf16_e4m3) {
      cuda_check(kvt_launch_copy_blocks_cast(src_base, dst_base, d + off * 3, cnt, src_cap, dst_cap, d_status_, grid, s),
                 "kvt_launch_copy_blocks_cast");
    } else {
      cuda_check(kvt_launch_copy_blocks(src_base, dst_base, d + off * 3, cnt, src_cap, dst_cap, d_status_, grid, s),
                 "kvt_launch_copy_blocks");
    }
  }
  used_ += n;
}

void DeviceStage::launch_resident(uint64_t src_base, uint64_t dst_base, const uint64_t* d_triples, size_t n,
                                  uint64_t src_cap, uint64_t dst_cap, int grid_ctas, uint32_t* status) {
  if (n == 0) return;
  uint32_t* st = status != nullptr ? status : d_status_;
  cuda_check(cudaSetDevice(device_), "cudaSetDevice");
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const size_t max_per_launch = env_kernel_copy_max_block_num();
  int grid = grid_ctas;
  if (grid <= 0) grid = std::max(1, static_cast<int>(2 * kvt_sm_count(device_) * env_kernel_copy_sm_usage()));
  for (size_t off = 0; off < n; off += max_per_launch) {
    const uint32_t cnt = static_cast<uint32_t>(std::min(max_per_launch, n - off));
    cuda_check(kvt_launch_copy_blocks(src_base, dst_base, d_triples + off * 3, cnt, src_cap, dst_cap, st, grid, s),
               "kvt_launch_copy_blocks");
  }
}

void DeviceStage::sync() {
  cuda_check(cudaSetDevice(device_), "cudaSetDevice");
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  cuda_check(cudaMemcpyAsync(h_status_.data(), d_status_, 8, cudaMemcpyDeviceToHost, s), "cudaMemcpyAsync(status)");
  cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
  used_ = 0;
  uint32_t st[2];
  memcpy(st, h_status_.data(), 8);
  if (st[0] != 0) {
    cudaMemsetAsync(d_status_, 0, 16, s);
    throw KVTransferException(ErrorKind::CUDA, "copy kernel rejected descriptor " + std::to_string(st[1]) +
                                                   " (status " + std::to_string(st[0]) + ")");
  }
}

}  // namespace kvx
