// Descriptor-driven copies on a CUDA stream, shared by the host-driven transports and the
// generic (any cache shape) path of the NVLink transport.  One DeviceStage belongs to one
// thread: it owns a non-blocking stream, a device array for {src_off, dst_off, len} triples,
// pinned staging for them and a status word, and turns a list of triples into one or more
// launches of kvt_copy_blocks (at most BLLM_KVTRANS_KERNEL_COPY_MAX_BLOCK_NUM descriptors per
// launch, like the reference's batching, kvtransfer/src/copy_kernels.cpp:770-823).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace kvx {

struct Triple {
  uint64_t src_off, dst_off, len;
};

// Pinned (and device-mapped) host buffer that grows on demand.
class PinnedBuffer {
 public:
  PinnedBuffer() = default;
  ~PinnedBuffer();
  PinnedBuffer(const PinnedBuffer&) = delete;
  char* reserve(size_t bytes, bool pinned);  // keeps contents only when no reallocation happens
  char* data() const { return host_; }
  uint64_t device_ptr() const { return dev_; }
  size_t capacity() const { return cap_; }
  bool pinned() const { return pinned_; }

 private:
  void release();
  char* host_{nullptr};
  uint64_t dev_{0};
  size_t cap_{0};
  bool pinned_{false};
};

class DeviceStage {
 public:
  explicit DeviceStage(int device);
  ~DeviceStage();
  DeviceStage(const DeviceStage&) = delete;
  // Launch the copy over descriptors that already sit in device memory (uploaded by the caller and
  // ordered before this stream by an event); does not wait.
  // `status` (device, 2 x u32) replaces the stage's own status words, so that several stages can report
  // into one place that the caller reads back itself.
  void launch_resident(uint64_t src_base, uint64_t dst_base, const uint64_t* d_triples, size_t n, uint64_t src_cap,
                       uint64_t dst_cap, int grid_ctas = 0, uint32_t* status = nullptr);
  // Enqueue the copy; does not wait.  host_side says which end is pinned host memory (HOST_NONE,
  // HOST_SRC, HOST_DST): with a host end the copy policy of the device may hand the list to the copy
  // engines (one cudaMemcpyAsync per descriptor, bounds checked here) instead of the kernel.  With
  // cast_bf16_e4m3 a descriptor's length counts values: 2 x len source bytes become len e4m3 bytes.
  enum { HOST_NONE = 0, HOST_SRC = 1, HOST_DST = 2 };
  void enqueue(uint64_t src_base, uint64_t dst_base, const std::vector<Triple>& triples, uint64_t src_cap,
               uint64_t dst_cap, int grid_ctas = 0, int host_side = HOST_NONE, bool cast_bf16_e4m3 = false);
  uint64_t memcpy_lists() const { return memcpy_lists_; }   // lists that went to the copy engines
  uint64_t kernel_lists() const { return kernel_lists_; }
  // Wait for everything enqueued and throw KVTransferException if the kernel flagged a descriptor.
  void sync();
  void* stream() const { return stream_; }
  int device() const { return device_; }
  // Make the stream wait for a cudaEvent_t before later work (no host wait).
  void wait_event(void* event);
  // Record this stage's own event behind everything enqueued so far and return it: another
  // stage can wait_event() on it, which joins the two streams without a host wait.
  void* record_done();

 private:
  int device_;
  void* stream_{nullptr};
  void* done_event_{nullptr};
  uint64_t* d_triples_{nullptr};
  size_t d_cap_{0};       // triples
  size_t used_{0};        // triples enqueued since the last sync
  uint32_t* d_status_{nullptr};
  PinnedBuffer h_triples_;
  PinnedBuffer h_status_;
  uint64_t memcpy_lists_{0};
  uint64_t kernel_lists_{0};
};

// Process-wide count of descriptor lists that went to the copy engines / to the copy kernel.
void copy_path_counters(uint64_t* memcpy_lists, uint64_t* kernel_lists);

void cuda_check(int err, const char* what);  // throws KVTransferException(CUDA)

}  // namespace kvx
