// Which engine moves a descriptor list between device memory and pinned host memory: the SMs
// (kvt_copy_blocks, one launch for the whole list) or the copy engines (one cudaMemcpyAsync per
// descriptor).  Few large runs favour the copy engines, many small ones the kernel; where the
// crossover lies depends on the box (PCIe generation, host memory), so it is measured once per
// process and device at start-up, per direction and per (descriptor count, descriptor size)
// bucket.  Same role as the reference's start-up profiler
// (kvtransfer/src/copy_kernels.cpp:495-631); with BLLM_KVTRANS_COPY_PROFILE_ENABLE=0 the static
// rule of the reference applies instead: copy engines when the list has at most
// BLLM_KVTRANS_COPY_MEMCPY_MAX_BLOCKS (16) descriptors, each of at least
// BLLM_KVTRANS_COPY_MEMCPY_BLOCK_THRESHOLD_BYTES (256 KiB).
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

namespace kvx {

enum class CopyDir : int { D2H = 0, H2D = 1 };
enum class CopyPath : int { KERNEL = 0, MEMCPY = 1 };

class CopyPolicy {
 public:
  static constexpr int kCountBuckets = 4;   // <= 4, <= 32, <= 512, more
  static constexpr int kSizeBuckets = 4;    // <= 16 KiB, <= 256 KiB, <= 2 MiB, more
  static int count_bucket(size_t n);
  static int size_bucket(size_t avg_len);

  // The policy of `device`; the first call measures (or applies the static rule) and may take
  // some tens of milliseconds.  Safe from any thread.
  static const CopyPolicy& get(int device);

  CopyPath choose(CopyDir dir, size_t n, size_t total_bytes, size_t min_len) const;
  bool measured() const { return measured_; }
  // One line per direction: the table as K (kernel) / M (memcpy) letters, count-major, with the
  // measured times in microseconds when there are any.
  std::string describe() const;

  // Builds a policy without touching a GPU (tests, forced modes): mode "kernel", "memcpy" or "static".
  static CopyPolicy fixed(const std::string& mode);
  static void reset_for_test();   // the next get() resolves the environment (and measures) again

 private:
  void measure(int device);
  bool measured_{false};
  bool static_rule_{true};
  size_t static_max_blocks_{16};
  size_t static_threshold_{256 * 1024};
  CopyPath table_[2][kCountBuckets][kSizeBuckets]{};
  float us_[2][kCountBuckets][kSizeBuckets][2]{};   // [.][.][.][path]
};

}  // namespace kvx
