// Descriptor-driven block copy for callers that must not allocate.
//
// Some callers of the copy path cannot tolerate a device or pinned-host allocation at call time:
// a transfer issued from inside a serving engine's steady state, where an allocation may
// synchronise the whole device or fragment a pool that the engine has sized to the last byte; an
// error-recovery path that runs when the device is already out of memory; a host thread that
// holds a lock the allocator also takes.  The ordinary entry point (kvt_launch_copy_blocks) leaves
// the descriptor array and the status word to the caller, who normally gets them from an
// allocator.  This variant keeps both in a fixed array that lives in the module's own device
// image, so the call itself neither allocates nor frees anything, on the device or on the host:
// it issues one async memset, one async copy of the descriptors, the kernel and (optionally) one
// async copy of the status words back.
//
// Limits and rules:
//   * at most KVT_NOALLOC_MAX_DESCS descriptors per call; more is rejected with
//     KVT_NOALLOC_ERR_TOO_MANY and nothing is launched;
//   * the first call on a device looks up the address of the scratch array
//     (cudaGetSymbolAddress, with that device current) and caches it; make that first call
//     before any stream capture begins.  Threads that make their first calls at the same time
//     each do the lookup and publish the same values (the address with release order, after the
//     SM count), so none of them can see a half-filled entry;
//   * host_triples is read by an async copy on the stream: in pinned memory it is read when the
//     stream reaches the copy, so it must stay untouched until then (an event recorded after
//     the call, or the status words' arrival, tells); pageable memory is staged before the call
//     returns;
//   * the status words are cleared on the stream before every launch;
//   * there is ONE scratch array per device: two calls on the same device that overlap in time
//     (different streams, or different threads) race on it.  Serialise them.
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "kvt_kernels.h"

namespace {

constexpr uint32_t kMaxDescs = KVT_NOALLOC_MAX_DESCS;
constexpr uint32_t kStatusWords = 64;   // 256 B: keeps the descriptor area 256-byte aligned too
constexpr int kMaxDevices = 64;

// [0, 64) u32 status words (word 0 = code, word 1 = detail), then 3 u64 per descriptor.
static __device__ __align__(256) unsigned char g_scratch[kStatusWords * 4 + (size_t)kMaxDescs * 24];

struct DevSlot {
  std::atomic<unsigned char*> ptr{nullptr};   // published last: a reader that sees it also sees sms
  std::atomic<int> sms{0};
};
DevSlot g_slots[kMaxDevices];

__device__ __forceinline__ void note_error(uint32_t* status, uint32_t code, uint32_t detail) {
  if (atomicCAS(status, 0u, code) == 0u) status[1] = detail;
}

__device__ __forceinline__ void span_copy(const char* __restrict__ s, char* __restrict__ d, uint32_t len, uint32_t lane,
                                          uint32_t stride) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d);
  if ((a & 15u) == 0) {
    const uint32_t n16 = len >> 4;
    const int4* s4 = reinterpret_cast<const int4*>(s);
    int4* d4 = reinterpret_cast<int4*>(d);
    uint32_t i = lane;
    for (; i + stride < n16; i += 2 * stride) {
      const int4 v0 = s4[i], v1 = s4[i + stride];
      d4[i] = v0;
      d4[i + stride] = v1;
    }
    for (; i < n16; i += stride) d4[i] = s4[i];
    for (uint32_t b = (n16 << 4) + lane; b < len; b += stride) d[b] = s[b];
  } else {
    for (uint32_t b = lane; b < len; b += stride) d[b] = s[b];
  }
}

// One warp per descriptor; scratch = status words followed by the descriptors.
__global__ void __launch_bounds__(256) kvt_copy_blocks_noalloc_kernel(const char* __restrict__ src,
                                                                       char* __restrict__ dst,
                                                                       unsigned char* __restrict__ scratch, uint32_t n,
                                                                       uint64_t src_cap, uint64_t dst_cap) {
  uint32_t* status = reinterpret_cast<uint32_t*>(scratch);
  const uint64_t* triples = reinterpret_cast<const uint64_t*>(scratch + kStatusWords * 4);
  const uint32_t wpc = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  for (uint32_t i = blockIdx.x * wpc + warp; i < n; i += gridDim.x * wpc) {
    const uint64_t so = triples[3 * i], dof = triples[3 * i + 1], len = triples[3 * i + 2];
    if (so > src_cap || len > src_cap - so || dof > dst_cap || len > dst_cap - dof || len > 0xffffffffull) {
      if (lane == 0) note_error(status, KVT_ERR_BLOCK_RANGE, i);
      continue;
    }
    span_copy(src + so, dst + dof, (uint32_t)len, lane, 32);
  }
}

// Set-up of the current device: one symbol lookup and one attribute query, both cached.
int device_slot(DevSlot** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return KVT_NOALLOC_ERR_BAD_ARGS;
  DevSlot& s = g_slots[dev];
  if (s.ptr.load(std::memory_order_acquire) == nullptr) {
    unsigned char* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_scratch);
    if (e != cudaSuccess) return (int)e;
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    s.sms.store(sms > 0 ? sms : 1, std::memory_order_relaxed);
    s.ptr.store(p, std::memory_order_release);
  }
  *out = &s;
  return 0;
}

}  // namespace

extern "C" int kvt_copy_blocks_noalloc(uint64_t src_base, uint64_t dst_base, const uint64_t* host_triples, uint32_t n,
                                       uint64_t src_capacity, uint64_t dst_capacity, uint32_t* host_status,
                                       void* stream) {
  if (n > kMaxDescs) return KVT_NOALLOC_ERR_TOO_MANY;
  if (n > 0 && (host_triples == nullptr || src_base == 0 || dst_base == 0)) return KVT_NOALLOC_ERR_BAD_ARGS;
  DevSlot* slot = nullptr;
  const int rc = device_slot(&slot);
  if (rc != 0) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  unsigned char* const scratch = slot->ptr.load(std::memory_order_acquire);
  cudaError_t e = cudaMemsetAsync(scratch, 0, kStatusWords * 4, st);
  if (e != cudaSuccess) return (int)e;
  if (n > 0) {
    e = cudaMemcpyAsync(scratch + kStatusWords * 4, host_triples, (size_t)n * 24, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return (int)e;
    const uint32_t wpc = 256 / 32;
    uint32_t grid = (n + wpc - 1) / wpc;
    const uint32_t cap = (uint32_t)slot->sms.load(std::memory_order_relaxed) * 8u;
    if (grid > cap) grid = cap;
    kvt_copy_blocks_noalloc_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const char*>(src_base),
                                                         reinterpret_cast<char*>(dst_base), scratch, n, src_capacity,
                                                         dst_capacity);
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  if (host_status != nullptr) {
    e = cudaMemcpyAsync(host_status, scratch, 8, cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}
