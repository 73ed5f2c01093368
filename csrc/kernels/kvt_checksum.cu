// Position-keyed checksum of byte ranges of one cache tensor: the device half of the end-to-end
// transfer check (BLLM_KVTRANS_CRC=1).
//
// The reference checks an RDMA transfer by CRC-32 over the source ranges on the sender's CPU (through a
// gdrcopy mapping) and over the destination ranges on the receiver's CPU (kvtransfer/src/
// rdma_channel.cpp:143-296, 845-852).  A CRC is a serial recurrence; a GPU wants a sum.  Here every byte
// contributes  mix32(((i & 0xFFFFFF) << 8) | byte)  where i is the byte's index inside its piece (a piece
// is one {offset, length} range of the transfer; both sides use the sender's piece list, so i is the same
// on both), and a piece's value is the 64-bit sum of its bytes' terms: independent of the order in which
// pieces and bytes are visited, sensitive to a byte's value and to its place in the piece.  Each GPU reads
// only its own memory: nothing crosses the link for the check except the piece list and one number.
//
// The host splits pieces into chunks of at most 64 KiB {offset, length, index of the first byte in its
// piece} so that one long merged piece still spreads over the whole GPU; kvt_checksum_host is the same
// function on the CPU (host-resident caches, and the oracle of the kernel's test).
#include <cuda_runtime.h>
#include <stdint.h>

#include "kvt_kernels.h"

namespace {

__host__ __device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x *= 0x9E3779B1u;
  x ^= x >> 15;
  x *= 0x85EBCA77u;
  x ^= x >> 13;
  return x;
}

__host__ __device__ __forceinline__ uint32_t term(uint32_t index, uint32_t byte) {
  return mix32(((index & 0xFFFFFFu) << 8) | byte);
}

__device__ __forceinline__ uint64_t word_terms(uint32_t w, uint32_t index) {
  return (uint64_t)term(index, w & 0xFFu) + term(index + 1, (w >> 8) & 0xFFu) + term(index + 2, (w >> 16) & 0xFFu) +
         term(index + 3, w >> 24);
}

__global__ void __launch_bounds__(256) kvt_checksum_kernel(const uint8_t* __restrict__ base, uint64_t capacity,
                                                           const KvtCheckChunk* __restrict__ chunks, uint32_t n,
                                                           unsigned long long* __restrict__ out,
                                                           uint32_t* __restrict__ status) {
  uint64_t acc = 0;
  for (uint32_t c = blockIdx.x; c < n; c += gridDim.x) {
    const KvtCheckChunk ch = chunks[c];
    if (ch.off > capacity || ch.len > capacity - ch.off) {   // never read outside the tensor: report and skip
      if (threadIdx.x == 0 && atomicCAS(status, 0u, KVT_ERR_BLOCK_RANGE) == 0u) status[1] = c;
      continue;
    }
    const uint8_t* p = base + ch.off;
    if (((reinterpret_cast<uintptr_t>(p) | ch.len) & 15u) == 0) {
      const uint4* p4 = reinterpret_cast<const uint4*>(p);
      for (uint32_t i = threadIdx.x; i < (ch.len >> 4); i += blockDim.x) {
        const uint4 v = p4[i];
        const uint32_t at = ch.index0 + (i << 4);
        acc += word_terms(v.x, at) + word_terms(v.y, at + 4) + word_terms(v.z, at + 8) + word_terms(v.w, at + 12);
      }
    } else {
      for (uint32_t i = threadIdx.x; i < ch.len; i += blockDim.x) acc += term(ch.index0 + i, p[i]);
    }
  }
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_down_sync(0xFFFFFFFFu, acc, d);
  if ((threadIdx.x & 31u) == 0 && acc != 0) atomicAdd(out, (unsigned long long)acc);
}

}  // namespace

extern "C" int kvt_launch_checksum(uint64_t base, uint64_t capacity, const KvtCheckChunk* d_chunks, uint32_t n,
                                   uint64_t* d_out, uint32_t* d_status, int grid_ctas, void* stream) {
  if (n == 0) return 0;
  const uint32_t grid = (uint32_t)(grid_ctas > 0 ? grid_ctas : 148 * 4);
  kvt_checksum_kernel<<<grid < n ? grid : n, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint8_t*>(base), capacity, d_chunks, n, reinterpret_cast<unsigned long long*>(d_out),
      d_status);
  return (int)cudaGetLastError();
}

extern "C" uint64_t kvt_checksum_host(const void* data, uint64_t len, uint32_t index0) {
  const uint8_t* p = static_cast<const uint8_t*>(data);
  uint64_t acc = 0;
  for (uint64_t i = 0; i < len; ++i) acc += term(index0 + (uint32_t)i, p[i]);
  return acc;
}
