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
// A transfer that changes the cache layout (NHD pages to HND pages, a head window of a TP-mismatched pair) has no
// common byte ranges, but it has common ROWS: the head_bytes of one (request, token, K or V, head).  The second
// kernel walks the block tables of one side with that side's strides (the KvtLayout of the fused transfer kernel)
// and keys every byte by its row's logical coordinates, which are the same on both sides; the sums agree exactly
// when every row arrived intact at the slot and head the layout rule names.
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

// blockIdx.y names the tensor instance (one per layer): the same chunks are summed over bases[y] into out[y].
__global__ void __launch_bounds__(256) kvt_checksum_kernel(const uint64_t* __restrict__ bases, uint64_t capacity,
                                                           const KvtCheckChunk* __restrict__ chunks, uint32_t n,
                                                           unsigned long long* __restrict__ out,
                                                           uint32_t* __restrict__ status) {
  const uint8_t* __restrict__ base = reinterpret_cast<const uint8_t*>(bases[blockIdx.y]);
  out += blockIdx.y;
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

// One CTA per token, one warp per (K or V, head) row of it.
__global__ void __launch_bounds__(256) kvt_checksum_attn_kernel(const uint64_t* __restrict__ bases, uint64_t capacity,
                                                                const KvtLayout lay, uint32_t head0, uint32_t n_heads,
                                                                const KvtCheckReq* __restrict__ reqs, uint32_t n_reqs,
                                                                uint32_t total_tokens, const uint32_t* __restrict__ pool,
                                                                uint32_t pool_len, unsigned long long* __restrict__ out,
                                                                uint32_t* __restrict__ status) {
  const uint8_t* __restrict__ base = reinterpret_cast<const uint8_t*>(bases[blockIdx.y]);
  out += blockIdx.y;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, n_warps = blockDim.x >> 5;
  const uint32_t rows = lay.kv_count * n_heads;
  uint64_t acc = 0;
  for (uint32_t u = blockIdx.x; u < total_tokens; u += gridDim.x) {
    uint32_t lo = 0, hi = n_reqs;
    while (hi - lo > 1) {
      const uint32_t mid = (lo + hi) >> 1;
      if (reqs[mid].first <= u) lo = mid; else hi = mid;
    }
    const KvtCheckReq r = reqs[lo];
    const uint32_t t = r.seen + (u - r.first);
    const uint32_t bi = t / lay.ntpb, slot = t % lay.ntpb;
    if (bi >= r.n_blocks || r.blk_off + bi >= pool_len) {
      if (threadIdx.x == 0 && atomicCAS(status, 0u, KVT_ERR_BLOCK_RANGE) == 0u) status[1] = u;
      continue;
    }
    const uint32_t blk = pool[r.blk_off + bi];
    if (blk >= lay.num_blocks) {
      if (threadIdx.x == 0 && atomicCAS(status, 0u, KVT_ERR_BLOCK_RANGE) == 0u) status[1] = u;
      continue;
    }
    for (uint32_t row = warp; row < rows; row += n_warps) {
      const uint32_t kv = row / n_heads, j = row % n_heads;
      const int64_t off = (int64_t)blk * lay.block_stride + (int64_t)kv * lay.kv_stride + (int64_t)slot * lay.token_stride +
                          (int64_t)(head0 + j) * lay.head_stride;
      if (off < 0 || (uint64_t)off > capacity || lay.head_bytes > capacity - (uint64_t)off) {
        if (lane == 0 && atomicCAS(status, 0u, KVT_ERR_BLOCK_RANGE) == 0u) status[1] = u;
        continue;
      }
      const uint32_t row_id = ((r.index * 131u + t) * lay.kv_count + kv) * n_heads + j;
      const uint32_t at0 = row_id * lay.head_bytes;
      const uint8_t* p = base + off;
      if (((reinterpret_cast<uintptr_t>(p) | lay.head_bytes) & 15u) == 0) {
        const uint4* p4 = reinterpret_cast<const uint4*>(p);
        for (uint32_t i = lane; i < (lay.head_bytes >> 4); i += 32) {
          const uint4 v = p4[i];
          const uint32_t at = at0 + (i << 4);
          acc += word_terms(v.x, at) + word_terms(v.y, at + 4) + word_terms(v.z, at + 8) + word_terms(v.w, at + 12);
        }
      } else {
        for (uint32_t i = lane; i < lay.head_bytes; i += 32) acc += term(at0 + i, p[i]);
      }
    }
  }
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_down_sync(0xFFFFFFFFu, acc, d);
  if (lane == 0 && acc != 0) atomicAdd(out, (unsigned long long)acc);
}

}  // namespace

extern "C" int kvt_launch_checksum_attn(const uint64_t* d_bases, uint32_t n_bases, uint64_t capacity, const KvtLayout* layout,
                                        uint32_t head0, uint32_t n_heads, const KvtCheckReq* d_reqs, uint32_t n_reqs,
                                        uint32_t total_tokens, const uint32_t* d_pool, uint32_t pool_len, uint64_t* d_out,
                                        uint32_t* d_status, int grid_ctas, void* stream) {
  if (n_reqs == 0 || total_tokens == 0 || n_heads == 0 || n_bases == 0) return 0;
  if (layout->ntpb == 0 || layout->head_bytes == 0 || layout->kv_count == 0 || n_bases > 65535u) return (int)cudaErrorInvalidValue;
  const uint32_t want = (uint32_t)(grid_ctas > 0 ? grid_ctas : 148 * 8);
  const uint32_t per = (want + n_bases - 1) / n_bases;        // the grid is spread over the tensors
  const dim3 grid(per < total_tokens ? (per > 0 ? per : 1) : total_tokens, n_bases);
  kvt_checksum_attn_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      d_bases, capacity, *layout, head0, n_heads, d_reqs, n_reqs, total_tokens, d_pool, pool_len,
      reinterpret_cast<unsigned long long*>(d_out), d_status);
  return (int)cudaGetLastError();
}

extern "C" int kvt_launch_checksum(const uint64_t* d_bases, uint32_t n_bases, uint64_t capacity, const KvtCheckChunk* d_chunks,
                                   uint32_t n, uint64_t* d_out, uint32_t* d_status, int grid_ctas, void* stream) {
  if (n == 0 || n_bases == 0) return 0;
  if (n_bases > 65535u) return (int)cudaErrorInvalidValue;
  const uint32_t want = (uint32_t)(grid_ctas > 0 ? grid_ctas : 148 * 8);
  const uint32_t per = (want + n_bases - 1) / n_bases;
  const dim3 grid(per < n ? (per > 0 ? per : 1) : n, n_bases);
  kvt_checksum_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      d_bases, capacity, d_chunks, n, reinterpret_cast<unsigned long long*>(d_out), d_status);
  return (int)cudaGetLastError();
}

extern "C" uint64_t kvt_checksum_host(const void* data, uint64_t len, uint32_t index0) {
  const uint8_t* p = static_cast<const uint8_t*>(data);
  uint64_t acc = 0;
  for (uint64_t i = 0; i < len; ++i) acc += term(index0 + (uint32_t)i, p[i]);
  return acc;
}
