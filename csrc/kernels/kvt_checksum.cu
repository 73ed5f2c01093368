// Position-keyed checksum of byte ranges of one cache tensor: the device half of the end-to-end
// transfer check (BLLM_KVTRANS_CRC=1).
//
// The reference checks an RDMA transfer by CRC-32 over the source ranges on the sender's CPU (through a
// gdrcopy mapping) and over the destination ranges on the receiver's CPU (kvtransfer/src/
// rdma_channel.cpp:143-296, 845-852).  A CRC is a serial recurrence; a GPU wants a sum.  Here a piece (one
// {offset, length} range of the transfer; both sides use the sender's piece list) is read as little-endian
// 32-bit words, the last one padded with zero bytes, and word k with value w contributes
//   term(k, w) = mix(w * 0x9E3779B1 ^ rotl(k * 0x85EBCA77, 13)),   mix(x) = (x ^ x >> 15) * 0xC2B2AE3D, then x ^ x >> 13
// to the piece's 64-bit sum: independent of the order in which pieces and words are visited, sensitive to a
// word's value and to its place in the piece, three multiplies per four bytes.  Where a piece starts in memory
// does not enter: a side whose copy of the piece is not word-aligned assembles the words from bytes.  Each GPU
// reads only its own memory: nothing crosses the link for the check except the piece list and one number.
//
// A transfer that changes the cache layout (NHD pages to HND pages, a head window of a TP-mismatched pair) has no
// common byte ranges, but it has common ROWS: the head_bytes of one (request, token, K or V, head).  The second
// kernel walks the block tables of one side with that side's strides (the KvtLayout of the fused transfer kernel)
// and keys every word by its row's logical coordinates, which are the same on both sides; the sums agree exactly
// when every row arrived intact at the slot and head the layout rule names.
//
// The host splits pieces into chunks of at most 64 KiB {offset, length, index of the first word in its
// piece} so that one long merged piece still spreads over the whole GPU; kvt_checksum_host is the same
// function on the CPU (host-resident caches, and the oracle of the kernel's test).
#include <cuda_runtime.h>
#include <stdint.h>

#include "kvt_kernels.h"

namespace {

__host__ __device__ __forceinline__ uint32_t term(uint32_t k, uint32_t w) {
  const uint32_t key = k * 0x85EBCA77u;
  uint32_t x = (w * 0x9E3779B1u) ^ ((key << 13) | (key >> 19));
  x ^= x >> 15;
  x *= 0xC2B2AE3Du;
  x ^= x >> 13;
  return x;
}

// Word k of a piece of `len` bytes at p, whatever p's alignment; bytes past the end read as zero.
__host__ __device__ __forceinline__ uint32_t word_at(const uint8_t* p, uint64_t len, uint64_t k) {
  const uint64_t at = k << 2;
  uint32_t w = 0;
#pragma unroll
  for (uint32_t b = 0; b < 4; ++b)
    if (at + b < len) w |= (uint32_t)p[at + b] << (8 * b);
  return w;
}

// Sum of the words [0, ceil(len / 4)) of the piece part at p, the first of which is word k0 of its piece; the
// calling threads are `lane` of `width`.
__device__ __forceinline__ uint64_t part_sum(const uint8_t* __restrict__ p, uint32_t len, uint32_t k0, uint32_t lane,
                                             uint32_t width) {
  uint64_t acc = 0;
  const uint32_t n_words = (len + 3u) >> 2;
  uint32_t done = 0;                                   // words covered by the vector path
  if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
    const uint4* p4 = reinterpret_cast<const uint4*>(p);
    const uint32_t n16 = len >> 4;
    for (uint32_t i = lane; i < n16; i += width) {
      const uint4 v = p4[i];
      const uint32_t k = k0 + (i << 2);
      acc += (uint64_t)term(k, v.x) + term(k + 1, v.y) + term(k + 2, v.z) + term(k + 3, v.w);
    }
    done = n16 << 2;
  }
  const bool aligned4 = (reinterpret_cast<uintptr_t>(p) & 3u) == 0;
  for (uint32_t k = done + lane; k < n_words; k += width) {
    const uint32_t w = (aligned4 && (k << 2) + 4u <= len) ? reinterpret_cast<const uint32_t*>(p)[k] : word_at(p, len, k);
    acc += term(k0 + k, w);
  }
  return acc;
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
    acc += part_sum(base + ch.off, ch.len, ch.index0, threadIdx.x, blockDim.x);
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
  const uint32_t row_words = (lay.head_bytes + 3u) >> 2;
  const uint32_t lanes_per_row = lay.head_bytes <= 256u ? 16u : 32u, rows_per_warp = 32u / lanes_per_row;
  const uint32_t sub = lane / lanes_per_row, sub_lane = lane % lanes_per_row;
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
    // rows of up to 256 bytes take half a warp each: two rows per warp per pass
    for (uint32_t row = warp * rows_per_warp + sub; row < rows; row += n_warps * rows_per_warp) {
      const uint32_t kv = row / n_heads, j = row % n_heads;
      const int64_t off = (int64_t)blk * lay.block_stride + (int64_t)kv * lay.kv_stride + (int64_t)slot * lay.token_stride +
                          (int64_t)(head0 + j) * lay.head_stride;
      if (off < 0 || (uint64_t)off > capacity || lay.head_bytes > capacity - (uint64_t)off) {
        if (sub_lane == 0 && atomicCAS(status, 0u, KVT_ERR_BLOCK_RANGE) == 0u) status[1] = u;
        continue;
      }
      const uint32_t row_id = ((r.index * 131u + t) * lay.kv_count + kv) * n_heads + j;
      acc += part_sum(base + off, lay.head_bytes, row_id * row_words, sub_lane, lanes_per_row);
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
  const uint64_t n_words = (len + 3u) >> 2;
  for (uint64_t k = 0; k < n_words; ++k) acc += term(index0 + (uint32_t)k, word_at(p, len, k));
  return acc;
}
