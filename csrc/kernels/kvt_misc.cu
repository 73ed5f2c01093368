// Smaller sm_100a kernels and the CUDA runtime helpers behind the C ABI:
//   * kvt_p2d_state   - block-relative strided segments; moves GDN / KDA / PLE recurrent state
//                       pages with the conv-row interleave of TP-mismatched ranks
//                       (offset rule of kvtransfer/src/parse_block_qwen3_next.cpp:440-502).
//   * kvt_copy_blocks - descriptor-driven copy of {src_off, dst_off, len} triples, the device
//                       end of the TCP / shared-memory staging path (what the reference's
//                       copy_d2h/h2d_direct kernels do, kvtransfer/src/copy_kernels.cu:105-281).
//   * bounded flag wait / flag set for completion signalling.
//   * peer-memory, IPC and mapped-host-memory helpers.
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

#include "kvt_kernels.h"

namespace {

__device__ __forceinline__ void set_status(uint32_t* status, uint32_t code, uint32_t detail) {
  if (status != nullptr) {
    if (atomicCAS(status, 0u, code) == 0u) status[1] = detail;
  }
}

// Copy `len` bytes with the widest vector both addresses allow.  Called by a whole CTA
// (stride = blockDim.x) or a warp (stride = 32).
__device__ __forceinline__ void copy_span(const char* __restrict__ s, char* __restrict__ d, uint32_t len,
                                          uint32_t lane, uint32_t stride) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d);
  if ((a & 15u) == 0) {
    const uint32_t n16 = len >> 4;
    const int4* s4 = reinterpret_cast<const int4*>(s);
    int4* d4 = reinterpret_cast<int4*>(d);
    uint32_t i = lane;
    for (; i + 3 * stride < n16; i += 4 * stride) {
      const int4 v0 = s4[i], v1 = s4[i + stride], v2 = s4[i + 2 * stride], v3 = s4[i + 3 * stride];
      d4[i] = v0;
      d4[i + stride] = v1;
      d4[i + 2 * stride] = v2;
      d4[i + 3 * stride] = v3;
    }
    for (; i < n16; i += stride) d4[i] = s4[i];
    for (uint32_t b = (n16 << 4) + lane; b < len; b += stride) d[b] = s[b];
  } else if ((a & 3u) == 0) {
    const uint32_t n4 = len >> 2;
    const int* s1 = reinterpret_cast<const int*>(s);
    int* d1 = reinterpret_cast<int*>(d);
    for (uint32_t i = lane; i < n4; i += stride) d1[i] = s1[i];
    for (uint32_t b = (n4 << 2) + lane; b < len; b += stride) d[b] = s[b];
  } else {
    for (uint32_t b = lane; b < len; b += stride) d[b] = s[b];
  }
}

__global__ void __launch_bounds__(512) kvt_p2d_state_kernel(const __grid_constant__ KvtStateLaunch p) {
  const uint32_t n_layers = p.layer_end - p.layer_begin;
  // Work item = (layer, page, rule, repetition); a warp takes one item when segments are
  // short, a CTA takes one when they are long.
  const uint32_t warps_per_cta = blockDim.x >> 5;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  for (uint32_t layer = 0; layer < n_layers; ++layer) {
    const char* src = reinterpret_cast<const char*>(p.src_layers[p.layer_begin + layer]);
    char* dst = reinterpret_cast<char*>(p.dst_layers[p.layer_begin + layer]);
    for (uint32_t r = 0; r < p.n_rules; ++r) {
      const KvtSegRule rule = p.rules[r];
      const uint64_t items = (uint64_t)p.n_pages * rule.count;
      if (rule.len >= 16384) {
        for (uint64_t it = blockIdx.x; it < items; it += gridDim.x) {
          const uint32_t page = (uint32_t)(it / rule.count);
          const uint32_t rep = (uint32_t)(it - (uint64_t)page * rule.count);
          const uint32_t sb = p.src_blocks[page], db = p.dst_blocks[page];
          if (sb >= p.src_num_blocks || db >= p.dst_num_blocks) {
            if (threadIdx.x == 0) set_status(p.status, KVT_ERR_BLOCK_RANGE, page);
            continue;
          }
          copy_span(src + (int64_t)sb * p.src_block_stride + rule.src_off + (int64_t)rep * rule.src_stride,
                    dst + (int64_t)db * p.dst_block_stride + rule.dst_off + (int64_t)rep * rule.dst_stride,
                    rule.len, threadIdx.x, blockDim.x);
        }
      } else {
        for (uint64_t it = (uint64_t)blockIdx.x * warps_per_cta + warp; it < items;
             it += (uint64_t)gridDim.x * warps_per_cta) {
          const uint32_t page = (uint32_t)(it / rule.count);
          const uint32_t rep = (uint32_t)(it - (uint64_t)page * rule.count);
          const uint32_t sb = p.src_blocks[page], db = p.dst_blocks[page];
          if (sb >= p.src_num_blocks || db >= p.dst_num_blocks) {
            if (lane == 0) set_status(p.status, KVT_ERR_BLOCK_RANGE, page);
            continue;
          }
          copy_span(src + (int64_t)sb * p.src_block_stride + rule.src_off + (int64_t)rep * rule.src_stride,
                    dst + (int64_t)db * p.dst_block_stride + rule.dst_off + (int64_t)rep * rule.dst_stride,
                    rule.len, lane, 32);
        }
      }
    }
  }
  if (p.flag != nullptr && p.done_counter != nullptr) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t prev = atomicAdd(p.done_counter, 1u);
      if (prev == gridDim.x - 1) {
        *p.done_counter = 0;
        __threadfence_system();
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p.flag), "l"(p.flag_value) : "memory");
      }
    }
  }
}

// A warp per 4 KiB segment.  The descriptors of one list are usually of one length (the pages of a
// cache tensor), so the segment count of the FIRST descriptor lays out the work: unit u is segment
// u % segs0 of descriptor u / segs0, and a descriptor longer than the first has its further
// segments taken by the same warps in a strided loop.  Few long descriptors thus spread over every
// SM as well as many short ones do.
constexpr uint32_t kCopySeg = 4096;

__global__ void __launch_bounds__(512) kvt_copy_blocks_kernel(const char* __restrict__ src, char* __restrict__ dst,
                                                               const uint64_t* __restrict__ triples, uint32_t n,
                                                               uint64_t src_cap, uint64_t dst_cap,
                                                               uint32_t* status) {
  const uint32_t warps_per_cta = blockDim.x >> 5;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint64_t len0 = triples[2];
  const uint32_t segs0 = len0 > kCopySeg ? (uint32_t)min((len0 + kCopySeg - 1) / kCopySeg, (uint64_t)65536) : 1u;
  const uint64_t total = (uint64_t)n * segs0;
  for (uint64_t u = (uint64_t)blockIdx.x * warps_per_cta + warp; u < total; u += (uint64_t)gridDim.x * warps_per_cta) {
    const uint32_t i = (uint32_t)(u / segs0);
    const uint32_t s0 = (uint32_t)(u - (uint64_t)i * segs0);
    const uint64_t so = triples[3 * i], dof = triples[3 * i + 1], len = triples[3 * i + 2];
    if (so > src_cap || len > src_cap - so || dof > dst_cap || len > dst_cap - dof || len > 0xffffffffull) {
      if (lane == 0 && s0 == 0) set_status(status, KVT_ERR_BLOCK_RANGE, i);
      continue;
    }
    for (uint64_t off = (uint64_t)s0 * kCopySeg; off < len; off += (uint64_t)segs0 * kCopySeg) {
      copy_span(src + so + off, dst + dof + off, (uint32_t)min((uint64_t)kCopySeg, len - off), lane, 32);
    }
  }
}

__global__ void __launch_bounds__(512) kvt_copy_blocks_multi_kernel(const __grid_constant__ KvtCopyMulti p) {
  const uint32_t warps_per_cta = blockDim.x >> 5;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  // per tensor: segments of its first descriptor lay out its units (see kvt_copy_blocks_kernel)
  uint32_t segs[KVT_COPY_MAX_TENSORS];
  uint64_t ends[KVT_COPY_MAX_TENSORS];
  uint64_t total = 0;
#pragma unroll
  for (uint32_t t = 0; t < KVT_COPY_MAX_TENSORS; ++t) {
    segs[t] = 1;
    if (t < p.n_tensors && p.count[t] > 0) {
      const uint64_t len0 = p.triples[3ull * p.first[t] + 2];
      if (len0 > kCopySeg) segs[t] = (uint32_t)min((len0 + kCopySeg - 1) / kCopySeg, (uint64_t)65536);
      total += (uint64_t)p.count[t] * segs[t];
    }
    ends[t] = total;
  }
  for (uint64_t u = (uint64_t)blockIdx.x * warps_per_cta + warp; u < total; u += (uint64_t)gridDim.x * warps_per_cta) {
    uint32_t t = 0;
#pragma unroll
    for (uint32_t k = 0; k + 1 < KVT_COPY_MAX_TENSORS; ++k) t += (u >= ends[k]) ? 1u : 0u;
    const uint64_t local = u - (t > 0 ? ends[t - 1] : 0);
    const uint32_t i = p.first[t] + (uint32_t)(local / segs[t]);
    const uint32_t s0 = (uint32_t)(local % segs[t]);
    const uint64_t so = p.triples[3ull * i], dof = p.triples[3ull * i + 1], len = p.triples[3ull * i + 2];
    if (so > p.src_cap[t] || len > p.src_cap[t] - so || dof > p.dst_cap[t] || len > p.dst_cap[t] - dof ||
        len > 0xffffffffull) {
      if (lane == 0 && s0 == 0) set_status(p.status, KVT_ERR_BLOCK_RANGE, i);
      continue;
    }
    const char* src = reinterpret_cast<const char*>(p.src_base[t]) + so;
    char* dst = reinterpret_cast<char*>(p.dst_base[t]) + dof;
    for (uint64_t off = (uint64_t)s0 * kCopySeg; off < len; off += (uint64_t)segs[t] * kCopySeg) {
      copy_span(src + off, dst + off, (uint32_t)min((uint64_t)kCopySeg, len - off), lane, 32);
    }
  }
}

__device__ __forceinline__ uint32_t cast4_bf16_e4m3(uint32_t lo, uint32_t hi) {
  // lo, hi: two bf16 pairs; returns four e4m3 bytes in memory order
  const float a = __uint_as_float(lo << 16), b = __uint_as_float(lo & 0xffff0000u);
  const float c = __uint_as_float(hi << 16), d = __uint_as_float(hi & 0xffff0000u);
  const uint32_t ab = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t cd = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return (ab & 0xffffu) | (cd << 16);
}

// A warp per 2048-value segment of a descriptor.
__global__ void __launch_bounds__(512) kvt_copy_blocks_cast_kernel(const char* __restrict__ src, char* __restrict__ dst,
                                                                    const uint64_t* __restrict__ triples, uint32_t n,
                                                                    uint64_t src_cap, uint64_t dst_cap, uint32_t* status) {
  constexpr uint32_t kSegVals = 2048;
  const uint32_t warps_per_cta = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint64_t len0 = triples[2];
  const uint32_t segs0 = len0 > kSegVals ? (uint32_t)min((len0 + kSegVals - 1) / kSegVals, (uint64_t)65536) : 1u;
  const uint64_t total = (uint64_t)n * segs0;
  for (uint64_t u = (uint64_t)blockIdx.x * warps_per_cta + warp; u < total; u += (uint64_t)gridDim.x * warps_per_cta) {
    const uint32_t i = (uint32_t)(u / segs0);
    const uint32_t s0 = (uint32_t)(u - (uint64_t)i * segs0);
    const uint64_t so = triples[3 * i], dof = triples[3 * i + 1], len = triples[3 * i + 2];
    if (len > 0x7fffffffull || so > src_cap || 2 * len > src_cap - so || dof > dst_cap || len > dst_cap - dof) {
      if (lane == 0 && s0 == 0) set_status(status, KVT_ERR_BLOCK_RANGE, i);
      continue;
    }
    for (uint64_t off = (uint64_t)s0 * kSegVals; off < len; off += (uint64_t)segs0 * kSegVals) {
      const uint32_t cnt = (uint32_t)min((uint64_t)kSegVals, len - off);
      const char* s = src + so + 2 * off;
      char* d = dst + dof + off;
      if (((reinterpret_cast<uintptr_t>(s) & 7u) | (reinterpret_cast<uintptr_t>(d) & 3u)) == 0) {
        const uint32_t n4 = cnt >> 2;   // four values per step: 8 bytes in, 4 bytes out
        const uint2* s2 = reinterpret_cast<const uint2*>(s);
        uint32_t* d1 = reinterpret_cast<uint32_t*>(d);
        for (uint32_t k = lane; k < n4; k += 32) {
          const uint2 v = s2[k];
          d1[k] = cast4_bf16_e4m3(v.x, v.y);
        }
        for (uint32_t k = (n4 << 2) + lane; k < cnt; k += 32) {
          const uint16_t h = reinterpret_cast<const uint16_t*>(s)[k];
          d[k] = (char)__nv_cvt_float_to_fp8(__uint_as_float((uint32_t)h << 16), __NV_SATFINITE, __NV_E4M3);
        }
      } else {
        for (uint32_t k = lane; k < cnt; k += 32) {
          const uint32_t h = (uint32_t)(unsigned char)s[2 * k] | ((uint32_t)(unsigned char)s[2 * k + 1] << 8);
          d[k] = (char)__nv_cvt_float_to_fp8(__uint_as_float(h << 16), __NV_SATFINITE, __NV_E4M3);
        }
      }
    }
  }
}

__global__ void kvt_wait_flag_kernel(const uint64_t* flag, uint64_t value, uint64_t timeout_ns, uint32_t* status) {
  uint64_t t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flag) : "memory");
    if (v >= value) return;
    uint64_t now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (now - t0 > timeout_ns) {
      set_status(status, KVT_ERR_FLAG_TIMEOUT, (uint32_t)v);
      return;
    }
    __nanosleep(200);
  }
}

__global__ void kvt_set_flag_kernel(uint64_t* flag, uint64_t value) {
  __threadfence_system();
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flag), "l"(value) : "memory");
}

int pick_grid(int grid_ctas) {
  if (grid_ctas > 0) return grid_ctas;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 0 ? sms : 1;
}

}  // namespace

extern "C" int kvt_launch_p2d_state(const KvtStateLaunch* args, int grid_ctas, int threads, void* stream) {
  if (args->n_pages == 0 || args->n_rules == 0 || args->layer_end <= args->layer_begin) return (int)cudaSuccess;
  if (threads <= 0) threads = 512;
  threads = (threads + 31) / 32 * 32;
  if (threads > 512) threads = 512;
  kvt_p2d_state_kernel<<<pick_grid(grid_ctas), threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*args);
  return (int)cudaGetLastError();
}

extern "C" int kvt_launch_copy_blocks(uint64_t src_base, uint64_t dst_base, const uint64_t* triples, uint32_t n,
                                      uint64_t src_capacity, uint64_t dst_capacity, uint32_t* status,
                                      int grid_ctas, void* stream) {
  if (n == 0) return (int)cudaSuccess;
  // two CTAs of 512 threads per SM by default: a warp keeps 2 KiB in flight
  kvt_copy_blocks_kernel<<<grid_ctas > 0 ? grid_ctas : 2 * pick_grid(0), 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const char*>(src_base), reinterpret_cast<char*>(dst_base), triples, n, src_capacity,
      dst_capacity, status);
  return (int)cudaGetLastError();
}

extern "C" int kvt_launch_copy_blocks_cast(uint64_t src_base, uint64_t dst_base, const uint64_t* triples, uint32_t n,
                                           uint64_t src_capacity, uint64_t dst_capacity, uint32_t* status,
                                           int grid_ctas, void* stream) {
  if (n == 0) return (int)cudaSuccess;
  kvt_copy_blocks_cast_kernel<<<grid_ctas > 0 ? grid_ctas : pick_grid(0), 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const char*>(src_base), reinterpret_cast<char*>(dst_base), triples, n, src_capacity, dst_capacity,
      status);
  return (int)cudaGetLastError();
}

extern "C" uint8_t kvt_bf16_to_e4m3(uint16_t bits) {
  const uint32_t sign = (bits >> 8) & 0x80u;
  const uint32_t mag = bits & 0x7fffu;
  if (mag > 0x7f80u) return (uint8_t)0x7fu;                           // NaN: the hardware conversion drops the sign
  uint32_t fb = mag << 16;
  float x;
  memcpy(&x, &fb, 4);
  if (x >= 464.0f) return (uint8_t)(sign | 0x7eu);                    // beyond the last tie: saturates to 448 (inf too)
  if (x < 0.015625f) {                                                // below the smallest normal 2^-6: steps of 2^-9
    const float q = nearbyintf(x * 512.0f);                           // round to nearest even (default rounding mode)
    return (uint8_t)(sign | (uint32_t)q);                             // q == 8 encodes 2^-6 by itself
  }
  int e;
  const float m = frexpf(x, &e);                                      // x = m * 2^e, m in [0.5, 1)
  int E = e - 1 + 7;
  float frac = nearbyintf((m * 2.0f - 1.0f) * 8.0f);
  if (frac >= 8.0f) {
    frac = 0.0f;
    E += 1;
  }
  const uint32_t code = ((uint32_t)E << 3) | (uint32_t)frac;
  return (uint8_t)(sign | (code > 0x7eu ? 0x7eu : code));
}

extern "C" int kvt_launch_copy_blocks_multi(const KvtCopyMulti* args, int grid_ctas, void* stream) {
  if (args->n_tensors == 0 || args->n_tensors > KVT_COPY_MAX_TENSORS) return (int)cudaErrorInvalidValue;
  uint64_t n = 0;
  for (uint32_t t = 0; t < args->n_tensors; ++t) n += args->count[t];
  if (n == 0) return (int)cudaSuccess;
  kvt_copy_blocks_multi_kernel<<<grid_ctas > 0 ? grid_ctas : 2 * pick_grid(0), 512, 0,
                                 reinterpret_cast<cudaStream_t>(stream)>>>(*args);
  return (int)cudaGetLastError();
}

extern "C" int kvt_launch_wait_flag(const uint64_t* flag, uint64_t value, uint64_t timeout_ns, uint32_t* status,
                                    void* stream) {
  kvt_wait_flag_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flag, value, timeout_ns, status);
  return (int)cudaGetLastError();
}

__global__ void kvt_stamp_kernel(uint64_t* slot) {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  *slot = t;
}

extern "C" int kvt_launch_stamp(uint64_t* slot, void* stream) {
  if (slot == nullptr || (reinterpret_cast<uintptr_t>(slot) & 7u) != 0) return (int)cudaErrorInvalidValue;
  kvt_stamp_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(slot);
  return (int)cudaGetLastError();
}

// Completion record of one batch.  Runs alone on a stream that has been ordered after every kernel of the
// batch: it moves the batch's status words and timer stamps into the record (mapped host memory), clears the
// status words for the slot's next batch and publishes the sequence number last, with release semantics at
// system scope, so that a host thread that reads the sequence number also reads the rest.
__global__ void kvt_complete_kernel(uint32_t* status, KvtCompletion* rec, uint64_t seq) {
  uint64_t now;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
  const uint32_t code = status[0], detail = status[1];
  const uint64_t t0 = *reinterpret_cast<const uint64_t*>(status + 2);
  rec->status = code;
  rec->detail = detail;
  rec->t_start_ns = t0;
  rec->t_end_ns = now;
  status[0] = 0;
  status[1] = 0;
  status[2] = 0;
  status[3] = 0;
  __threadfence_system();
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(&rec->seq), "l"(seq) : "memory");
}

extern "C" int kvt_launch_complete(uint32_t* status, KvtCompletion* record, uint64_t seq, void* stream) {
  if (status == nullptr || record == nullptr || (reinterpret_cast<uintptr_t>(record) & 7u) != 0 ||
      (reinterpret_cast<uintptr_t>(status) & 7u) != 0)
    return (int)cudaErrorInvalidValue;
  kvt_complete_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status, record, seq);
  return (int)cudaGetLastError();
}

extern "C" int kvt_launch_set_flag(uint64_t* flag, uint64_t value, void* stream) {
  kvt_set_flag_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flag, value);
  return (int)cudaGetLastError();
}

extern "C" int kvt_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

extern "C" int kvt_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return ok;
}

extern "C" int kvt_enable_peer_access(int dev, int peer) {
  int cur = 0;
  cudaGetDevice(&cur);
  cudaError_t e = cudaSetDevice(dev);
  if (e == cudaSuccess) {
    e = cudaDeviceEnablePeerAccess(peer, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
      cudaGetLastError();
      e = cudaSuccess;
    }
  }
  cudaSetDevice(cur);
  return (int)e;
}

extern "C" int kvt_p2p_attribute(int dev, int peer, int which) {
  cudaDeviceP2PAttr attr = cudaDevP2PAttrPerformanceRank;
  if (which == 1) attr = cudaDevP2PAttrAccessSupported;
  if (which == 2) attr = cudaDevP2PAttrNativeAtomicSupported;
  int v = 0;
  if (cudaDeviceGetP2PAttribute(&v, attr, dev, peer) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return v;
}

extern "C" int kvt_ipc_get_handle(uint64_t ptr, void* handle64, uint64_t* base, uint64_t* size) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes on the wire");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(ptr));
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, 64);
  // The handle names the whole allocation; report its range so the peer can rebase ptr.
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  *base = ptr;
  *size = 0;
  if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q) == cudaSuccess && fn != nullptr) {
    typedef int (*range_fn)(unsigned long long*, size_t*, unsigned long long);
    unsigned long long b = 0;
    size_t s = 0;
    if (reinterpret_cast<range_fn>(fn)(&b, &s, ptr) == 0) {
      *base = b;
      *size = s;
    }
  }
  return 0;
}

extern "C" int kvt_ipc_open_handle(const void* handle64, uint64_t* out_ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  *out_ptr = reinterpret_cast<uint64_t>(p);
  return (int)e;
}

extern "C" int kvt_ipc_close(uint64_t ptr) { return (int)cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)); }

extern "C" int kvt_malloc(uint64_t bytes, uint64_t* out_ptr) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  *out_ptr = reinterpret_cast<uint64_t>(p);
  return (int)e;
}

extern "C" int kvt_free(uint64_t ptr) { return (int)cudaFree(reinterpret_cast<void*>(ptr)); }

extern "C" int kvt_host_alloc_mapped(uint64_t bytes, uint64_t* host_ptr, uint64_t* dev_ptr) {
  void* h = nullptr;
  cudaError_t e = cudaHostAlloc(&h, bytes, cudaHostAllocMapped | cudaHostAllocPortable);
  if (e != cudaSuccess) return (int)e;
  void* d = nullptr;
  e = cudaHostGetDevicePointer(&d, h, 0);
  *host_ptr = reinterpret_cast<uint64_t>(h);
  *dev_ptr = reinterpret_cast<uint64_t>(d);
  return (int)e;
}

extern "C" int kvt_host_free(uint64_t host_ptr) { return (int)cudaFreeHost(reinterpret_cast<void*>(host_ptr)); }

extern "C" int kvt_host_register(uint64_t host_ptr, uint64_t bytes, uint64_t* dev_ptr) {
  cudaError_t e = cudaHostRegister(reinterpret_cast<void*>(host_ptr), bytes,
                                   cudaHostRegisterMapped | cudaHostRegisterPortable);
  if (e != cudaSuccess) return (int)e;
  void* d = nullptr;
  e = cudaHostGetDevicePointer(&d, reinterpret_cast<void*>(host_ptr), 0);
  *dev_ptr = reinterpret_cast<uint64_t>(d);
  return (int)e;
}

extern "C" int kvt_host_unregister(uint64_t host_ptr) {
  return (int)cudaHostUnregister(reinterpret_cast<void*>(host_ptr));
}

// ---- copy-engine paths: the in-run bandwidth ceilings and the library baseline of the benchmark ----
extern "C" int kvt_memcpy_async(uint64_t dst, uint64_t src, uint64_t bytes, void* stream) {
  return (int)cudaMemcpyAsync(reinterpret_cast<void*>(dst), reinterpret_cast<const void*>(src), bytes, cudaMemcpyDefault,
                              reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int kvt_memcpy_triples(uint64_t dst_base, uint64_t src_base, const uint64_t* host_triples, uint32_t n,
                                  void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  for (uint32_t i = 0; i < n; ++i) {
    const cudaError_t e = cudaMemcpyAsync(reinterpret_cast<void*>(dst_base + host_triples[3ull * i + 1]),
                                          reinterpret_cast<const void*>(src_base + host_triples[3ull * i]),
                                          host_triples[3ull * i + 2], cudaMemcpyDefault, st);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

extern "C" int kvt_sm_count(int dev) {
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return sms;
}

extern "C" const char* kvt_error_string(int err) { return cudaGetErrorString(static_cast<cudaError_t>(err)); }
