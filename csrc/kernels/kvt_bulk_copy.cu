// kvt_copy_blocks_bulk: the descriptor copy of kvt_copy_blocks_multi with the TMA engine doing the
// moving.  The byte ranges of the multi-tensor cache shapes (MLA latent and indexer pages, GDN / KDA
// state pages) are whole pages: long, 16-byte aligned runs.  One elected thread per CTA streams
// them through shared memory with untiled bulk copies (cp.async.bulk global -> shared on an
// mbarrier, shared -> global in a bulk group), several segments in flight, while the SMs' load /
// store units stay idle; the SIMT warps only take what the bulk engine cannot (a run or a tail
// that is not made of whole 16-byte words).  Destinations may be peer memory (stores); sources
// are local.  No copy here uses cluster multicast.  Every wait is bounded and reports through
// the status words.
#include <cuda_runtime.h>
#include <stdint.h>

#include "kvt_kernels.h"

namespace {

constexpr uint32_t kSeg = 8192;                 // bytes per bulk copy
constexpr int kMaxStagesB = 8;
constexpr long long kWaitCyclesB = 4000000000LL;  // ~2 s at 2 GHz

__device__ __forceinline__ void set_status(uint32_t* status, uint32_t code, uint32_t detail) {
  if (status != nullptr) {
    if (atomicCAS(status, 0u, code) == 0u) status[1] = detail;
  }
}
__device__ __forceinline__ uint32_t smem_u32(const void* ptr) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(ptr));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_dst),
               "l"(gsrc), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

struct Unit {
  const char* src;
  char* dst;
  uint32_t len;     // 0: nothing to do (out of range, or a segment beyond this descriptor's end)
  uint32_t desc;
  bool bad;
};

// Work layout shared by both passes: entry e contributes count[e] x segs[e] units, where segs[e]
// comes from the FIRST descriptor of the entry (pages of one tensor have one size); a descriptor
// longer than that has its further segments taken in a strided loop by the same unit.
struct Layout {
  uint32_t segs[KVT_COPY_MAX_TENSORS];
  uint64_t ends[KVT_COPY_MAX_TENSORS];
  uint64_t total;
};

// Units that a descriptor of this length is split over: one per 8 KiB segment, at most kMaxSegs
// (longer descriptors take further segments in later rounds).  The host's round count and the
// kernel's layout both come from here.
constexpr uint64_t kMaxSegs = 65536;
__host__ __device__ __forceinline__ uint32_t segs_of(uint64_t len) {
  if (len <= kSeg) return 1;
  const uint64_t s = (len + kSeg - 1) / kSeg;
  return (uint32_t)(s < kMaxSegs ? s : kMaxSegs);
}

__device__ __forceinline__ Layout make_layout(const KvtCopyMulti& p) {
  Layout l;
  l.total = 0;
#pragma unroll
  for (uint32_t t = 0; t < KVT_COPY_MAX_TENSORS; ++t) {
    l.segs[t] = 1;
    if (t < p.n_tensors && p.count[t] > 0) {
      const uint64_t len0 = p.triples[3ull * p.first[t] + 2];
      l.segs[t] = segs_of(len0);
      l.total += (uint64_t)p.count[t] * l.segs[t];
    }
    l.ends[t] = l.total;
  }
  return l;
}

// Segment number `round` (0, 1, ...) of unit u: its first segment is s0, the next s0 + segs, ...
__device__ __forceinline__ Unit decode(const KvtCopyMulti& p, const Layout& l, uint64_t u, uint32_t round) {
  Unit r;
  r.len = 0;
  r.bad = false;
  r.src = nullptr;
  r.dst = nullptr;
  uint32_t t = 0;
#pragma unroll
  for (uint32_t k = 0; k + 1 < KVT_COPY_MAX_TENSORS; ++k) t += (u >= l.ends[k]) ? 1u : 0u;
  const uint64_t local = u - (t > 0 ? l.ends[t - 1] : 0);
  const uint32_t i = p.first[t] + (uint32_t)(local / l.segs[t]);
  const uint32_t s0 = (uint32_t)(local % l.segs[t]);
  r.desc = i;
  const uint64_t so = p.triples[3ull * i], dof = p.triples[3ull * i + 1], len = p.triples[3ull * i + 2];
  if (so > p.src_cap[t] || len > p.src_cap[t] - so || dof > p.dst_cap[t] || len > p.dst_cap[t] - dof ||
      len > 0xffffffffull) {
    r.bad = s0 == 0 && round == 0;
    return r;
  }
  const uint64_t off = ((uint64_t)s0 + (uint64_t)round * l.segs[t]) * kSeg;
  if (off >= len) return r;
  r.src = reinterpret_cast<const char*>(p.src_base[t]) + so + off;
  r.dst = reinterpret_cast<char*>(p.dst_base[t]) + dof + off;
  r.len = (uint32_t)min((uint64_t)kSeg, len - off);
  return r;
}

__device__ __forceinline__ bool bulk_ok(const Unit& u) {
  return u.len != 0 && ((reinterpret_cast<uintptr_t>(u.src) | reinterpret_cast<uintptr_t>(u.dst) | u.len) & 15u) == 0;
}

__device__ __forceinline__ void simt_span(const char* __restrict__ s, char* __restrict__ d, uint32_t len, uint32_t lane) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d);
  if ((a & 15u) == 0) {
    const uint32_t n16 = len >> 4;
    const int4* s4 = reinterpret_cast<const int4*>(s);
    int4* d4 = reinterpret_cast<int4*>(d);
    for (uint32_t i = lane; i < n16; i += 32) d4[i] = s4[i];
    for (uint32_t b = (n16 << 4) + lane; b < len; b += 32) d[b] = s[b];
  } else if ((a & 3u) == 0) {
    const uint32_t n4 = len >> 2;
    const int* s1 = reinterpret_cast<const int*>(s);
    int* d1 = reinterpret_cast<int*>(d);
    for (uint32_t i = lane; i < n4; i += 32) d1[i] = s1[i];
    for (uint32_t b = (n4 << 2) + lane; b < len; b += 32) d[b] = s[b];
  } else {
    for (uint32_t b = lane; b < len; b += 32) d[b] = s[b];
  }
}

__global__ void __launch_bounds__(128) kvt_copy_blocks_bulk_kernel(const __grid_constant__ KvtCopyMulti p,
                                                                   const uint32_t n_stages, const uint32_t max_rounds) {
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)n_stages * kSeg);
  const Layout lay = make_layout(p);
  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < n_stages; ++s) mbar_init(smem_u32(&bars[s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  __syncthreads();
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  if (warp == 0) {
    // ---- bulk pass: lanes decode 32 units at a time, lane 0 runs the pipeline --------------------
    char* sdst[kMaxStagesB] = {};
    uint32_t slen[kMaxStagesB] = {};
    uint32_t issued = 0, stored = 0;
    bool failed = false;
    auto consume_one = [&]() {
      const uint32_t s = stored % n_stages;
      const uint32_t bar = smem_u32(&bars[s]);
      const uint32_t parity = (stored / n_stages) & 1u;
      const long long t0 = clock64();
      while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > kWaitCyclesB) {
          failed = true;
          break;
        }
      }
      if (failed) {
        set_status(p.status, KVT_ERR_TMA_TIMEOUT, stored);
        return;
      }
      bulk_store(sdst[s], smem_u32(smem + (size_t)s * kSeg), slen[s]);
      bulk_commit();
      ++stored;
    };
    for (uint32_t round = 0; round < max_rounds; ++round) {
      for (uint64_t batch = 0;; batch += 32) {
        const uint64_t u = blockIdx.x + (batch + lane) * (uint64_t)gridDim.x;
        Unit un;
        un.len = 0;
        un.src = nullptr;
        un.dst = nullptr;
        if (u < lay.total) un = decode(p, lay, u, round);
        const unsigned any = __ballot_sync(0xffffffffu, u < lay.total);
        unsigned mask = __ballot_sync(0xffffffffu, u < lay.total && bulk_ok(un));
        if (any == 0u) break;
        while (mask != 0u) {
          const int j = __ffs(mask) - 1;
          mask &= mask - 1u;
          const uint64_t j_src = __shfl_sync(0xffffffffu, reinterpret_cast<uint64_t>(un.src), j);
          const uint64_t j_dst = __shfl_sync(0xffffffffu, reinterpret_cast<uint64_t>(un.dst), j);
          const uint32_t j_len = __shfl_sync(0xffffffffu, un.len, j);
          if (lane == 0 && !failed) {
            if (n_stages == 1) {
              if (issued > stored) consume_one();
              if (!failed) bulk_wait_read<0>();
            } else if (issued - stored == n_stages - 1) {
              consume_one();
              // the stage refilled below was last read by the store issued one step earlier
              if (!failed) bulk_wait_read<1>();
            }
            if (!failed) {
              const uint32_t s = issued % n_stages;
              const uint32_t bar = smem_u32(&bars[s]);
              mbar_expect_tx(bar, j_len);
              bulk_load(smem_u32(smem + (size_t)s * kSeg), reinterpret_cast<const void*>(j_src), j_len, bar);
              sdst[s] = reinterpret_cast<char*>(j_dst);
              slen[s] = j_len;
              ++issued;
            }
          }
        }
      }
    }
    if (lane == 0) {
      while (!failed && stored < issued) consume_one();
      bulk_wait_all();
      fence_proxy_async();
    }
    __syncwarp();
  } else {
    // ---- SIMT pass: what the bulk engine cannot take, and the range reports ----------------------
    const uint32_t w = warp - 1, nw = (blockDim.x >> 5) - 1;
    for (uint32_t round = 0; round < max_rounds; ++round) {
      for (uint64_t k = w;; k += nw) {
        const uint64_t u = blockIdx.x + k * (uint64_t)gridDim.x;
        if (u >= lay.total) break;
        const Unit un = decode(p, lay, u, round);
        if (un.bad && lane == 0) set_status(p.status, KVT_ERR_BLOCK_RANGE, un.desc);
        if (un.len != 0 && !bulk_ok(un)) simt_span(un.src, un.dst, un.len, lane);
      }
    }
  }
}

}  // namespace

extern "C" uint32_t kvt_bulk_rounds(uint64_t first_len, uint64_t max_len) {
  // rounds x segs_of(first_len) x 8 KiB covers the longest descriptor
  const uint64_t segs0 = segs_of(first_len);
  const uint64_t segs_max = max_len > kSeg ? (max_len + kSeg - 1) / kSeg : 1;
  return (uint32_t)((segs_max + segs0 - 1) / segs0);
}

extern "C" int kvt_launch_copy_blocks_bulk(const KvtCopyMulti* args, uint32_t rounds, int grid_ctas, void* stream) {
  if (args->n_tensors == 0 || args->n_tensors > KVT_COPY_MAX_TENSORS || rounds == 0) return (int)cudaErrorInvalidValue;
  uint64_t n = 0;
  for (uint32_t t = 0; t < args->n_tensors; ++t) n += args->count[t];
  if (n == 0) return (int)cudaSuccess;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 1;
  // four CTAs per SM, each with four 8 KiB segments in flight: 128 KiB per SM on the way
  const int grid = grid_ctas > 0 ? grid_ctas : 4 * sms;
  const uint32_t stages = 4;
  const size_t smem = (size_t)stages * kSeg + kMaxStagesB * sizeof(uint64_t);
  kvt_copy_blocks_bulk_kernel<<<grid, 128, smem, reinterpret_cast<cudaStream_t>(stream)>>>(*args, stages, rounds);
  return (int)cudaGetLastError();
}
