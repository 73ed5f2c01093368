// kvt_walk: the block-table walk for the hybrid, MLA and state-page cache shapes.
//
// The reference expands every request of these shapes on the CPU into one {src, dst, len} triple per
// piece (GDN conv rows split by channel group, per-token head slices, kernel-block pages, KDA pages:
// kvtransfer/src/parse_block_qwen3_next.cpp:108-711, parse_block_dpsk.cpp:16-214, parse_block_kda.cpp:8-330,
// parse_block_kimi_k3.cpp:9-235), uploads the array and runs a copy kernel over it
// (kvtransfer/src/copy_kernels.cpp:363-439).  Here the host writes a handful of affine rules per request
// ("walk ops", kvt_kernels.h) and this kernel expands them while it copies: it reads the block tables,
// computes both offsets of every piece and moves it into the destination cache, which may be local
// memory, a peer GPU's memory mapped over NVLink, or mapped host memory.
//
// A CTA has two roles, as in kvt_bulk_copy.cu.  Warp 0 drives the TMA engine for the ops whose pieces are
// long and 16-byte aligned (whole pages, SSM state, kernel-block pages): its lanes decode 32 units at a
// time and lane 0 keeps several untiled bulk copies (global -> shared on an mbarrier, shared -> global in
// a bulk group) in flight.  The other warps take the remaining ops, a warp per unit, with the widest
// vector both addresses allow, and write the zero pieces of tail padding.  No load here uses cluster
// multicast.  Every wait is bounded; a bad table index, a piece beyond its tensor or a wait that ran out
// sets the status words and the piece is skipped.
#include <cuda_runtime.h>
#include <stdint.h>

#include "kvt_kernels.h"
#include "kvt_walk.h"

namespace {

constexpr int kMaxStagesW = 8;
constexpr long long kWaitCyclesW = 4000000000LL;  // ~2 s at 2 GHz

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

// Largest i with ops[i].first_unit <= u, over ops[0, n).
__device__ __forceinline__ uint32_t find_op(const KvtWalkOp* __restrict__ ops, uint32_t n, uint64_t u) {
  uint32_t lo = 0, hi = n;
  while (hi - lo > 1) {
    const uint32_t mid = (lo + hi) >> 1;
    if (ops[mid].first_unit <= u) lo = mid; else hi = mid;
  }
  return lo;
}

struct Resolved {
  const char* src;
  char* dst;
  int64_t src_step, dst_step;
  uint32_t len, n;
  bool zero;
};

// Unit `u` of class [ops, ops + n_ops) in layer `layer`: decoded, bounds-checked, as addresses.
__device__ __forceinline__ Resolved resolve(const KvtWalkLaunch& p, const KvtWalkOp* __restrict__ ops, uint32_t n_ops,
                                            uint64_t u, uint32_t layer, bool report) {
  Resolved r;
  r.src = nullptr;
  r.dst = nullptr;
  r.src_step = r.dst_step = 0;
  r.len = r.n = 0;
  r.zero = false;
  const uint32_t oi = find_op(ops, n_ops, u);
  const KvtWalkOp& op = ops[oi];
  const KvtWalkPieces pc = kvt_walk_unit(op, p.pool, u - op.first_unit);
  if (pc.error != 0) {
    if (report) set_status(p.status, KVT_ERR_BLOCK_RANGE, oi);
    return r;
  }
  if (pc.n == 0) return r;
  const uint32_t t = op.tensor;
  r.zero = (op.flags & KVT_WALK_ZERO) != 0;
  // the whole span of the unit's pieces must lie inside both tensors
  const int64_t s_last = pc.src_off + (int64_t)(pc.n - 1) * pc.src_step, d_last = pc.dst_off + (int64_t)(pc.n - 1) * pc.dst_step;
  const bool bad = t >= p.n_tensors || pc.dst_off < 0 || d_last < 0 || (uint64_t)pc.dst_off + pc.len > p.dst_cap[t] ||
                   (uint64_t)d_last + pc.len > p.dst_cap[t] ||
                   (!r.zero && (pc.src_off < 0 || s_last < 0 || (uint64_t)pc.src_off + pc.len > p.src_cap[t] ||
                                (uint64_t)s_last + pc.len > p.src_cap[t]));
  if (bad) {
    if (report) set_status(p.status, KVT_ERR_BLOCK_RANGE, oi);
    return r;
  }
  const uint64_t idx = (uint64_t)layer * p.n_tensors + t;
  r.src = r.zero ? nullptr : reinterpret_cast<const char*>(p.src_ptrs[idx]) + pc.src_off;
  r.dst = reinterpret_cast<char*>(p.dst_ptrs[idx]) + pc.dst_off;
  r.src_step = pc.src_step;
  r.dst_step = pc.dst_step;
  r.len = pc.len;
  r.n = pc.n;
  return r;
}

// Work item w = layer * units_per_layer + unit, with 32-bit divisions where the numbers allow.
__device__ __forceinline__ void split_unit(uint64_t w, uint64_t per_layer, uint64_t* unit, uint32_t* layer) {
  if (((w | per_layer) >> 32) == 0) {
    const uint32_t q = (uint32_t)w / (uint32_t)per_layer;
    *layer = q;
    *unit = (uint32_t)w - q * (uint32_t)per_layer;
  } else {
    *layer = (uint32_t)(w / per_layer);
    *unit = w % per_layer;
  }
}

__device__ __forceinline__ bool bulk_ok(const Resolved& r) {
  return r.n == 1 && !r.zero && r.len != 0 &&
         ((reinterpret_cast<uintptr_t>(r.src) | reinterpret_cast<uintptr_t>(r.dst) | r.len) & 15u) == 0;
}

// One warp copies (or zero-fills) the n pieces of a unit.
__device__ __forceinline__ void warp_pieces(const Resolved& r, uint32_t lane) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(r.src) | reinterpret_cast<uintptr_t>(r.dst) | (uintptr_t)r.src_step |
                      (uintptr_t)r.dst_step | r.len;
  if ((a & 15u) == 0) {
    const uint32_t cpp = r.len >> 4;                 // 16-byte chunks per piece
    const uint32_t total = cpp * r.n;
    for (uint32_t i = lane; i < total; i += 32) {
      const uint32_t j = i / cpp, c = i - j * cpp;
      int4 v = make_int4(0, 0, 0, 0);
      if (!r.zero) v = *reinterpret_cast<const int4*>(r.src + (int64_t)j * r.src_step + ((int64_t)c << 4));
      *reinterpret_cast<int4*>(r.dst + (int64_t)j * r.dst_step + ((int64_t)c << 4)) = v;
    }
  } else if ((a & 3u) == 0) {
    const uint32_t cpp = r.len >> 2;
    const uint32_t total = cpp * r.n;
    for (uint32_t i = lane; i < total; i += 32) {
      const uint32_t j = i / cpp, c = i - j * cpp;
      int v = 0;
      if (!r.zero) v = *reinterpret_cast<const int*>(r.src + (int64_t)j * r.src_step + ((int64_t)c << 2));
      *reinterpret_cast<int*>(r.dst + (int64_t)j * r.dst_step + ((int64_t)c << 2)) = v;
    }
  } else {
    const uint64_t total = (uint64_t)r.len * r.n;
    for (uint64_t i = lane; i < total; i += 32) {
      const uint32_t j = (uint32_t)(i / r.len), c = (uint32_t)(i - (uint64_t)j * r.len);
      r.dst[(int64_t)j * r.dst_step + c] = r.zero ? (char)0 : r.src[(int64_t)j * r.src_step + c];
    }
  }
}

__global__ void __launch_bounds__(256) kvt_walk_kernel(const __grid_constant__ KvtWalkLaunch p, const uint32_t n_stages) {
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)n_stages * KVT_WALK_SEG);
  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < n_stages; ++s) mbar_init(smem_u32(&bars[s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
  }
  __syncthreads();
  const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
  const uint32_t n_layers = p.layer_end - p.layer_begin;
  const KvtWalkOp* bulk_ops = p.ops;
  const KvtWalkOp* simt_ops = p.ops + p.n_bulk_ops;
  const uint64_t bulk_total = p.bulk_units * n_layers, simt_total = p.simt_units * n_layers;
  if (warp == 0) {
    // ---- bulk pass: lanes decode 32 units at a time, lane 0 runs the pipeline -----------------------
    char* sdst[kMaxStagesW] = {};
    uint32_t slen[kMaxStagesW] = {};
    uint32_t issued = 0, stored = 0;
    bool failed = false;
    auto consume_one = [&]() {
      const uint32_t s = stored % n_stages;
      const uint32_t bar = smem_u32(&bars[s]);
      const uint32_t parity = (stored / n_stages) & 1u;
      const long long t0 = clock64();
      while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > kWaitCyclesW) {
          failed = true;
          break;
        }
      }
      if (failed) {
        set_status(p.status, KVT_ERR_TMA_TIMEOUT, stored);
        return;
      }
      bulk_store(sdst[s], smem_u32(smem + (size_t)s * KVT_WALK_SEG), slen[s]);
      bulk_commit();
      ++stored;
    };
    for (uint64_t batch = 0;; batch += 32) {
      const uint64_t w = blockIdx.x + (batch + lane) * (uint64_t)gridDim.x;
      Resolved r;
      r.n = 0;
      r.len = 0;
      r.src = nullptr;
      r.dst = nullptr;
      r.zero = false;
      if (w < bulk_total) {
        uint64_t unit;
        uint32_t layer;
        split_unit(w, p.bulk_units, &unit, &layer);
        r = resolve(p, bulk_ops, p.n_bulk_ops, unit, p.layer_begin + layer, true);
      }
      const unsigned any = __ballot_sync(0xffffffffu, w < bulk_total);
      unsigned mask = __ballot_sync(0xffffffffu, w < bulk_total && bulk_ok(r));
      if (any == 0u) break;
      while (mask != 0u) {
        const int j = __ffs(mask) - 1;
        mask &= mask - 1u;
        const uint64_t j_src = __shfl_sync(0xffffffffu, reinterpret_cast<uint64_t>(r.src), j);
        const uint64_t j_dst = __shfl_sync(0xffffffffu, reinterpret_cast<uint64_t>(r.dst), j);
        const uint32_t j_len = __shfl_sync(0xffffffffu, r.len, j);
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
            bulk_load(smem_u32(smem + (size_t)s * KVT_WALK_SEG), reinterpret_cast<const void*>(j_src), j_len, bar);
            sdst[s] = reinterpret_cast<char*>(j_dst);
            slen[s] = j_len;
            ++issued;
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
    // ---- SIMT pass: the ops with short or strided pieces, zero fills, and whatever a bulk unit's
    //      addresses do not allow the TMA engine to take -------------------------------------------
    const uint32_t w0 = warp - 1, nw = (blockDim.x >> 5) - 1;
    for (uint64_t k = w0;; k += nw) {
      const uint64_t w = blockIdx.x + k * (uint64_t)gridDim.x;
      if (w >= simt_total) break;
      uint64_t unit;
      uint32_t layer;
      split_unit(w, p.simt_units, &unit, &layer);
      const Resolved r = resolve(p, simt_ops, p.n_simt_ops, unit, p.layer_begin + layer, lane == 0);
      if (r.n != 0) warp_pieces(r, lane);
    }
    for (uint64_t k = w0;; k += nw) {
      const uint64_t w = blockIdx.x + k * (uint64_t)gridDim.x;
      if (w >= bulk_total) break;
      uint64_t unit;
      uint32_t layer;
      split_unit(w, p.bulk_units, &unit, &layer);
      const Resolved r = resolve(p, bulk_ops, p.n_bulk_ops, unit, p.layer_begin + layer, false);
      if (r.n != 0 && !bulk_ok(r)) warp_pieces(r, lane);
    }
  }
}

}  // namespace

extern "C" int kvt_launch_walk(const KvtWalkLaunch* args, int grid_ctas, void* stream) {
  const KvtWalkLaunch& a = *args;
  if (a.layer_end <= a.layer_begin || (a.n_bulk_ops + a.n_simt_ops) == 0) return (int)cudaSuccess;
  if (a.n_tensors == 0 || a.n_tensors > KVT_WALK_MAX_TENSORS || a.ops == nullptr || a.pool == nullptr)
    return (int)cudaErrorInvalidValue;
  if ((a.n_bulk_ops != 0) != (a.bulk_units != 0) || (a.n_simt_ops != 0) != (a.simt_units != 0)) return (int)cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 1;
  // four CTAs per SM, each with two 8 KiB segments in flight through the TMA engine and seven SIMT warps.  Two
  // stages, not four: 16 KiB of shared memory per CTA lets the CTAs of the next layer's launch start beside
  // those of the running one (measured on the MLA step: 2495-2538 against 2225-2283 GB/s; three stages 2346,
  // one 1905; the hybrid GDN step is the same within its run-to-run spread)
  int grid = grid_ctas > 0 ? grid_ctas : 4 * sms;
  const uint64_t n_layers = a.layer_end - a.layer_begin;
  uint32_t threads = a.shape & 0xffffu, stages = a.shape >> 16;
  if (threads == 0) threads = 256;
  if (stages == 0) stages = 2;
  if (threads < 64 || threads > 256 || (threads & 31u) != 0 || stages > kMaxStagesW) return (int)cudaErrorInvalidValue;
  const uint64_t simt_warps = threads / 32 - 1;
  const uint64_t most = (a.bulk_units > a.simt_units / simt_warps ? a.bulk_units : (a.simt_units + simt_warps - 1) / simt_warps) * n_layers;
  if ((uint64_t)grid > most && most > 0) grid = (int)most;
  const size_t smem = (size_t)stages * KVT_WALK_SEG + kMaxStagesW * sizeof(uint64_t);
  kvt_walk_kernel<<<grid, threads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(a, stages);
  return (int)cudaGetLastError();
}
