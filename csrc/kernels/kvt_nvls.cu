// kvt_mc_fanout: replicate paged-cache blocks of THIS GPU into the same blocks of every GPU bound
// to an NVLink multicast object, with one store per 16 bytes (`multimem.st` through NVSwitch).
//
// Use: data that every tensor-parallel rank of a decode instance holds identically (the MLA
// latent and indexer caches, replicated KV heads when there are fewer KV heads than ranks).  The
// reference sends such data once per destination rank (one P rank fans out to d/p D ranks,
// blade_kvt/hybrid_connector/kvtbackend.py:637-664, kvtransfer/src/tx_stub.cpp:18-114), so the
// sender's link carries d/p copies.  Here the sender pushes ONE copy to one rank of the group and
// that rank's GPU replicates it: its NVLink egress carries the bytes once and the switch delivers
// them to every member (the issuing GPU included: same bytes to the same place).
//
// Only stores are multicast.  Sources are read with plain loads from local memory (the member's
// own cache, or a landing buffer the sender pushed into); nothing here loads through a multicast
// address.  Every rank of the group uses the same destination block ids for the request, which is
// how a TP group allocates anyway (one scheduler, one block table).
#include <cuda_runtime.h>
#include <stdint.h>

#include "kvt_kernels.h"
#include "kvt_walk.h"

namespace {

__device__ __forceinline__ void set_status(uint32_t* status, uint32_t code, uint32_t detail) {
  if (status != nullptr) {
    if (atomicCAS(status, 0u, code) == 0u) status[1] = detail;
  }
}

__device__ __forceinline__ int4 ld_nc_16(const void* p) {
  int4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void mc_st_16(void* mc, int4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(__int_as_float(v.x)),
               "f"(__int_as_float(v.y)), "f"(__int_as_float(v.z)), "f"(__int_as_float(v.w))
               : "memory");
}

constexpr uint32_t kSegBytes = 2048;   // a warp moves 32 lanes x 4 x 16 B per step

__global__ void __launch_bounds__(512) kvt_mc_fanout_kernel(const __grid_constant__ KvtMcFanout p) {
  const uint32_t n_layers = p.layer_end - p.layer_begin;
  const uint32_t segs = (p.block_len + kSegBytes - 1) / kSegBytes;
  const uint64_t per_layer = (uint64_t)p.n_blocks * segs;
  const uint64_t total = (uint64_t)n_layers * per_layer;
  const uint32_t warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  for (uint64_t w = (uint64_t)blockIdx.x * warps + warp; w < total; w += (uint64_t)gridDim.x * warps) {
    const uint32_t layer = (uint32_t)(w / per_layer);
    const uint64_t rem = w - (uint64_t)layer * per_layer;
    const uint32_t bi = (uint32_t)(rem / segs);
    const uint32_t seg = (uint32_t)(rem - (uint64_t)bi * segs);
    const uint32_t sb = p.src_blocks[bi], db = p.dst_blocks[bi];
    if (sb >= p.src_num_blocks || db >= p.dst_num_blocks) {
      if (lane == 0) set_status(p.status, KVT_ERR_BLOCK_RANGE, bi);
      continue;
    }
    const int64_t in_block = (int64_t)p.block_off + (int64_t)seg * kSegBytes;
    const char* src = reinterpret_cast<const char*>(p.src_layers[p.layer_begin + layer]) +
                      (int64_t)sb * p.src_block_stride + in_block;
    char* mc = reinterpret_cast<char*>(p.mc_layers[p.layer_begin + layer]) + (int64_t)db * p.dst_block_stride + in_block;
    const uint32_t len = min(kSegBytes, p.block_len - seg * kSegBytes);   // multiple of 16 (checked by the launcher)
    const uint32_t n16 = len >> 4;
    int4 v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t i = lane + 32u * k;
      if (i < n16) v[k] = ld_nc_16(src + ((size_t)i << 4));
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t i = lane + 32u * k;
      if (i < n16) mc_st_16(mc + ((size_t)i << 4), v[k]);
    }
  }
  // Completion word, multicast as well: a member that sees it (acquire at system scope) sees the
  // blocks.  The last CTA to finish publishes it after every CTA's stores have been fenced.
  if (p.mc_flag != nullptr && p.done_counter != nullptr) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t prev = atomicAdd(p.done_counter, 1u);
      if (prev == gridDim.x - 1) {
        *p.done_counter = 0;
        __threadfence_system();
        asm volatile("multimem.st.release.sys.global.u64 [%0], %1;" ::"l"(p.mc_flag), "l"(p.flag_value) : "memory");
      }
    }
  }
}

// ---- fan-out of what a walk plan wrote ----------------------------------------------------------------
// The member that received a request through walk ops (kvt_walk.cu) replicates exactly the bytes the ops
// wrote: every unit of every op is decoded with the shared kvt_walk_unit, and its DESTINATION pieces are
// read from this GPU's cache and stored to the same offsets of the multicast mapping.  Nothing but the
// transferred bytes is touched, so members may relay different requests, or different chunks of one
// request, without overwriting one another.
__device__ __forceinline__ void mc_st_16_weak(void* mc, int4 v) {
  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(__int_as_float(v.x)),
               "f"(__int_as_float(v.y)), "f"(__int_as_float(v.z)), "f"(__int_as_float(v.w))
               : "memory");
}

__device__ __forceinline__ void mc_st_4(void* mc, int v) {
  asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t find_walk_op(const KvtWalkOp* __restrict__ ops, uint32_t n, uint64_t u) {
  uint32_t lo = 0, hi = n;
  while (hi - lo > 1) {
    const uint32_t mid = (lo + hi) >> 1;
    if (ops[mid].first_unit <= u) lo = mid; else hi = mid;
  }
  return lo;
}

// One class of ops (bulk, simt or zero: first_unit counts within the class), `units` units per layer.
// FROM_SRC = false: the member that received the request stores what the ops WROTE (its own destination pieces).
// FROM_SRC = true: a sender whose GPU is bound to the group's multicast object stores the ops' SOURCE pieces
// straight to the group (and zeros for the zero-fill class): no member has to receive the request first.
template <bool FROM_SRC>
__global__ void __launch_bounds__(256) kvt_walk_fanout_kernel(const __grid_constant__ KvtWalkLaunch p,
                                                               const KvtWalkOp* __restrict__ ops, const uint32_t n_ops,
                                                               const uint64_t units, const uint64_t* __restrict__ mc_ptrs) {
  const bool weak = (p.shape & 0x80000000u) != 0;      // weak multicast stores (ordered by the fence at the end of the grid)
  const uint32_t n_layers = p.layer_end - p.layer_begin;
  const uint64_t total = units * n_layers;
  const uint32_t warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  for (uint64_t w = (uint64_t)blockIdx.x * warps + warp; w < total; w += (uint64_t)gridDim.x * warps) {
    const uint32_t layer = p.layer_begin + (uint32_t)(w / units);
    const uint64_t u = w % units;
    const uint32_t oi = find_walk_op(ops, n_ops, u);
    const KvtWalkOp& op = ops[oi];
    const KvtWalkPieces pc = kvt_walk_unit(op, p.pool, u - op.first_unit);
    if (pc.error != 0) {
      if (lane == 0) set_status(p.status, KVT_ERR_BLOCK_RANGE, oi);
      continue;
    }
    if (pc.n == 0) continue;
    const uint32_t t = op.tensor;
    const bool zero = FROM_SRC && (op.flags & KVT_WALK_ZERO) != 0;
    const int64_t d_last = pc.dst_off + (int64_t)(pc.n - 1) * pc.dst_step;
    bool bad = t >= p.n_tensors || pc.dst_off < 0 || d_last < 0 || (uint64_t)pc.dst_off + pc.len > p.dst_cap[t] ||
               (uint64_t)d_last + pc.len > p.dst_cap[t];
    if (FROM_SRC && !zero && !bad) {
      const int64_t s_last = pc.src_off + (int64_t)(pc.n - 1) * pc.src_step;
      bad = pc.src_off < 0 || s_last < 0 || (uint64_t)pc.src_off + pc.len > p.src_cap[t] || (uint64_t)s_last + pc.len > p.src_cap[t];
    }
    if (bad) {
      if (lane == 0) set_status(p.status, KVT_ERR_BLOCK_RANGE, oi);
      continue;
    }
    const uint64_t idx = (uint64_t)layer * p.n_tensors + t;
    // where the bytes are read: this GPU's copy of the destination pieces, or the source pieces
    const char* own = FROM_SRC ? (zero ? nullptr : reinterpret_cast<const char*>(p.src_ptrs[idx]) + pc.src_off)
                               : reinterpret_cast<const char*>(p.dst_ptrs[idx]) + pc.dst_off;
    const int64_t rd_step = FROM_SRC ? (zero ? 0 : pc.src_step) : pc.dst_step;
    char* mc = reinterpret_cast<char*>(mc_ptrs[idx]) + pc.dst_off;
    const uintptr_t a = reinterpret_cast<uintptr_t>(own) | reinterpret_cast<uintptr_t>(mc) | (uintptr_t)pc.dst_step |
                        (uintptr_t)rd_step | pc.len;
    if ((a & 15u) == 0) {
      // four independent 16-byte loads per lane before the first store: a unit is a few KiB, so the loop is
      // short and its latency, not its instruction count, is what a warp spends
      const uint32_t cpp = pc.len >> 4, n16 = cpp * pc.n;
      for (uint32_t i0 = lane; i0 < n16; i0 += 128) {
        int4 v[4];
        int64_t off[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t i = i0 + 32u * k;
          v[k] = make_int4(0, 0, 0, 0);
          off[k] = 0;
          if (i < n16) {
            const uint32_t j = i / cpp, c = i - j * cpp;
            off[k] = (int64_t)j * pc.dst_step + ((int64_t)c << 4);
            if (!zero) v[k] = ld_nc_16(own + (int64_t)j * rd_step + ((int64_t)c << 4));
          }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (i0 + 32u * k < n16) {
            if (weak) mc_st_16_weak(mc + off[k], v[k]); else mc_st_16(mc + off[k], v[k]);
          }
        }
      }
    } else if ((a & 3u) == 0) {
      const uint32_t cpp = pc.len >> 2, n4 = cpp * pc.n;
      for (uint32_t i = lane; i < n4; i += 32) {
        const uint32_t j = i / cpp, c = i - j * cpp;
        const int v = zero ? 0 : *reinterpret_cast<const int*>(own + (int64_t)j * rd_step + ((int64_t)c << 2));
        mc_st_4(mc + (int64_t)j * pc.dst_step + ((int64_t)c << 2), v);
      }
    } else {
      // multicast stores are at least four bytes wide; cache pieces are made of 2- and 4-byte elements in
      // multiples of two, so this is a geometry nobody registers
      if (lane == 0) set_status(p.status, KVT_ERR_BAD_ARGS, oi);
    }
  }
  __threadfence_system();      // the stores of this grid are performed before whatever follows on the stream
}

}  // namespace

namespace {

int launch_walk_fanout(const KvtWalkLaunch* args, uint32_t n_zero_ops, uint64_t zero_units, const uint64_t* mc_ptrs,
                       int grid_ctas, void* stream, bool from_src);

}  // namespace

extern "C" int kvt_launch_walk_fanout(const KvtWalkLaunch* args, uint32_t n_zero_ops, uint64_t zero_units,
                                      const uint64_t* mc_ptrs, int grid_ctas, void* stream) {
  return launch_walk_fanout(args, n_zero_ops, zero_units, mc_ptrs, grid_ctas, stream, false);
}

extern "C" int kvt_launch_walk_multicast(const KvtWalkLaunch* args, uint32_t n_zero_ops, uint64_t zero_units,
                                         const uint64_t* mc_ptrs, int grid_ctas, void* stream) {
  return launch_walk_fanout(args, n_zero_ops, zero_units, mc_ptrs, grid_ctas, stream, true);
}

namespace {

int launch_walk_fanout(const KvtWalkLaunch* args, uint32_t n_zero_ops, uint64_t zero_units, const uint64_t* mc_ptrs,
                       int grid_ctas, void* stream, bool from_src) {
  const KvtWalkLaunch& a = *args;
  if (a.layer_end <= a.layer_begin) return (int)cudaSuccess;
  if (a.n_tensors == 0 || a.n_tensors > KVT_WALK_MAX_TENSORS || a.ops == nullptr || a.pool == nullptr || mc_ptrs == nullptr ||
      (from_src ? a.src_ptrs == nullptr : a.dst_ptrs == nullptr))
    return (int)cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 1;
  const uint64_t n_layers = a.layer_end - a.layer_begin;
  const KvtWalkOp* ops = a.ops;
  const uint32_t counts[3] = {a.n_bulk_ops, a.n_simt_ops, n_zero_ops};
  const uint64_t units[3] = {a.bulk_units, a.simt_units, zero_units};
  for (int c = 0; c < 3; ++c) {
    if (counts[c] != 0 && units[c] != 0) {
      const uint64_t need = (units[c] * n_layers + 7) / 8;       // eight warps per CTA
      int grid = grid_ctas > 0 ? grid_ctas : 4 * sms;
      if ((uint64_t)grid > need) grid = (int)need;
      if (from_src)
        kvt_walk_fanout_kernel<true><<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a, ops, counts[c], units[c], mc_ptrs);
      else
        kvt_walk_fanout_kernel<false><<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a, ops, counts[c], units[c], mc_ptrs);
      const cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return (int)e;
    }
    ops += counts[c];
  }
  return (int)cudaSuccess;
}

}  // namespace

extern "C" int kvt_launch_mc_fanout(const KvtMcFanout* args, int grid_ctas, void* stream) {
  const KvtMcFanout& a = *args;
  if (a.n_blocks == 0 || a.layer_end <= a.layer_begin || a.block_len == 0) return (int)cudaSuccess;
  if (a.src_layers == nullptr || a.mc_layers == nullptr || a.src_blocks == nullptr || a.dst_blocks == nullptr)
    return (int)cudaErrorInvalidValue;
  // multimem.st.v4.f32 needs 16-byte aligned addresses: the ranges must be made of whole 16-byte words
  if ((a.block_len & 15u) != 0 || (a.block_off & 15u) != 0 || (a.src_block_stride & 15) != 0 ||
      (a.dst_block_stride & 15) != 0 || a.src_block_stride <= 0 || a.dst_block_stride <= 0)
    return (int)cudaErrorInvalidValue;
  if ((uint64_t)a.block_off + a.block_len > (uint64_t)a.src_block_stride ||
      (uint64_t)a.block_off + a.block_len > (uint64_t)a.dst_block_stride)
    return (int)cudaErrorInvalidValue;
  if (a.mc_flag != nullptr && ((reinterpret_cast<uintptr_t>(a.mc_flag) & 7u) != 0 || a.done_counter == nullptr))
    return (int)cudaErrorInvalidValue;
  int grid = grid_ctas;
  if (grid <= 0) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    grid = 2 * (sms > 0 ? sms : 1);
  }
  const uint64_t segs = (a.block_len + kSegBytes - 1) / kSegBytes;
  const uint64_t units = (uint64_t)(a.layer_end - a.layer_begin) * a.n_blocks * segs;
  const uint64_t need = (units + 15) / 16;
  if ((uint64_t)grid > need) grid = (int)need;
  kvt_mc_fanout_kernel<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return (int)cudaGetLastError();
}
