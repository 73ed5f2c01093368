#include "transport/verify.h"

#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <stdexcept>

#include "core/envcfg.h"
#include "core/fault_inject.h"
#include "core/util.h"
#include "kernels/kvt_kernels.h"
#include "transport/channel.h"
#include "transport/wire.h"

namespace kvx {

namespace {

inline uint64_t rotl64(uint64_t v, unsigned r) {
  r &= 63u;
  return r == 0 ? v : (v << r) | (v >> (64u - r));
}

inline uint64_t fold(uint64_t sum, uint32_t layer, uint32_t tensor) { return rotl64(sum, layer * 7u + tensor * 3u); }

void cu(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    cudaGetLastError();
    throw std::runtime_error(std::string("transfer check: ") + what + ": " + cudaGetErrorString(e));
  }
}

// Scratch of the device path, one per GPU, grown on demand and kept: the check is a diagnostic mode, so a
// growth step may allocate (and the free of the outgrown buffer may synchronise the device).
struct DeviceScratch {
  cudaStream_t stream{nullptr};
  KvtCheckChunk* chunks{nullptr};
  size_t chunk_cap{0};
  uint64_t* sums{nullptr};     // [sum_cap] sums, then 2 status words
  size_t sum_cap{0};
};

std::mutex g_mu;
std::map<int, DeviceScratch> g_scratch;

uint64_t checksum_device(Context* ctx, uint32_t lb, uint32_t le, const std::vector<std::vector<CheckRange>>& per_tensor) {
  const int dev = ctx->device_id();
  const auto& addrs = ctx->layer_data_address();
  const size_t n_tensors = per_tensor.size();
  // pieces cut to chunks; index0 restarts at every piece
  std::vector<KvtCheckChunk> host;
  std::vector<size_t> first(n_tensors + 1, 0);
  for (size_t t = 0; t < n_tensors; ++t) {
    for (const CheckRange& r : per_tensor[t]) {
      for (uint64_t done = 0; done < r.len; done += KVT_CHECK_CHUNK) {
        const uint64_t n = std::min<uint64_t>(KVT_CHECK_CHUNK, r.len - done);
        host.push_back(KvtCheckChunk{r.off + done, static_cast<uint32_t>(n), static_cast<uint32_t>(done)});
      }
    }
    first[t + 1] = host.size();
  }
  if (host.empty()) return 0;
  std::lock_guard<std::mutex> g(g_mu);
  cu(cudaSetDevice(dev), "cudaSetDevice");   // the calling threads are the transport's own: nothing to restore
  DeviceScratch& s = g_scratch[dev];
  uint64_t total = 0;
  {
    if (s.stream == nullptr) cu(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking), "stream");
    if (s.chunk_cap < host.size()) {
      if (s.chunks != nullptr) cudaFree(s.chunks);
      s.chunks = nullptr;
      s.chunk_cap = 0;
      const size_t want = std::max<size_t>(host.size() * 2, 4096);
      cu(cudaMalloc(reinterpret_cast<void**>(&s.chunks), want * sizeof(KvtCheckChunk)), "cudaMalloc");
      s.chunk_cap = want;
    }
    const size_t n_sums = static_cast<size_t>(le - lb) * n_tensors;
    if (s.sum_cap < n_sums) {
      if (s.sums != nullptr) cudaFree(s.sums);
      s.sums = nullptr;
      s.sum_cap = 0;
      const size_t want = std::max<size_t>(n_sums * 2, 256);
      cu(cudaMalloc(reinterpret_cast<void**>(&s.sums), (want + 1) * sizeof(uint64_t)), "cudaMalloc");
      s.sum_cap = want;
    }
    uint32_t* status = reinterpret_cast<uint32_t*>(s.sums + s.sum_cap);
    cu(cudaMemcpyAsync(s.chunks, host.data(), host.size() * sizeof(KvtCheckChunk), cudaMemcpyHostToDevice, s.stream), "upload");
    cu(cudaMemsetAsync(s.sums, 0, (s.sum_cap + 1) * sizeof(uint64_t), s.stream), "memset");
    const int sms = kvt_sm_count(dev);
    for (uint32_t l = lb; l < le; ++l) {
      for (size_t t = 0; t < n_tensors; ++t) {
        const size_t n = first[t + 1] - first[t];
        if (n == 0) continue;
        const int rc = kvt_launch_checksum(addrs[l][t], ctx->tensor_capacity(t), s.chunks + first[t], static_cast<uint32_t>(n),
                                           s.sums + (l - lb) * n_tensors + t, status, sms > 0 ? sms * 4 : 0, s.stream);
        if (rc != 0) cu(static_cast<cudaError_t>(rc), "launch");
      }
    }
    std::vector<uint64_t> out(n_sums + 1, 0);
    cu(cudaMemcpyAsync(out.data(), s.sums, n_sums * sizeof(uint64_t), cudaMemcpyDeviceToHost, s.stream), "download");
    cu(cudaMemcpyAsync(&out[n_sums], status, sizeof(uint64_t), cudaMemcpyDeviceToHost, s.stream), "download");
    cu(cudaStreamSynchronize(s.stream), "synchronize");
    if ((out[n_sums] & 0xFFFFFFFFu) != 0) throw std::out_of_range("transfer check: the kernel skipped a range outside its tensor");
    for (uint32_t l = lb; l < le; ++l)
      for (size_t t = 0; t < n_tensors; ++t) total += fold(out[(l - lb) * n_tensors + t], l, static_cast<uint32_t>(t));
  }
  return total;
}

}  // namespace

uint64_t checksum_cache(Context* ctx, uint32_t lb, uint32_t le, const std::vector<std::vector<CheckRange>>& per_tensor) {
  const auto& addrs = ctx->layer_data_address();
  if (lb > le || le > addrs.size()) throw std::out_of_range("transfer check: layer range outside the cache");
  for (uint32_t l = lb; l < le; ++l)
    if (addrs[l].size() != per_tensor.size()) throw std::out_of_range("transfer check: tensor count differs from the cache's");
  for (size_t t = 0; t < per_tensor.size(); ++t) {
    const uint64_t cap = ctx->tensor_capacity(t);
    for (const CheckRange& r : per_tensor[t])
      if (r.off > cap || r.len > cap - r.off) throw std::out_of_range("transfer check: range outside its tensor");
  }
  if (ctx->device_id() >= 0) return checksum_device(ctx, lb, le, per_tensor);
  uint64_t total = 0;
  for (uint32_t l = lb; l < le; ++l) {
    for (size_t t = 0; t < per_tensor.size(); ++t) {
      const char* base = reinterpret_cast<const char*>(addrs[l][t]);
      uint64_t sum = 0;
      for (const CheckRange& r : per_tensor[t]) sum += kvt_checksum_host(base + r.off, r.len, 0);
      total += fold(sum, l, static_cast<uint32_t>(t));
    }
  }
  return total;
}

// CHECK_REQ body: [layer_begin u32][layer_end u32][n_tensors u32][0 u32] { [n u64] { [off u64][len u64] } x n } x n_tensors
// response:      [RPC header][status u32][sum u64][elapsed_us i64]
CheckOutcome verify_transfer(Context* ctx, const WorkerInfo& dst, uint32_t lb, uint32_t le,
                             const std::vector<std::vector<IpcBlock>>& blocks) {
  CheckOutcome o;
  std::vector<std::vector<CheckRange>> src(blocks.size());
  std::string req(RPC_HEADER, '\0');
  const uint64_t reqid = new_id();
  put_rpc_header(req.data(), CHECK_REQ, reqid);
  put(req, lb);
  put(req, le);
  put(req, static_cast<uint32_t>(blocks.size()));
  put(req, static_cast<uint32_t>(0));
  for (size_t t = 0; t < blocks.size(); ++t) {
    uint64_t n = 0;
    for (const IpcBlock& b : blocks[t]) n += b.length != 0;
    put(req, n);
    src[t].reserve(n);
    for (const IpcBlock& b : blocks[t]) {
      if (b.length == 0) continue;
      src[t].push_back(CheckRange{b.src_offset, b.length});
      put(req, static_cast<uint64_t>(b.dst_offset));
      put(req, static_cast<uint64_t>(b.length));
    }
  }
  TimeWatch w;
  o.local = checksum_cache(ctx, lb, le, src);
  if (fault_inject_corrupt_check()) o.local ^= 1;
  o.local_us = w.get_elapse_us();

  TimeWatch wr;
  const int timeout_ms = env_rpc_timeout_s() * 1000;
  const std::string ip = dst.addr.empty() ? "127.0.0.1" : dst.addr;
  FdGuard sock(tcp_connect(ip, server_port_of(dst), timeout_ms));
  if (!sock.valid()) throw KVTransferException(ErrorKind::TRANSPORT, "transfer check: cannot reach the destination's server");
  std::string resp;
  if (!send_frame(sock.fd(), req.data(), req.size(), timeout_ms) || !recv_frame(sock.fd(), resp, timeout_ms) ||
      resp.size() < RPC_HEADER + 4 + 8) {
    throw KVTransferException(ErrorKind::TRANSPORT, "transfer check: no answer from the destination");
  }
  uint32_t status = 0;
  memcpy(&status, resp.data() + RPC_HEADER, 4);
  if (status != WIRE_OK)
    throw KVTransferException(ErrorKind::TRANSPORT, "transfer check: the destination refused the ranges, status=" + std::to_string(status));
  memcpy(&o.remote, resp.data() + RPC_HEADER + 4, 8);
  o.remote_us = wr.get_elapse_us();
  o.ok = o.local == o.remote;
  return o;
}

std::string answer_check(Context* ctx, const char* buf, size_t len) {
  const auto t0 = SteadyClock::now();
  uint32_t magic = 0;
  uint64_t reqid = 0;
  if (len >= RPC_HEADER) get_rpc_header(buf, &magic, &reqid);
  std::string resp(RPC_HEADER, '\0');
  put_rpc_header(resp.data(), CHECK_REQ, reqid);
  uint32_t status = WIRE_BAD_REQUEST;
  uint64_t sum = 0;
  const char* p = buf + std::min(len, RPC_HEADER);
  const char* end = buf + len;
  uint32_t lb = 0, le = 0, n_tensors = 0, zero = 0;
  if (take(p, end, &lb) && take(p, end, &le) && take(p, end, &n_tensors) && take(p, end, &zero) && n_tensors <= 64) {
    std::vector<std::vector<CheckRange>> dst(n_tensors);
    bool parsed = true;
    for (uint32_t t = 0; t < n_tensors && parsed; ++t) {
      uint64_t n = 0;
      parsed = take(p, end, &n) && n <= static_cast<uint64_t>(end - p) / sizeof(CheckRange);
      if (!parsed) break;
      dst[t].resize(n);
      if (n != 0) memcpy(dst[t].data(), p, n * sizeof(CheckRange));
      p += n * sizeof(CheckRange);
    }
    if (parsed) {
      try {
        sum = checksum_cache(ctx, lb, le, dst);
        status = WIRE_OK;
      } catch (const std::out_of_range& ex) {
        LOG(ERROR) << "KVT server rejected a transfer check,reqid=" << reqid << ",ex=" << ex.what();
      } catch (const std::exception& ex) {
        LOG(ERROR) << "KVT server transfer check failed,reqid=" << reqid << ",ex=" << ex.what();
        status = WIRE_INTERNAL;
      }
    }
  }
  put(resp, status);
  put(resp, sum);
  put(resp, static_cast<int64_t>(elapse_us(t0, SteadyClock::now())));
  return resp;
}

}  // namespace kvx
