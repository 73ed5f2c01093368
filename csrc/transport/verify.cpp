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
  char* buf{nullptr};          // the launch's descriptors (chunks, or requests + block ids)
  size_t buf_cap{0};
  uint64_t* sums{nullptr};     // [sum_cap] sums, then 2 status words
  size_t sum_cap{0};

  // Makes room for `bytes` of descriptors and `n_sums` sums, uploads the descriptors and clears the sums.
  uint32_t* prepare(const void* host, size_t bytes, size_t n_sums) {
    if (stream == nullptr) cu(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "stream");
    if (buf_cap < bytes) {
      if (buf != nullptr) cudaFree(buf);
      buf = nullptr;
      buf_cap = 0;
      const size_t want = std::max<size_t>(bytes * 2, 65536);
      cu(cudaMalloc(reinterpret_cast<void**>(&buf), want), "cudaMalloc");
      buf_cap = want;
    }
    if (sum_cap < n_sums) {
      if (sums != nullptr) cudaFree(sums);
      sums = nullptr;
      sum_cap = 0;
      const size_t want = std::max<size_t>(n_sums * 2, 256);
      cu(cudaMalloc(reinterpret_cast<void**>(&sums), (want + 1) * sizeof(uint64_t)), "cudaMalloc");
      sum_cap = want;
    }
    cu(cudaMemcpyAsync(buf, host, bytes, cudaMemcpyHostToDevice, stream), "upload");
    cu(cudaMemsetAsync(sums, 0, (sum_cap + 1) * sizeof(uint64_t), stream), "memset");
    return reinterpret_cast<uint32_t*>(sums + sum_cap);
  }

  // Waits for the launches and returns the n_sums sums; throws when a kernel skipped something out of range.
  std::vector<uint64_t> collect(size_t n_sums) {
    std::vector<uint64_t> out(n_sums + 1, 0);
    cu(cudaMemcpyAsync(out.data(), sums, n_sums * sizeof(uint64_t), cudaMemcpyDeviceToHost, stream), "download");
    cu(cudaMemcpyAsync(&out[n_sums], sums + sum_cap, sizeof(uint64_t), cudaMemcpyDeviceToHost, stream), "download");
    cu(cudaStreamSynchronize(stream), "synchronize");
    if ((out[n_sums] & 0xFFFFFFFFu) != 0) throw std::out_of_range("transfer check: the kernel skipped data outside its tensor");
    out.pop_back();
    return out;
  }
};

std::mutex g_mu;
std::map<int, DeviceScratch> g_scratch;

uint64_t checksum_device(Context* ctx, uint32_t lb, uint32_t le, const std::vector<std::vector<CheckRange>>& per_tensor) {
  const int dev = ctx->device_id();
  const auto& addrs = ctx->layer_data_address();
  const size_t n_tensors = per_tensor.size();
  // pieces cut to chunks of a whole number of words; index0 (in words) restarts at every piece
  static_assert(KVT_CHECK_CHUNK % 4 == 0, "a chunk boundary must be a word boundary of its piece");
  std::vector<KvtCheckChunk> host;
  std::vector<size_t> first(n_tensors + 1, 0);
  for (size_t t = 0; t < n_tensors; ++t) {
    for (const CheckRange& r : per_tensor[t]) {
      for (uint64_t done = 0; done < r.len; done += KVT_CHECK_CHUNK) {
        const uint64_t n = std::min<uint64_t>(KVT_CHECK_CHUNK, r.len - done);
        host.push_back(KvtCheckChunk{r.off + done, static_cast<uint32_t>(n), static_cast<uint32_t>(done >> 2)});
      }
    }
    first[t + 1] = host.size();
  }
  if (host.empty()) return 0;
  std::lock_guard<std::mutex> g(g_mu);
  cu(cudaSetDevice(dev), "cudaSetDevice");   // the calling threads are the transport's own: nothing to restore
  DeviceScratch& s = g_scratch[dev];
  const size_t n_layers = le - lb;
  const size_t n_sums = n_layers * n_tensors;
  // device image: [tensor t: the n_layers base addresses][chunks]; sums[t * n_layers + layer]
  std::vector<uint64_t> bases;
  bases.reserve(n_sums);
  for (size_t t = 0; t < n_tensors; ++t)
    for (uint32_t l = lb; l < le; ++l) bases.push_back(addrs[l][t]);
  std::string image(reinterpret_cast<const char*>(bases.data()), bases.size() * sizeof(uint64_t));
  const size_t chunks_at = image.size();
  image.append(reinterpret_cast<const char*>(host.data()), host.size() * sizeof(KvtCheckChunk));
  uint32_t* status = s.prepare(image.data(), image.size(), n_sums);
  const uint64_t* d_bases = reinterpret_cast<const uint64_t*>(s.buf);
  const KvtCheckChunk* d_chunks = reinterpret_cast<const KvtCheckChunk*>(s.buf + chunks_at);
  const int sms = kvt_sm_count(dev);
  for (size_t t = 0; t < n_tensors; ++t) {
    const size_t n = first[t + 1] - first[t];
    if (n == 0) continue;
    const int rc = kvt_launch_checksum(d_bases + t * n_layers, static_cast<uint32_t>(n_layers), ctx->tensor_capacity(t),
                                       d_chunks + first[t], static_cast<uint32_t>(n), s.sums + t * n_layers, status,
                                       sms > 0 ? sms * 8 : 0, s.stream);
    if (rc != 0) cu(static_cast<cudaError_t>(rc), "launch");
  }
  const std::vector<uint64_t> out = s.collect(n_sums);
  uint64_t total = 0;
  for (uint32_t l = lb; l < le; ++l)
    for (size_t t = 0; t < n_tensors; ++t) total += fold(out[t * n_layers + (l - lb)], l, static_cast<uint32_t>(t));
  return total;
}

CheckOutcome ask_destination(const WorkerInfo& dst, const std::string& req, CheckOutcome o) {
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
    throw KVTransferException(ErrorKind::TRANSPORT, "transfer check: the destination refused the request, status=" + std::to_string(status));
  memcpy(&o.remote, resp.data() + RPC_HEADER + 4, 8);
  o.remote_us = wr.get_elapse_us();
  o.ok = o.local == o.remote;
  return o;
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
  return ask_destination(dst, req, o);
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

// ---- row form ------------------------------------------------------------------------------------------------------
void AttnCheck::add(const std::vector<uint32_t>& blocks, uint32_t seen, uint32_t new_tokens, uint32_t index) {
  if (new_tokens == 0) return;
  KvtCheckReq r{};
  r.blk_off = static_cast<uint32_t>(pool.size());
  r.n_blocks = static_cast<uint32_t>(blocks.size());
  r.seen = seen;
  r.new_tokens = new_tokens;
  r.first = total_tokens;
  r.index = index;
  pool.insert(pool.end(), blocks.begin(), blocks.end());
  reqs.push_back(r);
  total_tokens += new_tokens;
}

namespace {

// Everything the kernel derives an address from, against the tensor: after this no product of a coordinate and a
// stride can leave [0, capacity] (the kernel still checks every row).
void validate_attn_check(const AttnCheck& c, uint64_t capacity) {
  const KvtLayout& l = c.layout;
  auto fits = [&](int64_t stride, uint64_t count) {
    return stride >= 0 && (count == 0 || static_cast<uint64_t>(stride) <= capacity / count);
  };
  const bool ok = l.ntpb != 0 && l.head_bytes != 0 && (l.kv_count == 1 || l.kv_count == 2) && l.num_blocks != 0 &&
                  c.n_heads != 0 && c.head0 <= l.num_heads && c.n_heads <= l.num_heads - c.head0 && l.head_bytes <= capacity &&
                  fits(l.block_stride, l.num_blocks) && fits(l.kv_stride, l.kv_count) && fits(l.token_stride, l.ntpb) &&
                  fits(l.head_stride, l.num_heads);
  if (!ok) throw std::out_of_range("transfer check: the layout does not fit the tensor");
  uint32_t expect_first = 0;
  for (const KvtCheckReq& r : c.reqs) {
    const uint64_t last = static_cast<uint64_t>(r.seen) + r.new_tokens;     // one past the last token
    if (r.new_tokens == 0 || r.first != expect_first || r.blk_off > c.pool.size() || r.n_blocks > c.pool.size() - r.blk_off ||
        last > static_cast<uint64_t>(r.n_blocks) * l.ntpb)
      throw std::out_of_range("transfer check: a request leaves its block table");
    expect_first += r.new_tokens;
  }
  if (expect_first != c.total_tokens) throw std::out_of_range("transfer check: token count differs from the requests'");
  for (uint32_t b : c.pool)
    if (b >= l.num_blocks) throw std::out_of_range("transfer check: block id outside the tensor");
}

// body of CHECK_ATTN_REQ: [layer_begin u32][layer_end u32][head0 u32][n_heads u32][KvtLayout][n_reqs u32][pool_len u32]
//                         [KvtCheckReq x n_reqs][u32 x pool_len]
void put_attn(std::string& s, uint32_t lb, uint32_t le, const AttnCheck& c) {
  put(s, lb);
  put(s, le);
  put(s, c.head0);
  put(s, c.n_heads);
  put(s, c.layout);
  put(s, static_cast<uint32_t>(c.reqs.size()));
  put(s, static_cast<uint32_t>(c.pool.size()));
  s.append(reinterpret_cast<const char*>(c.reqs.data()), c.reqs.size() * sizeof(KvtCheckReq));
  s.append(reinterpret_cast<const char*>(c.pool.data()), c.pool.size() * sizeof(uint32_t));
}

}  // namespace

uint64_t checksum_attn(Context* ctx, uint32_t lb, uint32_t le, const AttnCheck& c) {
  const auto& addrs = ctx->layer_data_address();
  if (lb > le || le > addrs.size()) throw std::out_of_range("transfer check: layer range outside the cache");
  const int dev = ctx->device_id();
  if (dev < 0) throw std::runtime_error("transfer check: the row form needs a device cache");
  for (uint32_t l = lb; l < le; ++l)
    if (addrs[l].size() != 1) throw std::out_of_range("transfer check: the row form describes one tensor per layer");
  const uint64_t capacity = ctx->tensor_capacity(0);
  validate_attn_check(c, capacity);
  if (c.reqs.empty() || lb == le) return 0;
  // device image: [the layers' base addresses][requests][block ids]
  std::vector<uint64_t> bases;
  for (uint32_t l = lb; l < le; ++l) bases.push_back(addrs[l][0]);
  std::string host(reinterpret_cast<const char*>(bases.data()), bases.size() * sizeof(uint64_t));
  const size_t reqs_at = host.size();
  host.append(reinterpret_cast<const char*>(c.reqs.data()), c.reqs.size() * sizeof(KvtCheckReq));
  const size_t pool_at = host.size();
  host.append(reinterpret_cast<const char*>(c.pool.data()), c.pool.size() * sizeof(uint32_t));
  std::lock_guard<std::mutex> g(g_mu);
  cu(cudaSetDevice(dev), "cudaSetDevice");
  DeviceScratch& s = g_scratch[dev];
  const size_t n_sums = le - lb;
  uint32_t* status = s.prepare(host.data(), host.size(), n_sums);
  const int sms = kvt_sm_count(dev);
  const int rc = kvt_launch_checksum_attn(reinterpret_cast<const uint64_t*>(s.buf), static_cast<uint32_t>(n_sums), capacity, &c.layout,
                                          c.head0, c.n_heads, reinterpret_cast<const KvtCheckReq*>(s.buf + reqs_at),
                                          static_cast<uint32_t>(c.reqs.size()), c.total_tokens,
                                          reinterpret_cast<const uint32_t*>(s.buf + pool_at), static_cast<uint32_t>(c.pool.size()),
                                          s.sums, status, sms > 0 ? sms * 8 : 0, s.stream);
  if (rc != 0) cu(static_cast<cudaError_t>(rc), "launch");
  const std::vector<uint64_t> out = s.collect(n_sums);
  uint64_t total = 0;
  for (uint32_t l = lb; l < le; ++l) total += fold(out[l - lb], l, 0);
  return total;
}

CheckOutcome verify_attn_transfer(Context* ctx, const WorkerInfo& dst, uint32_t lb, uint32_t le, const AttnCheck& src_side,
                                  const AttnCheck& dst_side) {
  CheckOutcome o;
  std::string req(RPC_HEADER, '\0');
  put_rpc_header(req.data(), CHECK_ATTN_REQ, new_id());
  put_attn(req, lb, le, dst_side);
  TimeWatch w;
  o.local = checksum_attn(ctx, lb, le, src_side);
  if (fault_inject_corrupt_check()) o.local ^= 1;
  o.local_us = w.get_elapse_us();
  return ask_destination(dst, req, o);
}

std::string answer_check_attn(Context* ctx, const char* buf, size_t len) {
  const auto t0 = SteadyClock::now();
  uint32_t magic = 0;
  uint64_t reqid = 0;
  if (len >= RPC_HEADER) get_rpc_header(buf, &magic, &reqid);
  std::string resp(RPC_HEADER, '\0');
  put_rpc_header(resp.data(), CHECK_ATTN_REQ, reqid);
  uint32_t status = WIRE_BAD_REQUEST;
  uint64_t sum = 0;
  const char* p = buf + std::min(len, RPC_HEADER);
  const char* end = buf + len;
  uint32_t lb = 0, le = 0, n_reqs = 0, pool_len = 0;
  AttnCheck c;
  if (take(p, end, &lb) && take(p, end, &le) && take(p, end, &c.head0) && take(p, end, &c.n_heads) && take(p, end, &c.layout) &&
      take(p, end, &n_reqs) && take(p, end, &pool_len) && n_reqs <= static_cast<size_t>(end - p) / sizeof(KvtCheckReq)) {
    c.reqs.resize(n_reqs);
    if (n_reqs != 0) memcpy(c.reqs.data(), p, n_reqs * sizeof(KvtCheckReq));
    p += n_reqs * sizeof(KvtCheckReq);
    if (pool_len <= static_cast<size_t>(end - p) / sizeof(uint32_t)) {
      c.pool.resize(pool_len);
      if (pool_len != 0) memcpy(c.pool.data(), p, pool_len * sizeof(uint32_t));
      for (const KvtCheckReq& r : c.reqs) c.total_tokens += r.new_tokens;
      try {
        sum = checksum_attn(ctx, lb, le, c);
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
