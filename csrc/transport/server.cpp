// Receiving side of the host-driven transports and control endpoint of the NVLink transport.
//
// One TCP listener per worker (BLLM_KVTRANS_PORT_BASE + worker_id, or an ephemeral port when
// that is taken; the bound port is published in WorkerInfo ext "port").  Each connection gets
// a thread that reads frames and
//   * scatters 'KVCa' data messages into the local cache - memcpy for host-resident caches,
//     the descriptor-driven copy kernel reading the pinned receive buffer for GPU caches
//     (receiver half of kvtransfer/src/tcp_channel.cpp:141-325);
//   * attaches a POSIX shm segment named by the sender and scatters blobs out of it;
//   * answers MEM_HANDLES_REQ with CUDA IPC handles of every layer tensor, which is how a
//     prefill worker's NVLink transport maps this worker's cache (the role the RDMA
//     rkey exchange plays in kvtransfer/src/rdma_channel.cpp:77-99,298-316);
//   * answers CHECK_REQ with the checksum of the named ranges of this worker's cache (the receiving half of
//     the end-to-end check, the role of resp_remote_crc in kvtransfer/src/rdma_channel.cpp:201-296).
#include <cuda_runtime.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <thread>

#include "core/envcfg.h"
#include "core/util.h"
#include "kernels/kvt_kernels.h"
#include "transport/channel.h"
#include "transport/device_stage.h"
#include "transport/pull_session.h"
#include "transport/verify.h"
#include "transport/wire.h"

namespace kvx {

int server_port_of(const WorkerInfo& w) {
  const int p = w.ext_int("port", 0);
  return p > 0 ? p : env_port_base() + static_cast<int>(w.worker_id);
}

namespace {

struct ShmSeg {
  char* base{nullptr};
  size_t bytes{0};
  uint64_t dev{0};  // device-mapped address when registered with CUDA
  bool registered{false};
  void reset() {
    if (base != nullptr) {
      if (registered) cudaHostUnregister(base);
      munmap(base, bytes);
    }
    base = nullptr;
    bytes = 0;
    dev = 0;
    registered = false;
  }
};

class TransferServer : public ITransferServer {
 public:
  ~TransferServer() override { stop(); }

  void start_server(Context* ctx) override {
    ctx_ = ctx;
    int want = env_port_base() + static_cast<int>(ctx->worker_id);
    int bound = 0;
    int fd = tcp_listen("0.0.0.0", want, 128, &bound);
    if (fd < 0) fd = tcp_listen("0.0.0.0", 0, 128, &bound);
    if (fd < 0) throw KVTransferException(ErrorKind::TRANSPORT, "transfer server: cannot listen");
    listen_fd_ = FdGuard(fd);
    port_ = bound;
    WorkerInfo* wi = ctx->worker_info_mutable();
    wi->ext["port"] = std::to_string(bound);
    wi->ext["host"] = std::to_string(this_host_id());
    wi->ext["pid"] = std::to_string(static_cast<int>(getpid()));
    wi->ext["dev"] = std::to_string(ctx->device_id());
    if (wi->addr.empty()) wi->addr = local_ip();
    stop_.store(false);
    accept_thd_ = std::thread([this] { accept_loop(); });
    LOG(INFO) << "KVT server listening. port=" << bound << " worker=" << wi->to_string();
  }

  int port() const override { return port_; }

  void stop() override {
    if (stop_.exchange(true)) return;
    if (listen_fd_.valid()) ::shutdown(listen_fd_.fd(), SHUT_RDWR);
    if (accept_thd_.joinable()) accept_thd_.join();
    listen_fd_.reset();
    std::vector<ConnThread> thds;
    {
      std::lock_guard<std::mutex> g(mu_);
      for (auto& kv : conns_) ::shutdown(kv.first, SHUT_RDWR);
      thds.swap(conn_thds_);
    }
    for (auto& t : thds)
      if (t.thd.joinable()) t.thd.join();
  }

 private:
  void accept_loop() {
    while (!stop_.load()) {
      struct pollfd p{listen_fd_.fd(), POLLIN, 0};
      int r = ::poll(&p, 1, 200);
      if (r <= 0) continue;
      int cfd = ::accept4(listen_fd_.fd(), nullptr, nullptr, SOCK_CLOEXEC);
      if (cfd < 0) continue;
      // replies are small and latency-bound: without this, Nagle + delayed ACK add ~40 ms per layer
      int one = 1;
      setsockopt(cfd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      std::vector<std::thread> ended;
      {
        std::lock_guard<std::mutex> g(mu_);
        // connections come and go over a long run: join the threads of those that ended
        for (auto it = conn_thds_.begin(); it != conn_thds_.end();) {
          if (it->done->load(std::memory_order_acquire)) {
            ended.push_back(std::move(it->thd));
            it = conn_thds_.erase(it);
          } else {
            ++it;
          }
        }
        conns_[cfd] = true;
        auto done = std::make_shared<std::atomic<bool>>(false);
        conn_thds_.push_back(ConnThread{std::thread([this, cfd, done] {
                                          serve(cfd);
                                          done->store(true, std::memory_order_release);
                                        }),
                                        done});
      }
      for (auto& t : ended)
        if (t.joinable()) t.join();
    }
  }

  // The longest frame a well-behaved peer sends: one layer's data for every tensor, plus its block
  // metadata (which a sender keeps far below the data it describes) and the headers.
  size_t frame_limit() const {
    size_t cap = 0;
    const auto& addrs = ctx_->layer_data_address();
    const size_t n_tensors = addrs.empty() ? 0 : addrs[0].size();
    for (size_t t = 0; t < n_tensors; ++t) cap += ctx_->tensor_capacity(t);
    const size_t lim = 2 * cap + (size_t{1} << 20);
    return std::min<size_t>(lim, 0xffffffffu);
  }

  void serve(int cfd) {
    FdGuard fd(cfd);
    std::unique_ptr<DeviceStage> stage;
    PinnedBuffer rx;
    ShmSeg shm;
    const bool gpu = ctx_->device_id() >= 0;
    // a pull session answers finished batches from the completion thread: every write to this connection is locked
    auto write_mu = std::make_shared<std::mutex>();
    std::shared_ptr<PullSession> pull;
    const size_t frame_max = frame_limit();
    try {
      if (gpu) stage = std::make_unique<DeviceStage>(ctx_->device_id());
      for (;;) {
        uint32_t n = 0;
        // Idle connections block here; stop() shuts the socket down to wake them.
        if (read_full(cfd, &n, 4, 0) != 4) break;
        if (n > frame_max) {      // nothing is pinned or read for a length no sender of ours produces
          LOG(ERROR) << "KVT server: frame of " << n << " bytes exceeds the limit of " << frame_max << ", closing";
          break;
        }
        char* buf = rx.reserve(n, gpu);
        if (n > 0 && read_full(cfd, buf, n, env_rpc_timeout_s() * 1000) != static_cast<ssize_t>(n)) break;
        if (n < 4) break;
        uint32_t magic = 0;
        memcpy(&magic, buf, 4);
        std::string resp;
        if (magic == KV_CACHE_DATA_MAGIC) {
          uint64_t reqid = 0;
          if (n < RPC_HEADER) break;
          get_rpc_header(buf, &magic, &reqid);
          resp = on_data(reqid, buf + RPC_HEADER, n - RPC_HEADER, buf, rx.device_ptr(), n, stage.get(), false, 0);
        } else if (magic == KV_CACHE_SHM_MAGIC) {
          uint64_t reqid = 0, seg_off = 0;
          if (n < RPC_HEADER + 8) break;
          get_rpc_header(buf, &magic, &reqid);
          memcpy(&seg_off, buf + RPC_HEADER, 8);
          resp = on_data(reqid, buf + RPC_HEADER + 8, n - RPC_HEADER - 8, shm.base, shm.dev, shm.bytes, stage.get(),
                         true, seg_off);
        } else if (magic == SHM_ATTACH_REQ) {
          resp = on_attach(buf, n, shm, gpu);
        } else if (magic == MEM_HANDLES_REQ) {
          resp = on_mem_handles(buf, n);
        } else if (magic == PULL_OPEN_REQ) {
          uint64_t reqid = 0;
          if (n < RPC_HEADER) break;
          get_rpc_header(buf, &magic, &reqid);
          uint32_t status = WIRE_BAD_REQUEST;
          if (gpu && env_nvlink_pull() != 0) {
            pull = std::make_shared<PullSession>(ctx_, cfd, write_mu);
            status = pull->open(buf + RPC_HEADER, n - RPC_HEADER);
            if (status != WIRE_OK) pull.reset();
          }
          resp.resize(RPC_HEADER);
          put_rpc_header(resp.data(), PULL_OPEN_REQ, reqid);
          put(resp, status);
        } else if (magic == PULL_PLAN_REQ || magic == PULL_LAYERS_REQ || magic == PULL_FLUSH_REQ) {
          uint64_t seq = 0;
          if (n < RPC_HEADER || !pull) break;
          get_rpc_header(buf, &magic, &seq);
          if (magic == PULL_PLAN_REQ) pull->on_plan(seq, buf + RPC_HEADER, n - RPC_HEADER);
          else if (magic == PULL_LAYERS_REQ) pull->on_layers(seq, buf + RPC_HEADER, n - RPC_HEADER);
          else pull->on_flush(seq, buf + RPC_HEADER, n - RPC_HEADER);
          continue;     // one-way: a flushed batch is answered with PULL_DONE when its completion record arrives
        } else if (magic == CHECK_REQ) {
          resp = answer_check(ctx_, buf, n);
        } else if (magic == CHECK_ATTN_REQ) {
          resp = answer_check_attn(ctx_, buf, n);
        } else if (magic == PING_REQ) {
          resp.assign(buf, std::min<size_t>(n, RPC_HEADER));
          put(resp, static_cast<uint32_t>(WIRE_OK));
        } else {
          LOG(ERROR) << "KVT server: unknown message magic=" << magic << " len=" << n;
          break;
        }
        std::lock_guard<std::mutex> wg(*write_mu);
        if (!send_frame(cfd, resp.data(), resp.size(), env_rpc_timeout_s() * 1000)) break;
      }
    } catch (const std::exception& ex) {
      LOG(ERROR) << "KVT server connection failed: " << ex.what();
    }
    if (pull) {
      pull->close();      // no more PULL_DONE frames; batches still completing keep the session alive until they end
      // the descriptor is about to close: wait (bounded) until nothing can write to it any more
      std::lock_guard<std::mutex> wg(*write_mu);
    }
    shm.reset();
    std::lock_guard<std::mutex> g(mu_);
    conns_.erase(cfd);
  }

  // body: the 'KVCa' message after its RPC header ([layer][num_tensors] + per-tensor metadata
  // [+ blob when !external]).  blob_host/blob_dev/blob_cap: the memory the blobs are read from
  // (the received frame itself, or the attached shm segment).
  std::string on_data(uint64_t reqid, const char* body, size_t len, const char* blob_host, uint64_t blob_dev,
                      size_t blob_cap, DeviceStage* stage, bool external, uint64_t seg_off) {
    const auto t_start = SteadyClock::now();
    std::string resp;
    auto reply = [&](uint32_t status) {
      resp.resize(RPC_HEADER);
      put_rpc_header(resp.data(), KV_CACHE_DATA_MAGIC, reqid);
      put(resp, status);
      put(resp, static_cast<int64_t>(elapse_us(t_start, SteadyClock::now())));
      return resp;
    };
    const char* p = body;
    const char* end = body + len;
    if (len < 2 * sizeof(size_t)) return reply(WIRE_BAD_REQUEST);
    size_t layer = 0, n_tensors = 0;
    take(p, end, &layer);
    take(p, end, &n_tensors);
    const auto& addrs = ctx_->layer_data_address();
    if (layer >= addrs.size() || n_tensors != addrs[layer].size()) {
      LOG(ERROR) << "KVT server: bad layer/tensor count. layer=" << layer << " tensors=" << n_tensors;
      return reply(WIRE_BAD_REQUEST);
    }
    size_t ext_cursor = seg_off;
    try {
      for (size_t t = 0; t < n_tensors; ++t) {
        size_t n_blocks = 0, blob_bytes = 0;
        if (!take(p, end, &n_blocks)) return reply(WIRE_BAD_REQUEST);
        if (n_blocks > static_cast<size_t>(end - p) / sizeof(IpcBlock)) return reply(WIRE_BAD_REQUEST);
        const char* meta = p;
        p += n_blocks * sizeof(IpcBlock);
        if (!take(p, end, &blob_bytes)) return reply(WIRE_BAD_REQUEST);
        size_t blob_off;
        if (external) {
          blob_off = ext_cursor;
          ext_cursor += blob_bytes;
          if (blob_host == nullptr || blob_off > blob_cap || blob_bytes > blob_cap - blob_off)
            return reply(WIRE_BAD_REQUEST);
        } else {
          if (blob_bytes > static_cast<size_t>(end - p)) return reply(WIRE_BAD_REQUEST);
          blob_off = static_cast<size_t>(p - blob_host);
          p += blob_bytes;
        }
        const size_t cap = ctx_->tensor_capacity(t);
        std::vector<Triple> triples;
        triples.reserve(n_blocks);
        size_t cursor = 0;
        for (size_t i = 0; i < n_blocks; ++i) {
          size_t f[3];
          memcpy(f, meta + i * sizeof(IpcBlock), sizeof(f));
          const size_t dst_off = f[1], blen = f[2];
          if (blen == 0 || dst_off > cap || blen > cap - dst_off || blen > blob_bytes - cursor) {
            LOG(ERROR) << "KVT server rejected invalid copy metadata,reqid=" << reqid << ",layer_idx=" << layer
                       << ",tensor_idx=" << t << ",block_idx=" << i << ",dst_offset=" << dst_off
                       << ",length=" << blen << ",capacity=" << cap;
            return reply(WIRE_BAD_REQUEST);
          }
          triples.push_back(Triple{blob_off + cursor, dst_off, blen});
          cursor += blen;
        }
        if (stage != nullptr) {
          stage->enqueue(blob_dev, addrs[layer][t], triples, blob_cap, cap, 0, DeviceStage::HOST_SRC);
        } else {
          char* dst = reinterpret_cast<char*>(addrs[layer][t]);
          for (const auto& tr : triples) memcpy(dst + tr.dst_off, blob_host + tr.src_off, tr.len);
        }
      }
      if (stage != nullptr) stage->sync();
    } catch (const std::exception& ex) {
      LOG(ERROR) << "KVT server scatter failed,reqid=" << reqid << ",ex=" << ex.what();
      return reply(WIRE_INTERNAL);
    }
    return reply(WIRE_OK);
  }

  std::string on_attach(const char* buf, size_t n, ShmSeg& shm, bool gpu) {
    uint32_t magic = 0, name_len = 0;
    uint64_t reqid = 0, bytes = 0;
    const char* p = buf;
    const char* end = buf + n;
    std::string resp(RPC_HEADER, '\0');
    uint32_t status = WIRE_BAD_REQUEST;
    if (n >= RPC_HEADER + 4) {
      get_rpc_header(p, &magic, &reqid);
      p += RPC_HEADER;
      take(p, end, &name_len);
      if (name_len < 256 && static_cast<size_t>(end - p) >= name_len + 8) {
        std::string name(p, name_len);
        p += name_len;
        take(p, end, &bytes);
        shm.reset();
        int sfd = shm_open(name.c_str(), O_RDWR, 0600);
        struct stat st {};
        if (sfd >= 0 && (fstat(sfd, &st) != 0 || bytes == 0 || bytes > static_cast<uint64_t>(st.st_size))) {
          // a mapping longer than the segment would fault on first touch
          LOG(ERROR) << "KVT server: shm attach of " << bytes << " bytes refused, segment has " << st.st_size;
          ::close(sfd);
          sfd = -1;
        }
        if (sfd >= 0) {
          void* m = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, sfd, 0);
          ::close(sfd);
          if (m != MAP_FAILED) {
            shm.base = static_cast<char*>(m);
            shm.bytes = bytes;
            status = WIRE_OK;
            if (gpu) {
              uint64_t dev = 0;
              if (kvt_host_register(reinterpret_cast<uint64_t>(m), bytes, &dev) == 0) {
                shm.dev = dev;
                shm.registered = true;
              } else {
                cudaGetLastError();
                shm.reset();
                status = WIRE_INTERNAL;
              }
            }
          }
        }
      }
    }
    put_rpc_header(resp.data(), SHM_ATTACH_REQ, reqid);
    put(resp, status);
    return resp;
  }

  std::string on_mem_handles(const char* buf, size_t n) {
    uint32_t magic = 0;
    uint64_t reqid = 0;
    if (n >= RPC_HEADER) get_rpc_header(buf, &magic, &reqid);
    PeerMemInfo info;
    info.pid = static_cast<int32_t>(getpid());
    info.device = ctx_->device_id();
    info.host_id = this_host_id();
    const auto& addrs = ctx_->layer_data_address();
    info.num_layers = static_cast<uint32_t>(addrs.size());
    info.num_tensors = addrs.empty() ? 0 : static_cast<uint32_t>(addrs[0].size());
    uint32_t status = WIRE_OK;
    std::lock_guard<std::mutex> g(handle_mu_);
    if (handle_cache_.empty() && ctx_->device_id() >= 0) {
      cudaSetDevice(ctx_->device_id());
      for (const auto& layer : addrs) {
        for (uint64_t ptr : layer) {
          PeerTensor t{};
          t.ptr = ptr;
          t.alloc_base = ptr;
          uint64_t base = 0, size = 0;
          if (kvt_ipc_get_handle(ptr, t.ipc_handle, &base, &size) == 0) {
            t.has_handle = 1;
            t.alloc_base = base;
          } else {
            cudaGetLastError();
            t.has_handle = 0;
          }
          handle_cache_.push_back(t);
        }
      }
    }
    info.tensors = handle_cache_;
    if (ctx_->device_id() < 0) status = WIRE_BAD_REQUEST;
    std::string resp(RPC_HEADER, '\0');
    put_rpc_header(resp.data(), MEM_HANDLES_REQ, reqid);
    put(resp, status);
    resp += info.serialize();
    return resp;
  }

  Context* ctx_{nullptr};
  FdGuard listen_fd_;
  int port_{0};
  std::atomic<bool> stop_{true};
  std::thread accept_thd_;
  std::mutex mu_;
  std::map<int, bool> conns_;
  struct ConnThread {
    std::thread thd;
    std::shared_ptr<std::atomic<bool>> done;   // set by the thread as its last act
  };
  std::vector<ConnThread> conn_thds_;
  std::mutex handle_mu_;
  std::vector<PeerTensor> handle_cache_;
};

}  // namespace

std::unique_ptr<ITransferServer> create_transfer_server() { return std::make_unique<TransferServer>(); }

}  // namespace kvx
