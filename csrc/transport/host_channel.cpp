// Sender side of the host-driven transports: TCP sockets and POSIX shared memory.
//
// Per layer the channel gathers the registered byte ranges of every cache tensor into one
// message (format in transport/wire.h; sender half of kvtransfer/src/tcp_channel.cpp:477-588)
// and hands it to the destination's server, which scatters it.  For a GPU-resident source the
// gather is a descriptor-driven copy kernel writing into mapped pinned memory; for a
// host-resident source it is memcpy.  With shared memory the blobs are gathered straight into
// a segment the receiver has mapped, and only the metadata crosses the socket.
// Connections: BLLM_KVTRANS_RDMA_SP sockets per target, layers round-robin over them.
#include <fcntl.h>
#include <sys/mman.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <future>
#include <sstream>

#include "core/envcfg.h"
#include "core/fault_inject.h"
#include "core/util.h"
#include "kernels/kvt_kernels.h"
#include "transport/channel.h"
#include "transport/device_stage.h"
#include "transport/wire.h"

namespace kvx {

namespace {

class HostChannel : public IChannel {
 public:
  HostChannel(Context* ctx, bool use_shm) : ctx_(ctx), use_shm_(use_shm) {}
  ~HostChannel() override { close(); }

  const char* name() const override { return use_shm_ ? "shm" : "tcp"; }

  void connect(const WorkerInfo& dst) override {
    dst_ = dst;
    const std::string ip = dst.addr.empty() ? "127.0.0.1" : dst.addr;
    const int port = server_port_of(dst);
    const int n = std::max(1, env_send_parallel());
    for (int i = 0; i < n; ++i) {
      fault_inject_throw();
      int fd = tcp_connect(ip, port, env_rpc_timeout_s() * 1000);
      if (fd < 0) {
        throw KVTransferException(ErrorKind::TRANSPORT, "connect to " + ip + ":" + std::to_string(port) +
                                                            " failed, errno=" + std::to_string(errno));
      }
      socks_.emplace_back(fd);
    }
    if (ctx_->device_id() >= 0) stage_ = std::make_unique<DeviceStage>(ctx_->device_id());
    active_ = true;
  }

  void register_data(std::vector<std::vector<IpcBlock>>& data, TPKind kind) override {
    data_.swap(data);
    data.clear();
    // The unscaled bf16 -> e4m3 cast of the reference's staged path (tcp_channel.cpp:411-447): only the
    // P>D planner emits fp8 lengths, and only single-tensor layers are cast.
    cast_ = env_bf162fp8_conversion() && kind == TPKind::PGTD && data_.size() == 1;
    origin_blocks_ = merged_blocks_ = 0;
    sb_min_ = SIZE_MAX;
    sb_max_ = sb_total_ = 0;
    blob_bytes_.assign(data_.size(), 0);
    for (size_t t = 0; t < data_.size(); ++t) {
      origin_blocks_ += data_[t].size();
      validate_ipc_block_bounds(data_[t], ctx_->tensor_capacity(t), IpcBlockOffset::SOURCE, name(), 0, t, cast_ ? 2 : 1);
      const MergeStats st = merge_interval(data_[t]);
      merged_blocks_ += st.count;
      if (st.count) {
        sb_min_ = std::min(sb_min_, st.min_len);
        sb_max_ = std::max(sb_max_, st.max_len);
      }
      sb_total_ += st.total_len;
      blob_bytes_[t] = st.total_len;
    }
    if (use_shm_) ensure_shm(sb_total_ * std::max<size_t>(1, ctx_->num_layers() > 4 ? 4 : ctx_->num_layers()));
    pending_.clear();
    send_us_ = gather_us_ = 0;
    inflight_bytes_ = 0;
  }

  void send_data(size_t layer, Step* step) override {
    (void)step;
    TimeWatch tw;
    const uint64_t reqid = new_id();
    const auto& addrs = ctx_->layer_data_address();
    RTASSERT(layer < addrs.size());
    RTASSERT(addrs[layer].size() == data_.size());
    // ---- metadata ------------------------------------------------------------------------
    std::string head;
    head.resize(RPC_HEADER);
    put_rpc_header(head.data(), use_shm_ ? KV_CACHE_SHM_MAGIC : KV_CACHE_DATA_MAGIC, reqid);
    size_t seg_off = 0;
    if (use_shm_) {
      // ring allocation inside the segment; the receiver acks a layer before its slot is reused
      if (shm_cursor_ + sb_total_ > shm_bytes_) {
        drain(0);
        shm_cursor_ = 0;
      }
      seg_off = shm_cursor_;
      put(head, static_cast<uint64_t>(seg_off));
    }
    put(head, static_cast<size_t>(layer));
    put(head, static_cast<size_t>(data_.size()));
    // ---- blobs ------------------------------------------------------------------------------
    const size_t inline_bytes = use_shm_ ? 0 : sb_total_;
    std::string& msg = msg_buf_;
    msg.clear();
    char* blob_base = nullptr;
    uint64_t blob_dev = 0;
    size_t blob_cap = 0;
    TxSlot* slot = nullptr;
    size_t meta_bytes = head.size();
    for (size_t t = 0; t < data_.size(); ++t) meta_bytes += 2 * sizeof(size_t) + data_[t].size() * sizeof(IpcBlock);
    if (use_shm_) {
      blob_base = shm_base_;
      blob_dev = shm_dev_;
      blob_cap = shm_bytes_;
    } else {
      // One frame buffer per connection, pinned when the source is a GPU, holding metadata and blobs
      // contiguously.  The connection's previous frame must have been acknowledged before its buffer is
      // refilled; frames on the other connections are still on their way meanwhile.
      if (slots_.size() != socks_.size()) {
        slots_.clear();
        for (size_t i = 0; i < socks_.size(); ++i) slots_.emplace_back(std::make_unique<TxSlot>());
      }
      slot = slots_[rr_ % slots_.size()].get();
      wait_slot(*slot);
      slot->buf.reserve(meta_bytes + inline_bytes, stage_ != nullptr);
      blob_base = slot->buf.data();
      blob_dev = slot->buf.device_ptr();
      blob_cap = slot->buf.capacity();
    }
    std::string meta = head;
    size_t cursor = use_shm_ ? seg_off : 0;  // offset inside blob_base where the next blob goes
    size_t inline_cursor = 0;                // only for !shm: position inside the frame
    std::vector<std::pair<size_t, size_t>> blob_pos(data_.size());
    if (!use_shm_) {
      // frame layout is sequential: compute where each blob lands
      inline_cursor = head.size();
      for (size_t t = 0; t < data_.size(); ++t) {
        inline_cursor += sizeof(size_t) + data_[t].size() * sizeof(IpcBlock) + sizeof(size_t);
        blob_pos[t] = {inline_cursor, blob_bytes_[t]};
        inline_cursor += blob_bytes_[t];
      }
    } else {
      for (size_t t = 0; t < data_.size(); ++t) {
        blob_pos[t] = {cursor, blob_bytes_[t]};
        cursor += blob_bytes_[t];
      }
    }
    TimeWatch gw;
    for (size_t t = 0; t < data_.size(); ++t) {
      std::vector<Triple> triples;
      triples.reserve(data_[t].size());
      size_t c = blob_pos[t].first;
      for (const auto& b : data_[t]) {
        triples.push_back(Triple{b.src_offset, c, b.length});
        c += b.length;
      }
      if (stage_ != nullptr) {
        stage_->enqueue(addrs[layer][t], blob_dev, triples, ctx_->tensor_capacity(t), blob_cap, 0, DeviceStage::HOST_DST,
                        cast_);
      } else if (cast_) {
        const char* src = reinterpret_cast<const char*>(addrs[layer][t]);
        for (const auto& tr : triples) {
          const char* sp = src + tr.src_off;
          char* dp = blob_base + tr.dst_off;
          for (uint64_t k = 0; k < tr.len; ++k) {
            uint16_t h;
            memcpy(&h, sp + 2 * k, 2);
            dp[k] = static_cast<char>(kvt_bf16_to_e4m3(h));
          }
        }
      } else {
        const char* src = reinterpret_cast<const char*>(addrs[layer][t]);
        for (const auto& tr : triples) memcpy(blob_base + tr.dst_off, src + tr.src_off, tr.len);
      }
    }
    if (stage_ != nullptr) stage_->sync();
    gather_us_ += gw.get_elapse_us();
    // ---- send ---------------------------------------------------------------------------------
    FdGuard& sock = socks_[rr_++ % socks_.size()];
    bool ok;
    if (use_shm_) {
      for (size_t t = 0; t < data_.size(); ++t) {
        put(meta, static_cast<size_t>(data_[t].size()));
        meta.append(reinterpret_cast<const char*>(data_[t].data()), data_[t].size() * sizeof(IpcBlock));
        put(meta, static_cast<size_t>(blob_bytes_[t]));
      }
      ok = send_frame(sock.fd(), meta.data(), meta.size(), env_rpc_timeout_s() * 1000);
      shm_cursor_ = cursor;
    } else {
      // write metadata pieces between the already gathered blobs
      char* p = slot->buf.data();
      memcpy(p, head.data(), head.size());
      p += head.size();
      for (size_t t = 0; t < data_.size(); ++t) {
        const size_t n = data_[t].size();
        memcpy(p, &n, sizeof(size_t));
        p += sizeof(size_t);
        memcpy(p, data_[t].data(), n * sizeof(IpcBlock));
        p += n * sizeof(IpcBlock);
        memcpy(p, &blob_bytes_[t], sizeof(size_t));
        p += sizeof(size_t);
        p += blob_bytes_[t];
      }
      // the frame leaves, and its acknowledgement comes back, on a thread of its own: the next layer is
      // gathered and sent on another connection meanwhile
      const int fd = sock.fd();
      const char* frame = slot->buf.data();
      const size_t frame_bytes = static_cast<size_t>(p - slot->buf.data());
      const int timeout_ms = env_rpc_timeout_s() * 1000;
      slot->layer = layer;
      slot->fut = std::async(std::launch::async, [fd, frame, frame_bytes, timeout_ms, reqid]() -> int64_t {
        if (!send_frame(fd, frame, frame_bytes, timeout_ms)) {
          throw KVTransferException(ErrorKind::TRANSPORT, "tcp send failed, errno=" + std::to_string(errno));
        }
        std::string resp;
        if (!recv_frame(fd, resp, timeout_ms)) throw KVTransferException(ErrorKind::TIMEOUT, "tcp ack timeout/closed");
        uint32_t magic = 0, status = WIRE_INTERNAL;
        uint64_t got = 0;
        int64_t us = 0;
        if (resp.size() >= RPC_HEADER + 4) {
          get_rpc_header(resp.data(), &magic, &got);
          memcpy(&status, resp.data() + RPC_HEADER, 4);
          if (resp.size() >= RPC_HEADER + 12) memcpy(&us, resp.data() + RPC_HEADER + 4, 8);
        }
        if (status != WIRE_OK || got != reqid) {
          throw KVTransferException(ErrorKind::TRANSPORT, "tcp receiver rejected the layer, status=" + std::to_string(status));
        }
        return us;
      });
      send_us_ += tw.get_elapse_us();
      return;
    }
    if (!ok) {
      active_ = false;
      throw KVTransferException(ErrorKind::TRANSPORT, std::string(name()) + " send failed, errno=" + std::to_string(errno));
    }
    pending_.push_back(Pending{reqid, &sock, layer});   // shm slots are distinct until the ring wraps
    send_us_ += tw.get_elapse_us();
  }

  void flush(std::string& out) override {
    TimeWatch tw;
    drain(0);
    for (auto& sl : slots_) wait_slot(*sl);
    std::ostringstream ss;
    ss << "Proto=" << name() << (cast_ ? ",Cast=bf16->e4m3" : "") << ",OriginSbNum=" << origin_blocks_ << ",MergedSbNum=" << merged_blocks_
       << ",SbSizeMin=" << (sb_min_ == SIZE_MAX ? 0 : sb_min_) << ",SbSizeMax=" << sb_max_ << ",SbSizeTotal=" << sb_total_
       << ",SendUs=" << send_us_ << ",D2HUs=" << gather_us_ << ",H2DUsMax=" << recv_us_max_
       << ",FlushUs=" << tw.get_elapse_us();
    out = ss.str();
    data_.clear();
  }

  // Between batches nothing is outstanding on the connections, so anything readable is the peer hanging up
  // (its process ended, or its server was stopped): the stub then builds a fresh channel, resolving the
  // destination again, before the next batch instead of failing that batch on a dead socket
  // (the role of XChannel::IsActive in kvtransfer/src/protocol/barex_protocol.cpp:701-711).
  bool is_active() override {
    if (!active_) return false;
    for (const auto& s : socks_) {
      struct pollfd p{s.fd(), POLLIN | POLLRDHUP, 0};
      if (::poll(&p, 1, 0) > 0 && (p.revents & (POLLIN | POLLRDHUP | POLLHUP | POLLERR)) != 0) {
        active_ = false;
        break;
      }
    }
    return active_;
  }

  void close() override {
    for (auto& sl : slots_) {
      try {
        if (sl->fut.valid()) sl->fut.get();   // the sender thread uses the socket and the buffer
      } catch (const std::exception&) {
      }
    }
    slots_.clear();
    socks_.clear();
    active_ = false;
    if (shm_base_ != nullptr) {
      if (shm_registered_) kvt_host_unregister_(shm_base_);
      munmap(shm_base_, shm_bytes_);
      shm_base_ = nullptr;
    }
    if (!shm_name_.empty()) {
      shm_unlink(shm_name_.c_str());
      shm_name_.clear();
    }
  }

 private:
  struct Pending {
    uint64_t reqid;
    FdGuard* sock;
    size_t layer;
  };
  struct TxSlot {
    PinnedBuffer buf;
    std::future<int64_t> fut;   // valid while a frame of this connection is unacknowledged
    size_t layer{0};
  };

  void wait_slot(TxSlot& sl) {
    if (!sl.fut.valid()) return;
    try {
      recv_us_max_ = std::max(recv_us_max_, sl.fut.get());
    } catch (const std::exception& ex) {
      active_ = false;
      throw KVTransferException(ErrorKind::TRANSPORT, std::string(ex.what()) + " (layer " + std::to_string(sl.layer) + ")");
    }
  }

  static void kvt_host_unregister_(char* p) { kvt_host_unregister(reinterpret_cast<uint64_t>(p)); }

  // Wait for acknowledgements until at most `keep` remain.
  void drain(size_t keep) {
    while (pending_.size() > keep) {
      Pending pd = pending_.front();
      pending_.erase(pending_.begin());
      std::string resp;
      if (!recv_frame(pd.sock->fd(), resp, env_rpc_timeout_s() * 1000)) {
        active_ = false;
        throw KVTransferException(ErrorKind::TIMEOUT, std::string(name()) + " ack timeout/closed for layer " +
                                                          std::to_string(pd.layer));
      }
      uint32_t magic = 0, status = WIRE_INTERNAL;
      uint64_t reqid = 0;
      int64_t us = 0;
      if (resp.size() >= RPC_HEADER + 4) {
        get_rpc_header(resp.data(), &magic, &reqid);
        memcpy(&status, resp.data() + RPC_HEADER, 4);
        if (resp.size() >= RPC_HEADER + 12) memcpy(&us, resp.data() + RPC_HEADER + 4, 8);
      }
      recv_us_max_ = std::max(recv_us_max_, us);
      if (status != WIRE_OK || reqid != pd.reqid) {
        active_ = false;
        throw KVTransferException(ErrorKind::TRANSPORT, std::string(name()) + " receiver rejected layer " +
                                                            std::to_string(pd.layer) + " status=" +
                                                            std::to_string(status));
      }
    }
  }

  void ensure_shm(size_t want) {
    want = std::max<size_t>(want, 1 << 20);
    want = (want + 4095) & ~size_t{4095};
    if (shm_base_ != nullptr && want <= shm_bytes_) return;
    if (shm_base_ != nullptr) {
      drain(0);
      if (shm_registered_) kvt_host_unregister_(shm_base_);
      munmap(shm_base_, shm_bytes_);
      shm_base_ = nullptr;
    }
    static std::atomic<int> seq{0};
    shm_name_ = "/kvx_" + std::to_string(getpid()) + "_" + std::to_string(seq.fetch_add(1));
    int fd = shm_open(shm_name_.c_str(), O_CREAT | O_RDWR | O_EXCL, 0600);
    if (fd < 0) throw KVTransferException(ErrorKind::TRANSPORT, "shm_open failed");
    if (ftruncate(fd, static_cast<off_t>(want)) != 0) {
      ::close(fd);
      shm_unlink(shm_name_.c_str());
      throw KVTransferException(ErrorKind::TRANSPORT, "shm ftruncate failed");
    }
    void* m = mmap(nullptr, want, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) throw KVTransferException(ErrorKind::TRANSPORT, "shm mmap failed");
    shm_base_ = static_cast<char*>(m);
    shm_bytes_ = want;
    shm_cursor_ = 0;
    shm_dev_ = 0;
    shm_registered_ = false;
    if (stage_ != nullptr) {
      uint64_t dev = 0;
      cuda_check(host_register(shm_base_, want, &dev), "cudaHostRegister(shm)");
      shm_dev_ = dev;
      shm_registered_ = true;
    }
    // Tell every connection's server thread to map the segment.  Whatever happens, the name goes away before this
    // function returns: the mappings keep the memory alive for as long as both sides use it, and a process that
    // dies (or never closes its channels) leaves nothing behind in /dev/shm.
    struct Unlink {
      std::string* name;
      ~Unlink() {
        shm_unlink(name->c_str());
        name->clear();
      }
    } unlink_on_exit{&shm_name_};
    for (auto& s : socks_) {
      std::string req(RPC_HEADER, '\0');
      const uint64_t reqid = new_id();
      put_rpc_header(req.data(), SHM_ATTACH_REQ, reqid);
      put(req, static_cast<uint32_t>(shm_name_.size()));
      req += shm_name_;
      put(req, static_cast<uint64_t>(want));
      std::string resp;
      uint32_t status = WIRE_INTERNAL;
      if (send_frame(s.fd(), req.data(), req.size(), env_rpc_timeout_s() * 1000) &&
          recv_frame(s.fd(), resp, env_rpc_timeout_s() * 1000) && resp.size() >= RPC_HEADER + 4) {
        memcpy(&status, resp.data() + RPC_HEADER, 4);
      }
      if (status != WIRE_OK) {
        active_ = false;
        throw KVTransferException(ErrorKind::TRANSPORT, "receiver could not attach shm segment " + std::string(shm_name_));
      }
    }
  }

  static int host_register(char* p, size_t bytes, uint64_t* dev) {
    return kvt_host_register(reinterpret_cast<uint64_t>(p), bytes, dev);
  }

  Context* ctx_;
  const bool use_shm_;
  WorkerInfo dst_;
  std::vector<FdGuard> socks_;
  size_t rr_{0};
  bool active_{false};
  std::unique_ptr<DeviceStage> stage_;
  std::vector<std::vector<IpcBlock>> data_;
  std::vector<size_t> blob_bytes_;
  bool cast_{false};   // gather casts bf16 -> e4m3 (descriptor lengths are fp8 bytes)
  std::vector<std::unique_ptr<TxSlot>> slots_;   // TCP: one frame buffer and one sender per connection
  std::string msg_buf_;
  std::vector<Pending> pending_;
  size_t origin_blocks_{0}, merged_blocks_{0}, sb_min_{0}, sb_max_{0}, sb_total_{0};
  int64_t send_us_{0}, gather_us_{0}, recv_us_max_{0};
  size_t inflight_bytes_{0};
  // shared memory
  std::string shm_name_;
  char* shm_base_{nullptr};
  size_t shm_bytes_{0};
  size_t shm_cursor_{0};
  uint64_t shm_dev_{0};
  bool shm_registered_{false};
};

}  // namespace

Channel make_tcp_channel(Context* ctx, bool use_shm) { return std::make_shared<HostChannel>(ctx, use_shm); }

}  // namespace kvx
