// NVLink transport: kernels on the prefill GPU store straight into the decode GPU's paged
// cache through peer-mapped memory (NVLink 5 / NVSwitch).  No staging buffer, no library copy.
//
// connect() asks the destination's server for the CUDA IPC handles of its layer tensors
// (MEM_HANDLES_REQ) and maps them; a destination in the same process is used by pointer after
// enabling peer access.  Two data paths share the channel:
//   * fused:   register_tasks() packs the requests' block tables; send_data(layer) launches
//              kvt_p2d_attn, which walks the tables, converts the layout (NHD<->HND), re-shards
//              heads for TP-mismatched pairs, optionally quantises to block-scaled e4m3 and
//              stores into the peer cache.  Serves cache shapes 1, 2 and 5 on either side.
//   * generic: register_data() takes the planner's IpcBlocks (any cache shape, including hybrid
//              GDN / MLA / KDA pages) and send_data(layer) runs the descriptor-driven copy
//              kernel from the local tensor into the peer tensor.
// The channel is device ordered: send_data(layer) makes its stream wait for the layer's CUDA
// event and returns; nothing on the host waits for the forward pass.  flush() waits for the
// transfer streams and turns a kernel status word into an exception.
// Only plain peer stores are used here; loads with cluster multicast are never issued.
#include <cuda_runtime.h>
#include <unistd.h>

#include <map>
#include <mutex>
#include <sstream>

#include "core/envcfg.h"
#include "core/fault_inject.h"
#include "core/util.h"
#include "kernels/kvt_kernels.h"
#include "plan/device_plan.h"
#include "transport/channel.h"
#include "transport/device_stage.h"
#include "transport/wire.h"

namespace kvx {

namespace {

// IPC mappings are per process; a handle must be opened once and shared by all channels.
struct IpcCache {
  std::mutex mu;
  std::map<std::pair<int32_t, uint64_t>, uint64_t> mapped;  // (pid, alloc_base) -> local address
};
IpcCache& ipc_cache() {
  static IpcCache c;
  return c;
}

template <typename T>
struct DevArray {
  T* p{nullptr};
  size_t n{0};
  ~DevArray() {
    if (p != nullptr) cudaFree(p);
  }
  void upload(const std::vector<T>& v) {
    if (p != nullptr) cudaFree(p);
    p = nullptr;
    n = v.size();
    if (n == 0) return;
    cuda_check(cudaMalloc(reinterpret_cast<void**>(&p), n * sizeof(T)), "cudaMalloc");
    cuda_check(cudaMemcpy(p, v.data(), n * sizeof(T), cudaMemcpyHostToDevice), "cudaMemcpy");
  }
};

struct alignas(64) TensorMapBytes {
  char b[128];
};

class NvlinkChannel : public IChannel {
 public:
  explicit NvlinkChannel(Context* ctx) : ctx_(ctx) {}
  ~NvlinkChannel() override { close(); }
  const char* name() const override { return "nvlink"; }
  bool device_ordered() const override { return true; }

  void connect(const WorkerInfo& dst) override {
    RTASSERT(ctx_->device_id() >= 0);
    dst_ = dst;
    fault_inject_throw();
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    // ---- fetch and map the destination's memory ------------------------------------------
    const std::string ip = dst.addr.empty() ? "127.0.0.1" : dst.addr;
    FdGuard sock(tcp_connect(ip, server_port_of(dst), env_rpc_timeout_s() * 1000));
    if (!sock.valid()) throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: cannot reach destination control port");
    std::string req(RPC_HEADER, '\0');
    put_rpc_header(req.data(), MEM_HANDLES_REQ, new_id());
    std::string resp;
    if (!send_frame(sock.fd(), req.data(), req.size(), env_rpc_timeout_s() * 1000) ||
        !recv_frame(sock.fd(), resp, env_rpc_timeout_s() * 1000) || resp.size() < RPC_HEADER + 4) {
      throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: memory-handle exchange failed");
    }
    uint32_t status = 0;
    memcpy(&status, resp.data() + RPC_HEADER, 4);
    PeerMemInfo info;
    if (status != WIRE_OK || !PeerMemInfo::parse(resp.data() + RPC_HEADER + 4, resp.size() - RPC_HEADER - 4, &info)) {
      throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: destination has no device memory to map");
    }
    if (info.host_id != this_host_id()) {
      throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: destination is on another host");
    }
    RTASSERT(info.num_layers == ctx_->num_layers());
    const bool same_process = info.pid == static_cast<int32_t>(getpid());
    dst_remote_ = info.device != ctx_->device_id();
    if (info.device != ctx_->device_id() && same_process) {
      if (!kvt_can_access_peer(ctx_->device_id(), info.device))
        throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: no peer access to the destination GPU");
      cuda_check(kvt_enable_peer_access(ctx_->device_id(), info.device), "cudaDeviceEnablePeerAccess");
    }
    dst_ptrs_.assign(info.num_layers, std::vector<uint64_t>(info.num_tensors, 0));
    for (uint32_t l = 0; l < info.num_layers; ++l) {
      for (uint32_t t = 0; t < info.num_tensors; ++t) {
        const PeerTensor& pt = info.tensors[static_cast<size_t>(l) * info.num_tensors + t];
        if (same_process) {
          dst_ptrs_[l][t] = pt.ptr;
          continue;
        }
        if (!pt.has_handle) throw KVTransferException(ErrorKind::TRANSPORT, "nvlink: destination tensor has no IPC handle");
        IpcCache& c = ipc_cache();
        std::lock_guard<std::mutex> g(c.mu);
        auto key = std::make_pair(info.pid, pt.alloc_base);
        auto it = c.mapped.find(key);
        if (it == c.mapped.end()) {
          uint64_t local = 0;
          cuda_check(kvt_ipc_open_handle(pt.ipc_handle, &local), "cudaIpcOpenMemHandle");
          it = c.mapped.emplace(key, local).first;
        }
        dst_ptrs_[l][t] = it->second + (pt.ptr - pt.alloc_base);
      }
    }
    // ---- streams -----------------------------------------------------------------------------
    const int n_streams = std::max(1, env_nvlink_streams());
    for (int i = 0; i < n_streams; ++i) stages_.emplace_back(std::make_unique<DeviceStage>(ctx_->device_id()));
    void* st = nullptr;
    cuda_check(cudaMalloc(&st, 64), "cudaMalloc(status)");
    cuda_check(cudaMemset(st, 0, 64), "cudaMemset");
    d_status_ = static_cast<uint32_t*>(st);
    h_status_.reserve(64, true);
    src_shape_ = ctx_->worker_info().cache_shape_or(env_cache_shape());
    dst_shape_ = dst.cache_shape_or(src_shape_);
    dst_mx_ = dst.ext_int("mx", env_dst_mxfp8()) != 0;
    active_ = true;
    LOG(INFO) << "nvlink channel connected. dst=" << dst.to_string() << " same_process=" << same_process
              << " src_shape=" << src_shape_ << " dst_shape=" << dst_shape_ << " dst_mx=" << dst_mx_;
  }

  bool register_tasks(const PlanEnv& env, const std::vector<const ReqSendTask*>& tasks) override {
    fused_ = false;
    generic_.clear();
    if (dst_ptrs_.empty() || dst_ptrs_[0].size() != 1) return false;
    PlanEnv e = env;
    e.cache_shape = src_shape_;
    PlannerChoice choice;
    try {
      choice = bind_planner(e);
    } catch (const std::exception&) {
      return false;
    }
    DeviceAttnParams p;
    std::string why;
    if (!device_attn_params(e, choice.kind, src_shape_, dst_shape_, dst_mx_, &p, &why)) {
      if (src_shape_ != dst_shape_ || dst_mx_) {
        throw KVTransferException(ErrorKind::INVALID_OPERATION,
                                  "nvlink: cross-layout / fp8 transfer needs the fused kernel but " + why);
      }
      return false;
    }
    params_ = p;
    if (p.skip) {
      plan_ = PackedPlan{};
      fused_ = true;
      return true;
    }
    plan_ = pack_device_plan(tasks, 0, p.tile_tokens, p.dst.ntpb, false);
    if (plan_.n_reqs == 0) {
      fused_ = true;
      return true;
    }
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    ensure_layer_arrays();
    // upload the plan on stream 0; the other streams wait for it
    cudaStream_t s0 = static_cast<cudaStream_t>(stages_[0]->stream());
    const size_t bytes = plan_.blob.size();
    if (bytes > d_plan_cap_) {
      if (d_plan_ != nullptr) cuda_check(cudaFree(d_plan_), "cudaFree");
      d_plan_cap_ = std::max<size_t>(bytes * 2, 1 << 16);
      cuda_check(cudaMalloc(reinterpret_cast<void**>(&d_plan_), d_plan_cap_), "cudaMalloc(plan)");
    }
    memcpy(h_plan_.reserve(bytes, true), plan_.blob.data(), bytes);
    cuda_check(cudaMemcpyAsync(d_plan_, h_plan_.data(), bytes, cudaMemcpyHostToDevice, s0), "cudaMemcpyAsync(plan)");
    if (plan_event_ == nullptr) {
      cudaEvent_t ev;
      cuda_check(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate");
      plan_event_ = ev;
    }
    stamp_start(s0);
    cuda_check(cudaEventRecord(static_cast<cudaEvent_t>(plan_event_), s0), "cudaEventRecord");
    begin_batch();
    fused_ = true;
    moved_bytes_per_layer_ = 0;
    for (const ReqSendTask* t : tasks)
      moved_bytes_per_layer_ += static_cast<size_t>(t->new_tokens) * 2 * p.n_heads * p.src.head_bytes;
    return true;
  }

  void register_data(std::vector<std::vector<IpcBlock>>& data, TPKind kind) override {
    if (env_bf162fp8_conversion() && kind == TPKind::PGTD) {
      throw KVTransferException(ErrorKind::INVALID_OPERATION,
                                "nvlink: the unscaled bf16->fp8 cast belongs to the host-staged transports; over NVLink an "
                                "fp8 decode cache is filled by the block-scaled quantiser (BLLM_KVTRANS_DST_MXFP8)");
    }
    fused_ = false;
    generic_.assign(data.size(), {});
    moved_bytes_per_layer_ = 0;
    origin_blocks_ = merged_blocks_ = 0;
    for (size_t t = 0; t < data.size(); ++t) {
      origin_blocks_ += data[t].size();
      validate_ipc_block_bounds(data[t], ctx_->tensor_capacity(t), IpcBlockOffset::SOURCE, "nvlink", 0, t);
      const MergeStats st = merge_interval(data[t]);
      merged_blocks_ += st.count;
      moved_bytes_per_layer_ += st.total_len;
      generic_[t].reserve(data[t].size());
      for (const auto& b : data[t]) generic_[t].push_back(Triple{b.src_offset, b.dst_offset, b.length});
    }
    data.clear();
    upload_generic();
  }

  // The descriptor lists are the same for every layer of the batch: upload them once (on stream 0,
  // the other streams wait for the upload) instead of once per layer.
  void upload_generic() {
    size_t total = 0;
    generic_off_.assign(generic_.size(), 0);
    generic_rounds_ = 1;
    for (size_t t = 0; t < generic_.size(); ++t) {
      generic_off_[t] = total;
      total += generic_[t].size();
      if (generic_[t].empty()) continue;
      uint64_t longest = 0;
      for (const Triple& tr : generic_[t]) longest = std::max<uint64_t>(longest, tr.len);
      generic_rounds_ = std::max(generic_rounds_, kvt_bulk_rounds(generic_[t][0].len, longest));
    }
    if (total == 0) return;
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    const size_t bytes = total * sizeof(Triple);
    if (bytes > d_plan_cap_) {
      for (auto& s : stages_) s->sync();   // nothing may still read the old buffer
      if (d_plan_ != nullptr) cuda_check(cudaFree(d_plan_), "cudaFree");
      d_plan_cap_ = std::max<size_t>(bytes * 2, 1 << 16);
      cuda_check(cudaMalloc(reinterpret_cast<void**>(&d_plan_), d_plan_cap_), "cudaMalloc(descriptors)");
    }
    char* h = h_plan_.reserve(bytes, true);
    for (size_t t = 0; t < generic_.size(); ++t)
      if (!generic_[t].empty()) memcpy(h + generic_off_[t] * sizeof(Triple), generic_[t].data(), generic_[t].size() * sizeof(Triple));
    cudaStream_t s0 = static_cast<cudaStream_t>(stages_[0]->stream());
    cuda_check(cudaMemcpyAsync(d_plan_, h, bytes, cudaMemcpyHostToDevice, s0), "cudaMemcpyAsync(descriptors)");
    if (plan_event_ == nullptr) {
      cudaEvent_t ev;
      cuda_check(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate");
      plan_event_ = ev;
    }
    stamp_start(s0);
    cuda_check(cudaEventRecord(static_cast<cudaEvent_t>(plan_event_), s0), "cudaEventRecord");
    begin_batch();
  }

  bool send_layers(size_t layer_begin, size_t layer_end, Step* step) override {
    (void)step;
    if (!fused_ || layer_end <= layer_begin) return false;
    if (plan_.n_reqs == 0) return true;
    // One launch saves ~100 us of launch and event overhead, which is what matters for a small
    // migration; a large one is faster layer by layer over several streams (measured crossover
    // around half a GiB).
    if (moved_bytes_per_layer_ * (layer_end - layer_begin) > (512ull << 20)) return false;
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    // one launch over the layer range on the stream that carried the plan; layer events are
    // recorded in order on one stream, so the last one implies the others
    DeviceStage& st = *stages_[0];
    st.wait_event(ctx_->cuda_barrier()->event(static_cast<uint32_t>(layer_end - 1)));
    launch_fused(layer_begin, layer_end, st);
    return true;
  }

  void launch_fused(size_t layer_begin, size_t layer_end, DeviceStage& st) {
    {
      KvtAttnLaunch a{};
      a.src_layers = d_src_layers_.p;
      a.dst_layers = d_dst_layers_.p;
      a.src_maps = use_tma_ ? d_src_maps_.p : nullptr;
      a.dst_maps = use_tma_ ? d_dst_maps_.p : nullptr;
      a.src = params_.src;
      a.dst = params_.dst;
      a.layer_begin = static_cast<uint32_t>(layer_begin);
      a.layer_end = static_cast<uint32_t>(layer_end);
      a.reqs = reinterpret_cast<const KvtReqDesc*>(d_plan_);
      a.n_reqs = plan_.n_reqs;
      a.total_tiles = plan_.total_tiles;
      a.block_ids = reinterpret_cast<const uint32_t*>(d_plan_ + plan_.pool_offset);
      a.tile_tokens = params_.tile_tokens;
      a.src_head0 = params_.src_head0;
      a.dst_head0 = params_.dst_head0;
      a.n_heads = params_.n_heads;
      a.mode = params_.mode;
      a.status = d_status_;
      a.dst_remote = dst_remote_ ? 1u : 0u;
      int grid = env_nvlink_ctas();
      // four small CTAs per SM, scaled by the SM-usage knob that bounds what a transfer may take from the forward pass
      if (grid <= 0) grid = std::max(1, static_cast<int>(4 * kvt_sm_count(ctx_->device_id()) * env_kernel_copy_sm_usage()));
      cuda_check(kvt_launch_p2d_attn(&a, grid, 0, use_tma_ ? 1 : 0, st.stream()), "kvt_launch_p2d_attn");
    }
  }

  void send_data(size_t layer, Step* step) override {
    (void)step;
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    DeviceStage& st = use_stage(layer % stages_.size());
    st.wait_event(ctx_->cuda_barrier()->event(static_cast<uint32_t>(layer)));
    if (fused_) {
      if (plan_.n_reqs != 0) launch_fused(layer, layer + 1, st);
      return;
    }
    const auto& addrs = ctx_->layer_data_address();
    RTASSERT(layer < addrs.size() && layer < dst_ptrs_.size());
    if (launch_generic_multi(layer, layer + 1, st)) return;
    for (size_t t = 0; t < generic_.size(); ++t) {
      if (generic_[t].empty()) continue;
      const size_t dst_cap = dst_.block_sizes.at(t) * static_cast<size_t>(dst_.layer_num_blocks);
      const uint64_t* d = reinterpret_cast<const uint64_t*>(d_plan_) + generic_off_[t] * 3;
      st.launch_resident(addrs[layer][t], dst_ptrs_[layer][t], d, generic_[t].size(), ctx_->tensor_capacity(t), dst_cap, 0,
                         d_status_);
    }
  }

  // Every tensor of layers [lo, hi) in one launch when they fit the kernel's entry table.
  bool launch_generic_multi(size_t lo, size_t hi, DeviceStage& st) {
    size_t per_layer = 0;
    for (const auto& g : generic_) per_layer += g.empty() ? 0 : 1;
    if (per_layer == 0) return true;
    if (per_layer * (hi - lo) > KVT_COPY_MAX_TENSORS) return false;
    const auto& addrs = ctx_->layer_data_address();
    KvtCopyMulti m{};
    uint32_t e = 0;
    for (size_t layer = lo; layer < hi; ++layer) {
      for (size_t t = 0; t < generic_.size(); ++t) {
        if (generic_[t].empty()) continue;
        m.src_base[e] = addrs[layer][t];
        m.dst_base[e] = dst_ptrs_[layer][t];
        m.src_cap[e] = ctx_->tensor_capacity(t);
        m.dst_cap[e] = dst_.block_sizes.at(t) * static_cast<uint64_t>(dst_.layer_num_blocks);
        m.first[e] = static_cast<uint32_t>(generic_off_[t]);
        m.count[e] = static_cast<uint32_t>(generic_[t].size());
        ++e;
      }
    }
    m.n_tensors = e;
    m.triples = reinterpret_cast<const uint64_t*>(d_plan_);
    m.status = d_status_;
    if (env_use_tma() != 0) {
      // pages are long 16-byte aligned runs: the TMA engine moves them, four CTAs per SM
      const int grid = std::max(1, static_cast<int>(4 * kvt_sm_count(ctx_->device_id()) * env_kernel_copy_sm_usage()));
      cuda_check(kvt_launch_copy_blocks_bulk(&m, generic_rounds_, grid, st.stream()), "kvt_launch_copy_blocks_bulk");
      return true;
    }
    const int grid = std::max(1, static_cast<int>(2 * kvt_sm_count(ctx_->device_id()) * env_kernel_copy_sm_usage()));
    cuda_check(kvt_launch_copy_blocks_multi(&m, grid, st.stream()), "kvt_launch_copy_blocks_multi");
    return true;
  }

  size_t send_range(size_t lo, size_t hi, Step* step) override {
    if (fused_ || hi <= lo + 1) {   // the fused kernel gains nothing from longer launches (measured)
      send_data(lo, step);
      return 1;
    }
    size_t per_layer = 0;
    for (const auto& g : generic_) per_layer += g.empty() ? 0 : 1;
    const size_t fit = per_layer == 0 ? hi - lo : KVT_COPY_MAX_TENSORS / per_layer;
    const size_t n = std::max<size_t>(1, std::min(hi - lo, fit));
    if (n == 1) {
      send_data(lo, step);
      return 1;
    }
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    const auto& addrs = ctx_->layer_data_address();
    RTASSERT(lo + n <= addrs.size() && lo + n <= dst_ptrs_.size());
    DeviceStage& st = use_stage((range_rr_++) % stages_.size());
    // layer events are recorded in order on one stream: the last of the range implies the others
    st.wait_event(ctx_->cuda_barrier()->event(static_cast<uint32_t>(lo + n - 1)));
    if (!launch_generic_multi(lo, lo + n, st)) {
      send_data(lo, step);
      return 1;
    }
    return n;
  }

  void flush(std::string& out) override {
    TimeWatch tw;
    cuda_check(cudaSetDevice(ctx_->device_id()), "cudaSetDevice");
    fault_inject_throw();
    {
      // one host wait for the batch: the other streams are joined into the first on the device, the
      // kernels' shared status words follow them, and the host waits for that copy alone
      cudaStream_t s0 = static_cast<cudaStream_t>(stages_[0]->stream());
      for (size_t i = 1; i < stages_.size() && i < stage_used_.size(); ++i)
        if (stage_used_[i]) stages_[0]->wait_event(stages_[i]->record_done());
      begin_batch();
      if (stamps_) cuda_check(kvt_launch_stamp(reinterpret_cast<uint64_t*>(d_status_) + 2, s0), "kvt_launch_stamp");
      cuda_check(cudaMemcpyAsync(h_status_.data(), d_status_, 24, cudaMemcpyDeviceToHost, s0), "cudaMemcpyAsync(status)");
      cuda_check(cudaStreamSynchronize(s0), "cudaStreamSynchronize");
      uint32_t st[2];
      memcpy(st, h_status_.data(), 8);
      if (stamps_) {
        uint64_t t[2];
        memcpy(t, h_status_.data() + 8, 16);
        device_us_ = t[1] >= t[0] ? static_cast<int64_t>((t[1] - t[0]) / 1000) : -1;
      }
      if (st[0] != 0) {
        cudaMemset(d_status_, 0, 64);
        throw KVTransferException(ErrorKind::CUDA, std::string(fused_ ? "transfer" : "copy") + " kernel reported status " +
                                                       std::to_string(st[0]) + " detail " + std::to_string(st[1]));
      }
    }
    std::ostringstream ss;
    ss << "Proto=nvlink,Path=" << (fused_ ? "fused" : "descriptors") << ",OriginSbNum=" << origin_blocks_
       << ",MergedSbNum=" << merged_blocks_ << ",BytesPerLayer=" << moved_bytes_per_layer_
       << ",Tiles=" << plan_.total_tiles << ",FlushUs=" << tw.get_elapse_us();
    if (stamps_) ss << ",DeviceUs=" << device_us_;   // GPU timer from the plan upload to the last kernel of the batch
    out = ss.str();
    generic_.clear();
  }

  bool is_active() override { return active_; }

  void close() override {
    if (!active_ && stages_.empty()) return;
    active_ = false;
    if (ctx_->device_id() >= 0) cudaSetDevice(ctx_->device_id());
    stages_.clear();
    if (d_status_ != nullptr) cudaFree(d_status_);
    d_status_ = nullptr;
    if (d_plan_ != nullptr) cudaFree(d_plan_);
    d_plan_ = nullptr;
    if (plan_event_ != nullptr) cudaEventDestroy(static_cast<cudaEvent_t>(plan_event_));
    plan_event_ = nullptr;
  }

 private:
  // Stream 0 carries the plan; another stream joins it (waits for the upload) when the batch first uses
  // it, and flush() joins back only the streams that were used: a batch of one launch makes no join at all.
  void begin_batch() { stage_used_.assign(stages_.size(), 0); }

  DeviceStage& use_stage(size_t i) {
    if (stage_used_.size() != stages_.size()) stage_used_.assign(stages_.size(), 0);
    if (i != 0 && !stage_used_[i]) {
      stages_[i]->wait_event(plan_event_);
      stage_used_[i] = 1;
    }
    return *stages_[i];
  }

  void stamp_start(cudaStream_t s0) {
    if (stamps_) cuda_check(kvt_launch_stamp(reinterpret_cast<uint64_t*>(d_status_) + 1, s0), "kvt_launch_stamp");
  }

  void ensure_layer_arrays() {
    if (d_src_layers_.p != nullptr) return;
    std::vector<uint64_t> src, dst;
    for (const auto& l : ctx_->layer_data_address()) src.push_back(l.at(0));
    for (const auto& l : dst_ptrs_) dst.push_back(l.at(0));
    d_src_layers_.upload(src);
    d_dst_layers_.upload(dst);
    use_tma_ = false;
    if (env_use_tma() != 0 && params_.mode == KVT_MODE_COPY) {
      std::vector<TensorMapBytes> sm(src.size()), dm(dst.size());
      bool ok = true;
      for (size_t i = 0; i < src.size() && ok; ++i) {
        ok = kvt_encode_tensor_map(sm[i].b, src[i], &params_.src, params_.n_heads, params_.tile_tokens) == 0 &&
             kvt_encode_tensor_map(dm[i].b, dst[i], &params_.dst, params_.n_heads, params_.tile_tokens) == 0;
      }
      if (ok) {
        d_src_maps_.upload(sm);
        d_dst_maps_.upload(dm);
        use_tma_ = true;
      } else {
        LOG(WARNING) << "nvlink: tensor maps not encodable for this layout, using the SIMT path";
      }
    }
  }

  Context* ctx_;
  WorkerInfo dst_;
  bool active_{false};
  std::vector<std::vector<uint64_t>> dst_ptrs_;
  std::vector<std::unique_ptr<DeviceStage>> stages_;
  int src_shape_{0}, dst_shape_{0};
  bool dst_mx_{false};
  // fused path
  bool fused_{false};
  bool use_tma_{false};
  DeviceAttnParams params_{};
  PackedPlan plan_;
  char* d_plan_{nullptr};
  size_t d_plan_cap_{0};
  PinnedBuffer h_plan_;
  void* plan_event_{nullptr};
  DevArray<uint64_t> d_src_layers_, d_dst_layers_;
  DevArray<TensorMapBytes> d_src_maps_, d_dst_maps_;
  size_t range_rr_{0};
  bool dst_remote_{false};       // the destination cache lives on another GPU
  std::vector<char> stage_used_;
  uint32_t generic_rounds_{1};   // bulk copy kernel: segment rounds the longest descriptor needs
  uint32_t* d_status_{nullptr};   // 64 bytes: [0] code, [1] detail, bytes 8..15 start stamp, bytes 16..23 end stamp
  const bool stamps_{env_device_timestamps()};
  int64_t device_us_{-1};
  PinnedBuffer h_status_;
  // generic path
  std::vector<std::vector<Triple>> generic_;
  std::vector<size_t> generic_off_;   // first descriptor of each tensor inside the uploaded buffer
  size_t origin_blocks_{0}, merged_blocks_{0}, moved_bytes_per_layer_{0};
};

}  // namespace

Channel make_nvlink_channel(Context* ctx) { return std::make_unique<NvlinkChannel>(ctx); }

Channel ChannelFactory::create(const WorkerInfo& dst) {
  const uint8_t mine = ctx_->worker_info().transfer_protocols;
  const uint8_t theirs = dst.transfer_protocols;
  auto both = [&](TransferProtocol::Kind k) { return (mine & k) != 0 && (theirs & k) != 0; };
  const std::string host = dst.ext_str("host");
  const bool same_host = !host.empty() && host == std::to_string(this_host_id());
  TransferProtocol::Kind pick = TransferProtocol::UNKNOWN;
  if (proto_.has_value()) {
    pick = proto_->type;
  } else if (both(TransferProtocol::NVLINK) && same_host && ctx_->device_id() >= 0 && dst.ext_int("dev", -1) >= 0) {
    pick = TransferProtocol::NVLINK;
  } else if (both(TransferProtocol::SHM) && same_host) {
    pick = TransferProtocol::SHM;
  } else if (both(TransferProtocol::TCP)) {
    pick = TransferProtocol::TCP;
  }
  Channel ch;
  switch (pick) {
    case TransferProtocol::NVLINK: ch = make_nvlink_channel(ctx_); break;
    case TransferProtocol::SHM: ch = make_tcp_channel(ctx_, true); break;
    case TransferProtocol::TCP: ch = make_tcp_channel(ctx_, false); break;
    default:
      throw KVTransferException(ErrorKind::TRANSPORT, "no transfer protocol in common with " + dst.to_string());
  }
  ch->connect(dst);
  return ch;
}

}  // namespace kvx
