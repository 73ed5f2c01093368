// pybind11 bindings of the engine.  Module-level functions keep the names and argument order
// of the reference binding (kvtransfer/kvtransfer_pybind.cpp:415-522) and act on one
// process-global client / server, as there.  `KvClient` / `KvServer` expose the same engine as
// objects so that several workers can live in one process (tests, single-process demos).
#include <chrono>

#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "core/client.h"
#include "core/completion.h"
#include "core/envcfg.h"
#include "transport/copy_policy.h"
#include "transport/device_stage.h"
#include "core/gdr.h"
#include "core/monitor.h"
#include "core/fault_inject.h"
#include "kernels/kvt_kernels.h"
#include "naming/naming.h"
#include "plan/device_plan.h"
#include "plan/planner.h"
#include "topo/topology.h"
#include "transport/channel.h"
#include "transport/peer_memory.h"

namespace py = pybind11;

namespace kvx {

namespace {

struct HybridArgs {
  int num_kv_heads = -1;
  uint32_t num_gdn_layers = 3;
  uint32_t indexer_blk_ntpb = 0;
  uint32_t hybrid_indexer_token_size = 0;
  uint32_t gdn_conv_elem_size = 1;
  uint32_t gdn_ssm_elem_size = 1;
  std::vector<size_t> conv_state_shape, ssm_state_shape, gdn_conv_channel_dims;
  bool kda_conv_dim_first = false;
  uint32_t hybrid_attn_token_size = 0;
  uint64_t kda_page_stride = 0;
  uint32_t attn_pack_size = 1;
  uint32_t num_ple_layers = 0;
  uint32_t ple_block_group = 0;
  uint32_t ple_conv_elem_size = 1;
  std::vector<size_t> ple_conv_state_shape, ple_conv_channel_dims;
  // the worker's cache as a member of an NVLink multicast group: multicast address per [layer][tensor], group size
  std::vector<std::vector<uint64_t>> mc_layers;
  uint32_t mc_size = 0;
};

void apply_hybrid(WorkerInfo* wi, const HybridArgs& h) {
  wi->num_kv_heads = h.num_kv_heads;
  wi->num_gdn_layers = h.num_gdn_layers;
  wi->hybrid_indexer_token_size = h.hybrid_indexer_token_size;
  wi->gdn_conv_elem_size = h.gdn_conv_elem_size;
  wi->gdn_ssm_elem_size = h.gdn_ssm_elem_size;
  wi->conv_state_shape = h.conv_state_shape;
  wi->ssm_state_shape = h.ssm_state_shape;
  wi->gdn_conv_channel_dims = h.gdn_conv_channel_dims;
  wi->kda_conv_dim_first = h.kda_conv_dim_first;
  wi->hybrid_attn_token_size = h.hybrid_attn_token_size;
  wi->kda_page_stride = h.kda_page_stride;
  wi->num_ple_layers = h.num_ple_layers;
  wi->ple_block_group = h.ple_block_group;
  wi->ple_conv_elem_size = h.ple_conv_elem_size;
  wi->ple_conv_state_shape = h.ple_conv_state_shape;
  wi->ple_conv_channel_dims = h.ple_conv_channel_dims;
}

uint8_t protocol_mask(const std::vector<TransferProtocol>& protocols, int device_id) {
  uint8_t mask = 0;
  for (const auto& p : protocols) mask |= static_cast<uint8_t>(p.type);
  if (mask == 0) {
    mask = TransferProtocol::TCP | TransferProtocol::SHM;
    if (device_id >= 0) mask |= TransferProtocol::NVLINK;
  }
  return mask;
}

std::unique_ptr<Context> make_context(const std::string& inst, uint32_t tp_size, uint32_t worker_id,
                                      uint32_t worker_tp_rank, int device_id, const std::vector<size_t>& block_sizes,
                                      const std::vector<size_t>& token_sizes, uint32_t layer_num_blocks,
                                      const std::vector<std::vector<uint64_t>>& layers,
                                      const std::vector<TransferProtocol>& protocols, const HybridArgs& h,
                                      int cache_shape, bool mx_scaled) {
  RTASSERT(block_sizes.size() == token_sizes.size());
  auto ctx = std::make_unique<Context>(inst, worker_id);
  ctx->set_tp(tp_size, worker_tp_rank);
  WorkerInfo* wi = ctx->worker_info_mutable();
  // attn_pack_size must be known before set_block_params derives tokens-per-kernel-block
  wi->attn_pack_size = h.attn_pack_size == 0 ? 1 : h.attn_pack_size;
  std::vector<std::vector<LayerInfo>> infos;
  for (const auto& layer : layers) {
    RTASSERT(layer.size() == block_sizes.size());
    std::vector<LayerInfo> li;
    for (size_t t = 0; t < layer.size(); ++t) li.emplace_back(token_sizes[t], block_sizes[t], layer[t]);
    infos.push_back(std::move(li));
  }
  ctx->set_block_params(block_sizes, token_sizes, layer_num_blocks, h.indexer_blk_ntpb);
  ctx->set_layer_info(device_id, infos);
  apply_hybrid(wi, h);
  ctx->set_protocols(protocol_mask(protocols, device_id));
  const int shape = cache_shape > 0 ? cache_shape : env_cache_shape();
  wi->ext["shape"] = std::to_string(shape);
  if (mx_scaled) wi->ext["mx"] = "1";
  if (h.num_kv_heads > 0) {
    const int per_rank = static_cast<uint32_t>(h.num_kv_heads) >= tp_size ? h.num_kv_heads / static_cast<int>(tp_size) : 1;
    wi->ext["heads"] = std::to_string(per_rank);
  }
  wi->ext["dev"] = std::to_string(device_id);
  if (!h.mc_layers.empty() && h.mc_size > 1) {
    RTASSERT(h.mc_layers.size() == layers.size());
    for (size_t l = 0; l < layers.size(); ++l) RTASSERT(h.mc_layers[l].size() == layers[l].size());
    ctx->set_multicast_address(h.mc_layers);
    wi->ext["mcn"] = std::to_string(h.mc_size);     // senders may hand this worker a request for the whole group
  }
  return ctx;
}

class KvClient {
 public:
  KvClient(const std::string& inst, uint32_t tp_size, uint32_t worker_id, uint32_t worker_tp_rank, int device_id,
           std::vector<size_t> block_sizes, std::vector<size_t> token_sizes, uint32_t layer_num_blocks,
           const std::string& naming_url, const std::vector<uint64_t>& events,
           const std::vector<std::vector<uint64_t>>& layers, const std::vector<TransferProtocol>& protocols,
           const HybridArgs& h, int cache_shape, const std::string& send_done_addr = "") {
    auto ctx = make_context(inst, tp_size, worker_id, worker_tp_rank, device_id, block_sizes, token_sizes,
                            layer_num_blocks, layers, protocols, h, cache_shape, false);
    if (!send_done_addr.empty()) ctx->worker_info_mutable()->ext["sdaddr"] = send_done_addr;
    if (!events.empty()) {
      RTASSERT(events.size() == layers.size());
      ctx->set_cuda_barrier(std::make_unique<CudaEventBarrier>(events));
    }
    std::shared_ptr<INamingClient> naming;
    if (!naming_url.empty() && naming_url.rfind("fake", 0) != 0) {
      naming = NamingManager::instance().connect_naming(inst, naming_url);
    }
    Context* raw = ctx.get();
    auto factory = std::make_unique<KvSendStubFactory>(raw, naming);
    client_ = std::make_unique<KvTransferClient>(std::move(ctx), std::move(factory));
  }
  KvTransferClient* get() { return client_.get(); }

 private:
  std::unique_ptr<KvTransferClient> client_;
};

class KvServer {
 public:
  KvServer(const std::string& inst, uint32_t tp_size, uint32_t worker_id, uint32_t worker_tp_rank, int device_id,
           std::vector<size_t> block_sizes, std::vector<size_t> token_sizes, uint32_t layer_num_blocks,
           const std::string& naming_url, const std::vector<std::vector<uint64_t>>& layers,
           const std::vector<TransferProtocol>& protocols, const HybridArgs& h, int cache_shape, bool mx_scaled) {
    ctx_ = make_context(inst, tp_size, worker_id, worker_tp_rank, device_id, block_sizes, token_sizes,
                        layer_num_blocks, layers, protocols, h, cache_shape, mx_scaled);
    server_ = create_transfer_server();
    server_->start_server(ctx_.get());
    if (!naming_url.empty() && naming_url.rfind("fake", 0) != 0) {
      naming_ = NamingManager::instance().connect_naming(inst, naming_url);
      WorkerNamingClient(naming_).register_worker(ctx_->worker_info());
    }
    LOG(INFO) << "init_kv_transfer_server. worker_info=" << ctx_->worker_info().to_string();
  }
  ~KvServer() { stop(); }
  void stop() {
    if (server_) server_->stop();
  }
  std::string worker_info() const { return ctx_->worker_info().to_string(); }
  int port() const { return server_->port(); }
  Context* context() { return ctx_.get(); }

 private:
  std::unique_ptr<Context> ctx_;
  std::unique_ptr<ITransferServer> server_;
  std::shared_ptr<INamingClient> naming_;
};

std::unique_ptr<KvClient> g_client;
std::unique_ptr<KvServer> g_server;

KvTransferClient* need_client() {
  if (!g_client) throw KVTransferException(ErrorKind::INVALID_OPERATION, "kv client is not initialized");
  return g_client->get();
}

std::optional<WorkerInfo> parse_py_worker_info(const py::handle& h) {
  if (h.is_none()) return std::nullopt;
  if (py::isinstance<py::str>(h)) {
    const std::string s = h.cast<std::string>();
    if (s.empty()) return std::nullopt;
    return WorkerInfo::from_string(s);
  }
  throw py::type_error("dst_worker_info must be None or str");
}

HybridArgs hybrid_from_kwargs(const py::kwargs& kw) {
  HybridArgs h;
  auto geti = [&](const char* k, auto& dst) {
    if (kw.contains(k)) dst = kw[k].cast<std::decay_t<decltype(dst)>>();
  };
  geti("num_kv_heads", h.num_kv_heads);
  geti("num_gdn_layers", h.num_gdn_layers);
  geti("indexer_blk_ntpb", h.indexer_blk_ntpb);
  geti("hybrid_indexer_token_size", h.hybrid_indexer_token_size);
  geti("gdn_conv_elem_size", h.gdn_conv_elem_size);
  geti("gdn_ssm_elem_size", h.gdn_ssm_elem_size);
  geti("conv_state_shape", h.conv_state_shape);
  geti("ssm_state_shape", h.ssm_state_shape);
  geti("gdn_conv_channel_dims", h.gdn_conv_channel_dims);
  geti("kda_conv_dim_first", h.kda_conv_dim_first);
  geti("hybrid_attn_token_size", h.hybrid_attn_token_size);
  geti("kda_page_stride", h.kda_page_stride);
  geti("attn_pack_size", h.attn_pack_size);
  geti("num_ple_layers", h.num_ple_layers);
  geti("ple_block_group", h.ple_block_group);
  geti("ple_conv_elem_size", h.ple_conv_elem_size);
  geti("ple_conv_state_shape", h.ple_conv_state_shape);
  geti("ple_conv_channel_dims", h.ple_conv_channel_dims);
  geti("mc_layers", h.mc_layers);
  geti("mc_size", h.mc_size);
  return h;
}

void bind_worker_info(py::module_& m) {
  py::class_<WorkerInfo>(m, "WorkerInfo")
      .def(py::init<>())
      .def_static("from_string", &WorkerInfo::from_string)
      .def("to_string", &WorkerInfo::to_string)
      .def("__str__", &WorkerInfo::to_string)
      .def_readwrite("inst_id", &WorkerInfo::inst_id)
      .def_readwrite("worker_id", &WorkerInfo::worker_id)
      .def_readwrite("engine_tp_size", &WorkerInfo::engine_tp_size)
      .def_readwrite("worker_tp_rank", &WorkerInfo::worker_tp_rank)
      .def_readwrite("block_sizes", &WorkerInfo::block_sizes)
      .def_readwrite("token_sizes", &WorkerInfo::token_sizes)
      .def_readwrite("layer_num_blocks", &WorkerInfo::layer_num_blocks)
      .def_readwrite("num_layers", &WorkerInfo::num_layers)
      .def_readwrite("transfer_protocols", &WorkerInfo::transfer_protocols)
      .def_readwrite("attn_kernel_blk_ntpb", &WorkerInfo::attn_kernel_blk_ntpb)
      .def_readwrite("indexer_blk_ntpb", &WorkerInfo::indexer_blk_ntpb)
      .def_readwrite("attn_pack_size", &WorkerInfo::attn_pack_size)
      .def_readwrite("kda_page_stride", &WorkerInfo::kda_page_stride)
      .def_readwrite("addr", &WorkerInfo::addr)
      .def_readwrite("ext", &WorkerInfo::ext)
      .def_readwrite("num_kv_heads", &WorkerInfo::num_kv_heads)
      .def_readwrite("num_gdn_layers", &WorkerInfo::num_gdn_layers)
      .def_readwrite("hybrid_indexer_token_size", &WorkerInfo::hybrid_indexer_token_size)
      .def_readwrite("gdn_conv_elem_size", &WorkerInfo::gdn_conv_elem_size)
      .def_readwrite("gdn_ssm_elem_size", &WorkerInfo::gdn_ssm_elem_size)
      .def_readwrite("conv_state_shape", &WorkerInfo::conv_state_shape)
      .def_readwrite("ssm_state_shape", &WorkerInfo::ssm_state_shape)
      .def_readwrite("gdn_conv_channel_dims", &WorkerInfo::gdn_conv_channel_dims)
      .def_readwrite("num_ple_layers", &WorkerInfo::num_ple_layers)
      .def_readwrite("ple_block_group", &WorkerInfo::ple_block_group)
      .def_readwrite("ple_conv_elem_size", &WorkerInfo::ple_conv_elem_size)
      .def_readwrite("ple_conv_state_shape", &WorkerInfo::ple_conv_state_shape)
      .def_readwrite("ple_conv_channel_dims", &WorkerInfo::ple_conv_channel_dims)
      .def_readwrite("kda_conv_dim_first", &WorkerInfo::kda_conv_dim_first)
      .def_readwrite("hybrid_attn_token_size", &WorkerInfo::hybrid_attn_token_size);
}

// Planner exposed for tests and for Python-side transports (pinned store, migration):
// returns, per cache tensor, a list of (src_offset, dst_offset, length).
py::tuple py_plan(const WorkerInfo& src, const WorkerInfo& dst, int cache_shape,
                  const std::vector<std::tuple<std::string, uint32_t, uint32_t, bool, BlockIds, BlockIds>>& tasks,
                  bool cast_fp8, bool pad_last, bool merge) {
  PlanEnv env;
  env.src = &src;
  env.dst = &dst;
  env.cache_shape = cache_shape;
  env.cast_bf16_to_fp8 = cast_fp8;
  env.pad_last_attn_block = pad_last;
  PlannerChoice c = bind_planner(env);
  std::vector<std::vector<IpcBlock>> out;
  for (const auto& t : tasks) {
    auto info = std::make_shared<RequestInfo>(dst.inst_id, dst.worker_id, std::get<0>(t), std::get<4>(t), std::get<5>(t));
    ReqSendTask task(info, std::get<1>(t), std::get<2>(t), std::get<3>(t));
    plan_request(c, env, task, out);
  }
  py::list per_tensor;
  for (auto& v : out) {
    if (merge) merge_interval(v);
    py::list l;
    for (const auto& b : v) l.append(py::make_tuple(b.src_offset, b.dst_offset, b.length));
    per_tensor.append(l);
  }
  const char* kind = c.kind == TPKind::PEQD ? "PEQD" : (c.kind == TPKind::PGTD ? "PGTD" : "PLTD");
  return py::make_tuple(per_tensor, std::string(kind), env.valid_ranks.to_string(), env.kvt_tp_size, env.kvt_tp_rank);
}

// Host cost of planning one batch, without the conversion to Python objects: microseconds per call of
// (planner, then merge when asked), averaged over `iters` calls.
double py_plan_time_us(const WorkerInfo& src, const WorkerInfo& dst, int cache_shape,
                       const std::vector<std::tuple<std::string, uint32_t, uint32_t, bool, BlockIds, BlockIds>>& tasks,
                       bool merge, int iters) {
  PlanEnv env;
  env.src = &src;
  env.dst = &dst;
  env.cache_shape = cache_shape;
  PlannerChoice c = bind_planner(env);
  std::vector<ReqSendTask> reqs;
  for (const auto& t : tasks) {
    auto info = std::make_shared<RequestInfo>(dst.inst_id, dst.worker_id, std::get<0>(t), std::get<4>(t), std::get<5>(t));
    reqs.emplace_back(info, std::get<1>(t), std::get<2>(t), std::get<3>(t));
  }
  if (iters < 1) iters = 1;
  const auto t0 = std::chrono::steady_clock::now();
  size_t sink = 0;
  for (int i = 0; i < iters; ++i) {
    std::vector<std::vector<IpcBlock>> out;
    for (const auto& r : reqs) plan_request(c, env, r, out);
    for (auto& v : out) {
      if (merge) merge_interval(v);
      sink += v.size();
    }
  }
  const auto t1 = std::chrono::steady_clock::now();
  if (sink == static_cast<size_t>(-1)) throw std::runtime_error("unreachable");
  return std::chrono::duration<double, std::micro>(t1 - t0).count() / iters;
}

}  // namespace

void bind_engine(py::module_& m) {
  py::register_exception<KVTransferException>(m, "KVTransferError", PyExc_RuntimeError);
  py::register_exception<RtAssertError>(m, "KVTransferAssertError", PyExc_AssertionError);

  py::class_<TransferProtocol> protocol(m, "TransferProtocol");
  protocol.def(py::init<TransferProtocol::Kind>())
      .def_readwrite("type", &TransferProtocol::type)
      .def("to_string", &TransferProtocol::to_string)
      .def("__str__", &TransferProtocol::to_string)
      .def("__repr__", &TransferProtocol::to_string);
  py::enum_<TransferProtocol::Kind>(protocol, "Kind")
      .value("RDMA_DIRECT", TransferProtocol::RDMA_DIRECT)
      .value("TCP", TransferProtocol::TCP)
      .value("NVLINK", TransferProtocol::NVLINK)
      .value("SHM", TransferProtocol::SHM)
      .export_values();

  py::class_<ReqMeta>(m, "ReqMeta")
      .def(py::init<>())
      .def_readwrite("dst_inst", &ReqMeta::dst_inst)
      .def_readwrite("dst_worker", &ReqMeta::dst_worker)
      .def_readwrite("reqid", &ReqMeta::reqid)
      .def_readwrite("seen_tokens", &ReqMeta::seen_tokens)
      .def_readwrite("new_tokens", &ReqMeta::new_tokens)
      .def_readwrite("src_block_ids", &ReqMeta::src_block_ids)
      .def_readwrite("dst_block_ids", &ReqMeta::dst_block_ids)
      .def_property(
          "dst_worker_info",
          [](const ReqMeta& r) -> py::object {
            if (!r.dst_worker_info) return py::none();
            return py::str(r.dst_worker_info->to_string());
          },
          [](ReqMeta& r, const py::object& v) { r.dst_worker_info = parse_py_worker_info(v); });

  bind_worker_info(m);

  py::class_<INamingClient, std::shared_ptr<INamingClient>>(m, "NamingClient")
      .def("get", &INamingClient::get, py::call_guard<py::gil_scoped_release>())
      .def("search", &INamingClient::search, py::call_guard<py::gil_scoped_release>())
      .def("store", &INamingClient::store, py::call_guard<py::gil_scoped_release>())
      .def("remove", &INamingClient::remove, py::call_guard<py::gil_scoped_release>())
      .def("list", [](INamingClient& c) { return c.list(); }, py::call_guard<py::gil_scoped_release>())
      .def("get_schema", &INamingClient::get_schema)
      .def_readonly("inst_id", &INamingClient::inst_id);
  m.def("connect_naming", [](const std::string& name, const std::string& url) {
    return NamingManager::instance().connect_naming(name, url);
  }, py::call_guard<py::gil_scoped_release>());
  py::class_<KvStoreServer>(m, "KvStoreServer")
      .def(py::init<>())
      .def("start", &KvStoreServer::start, py::arg("port") = 0, py::call_guard<py::gil_scoped_release>())
      .def("stop", &KvStoreServer::stop, py::call_guard<py::gil_scoped_release>());
  m.def("parse_eas_document", [](const std::string& json) {
    int64_t v = -1;
    std::map<std::string, std::map<std::string, std::string>> doc;
    const bool ok = parse_eas_document(json, &v, &doc);
    return py::make_tuple(ok, v, doc);
  });

  // ---- object API ---------------------------------------------------------------------------
  py::class_<KvClient>(m, "KvClient")
      .def(py::init([](const std::string& inst, uint32_t tp, uint32_t wid, uint32_t rank, int dev,
                       std::vector<size_t> bs, std::vector<size_t> ts, uint32_t nblocks, const std::string& url,
                       const std::vector<uint64_t>& events, const std::vector<std::vector<uint64_t>>& layers,
                       const std::vector<TransferProtocol>& protocols, int cache_shape, const py::kwargs& kw) {
             HybridArgs h = hybrid_from_kwargs(kw);
             std::string sd;
             if (kw.contains("send_done_addr") && !kw["send_done_addr"].is_none()) sd = kw["send_done_addr"].cast<std::string>();
             py::gil_scoped_release rel;
             return std::make_unique<KvClient>(inst, tp, wid, rank, dev, std::move(bs), std::move(ts), nblocks, url,
                                               events, layers, protocols, h, cache_shape, sd);
           }),
           py::arg("inst_name"), py::arg("tp_size"), py::arg("worker_id"), py::arg("worker_tp_rank"),
           py::arg("device_id"), py::arg("block_sizes"), py::arg("token_sizes"), py::arg("layer_num_blocks"),
           py::arg("naming_url"), py::arg("events"), py::arg("layers"), py::arg("protocols"),
           py::arg("cache_shape") = -1)
      .def("submit_req_send2",
           [](KvClient& c, const std::string& dst_inst, uint32_t dst_worker, const std::string& reqid, uint32_t seen,
              uint32_t new_tokens, bool last, const BlockIds& src, const BlockIds& dst, const py::object& info,
              size_t stepid, uint32_t substepid, uint32_t fanout) {
             std::optional<std::string> s;
             if (!info.is_none()) s = info.cast<std::string>();
             c.get()->submit_req_send(dst_inst, dst_worker, reqid, seen, new_tokens, last, src, dst, s, stepid, substepid,
                                      fanout);
           },
           py::arg("dst_inst"), py::arg("dst_worker"), py::arg("reqid"), py::arg("seen_tokens"), py::arg("new_tokens"),
           py::arg("has_last_token"), py::arg("src_block_ids"), py::arg("dst_block_ids"),
           py::arg("dst_worker_info") = py::none(), py::arg("stepid") = 1024, py::arg("substepid") = 0,
           py::arg("fanout") = 0)
      .def("submit_delta_send",
           [](KvClient& c, const std::string& reqid, uint32_t seen, uint32_t new_tokens, bool last, size_t stepid,
              uint32_t substepid) { c.get()->submit_delta_send(reqid, seen, new_tokens, last, stepid, substepid); },
           py::arg("reqid"), py::arg("seen_tokens"), py::arg("new_tokens"), py::arg("has_last_token"),
           py::arg("stepid") = 1024, py::arg("substepid") = 0)
      .def("start_req_send",
           [](KvClient& c, std::vector<ReqMeta> metas, size_t stepid, uint32_t substepid) {
             c.get()->start_req_send(metas, stepid, substepid);
           },
           py::arg("metas"), py::arg("stepid") = 1024, py::arg("substepid") = 0)
      .def("start_send_substep",
           [](KvClient& c, size_t stepid, uint32_t substepid, std::vector<ReqMeta> metas) {
             c.get()->start_send_substep(stepid, substepid, metas);
           })
      .def("start_send", [](KvClient& c, size_t stepid, size_t sched) { return c.get()->start_send(stepid, sched); },
           py::arg("stepid") = 1024, py::arg("sched_tokens") = 1)
      .def("notify_event_record", [](KvClient& c, size_t stepid) { c.get()->notify_event_record(stepid); })
      .def("flush_send", [](KvClient& c, size_t stepid) { c.get()->flush_send(stepid); })
      .def("drain", [](KvClient& c) { c.get()->drain(); }, py::call_guard<py::gil_scoped_release>())
      .def("wait_inflight",
           [](KvClient& c, uint64_t max_batches, double timeout_s) {
             return c.get()->context()->inflight().wait_at_most(
                 max_batches, std::chrono::milliseconds(static_cast<int64_t>(timeout_s * 1000)));
           },
           py::arg("max_batches") = 0, py::arg("timeout_s") = 30.0, py::call_guard<py::gil_scoped_release>(),
           "Wait until at most max_batches batches are still in flight; False when the timeout ran out.")
      .def("inflight", [](KvClient& c) { return c.get()->context()->inflight().inflight(); })
      .def("finished_batches", [](KvClient& c) { return c.get()->context()->inflight().finished(); })
      .def("failed_batches", [](KvClient& c) { return c.get()->context()->inflight().failed(); })
      .def("target_size", [](KvClient& c) { return c.get()->target_size(); })
      .def("target_try_shrink", [](KvClient& c, size_t cap) { c.get()->target_try_shrink(cap); },
           py::call_guard<py::gil_scoped_release>())
      .def("worker_info", [](KvClient& c) { return c.get()->context()->worker_info().to_string(); });

  py::class_<KvServer>(m, "KvServer")
      .def(py::init([](const std::string& inst, uint32_t tp, uint32_t wid, uint32_t rank, int dev,
                       std::vector<size_t> bs, std::vector<size_t> ts, uint32_t nblocks, const std::string& url,
                       const std::vector<std::vector<uint64_t>>& layers,
                       const std::vector<TransferProtocol>& protocols, int cache_shape, bool mx_scaled,
                       const py::kwargs& kw) {
             HybridArgs h = hybrid_from_kwargs(kw);
             py::gil_scoped_release rel;
             return std::make_unique<KvServer>(inst, tp, wid, rank, dev, std::move(bs), std::move(ts), nblocks, url,
                                               layers, protocols, h, cache_shape, mx_scaled);
           }),
           py::arg("inst_name"), py::arg("tp_size"), py::arg("worker_id"), py::arg("worker_tp_rank"),
           py::arg("device_id"), py::arg("block_sizes"), py::arg("token_sizes"), py::arg("layer_num_blocks"),
           py::arg("naming_url"), py::arg("layers"), py::arg("protocols"), py::arg("cache_shape") = -1,
           py::arg("mx_scaled") = false)
      .def("worker_info", &KvServer::worker_info)
      .def("port", &KvServer::port)
      .def("stop", &KvServer::stop, py::call_guard<py::gil_scoped_release>());

  // ---- module-level API with the reference's names ---------------------------------------------
  m.def(
      "init_kv_transfer_client",
      [](const std::string& inst, uint32_t tp, uint32_t wid, uint32_t rank, int dev, std::vector<size_t> bs,
         std::vector<size_t> ts, uint32_t nblocks, const std::string& url, const std::vector<uint64_t>& events,
         const std::vector<std::vector<uint64_t>>& layers, const std::vector<TransferProtocol>& protocols,
         const py::kwargs& kw) {
        if (g_client) return;
        int cache_shape = -1;
        if (kw.contains("cache_shape")) cache_shape = kw["cache_shape"].cast<int>();
        HybridArgs h = hybrid_from_kwargs(kw);
        py::gil_scoped_release rel;
        g_client = std::make_unique<KvClient>(inst, tp, wid, rank, dev, std::move(bs), std::move(ts), nblocks, url,
                                              events, layers, protocols, h, cache_shape);
      },
      py::arg("inst_name"), py::arg("tp_size"), py::arg("worker_id"), py::arg("worker_tp_rank"), py::arg("device_id"),
      py::arg("block_sizes"), py::arg("token_sizes"), py::arg("layer_num_blocks"), py::arg("naming_url"),
      py::arg("events"), py::arg("layers"), py::arg("protocols"), "init kv transfer client;");
  m.def(
      "init_kv_transfer_server",
      [](const std::string& inst, uint32_t tp, uint32_t wid, uint32_t rank, int dev, std::vector<size_t> bs,
         std::vector<size_t> ts, uint32_t nblocks, const std::string& url,
         const std::vector<std::vector<uint64_t>>& layers, const std::vector<TransferProtocol>& protocols,
         const py::kwargs& kw) {
        if (g_server) return;
        int cache_shape = -1;
        bool mx = false;
        if (kw.contains("cache_shape")) cache_shape = kw["cache_shape"].cast<int>();
        if (kw.contains("mx_scaled")) mx = kw["mx_scaled"].cast<bool>();
        HybridArgs h = hybrid_from_kwargs(kw);
        py::gil_scoped_release rel;
        g_server = std::make_unique<KvServer>(inst, tp, wid, rank, dev, std::move(bs), std::move(ts), nblocks, url,
                                              layers, protocols, h, cache_shape, mx);
      },
      py::arg("inst_name"), py::arg("tp_size"), py::arg("worker_id"), py::arg("worker_tp_rank"), py::arg("device_id"),
      py::arg("block_sizes"), py::arg("token_sizes"), py::arg("layer_num_blocks"), py::arg("naming_url"),
      py::arg("layers"), py::arg("protocols"), "init kv transfer server;");
  m.def("shutdown_kv_transfer", [] {
    py::gil_scoped_release rel;
    if (g_client) g_client->get()->drain();
    g_client.reset();
    g_server.reset();
  });
  m.def("add_target", [](const std::string&, uint32_t, uint32_t, uint32_t, const py::object&) {
    // targets are created on demand from the requests; explicit registration is not supported
    // (the reference asserts here too, kvtransfer/src/client.cpp:243-254)
    throw KVTransferException(ErrorKind::INVALID_OPERATION, "add_target is not supported: targets are created lazily");
  });
  m.def(
      "submit_req_send2",
      [](const std::string& dst_inst, uint32_t dst_worker, const std::string& reqid, uint32_t seen, uint32_t new_tokens,
         bool last, const BlockIds& src, const BlockIds& dst, const py::object& info, size_t stepid,
         uint32_t substepid, uint32_t fanout) {
        std::optional<std::string> s;
        if (!info.is_none()) s = info.cast<std::string>();
        need_client()->submit_req_send(dst_inst, dst_worker, reqid, seen, new_tokens, last, src, dst, s, stepid,
                                       substepid, fanout);
      },
      py::arg("dst_inst"), py::arg("dst_worker"), py::arg("reqid"), py::arg("seen_tokens"), py::arg("new_tokens"),
      py::arg("has_last_token"), py::arg("src_block_ids"), py::arg("dst_block_ids"), py::arg("dst_worker_info") = py::none(),
      py::arg("stepid") = 1024, py::arg("substepid") = 0, py::arg("fanout") = 0, "submit kv send to kv client;");
  m.def("start_req_send", [](std::vector<ReqMeta> metas, size_t stepid, uint32_t substepid) {
    need_client()->start_req_send(metas, stepid, substepid);
  });
  m.def("submit_delta_send", [](const std::string& reqid, uint32_t seen, uint32_t new_tokens, bool last, size_t stepid,
                                uint32_t substepid) {
    need_client()->submit_delta_send(reqid, seen, new_tokens, last, stepid, substepid);
  });
  m.def("start_send", [](size_t stepid, size_t sched) { return need_client()->start_send(stepid, sched); });
  m.def("start_send_substep", [](size_t stepid, uint32_t substepid, std::vector<ReqMeta> metas) {
    need_client()->start_send_substep(stepid, substepid, metas);
  });
  m.def("notify_event_record", [](size_t stepid) { need_client()->notify_event_record(stepid); });
  m.def("flush_send", [](size_t stepid) { need_client()->flush_send(stepid); });
  m.def(
      "current_worker_info",
      [](const std::string& kind) -> std::string {
        if ((kind == "client" || kind == "any") && g_client) return g_client->get()->context()->worker_info().to_string();
        if ((kind == "server" || kind == "any") && g_server) return g_server->worker_info();
        return {};
      },
      py::arg("kind") = "any");
  m.def("lib_support_transfer_protocols", [] {
    std::vector<TransferProtocol> v{TransferProtocol(TransferProtocol::TCP), TransferProtocol(TransferProtocol::SHM)};
    if (kvt_device_count() > 0) v.emplace_back(TransferProtocol::NVLINK);
    return v;
  });

  // ---- planner / codecs / test hooks ------------------------------------------------------------
  m.def("compute_valid_ranks_pd", [](uint32_t p, uint32_t d, int heads) {
    return compute_valid_ranks_pd(p, d, heads).to_string();
  });
  // The same planner recording walk ops: what the NVLINK transport uploads for the device walk.
  py::class_<WalkPlan>(m, "WalkPlan")
      .def_property_readonly("n_ops", [](const WalkPlan& w) { return w.ops.size(); })
      .def_readonly("n_bulk", &WalkPlan::n_bulk)
      .def_readonly("n_simt", &WalkPlan::n_simt)
      .def_readonly("n_zero", &WalkPlan::n_zero)
      .def_readonly("bulk_units", &WalkPlan::bulk_units)
      .def_readonly("simt_units", &WalkPlan::simt_units)
      .def_readonly("zero_units", &WalkPlan::zero_units)
      .def_readonly("bytes", &WalkPlan::bytes)
      .def_property_readonly("pool_len", [](const WalkPlan& w) { return w.pool.size(); })
      .def_property_readonly("pool_offset", [](const WalkPlan& w) { return w.ops.size() * sizeof(KvtWalkOp); })
      .def("blob", [](const WalkPlan& w) {
        std::string b(w.ops.size() * sizeof(KvtWalkOp) + w.pool.size() * sizeof(uint32_t), '\0');
        if (!w.ops.empty()) memcpy(b.data(), w.ops.data(), w.ops.size() * sizeof(KvtWalkOp));
        if (!w.pool.empty()) memcpy(b.data() + w.ops.size() * sizeof(KvtWalkOp), w.pool.data(), w.pool.size() * sizeof(uint32_t));
        return py::bytes(b);
      }, "ops followed by the block-table pool, as uploaded to the device")
      .def("expand", [](const WalkPlan& w, const std::vector<uint64_t>& src_caps, const std::vector<uint64_t>& dst_caps) {
        py::list out;
        for (const WalkPiece& p : expand_walk_plan(w, src_caps, dst_caps))
          out.append(py::make_tuple(p.tensor, p.zero, p.src_offset, p.dst_offset, p.length));
        return out;
      }, "every piece the device walk moves: (tensor, zero_fill, src_offset, dst_offset, length)");
  m.def("plan_walk", [](const WorkerInfo& src, const WorkerInfo& dst, int cache_shape,
                        const std::vector<std::tuple<std::string, uint32_t, uint32_t, bool, BlockIds, BlockIds>>& tasks,
                        bool pad_last) {
    PlanEnv env;
    env.src = &src;
    env.dst = &dst;
    env.cache_shape = cache_shape;
    env.pad_last_attn_block = pad_last;
    PlannerChoice c = bind_planner(env);
    WalkPlan plan;
    for (const auto& t : tasks) {
      auto info = std::make_shared<RequestInfo>(dst.inst_id, dst.worker_id, std::get<0>(t), std::get<4>(t), std::get<5>(t));
      ReqSendTask task(info, std::get<1>(t), std::get<2>(t), std::get<3>(t));
      plan_request_ops(c, env, task, plan);
    }
    plan.finalize(src.layer_num_blocks, dst.layer_num_blocks);
    return plan;
  }, py::arg("src"), py::arg("dst"), py::arg("cache_shape"), py::arg("tasks"), py::arg("pad_last") = true);
  m.attr("KVT_WALK_OP_BYTES") = static_cast<int>(sizeof(KvtWalkOp));
  m.def("kvt_launch_walk", [](uint64_t src_ptrs, uint64_t dst_ptrs, uint32_t n_tensors, uint32_t layer_begin, uint32_t layer_end,
                              const std::vector<uint64_t>& src_caps, const std::vector<uint64_t>& dst_caps, uint64_t ops,
                              uint32_t n_bulk, uint32_t n_simt, uint64_t bulk_units, uint64_t simt_units, uint64_t pool,
                              uint32_t pool_len, uint64_t status, int grid, uint64_t stream) {
    if (n_tensors == 0 || n_tensors > KVT_WALK_MAX_TENSORS || src_caps.size() != n_tensors || dst_caps.size() != n_tensors)
      throw std::invalid_argument("kvt_launch_walk: 1..8 tensors with one capacity each");
    KvtWalkLaunch a{};
    a.src_ptrs = reinterpret_cast<const uint64_t*>(src_ptrs);
    a.dst_ptrs = reinterpret_cast<const uint64_t*>(dst_ptrs);
    a.n_tensors = n_tensors;
    a.layer_begin = layer_begin;
    a.layer_end = layer_end;
    for (uint32_t t = 0; t < n_tensors; ++t) {
      a.src_cap[t] = src_caps[t];
      a.dst_cap[t] = dst_caps[t];
    }
    a.ops = reinterpret_cast<const KvtWalkOp*>(ops);
    a.n_bulk_ops = n_bulk;
    a.n_simt_ops = n_simt;
    a.bulk_units = bulk_units;
    a.simt_units = simt_units;
    a.pool = reinterpret_cast<const uint32_t*>(pool);
    a.pool_len = pool_len;
    a.status = reinterpret_cast<uint32_t*>(status);
    const int e = kvt_launch_walk(&a, grid, reinterpret_cast<void*>(stream));
    if (e != 0) throw std::runtime_error(std::string("kvt_launch_walk: ") + kvt_error_string(e));
  }, py::arg("src_ptrs"), py::arg("dst_ptrs"), py::arg("n_tensors"), py::arg("layer_begin"), py::arg("layer_end"),
     py::arg("src_caps"), py::arg("dst_caps"), py::arg("ops"), py::arg("n_bulk"), py::arg("n_simt"), py::arg("bulk_units"),
     py::arg("simt_units"), py::arg("pool"), py::arg("pool_len"), py::arg("status"), py::arg("grid") = 0, py::arg("stream") = 0);
  m.def("plan_ipc_blocks", &py_plan, py::arg("src"), py::arg("dst"), py::arg("cache_shape"), py::arg("tasks"),
        py::arg("cast_fp8") = false, py::arg("pad_last") = true, py::arg("merge") = false);
  m.def("plan_time_us", &py_plan_time_us, py::arg("src"), py::arg("dst"), py::arg("cache_shape"), py::arg("tasks"),
        py::arg("merge") = true, py::arg("iters") = 100);
  m.def("merge_interval", [](std::vector<std::tuple<size_t, size_t, size_t>> v) {
    std::vector<IpcBlock> b;
    for (auto& t : v) b.emplace_back(std::get<0>(t), std::get<1>(t), std::get<2>(t));
    MergeStats st = merge_interval(b);
    py::list out;
    for (auto& x : b) out.append(py::make_tuple(x.src_offset, x.dst_offset, x.length));
    return py::make_tuple(out, st.min_len, st.max_len, st.total_len, st.count);
  });
  m.def("encode_send_done", [](uint32_t rank, const std::vector<std::tuple<std::string, uint32_t, bool>>& reqs,
                               int head_kind) {
    std::vector<std::shared_ptr<RequestInfo>> infos;
    std::vector<ReqSendTask> tasks;
    for (const auto& r : reqs) {
      infos.push_back(std::make_shared<RequestInfo>("d", 0, std::get<0>(r), BlockIds{}, BlockIds{}));
      infos.back()->set_state(std::get<2>(r) ? ReqState::OK : ReqState::FAILED);
      tasks.emplace_back(infos.back(), 0, std::get<1>(r), true);
    }
    std::vector<const ReqSendTask*> ptrs;
    for (auto& t : tasks) ptrs.push_back(&t);
    int resp = 0;
    auto buf = SendDoneNotifier::encode(rank, ptrs, head_kind, &resp);
    return py::make_tuple(py::bytes(buf.data(), buf.size()), resp);
  });
  m.def("fault_inject_arm", &fault_inject_arm);
  m.def("fault_inject_arm_drop_completion", &fault_inject_arm_drop_completion);
  m.def("fault_inject_arm_corrupt_check", &fault_inject_arm_corrupt_check);
  m.def("completions_pending", [] { return CompletionPoller::instance().pending(); });
  m.def("ipc_mappings_open", [] { return ipc_mappings_open(); },
        "Peer allocations this process has mapped through CUDA IPC handles right now.");
  m.def("envcfg_reset_for_test", &envcfg_reset_for_test);
  m.def("env_cache_shape", &env_cache_shape);
  m.def("env_port_base", &env_port_base);
  m.def("new_id", &new_id);
  m.def("monitor_start", &monitor_start, "start the process monitor; returns its TCP port");
  m.def("monitor_stop", &monitor_stop);
  m.def("monitor_port", &monitor_port);
  m.def("monitor_handle_line", &monitor_handle_line);
  m.def("envcfg_dump", &envcfg_dump);
  m.def("copy_policy_describe", [](int device) {
    py::gil_scoped_release nogil;
    return CopyPolicy::get(device).describe();
  }, py::arg("device"), "Copy policy of a device (measures at the first call unless the environment forces a path).");
  m.def("copy_policy_choose", [](const std::string& mode, int dir, size_t n, size_t total, size_t min_len) {
    return static_cast<int>(CopyPolicy::fixed(mode).choose(static_cast<CopyDir>(dir), n, total, min_len));
  }, py::arg("mode"), py::arg("dir"), py::arg("n"), py::arg("total_bytes"), py::arg("min_len"),
        "Decision (0 kernel, 1 memcpy) of a fixed policy: mode 'kernel', 'memcpy' or 'static'.");
  m.def("copy_policy_bucket", [](size_t n, size_t avg_len) {
    return std::make_pair(CopyPolicy::count_bucket(n), CopyPolicy::size_bucket(avg_len));
  });
  m.def("copy_policy_reset_for_test", &CopyPolicy::reset_for_test);
  m.def("copy_path_counters", []() {
    uint64_t a = 0, b = 0;
    copy_path_counters(&a, &b);
    return std::make_pair(a, b);
  }, "(descriptor lists moved by the copy engines, by the copy kernel) in this process.");
  m.def("gdr_available", [] {
    std::string why;
    const bool ok = gdr_available(&why);
    return py::make_tuple(ok, why);
  });
  m.def("crc32_bytes", [](py::bytes b, uint32_t seed) {
    const std::string s = b;
    return crc32_bytes(s.data(), s.size(), seed);
  }, py::arg("data"), py::arg("seed") = 0);
  m.def("discover_topology", [] { return discover_topology().to_json(); },
        "NVLink / NVSwitch topology of this process's visible GPUs as a JSON string");
  m.attr("EMPTY_STEP_ID") = EMPTY_STEP_ID;
  m.attr("MAX_TP_SIZE") = MAX_TP_SIZE;
}

}  // namespace kvx
