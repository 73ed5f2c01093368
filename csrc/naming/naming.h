// Naming / discovery: where workers publish their WorkerInfo and find each other's.
//
// Interface and key scheme follow the reference (kvtransfer/include/naming.h:18-97): a client
// is bound to one instance id, stores key/value pairs under it, reads any instance's keys and
// lists live instances; a worker is published under "worker_{id}".  Back ends by URL schema:
//   file:<dir>            directory per instance, atomic tmp+rename writes, "_timestamp_"
//                         keep-alive, liveness = age below BLLM_KVTRANS_FSNAMING_TOLERATE_S
//                         (kvtransfer/src/filesys_naming.cpp:15-161)
//   tcpstore:<ip>:<port>  a small TCP key/value store (the reference wraps c10d::TCPStore,
//                         kvtransfer/src/tcpstore_naming.cpp:27-71; this engine has no torch
//                         dependency and ships its own server, KvStoreServer)
//   eas:<ip>:<port>/<path> HTTP/JSON service with a versioned cache (kvtransfer/src/eas_naming.cpp)
//   mem:<name>            in-process map (tests)
//   fake:                 no service: the destination WorkerInfo travels inside each request
#pragma once
#include <atomic>
#include <filesystem>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <shared_mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "core/types.h"
#include "core/util.h"

namespace kvx {

typedef std::string Schema;

class INamingClient {
 public:
  const InstanceId inst_id;
  explicit INamingClient(InstanceId n) : inst_id(std::move(n)) {}
  virtual Schema get_schema() = 0;
  virtual void connect(const Schema& schema, const std::string& path) = 0;
  virtual void store(const std::string& k, const std::string& v) = 0;
  virtual void remove(const std::string& key) = 0;
  virtual std::optional<std::string> get(const InstanceId& inst, const std::string& k) = 0;
  virtual std::vector<std::string> search(const InstanceId& inst, const std::string& prefix) = 0;
  virtual const std::vector<std::string>& list() = 0;
  virtual ~INamingClient() = default;
};

class INamingWorkerClient {
 public:
  virtual void register_worker(const WorkerInfo& w) = 0;
  virtual std::optional<WorkerInfo> get_worker_info(const InstanceId& inst, WorkerId wid) = 0;
  virtual ~INamingWorkerClient() = default;
};

// Publishes / resolves workers through a key/value naming client under "worker_{id}".
class WorkerNamingClient : public INamingWorkerClient {
 public:
  explicit WorkerNamingClient(std::shared_ptr<INamingClient> c) : client_(std::move(c)) {}
  void register_worker(const WorkerInfo& w) override { client_->store("worker_" + std::to_string(w.worker_id), w.to_string()); }
  std::optional<WorkerInfo> get_worker_info(const InstanceId& inst, WorkerId wid) override {
    auto v = client_->get(inst, "worker_" + std::to_string(wid));
    if (!v.has_value()) return std::nullopt;
    return WorkerInfo::from_string(*v);
  }

 private:
  std::shared_ptr<INamingClient> client_;
};

// Destination info carried by the request itself (fake:// naming).
class FakeNamingWorkerClient : public INamingWorkerClient {
 public:
  explicit FakeNamingWorkerClient(WorkerInfo info) : info_(std::move(info)) {}
  void register_worker(const WorkerInfo&) override {}
  std::optional<WorkerInfo> get_worker_info(const InstanceId&, WorkerId) override { return info_; }

 private:
  WorkerInfo info_;
};

class FileSysNaming : public INamingClient {
 public:
  explicit FileSysNaming(const InstanceId& n) : INamingClient(n) {}
  ~FileSysNaming() override;
  Schema get_schema() override { return "file"; }
  void connect(const Schema& schema, const std::string& path) override;
  void store(const std::string& k, const std::string& v) override;
  void remove(const std::string& key) override;
  std::optional<std::string> get(const InstanceId& inst, const std::string& k) override;
  std::vector<std::string> search(const InstanceId& inst, const std::string& prefix) override;
  const std::vector<std::string>& list() override;

 private:
  void write_file(const std::string& name, const std::string& content);
  std::filesystem::path root_, mine_;
  std::thread keepalive_;
  std::atomic<bool> stop_{false};
  std::mutex list_mu_;
  std::vector<std::string> list_cache_;
  Timepoint list_at_{};
};

class MemNaming : public INamingClient {
 public:
  explicit MemNaming(const InstanceId& n) : INamingClient(n) {}
  Schema get_schema() override { return "mem"; }
  void connect(const Schema&, const std::string& path) override { space_ = path; }
  void store(const std::string& k, const std::string& v) override;
  void remove(const std::string& key) override;
  std::optional<std::string> get(const InstanceId& inst, const std::string& k) override;
  std::vector<std::string> search(const InstanceId& inst, const std::string& prefix) override;
  const std::vector<std::string>& list() override;

 private:
  std::string space_;
  std::vector<std::string> list_cache_;
};

// Tiny TCP key/value store.  Requests are frames "[u8 op][u32 klen][key][u32 vlen][value]";
// ops: 1 set, 2 get, 3 delete, 4 list-keys-with-prefix.  Keys are "inst/key".
class KvStoreServer {
 public:
  KvStoreServer() = default;
  ~KvStoreServer() { stop(); }
  int start(int port);  // returns the bound port
  void stop();

 private:
  void serve(int fd);
  FdGuard listen_;
  std::thread accept_;
  std::vector<std::thread> conns_;
  std::atomic<bool> stop_{true};
  std::mutex mu_;
  std::map<std::string, std::string> kv_;
  std::vector<int> fds_;
};

class TcpStoreNaming : public INamingClient {
 public:
  explicit TcpStoreNaming(const InstanceId& n) : INamingClient(n) {}
  Schema get_schema() override { return "tcpstore"; }
  void connect(const Schema& schema, const std::string& path) override;  // "ip:port"
  void store(const std::string& k, const std::string& v) override;
  void remove(const std::string& key) override;
  std::optional<std::string> get(const InstanceId& inst, const std::string& k) override;
  std::vector<std::string> search(const InstanceId& inst, const std::string& prefix) override;
  const std::vector<std::string>& list() override;

 private:
  std::string rpc(uint8_t op, const std::string& key, const std::string& val, bool* found);
  std::mutex mu_;
  std::string ip_;
  int port_{0};
  FdGuard sock_;
  std::vector<std::string> list_cache_;
};

// HTTP fetch used by the EAS naming client; replaceable in tests.
class IHttpClient {
 public:
  virtual ~IHttpClient() = default;
  // Returns the body of GET http://host:port/path, or nullopt.
  virtual std::optional<std::string> get(const std::string& host, int port, const std::string& path) = 0;
};
std::unique_ptr<IHttpClient> make_socket_http_client();

// EAS-style discovery: GET returns {"version": N, "instances": {"<inst>": {"<key>": "<value>", ...}, ...}}.
// The document is cached and only re-parsed when the version changes; store() is not supported by
// the service (instances are registered out of band), so it keeps a local overlay.
class EasNaming : public INamingClient {
 public:
  EasNaming(const InstanceId& n, std::unique_ptr<IHttpClient> http) : INamingClient(n), http_(std::move(http)) {}
  Schema get_schema() override { return "eas"; }
  void connect(const Schema& schema, const std::string& path) override;  // "host:port/path"
  void store(const std::string& k, const std::string& v) override;
  void remove(const std::string& key) override;
  std::optional<std::string> get(const InstanceId& inst, const std::string& k) override;
  std::vector<std::string> search(const InstanceId& inst, const std::string& prefix) override;
  const std::vector<std::string>& list() override;
  int64_t version() const { return version_; }

 private:
  void refresh();
  std::unique_ptr<IHttpClient> http_;
  std::string host_, path_;
  int port_{80};
  std::mutex mu_;
  int64_t version_{-1};
  Timepoint fetched_at_{};
  std::map<std::string, std::map<std::string, std::string>> doc_;
  std::map<std::string, std::string> overlay_;
  std::vector<std::string> list_cache_;
};

class NamingManager {
 public:
  // url = "<schema>:<path>".  Clients are cached per (instance, url).
  std::shared_ptr<INamingClient> connect_naming(const InstanceId& myname, const std::string& url);
  static NamingManager& instance();

 private:
  std::mutex mu_;
  std::unordered_map<std::string, std::shared_ptr<INamingClient>> clients_;
};

// Minimal JSON reader for the EAS document (objects, strings, integers).
bool parse_eas_document(const std::string& json, int64_t* version,
                        std::map<std::string, std::map<std::string, std::string>>* out);

}  // namespace kvx
