#include "naming/naming.h"

#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>

#include "core/envcfg.h"

namespace kvx {

namespace fs = std::filesystem;

static long unix_now() {
  return std::chrono::duration_cast<std::chrono::seconds>(std::chrono::system_clock::now().time_since_epoch()).count();
}

// ---- file system ---------------------------------------------------------------------------
FileSysNaming::~FileSysNaming() {
  stop_.store(true);
  if (keepalive_.joinable()) keepalive_.join();
}

void FileSysNaming::connect(const Schema&, const std::string& path) {
  if (!fs::exists(path) || !fs::is_directory(path)) throw std::runtime_error("parent directory not exist: " + path);
  root_ = path;
  mine_ = root_ / inst_id;
  std::error_code ec;
  fs::create_directories(mine_, ec);
  write_file("_timestamp_", std::to_string(unix_now()));
  if (!keepalive_.joinable()) {
    keepalive_ = std::thread([this] {
      // sleep in short slices so that destruction does not wait a whole interval
      long waited_ms = 0;
      while (!stop_.load(std::memory_order_relaxed)) {
        std::this_thread::sleep_for(std::chrono::milliseconds(50));
        waited_ms += 50;
        if (waited_ms >= 1000L * env_fsnaming_keepalive_interval_s()) {
          waited_ms = 0;
          try {
            write_file("_timestamp_", std::to_string(unix_now()));
          } catch (const std::exception& ex) {
            LOG(WARNING) << "file naming keep-alive failed: " << ex.what();
          }
        }
      }
    });
  }
}

void FileSysNaming::store(const std::string& k, const std::string& v) {
  if (k.find('/') != std::string::npos) throw std::runtime_error("unsupported key format: " + k);
  write_file(k, v);
}

void FileSysNaming::remove(const std::string& key) {
  if (std::remove((mine_ / key).c_str()) != 0) throw std::runtime_error("failed to remove file: " + key);
}

static std::optional<std::string> first_line(const fs::path& p) {
  std::ifstream in(p);
  if (!in) return std::nullopt;
  std::string line;
  std::getline(in, line);
  if (line.empty()) return std::nullopt;
  return line;
}

std::optional<std::string> FileSysNaming::get(const InstanceId& inst, const std::string& k) {
  const fs::path dir = root_ / inst;
  std::error_code ec;
  if (!fs::is_directory(dir, ec)) return std::nullopt;
  return first_line(dir / k);
}

std::vector<std::string> FileSysNaming::search(const InstanceId& inst, const std::string& prefix) {
  std::vector<std::string> out;
  const fs::path dir = root_ / inst;
  std::error_code ec;
  if (!fs::is_directory(dir, ec)) return out;
  for (const auto& entry : fs::directory_iterator(dir, ec)) {
    const std::string name = entry.path().filename().string();
    if (name.rfind(prefix, 0) == 0 && name.find(".tmp") == std::string::npos) {
      auto v = first_line(entry.path());
      if (v.has_value()) out.push_back(std::move(*v));
    }
  }
  return out;
}

const std::vector<std::string>& FileSysNaming::list() {
  std::lock_guard<std::mutex> g(list_mu_);
  const auto now_tp = SteadyClock::now();
  if (!list_cache_.empty() && elapse_us(list_at_, now_tp) < 2000 * 1000) return list_cache_;
  list_cache_.clear();
  std::error_code ec;
  const long now = unix_now();
  const long tolerate = env_fsnaming_tolerate_interval_s();
  for (const auto& entry : fs::directory_iterator(root_, ec)) {
    if (!entry.is_directory(ec)) continue;
    const std::string inst = entry.path().filename().string();
    auto ts = get(inst, "_timestamp_");
    if (!ts.has_value()) continue;
    try {
      const long last = std::stol(*ts);
      if (last >= now || now - last < tolerate) list_cache_.push_back(inst);
    } catch (const std::exception& e) {
      LOG(WARNING) << "invalid timestamp: " << *ts << ", " << e.what();
    }
  }
  list_at_ = now_tp;
  return list_cache_;
}

void FileSysNaming::write_file(const std::string& name, const std::string& content) {
  // temp file + rename: a reader never sees a half-written value
  const std::string full = (mine_ / name).string();
  std::string tmpl = full + ".tmpXXXXXX";
  std::vector<char> buf(tmpl.begin(), tmpl.end());
  buf.push_back('\0');
  int fd = mkstemp(buf.data());
  if (fd < 0) throw std::runtime_error("FileSysNaming.write_file: mkstemp failed. err=" + std::string(strerror(errno)));
  const std::string line = content + "\n";
  ssize_t w = ::write(fd, line.data(), line.size());
  ::close(fd);
  if (w != static_cast<ssize_t>(line.size()) || rename(buf.data(), full.c_str()) != 0) {
    ::unlink(buf.data());
    throw std::runtime_error("FileSysNaming.write_file: write/rename failed. err=" + std::string(strerror(errno)));
  }
}

// ---- in-process -----------------------------------------------------------------------------
namespace {
// never destroyed: clients on other threads may outlive the main thread's exit handlers
std::mutex& g_mem_mu = *new std::mutex;
using MemSpaces = std::map<std::string, std::map<std::string, std::map<std::string, std::string>>>;   // space -> inst -> kv
MemSpaces& g_mem = *new MemSpaces;
}  // namespace

void MemNaming::store(const std::string& k, const std::string& v) {
  std::lock_guard<std::mutex> g(g_mem_mu);
  g_mem[space_][inst_id][k] = v;
}
void MemNaming::remove(const std::string& key) {
  std::lock_guard<std::mutex> g(g_mem_mu);
  g_mem[space_][inst_id].erase(key);
}
std::optional<std::string> MemNaming::get(const InstanceId& inst, const std::string& k) {
  std::lock_guard<std::mutex> g(g_mem_mu);
  auto& sp = g_mem[space_];
  auto it = sp.find(inst);
  if (it == sp.end()) return std::nullopt;
  auto kv = it->second.find(k);
  if (kv == it->second.end()) return std::nullopt;
  return kv->second;
}
std::vector<std::string> MemNaming::search(const InstanceId& inst, const std::string& prefix) {
  std::lock_guard<std::mutex> g(g_mem_mu);
  std::vector<std::string> out;
  auto& sp = g_mem[space_];
  auto it = sp.find(inst);
  if (it == sp.end()) return out;
  for (const auto& kv : it->second)
    if (kv.first.rfind(prefix, 0) == 0) out.push_back(kv.second);
  return out;
}
const std::vector<std::string>& MemNaming::list() {
  std::lock_guard<std::mutex> g(g_mem_mu);
  list_cache_.clear();
  for (const auto& kv : g_mem[space_]) list_cache_.push_back(kv.first);
  return list_cache_;
}

// ---- TCP key/value store ----------------------------------------------------------------------
namespace {
bool send_msg(int fd, uint8_t op, const std::string& k, const std::string& v) {
  std::string m;
  m.push_back(static_cast<char>(op));
  uint32_t kl = static_cast<uint32_t>(k.size()), vl = static_cast<uint32_t>(v.size());
  m.append(reinterpret_cast<const char*>(&kl), 4);
  m += k;
  m.append(reinterpret_cast<const char*>(&vl), 4);
  m += v;
  return write_full(fd, m.data(), m.size(), 5000) == static_cast<ssize_t>(m.size());
}
bool recv_msg(int fd, uint8_t* op, std::string* k, std::string* v, int timeout_ms) {
  uint32_t kl = 0, vl = 0;
  if (read_full(fd, op, 1, timeout_ms) != 1) return false;
  if (read_full(fd, &kl, 4, 5000) != 4 || kl > (1u << 20)) return false;
  k->resize(kl);
  if (kl && read_full(fd, k->data(), kl, 5000) != static_cast<ssize_t>(kl)) return false;
  if (read_full(fd, &vl, 4, 5000) != 4 || vl > (1u << 26)) return false;
  v->resize(vl);
  if (vl && read_full(fd, v->data(), vl, 5000) != static_cast<ssize_t>(vl)) return false;
  return true;
}
}  // namespace

int KvStoreServer::start(int port) {
  int bound = 0;
  int fd = tcp_listen("0.0.0.0", port, 64, &bound);
  if (fd < 0) throw std::runtime_error("KvStoreServer: cannot listen");
  listen_ = FdGuard(fd);
  stop_.store(false);
  accept_ = std::thread([this] {
    while (!stop_.load()) {
      struct pollfd p{listen_.fd(), POLLIN, 0};
      if (::poll(&p, 1, 100) <= 0) continue;
      int c = ::accept4(listen_.fd(), nullptr, nullptr, SOCK_CLOEXEC);
      if (c < 0) continue;
      std::lock_guard<std::mutex> g(mu_);
      fds_.push_back(c);
      conns_.emplace_back([this, c] { serve(c); });
    }
  });
  return bound;
}

void KvStoreServer::stop() {
  if (stop_.exchange(true)) return;
  if (accept_.joinable()) accept_.join();
  std::vector<std::thread> t;
  {
    std::lock_guard<std::mutex> g(mu_);
    for (int f : fds_) ::shutdown(f, SHUT_RDWR);
    t.swap(conns_);
  }
  for (auto& th : t)
    if (th.joinable()) th.join();
  listen_.reset();
}

void KvStoreServer::serve(int fd) {
  FdGuard guard(fd);
  for (;;) {
    uint8_t op = 0;
    std::string k, v;
    if (!recv_msg(fd, &op, &k, &v, 0)) return;
    std::string out;
    uint8_t rc = 0;
    {
      std::lock_guard<std::mutex> g(mu_);
      if (op == 1) {
        kv_[k] = v;
      } else if (op == 2) {
        auto it = kv_.find(k);
        if (it != kv_.end()) {
          rc = 1;
          out = it->second;
        }
      } else if (op == 3) {
        kv_.erase(k);
      } else if (op == 4) {
        for (auto it = kv_.lower_bound(k); it != kv_.end() && it->first.rfind(k, 0) == 0; ++it) {
          out += it->first;
          out.push_back('\0');
          out += it->second;
          out.push_back('\0');
        }
      }
    }
    if (!send_msg(fd, rc, "", out)) return;
  }
}

void TcpStoreNaming::connect(const Schema&, const std::string& path) {
  auto pos = path.rfind(':');
  if (pos == std::string::npos) throw std::runtime_error("tcpstore naming url must be tcpstore:<ip>:<port>");
  ip_ = path.substr(0, pos);
  port_ = atoi(path.c_str() + pos + 1);
  store("_timestamp_", std::to_string(unix_now()));
}

std::string TcpStoreNaming::rpc(uint8_t op, const std::string& key, const std::string& val, bool* found) {
  std::lock_guard<std::mutex> g(mu_);
  for (int attempt = 0; attempt < 2; ++attempt) {
    if (!sock_.valid()) sock_ = FdGuard(tcp_connect(ip_, port_, 3000));
    if (!sock_.valid()) continue;
    uint8_t rc = 0;
    std::string k, v;
    if (send_msg(sock_.fd(), op, key, val) && recv_msg(sock_.fd(), &rc, &k, &v, 5000)) {
      if (found != nullptr) *found = rc == 1;
      return v;
    }
    sock_.reset();  // stale connection: reconnect once
  }
  throw KVTransferException(ErrorKind::NAMING, "tcpstore naming: server unreachable at " + ip_ + ":" + std::to_string(port_));
}

void TcpStoreNaming::store(const std::string& k, const std::string& v) { rpc(1, inst_id + "/" + k, v, nullptr); }
void TcpStoreNaming::remove(const std::string& key) { rpc(3, inst_id + "/" + key, "", nullptr); }
std::optional<std::string> TcpStoreNaming::get(const InstanceId& inst, const std::string& k) {
  bool found = false;
  std::string v = rpc(2, inst + "/" + k, "", &found);
  if (!found) return std::nullopt;
  return v;
}
static std::vector<std::pair<std::string, std::string>> split_pairs(const std::string& blob) {
  std::vector<std::pair<std::string, std::string>> out;
  size_t p = 0;
  while (p < blob.size()) {
    size_t e1 = blob.find('\0', p);
    if (e1 == std::string::npos) break;
    size_t e2 = blob.find('\0', e1 + 1);
    if (e2 == std::string::npos) break;
    out.emplace_back(blob.substr(p, e1 - p), blob.substr(e1 + 1, e2 - e1 - 1));
    p = e2 + 1;
  }
  return out;
}
std::vector<std::string> TcpStoreNaming::search(const InstanceId& inst, const std::string& prefix) {
  std::vector<std::string> out;
  for (auto& kv : split_pairs(rpc(4, inst + "/" + prefix, "", nullptr))) out.push_back(std::move(kv.second));
  return out;
}
const std::vector<std::string>& TcpStoreNaming::list() {
  auto pairs = split_pairs(rpc(4, "", "", nullptr));
  list_cache_.clear();
  for (const auto& kv : pairs) {
    const auto pos = kv.first.find("/_timestamp_");
    if (pos != std::string::npos && pos + 12 == kv.first.size()) list_cache_.push_back(kv.first.substr(0, pos));
  }
  return list_cache_;
}

// ---- EAS (HTTP/JSON) ----------------------------------------------------------------------------
namespace {
class SocketHttpClient : public IHttpClient {
 public:
  std::optional<std::string> get(const std::string& host, int port, const std::string& path) override {
    FdGuard s(tcp_connect(host, port, 3000));
    if (!s.valid()) return std::nullopt;
    const std::string req = "GET " + path + " HTTP/1.0\r\nHost: " + host + "\r\nConnection: close\r\n\r\n";
    if (write_full(s.fd(), req.data(), req.size(), 3000) != static_cast<ssize_t>(req.size())) return std::nullopt;
    std::string resp;
    char buf[4096];
    for (;;) {
      struct pollfd p{s.fd(), POLLIN, 0};
      if (::poll(&p, 1, 5000) <= 0) break;
      ssize_t r = ::recv(s.fd(), buf, sizeof(buf), 0);
      if (r <= 0) break;
      resp.append(buf, static_cast<size_t>(r));
      if (resp.size() > (64u << 20)) return std::nullopt;
    }
    const auto hdr_end = resp.find("\r\n\r\n");
    if (hdr_end == std::string::npos || resp.compare(0, 5, "HTTP/") != 0) return std::nullopt;
    const auto sp = resp.find(' ');
    if (sp == std::string::npos || resp.compare(sp + 1, 3, "200") != 0) return std::nullopt;
    return resp.substr(hdr_end + 4);
  }
};

struct JsonCursor {
  const std::string& s;
  size_t i{0};
  void ws() {
    while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i;
  }
  bool eat(char c) {
    ws();
    if (i < s.size() && s[i] == c) {
      ++i;
      return true;
    }
    return false;
  }
  bool str(std::string* out) {
    ws();
    if (i >= s.size() || s[i] != '"') return false;
    ++i;
    out->clear();
    while (i < s.size() && s[i] != '"') {
      if (s[i] == '\\' && i + 1 < s.size()) {
        ++i;
        switch (s[i]) {
          case 'n': out->push_back('\n'); break;
          case 't': out->push_back('\t'); break;
          default: out->push_back(s[i]);
        }
      } else {
        out->push_back(s[i]);
      }
      ++i;
    }
    if (i >= s.size()) return false;
    ++i;
    return true;
  }
  bool integer(int64_t* v) {
    ws();
    size_t st = i;
    if (i < s.size() && (s[i] == '-' || s[i] == '+')) ++i;
    while (i < s.size() && s[i] >= '0' && s[i] <= '9') ++i;
    if (i == st) return false;
    *v = std::stoll(s.substr(st, i - st));
    return true;
  }
};
}  // namespace

std::unique_ptr<IHttpClient> make_socket_http_client() { return std::make_unique<SocketHttpClient>(); }

bool parse_eas_document(const std::string& json, int64_t* version,
                        std::map<std::string, std::map<std::string, std::string>>* out) {
  JsonCursor c{json};
  out->clear();
  *version = -1;
  if (!c.eat('{')) return false;
  if (c.eat('}')) return true;
  do {
    std::string key;
    if (!c.str(&key) || !c.eat(':')) return false;
    if (key == "version") {
      if (!c.integer(version)) return false;
    } else if (key == "instances") {
      if (!c.eat('{')) return false;
      if (!c.eat('}')) {
        do {
          std::string inst;
          if (!c.str(&inst) || !c.eat(':') || !c.eat('{')) return false;
          auto& kv = (*out)[inst];
          if (!c.eat('}')) {
            do {
              std::string k, v;
              if (!c.str(&k) || !c.eat(':') || !c.str(&v)) return false;
              kv[k] = v;
            } while (c.eat(','));
            if (!c.eat('}')) return false;
          }
        } while (c.eat(','));
        if (!c.eat('}')) return false;
      }
    } else {
      // skip a scalar we do not know
      std::string dummy;
      int64_t n;
      if (!c.str(&dummy) && !c.integer(&n)) return false;
    }
  } while (c.eat(','));
  return c.eat('}');
}

void EasNaming::connect(const Schema&, const std::string& path) {
  // host:port/path
  auto slash = path.find('/');
  std::string hp = slash == std::string::npos ? path : path.substr(0, slash);
  path_ = slash == std::string::npos ? "/" : path.substr(slash);
  auto colon = hp.rfind(':');
  host_ = colon == std::string::npos ? hp : hp.substr(0, colon);
  port_ = colon == std::string::npos ? 80 : atoi(hp.c_str() + colon + 1);
  std::lock_guard<std::mutex> g(mu_);
  refresh();
}

void EasNaming::refresh() {
  const auto now = SteadyClock::now();
  if (version_ >= 0 && elapse_us(fetched_at_, now) < 1000 * 1000) return;
  fetched_at_ = now;
  auto body = http_->get(host_, port_, path_);
  if (!body.has_value()) {
    LOG(WARNING) << "eas naming: fetch failed, keeping version " << version_;
    return;
  }
  // cheap version probe before a full parse
  int64_t v = -1;
  std::map<std::string, std::map<std::string, std::string>> doc;
  if (!parse_eas_document(*body, &v, &doc)) {
    LOG(WARNING) << "eas naming: malformed document ignored";
    return;
  }
  if (v == version_ && v >= 0) return;
  version_ = v;
  doc_.swap(doc);
}

void EasNaming::store(const std::string& k, const std::string& v) {
  std::lock_guard<std::mutex> g(mu_);
  overlay_[k] = v;
}
void EasNaming::remove(const std::string& key) {
  std::lock_guard<std::mutex> g(mu_);
  overlay_.erase(key);
}
std::optional<std::string> EasNaming::get(const InstanceId& inst, const std::string& k) {
  std::lock_guard<std::mutex> g(mu_);
  if (inst == inst_id) {
    auto it = overlay_.find(k);
    if (it != overlay_.end()) return it->second;
  }
  refresh();
  auto it = doc_.find(inst);
  if (it == doc_.end()) return std::nullopt;
  auto kv = it->second.find(k);
  if (kv == it->second.end()) return std::nullopt;
  return kv->second;
}
std::vector<std::string> EasNaming::search(const InstanceId& inst, const std::string& prefix) {
  std::lock_guard<std::mutex> g(mu_);
  refresh();
  std::vector<std::string> out;
  auto it = doc_.find(inst);
  if (it == doc_.end()) return out;
  for (const auto& kv : it->second)
    if (kv.first.rfind(prefix, 0) == 0) out.push_back(kv.second);
  return out;
}
const std::vector<std::string>& EasNaming::list() {
  std::lock_guard<std::mutex> g(mu_);
  refresh();
  list_cache_.clear();
  for (const auto& kv : doc_) list_cache_.push_back(kv.first);
  return list_cache_;
}

// ---- manager -----------------------------------------------------------------------------------
NamingManager& NamingManager::instance() {
  static NamingManager& m = *new NamingManager;   // never destroyed (see g_mem)
  return m;
}

std::shared_ptr<INamingClient> NamingManager::connect_naming(const InstanceId& myname, const std::string& url) {
  const auto pos = url.find(':');
  if (pos == std::string::npos) throw std::runtime_error("invalid naming url: " + url);
  const std::string schema = url.substr(0, pos);
  std::string path = url.substr(pos + 1);
  while (path.rfind("//", 0) == 0) path = path.substr(2);
  std::lock_guard<std::mutex> g(mu_);
  const std::string key = myname + "@" + url;
  auto it = clients_.find(key);
  if (it != clients_.end()) return it->second;
  std::shared_ptr<INamingClient> c;
  if (schema == "file") c = std::make_shared<FileSysNaming>(myname);
  else if (schema == "mem") c = std::make_shared<MemNaming>(myname);
  else if (schema == "tcpstore") c = std::make_shared<TcpStoreNaming>(myname);
  else if (schema == "eas") c = std::make_shared<EasNaming>(myname, make_socket_http_client());
  else throw std::runtime_error("unsupported naming schema: " + schema);
  c->connect(schema, path);
  clients_[key] = c;
  return c;
}

}  // namespace kvx
