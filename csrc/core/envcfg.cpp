#include "core/envcfg.h"

#include <arpa/inet.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

namespace kvx {

namespace {
// Process-lifetime state that worker threads (naming keep-alive, senders, servers) read until the very end of
// the process: allocated once and never destroyed, so that a thread still running while the main thread runs
// its exit handlers never touches a destroyed object.
std::mutex& g_mu = *new std::mutex;
std::map<std::string, long>& g_int_cache = *new std::map<std::string, long>;
std::map<std::string, double>& g_dbl_cache = *new std::map<std::string, double>;
bool g_quiet = getenv("BLLM_KVTRANS_QUIET_ENV") != nullptr;

void echo(const char* env, const char* val, const std::string& def) {
  if (g_quiet) return;
  fprintf(stderr, "kvtenv: env=%s val=%s def=%s\n", env, val == nullptr ? "NULL" : val, def.c_str());
  fflush(stdout);
}

// Positive integer env (values <= 0 fall back to the default).
long posint(const char* env, long def) {
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_int_cache.find(env);
  if (it != g_int_cache.end()) return it->second;
  const char* v = getenv(env);
  echo(env, v, std::to_string(def));
  long out = def;
  if (v != nullptr) {
    long parsed = atol(v);
    if (parsed > 0) out = parsed;
  }
  g_int_cache[env] = out;
  return out;
}

// Any integer env (including 0 and negatives).
long anyint(const char* env, long def) {
  std::lock_guard<std::mutex> g(g_mu);
  auto it = g_int_cache.find(env);
  if (it != g_int_cache.end()) return it->second;
  const char* v = getenv(env);
  echo(env, v, std::to_string(def));
  long out = def;
  if (v != nullptr && *v != '\0') out = atol(v);
  g_int_cache[env] = out;
  return out;
}

struct SendDoneAddr {
  bool parsed = false;
  bool valid = false;
  sockaddr_in addr{};
};
SendDoneAddr g_send_done;
std::vector<std::pair<uint64_t, int>>& g_reserve = *new std::vector<std::pair<uint64_t, int>>;
bool g_reserve_parsed = false;
std::string& g_nic = *new std::string;
bool g_nic_parsed = false;
}  // namespace

int env_heap_prof() { return (int)anyint("BLLM_KVTRANS_HEAP_PROF", 0); }
int env_send_parallel() { return (int)posint("BLLM_KVTRANS_RDMA_SP", 1); }
int env_ctx_tpsize() { return (int)posint("BLLM_KVTRANS_CTX_TPSIZE", 4); }
int env_conn_tpsize() { return (int)posint("BLLM_KVTRANS_CONN_TPSIZE", 4); }
int env_h2d_sync_tpsize() { return (int)posint("BLLM_KVTRANS_H2D_SYNC_TPSIZE", 4); }
int env_fsnaming_keepalive_interval_s() { return (int)posint("BLLM_KVTRANS_FSNAMING_KEEPALIVE_S", 3); }
int env_fsnaming_tolerate_interval_s() { return (int)posint("BLLM_KVTRANS_FSNAMING_TOLERATE_S", 9); }
int env_debug_tx_failrate() { return (int)posint("BLLM_KVTRANS_DEBUG_TX_FAILRATE", 1); }
int env_debug_tx_delay_ms() { return (int)posint("BLLM_KVTRANS_DEBUG_TX_DELAYMS", 1); }
int env_cache_shape() { return (int)posint("BLLM_KVTRANS_CACHE_SHAPE", RAGGED_FLASH_CACHE_SHAPE); }
int env_send_done_head_kind() { return (int)posint("BLLM_KVTRANS_SDH_KIND", SEND_SAVE_DONE_HEAD_KIND); }
int env_rpc_timeout_s() { return (int)posint("BLLM_KVTRANS_RPC_TIMEOUT_S", 7); }
int env_crc() { return (int)anyint("BLLM_KVTRANS_CRC", 0); }
int env_port_base() { return (int)posint("BLLM_KVTRANS_PORT_BASE", 31218); }
int env_send_tpsize() { return (int)posint("BLLM_KVTRANS_SEND_TPSIZE", 16); }
int env_txstub_cap() { return (int)posint("BLLM_KVTRANS_TXSTUB_CAP", 640); }
int env_waitlayer_tpsize() { return (int)posint("BLLM_KVTRANS_WAITLAYER_TPSIZE", 2); }
int env_shrink_tpsize() { return (int)posint("BLLM_KVTRANS_SHRINK_TPSIZE", 1); }
int env_attn_kernel_blk_size() { return (int)anyint("BLLM_KVTRANS_ATTN_KERNEL_BLK_SIZE", -1); }
size_t env_kernel_copy_max_block_num() noexcept { return (size_t)posint("BLLM_KVTRANS_KERNEL_COPY_MAX_BLOCK_NUM", 8192); }
bool env_bf162fp8_conversion() noexcept { return anyint("BLLM_KVTRANS_BF162FP8_CONV", 0) != 0; }
bool env_pad_last_attn_block() noexcept { return anyint("BLLM_KVTRANS_PAD_LAST_ATTN_BLOCK", 1) != 0; }
bool env_rdma_staged() noexcept { return anyint("BLLM_KVTRANS_RDMA_STAGED", 0) != 0; }
int env_nvlink_ctas() { return (int)anyint("BLLM_KVTRANS_NVLINK_CTAS", 0); }
int env_nvlink_streams() { return (int)posint("BLLM_KVTRANS_NVLINK_STREAMS", 8); }
int env_dst_mxfp8() { return (int)anyint("BLLM_KVTRANS_DST_MXFP8", 0); }
int env_use_tma() { return (int)anyint("BLLM_KVTRANS_USE_TMA", 1); }
int env_completion_timeout_ms() { return (int)posint("BLLM_KVTRANS_COMPLETION_TIMEOUT_MS", env_rpc_timeout_s() * 1000); }
int env_nvlink_pull() { return (int)anyint("BLLM_KVTRANS_NVLINK_PULL", 1); }
int env_nvlink_walk() { return (int)anyint("BLLM_KVTRANS_NVLINK_WALK", 1); }
int env_fanout_weak() { return (int)anyint("BLLM_KVTRANS_FANOUT_WEAK", 0); }
int env_walk_threads() { return (int)anyint("BLLM_KVTRANS_WALK_THREADS", 0); }
int env_walk_stages() { return (int)anyint("BLLM_KVTRANS_WALK_STAGES", 0); }
int env_tile_order() { return (int)anyint("BLLM_KVTRANS_TILE_ORDER", -1); }
int env_store_form() { return (int)anyint("BLLM_KVTRANS_STORE_FORM", -1); }
bool env_copy_profile_enable() { return anyint("BLLM_KVTRANS_COPY_PROFILE_ENABLE", 1) != 0; }
size_t env_copy_memcpy_max_blocks() { return (size_t)posint("BLLM_KVTRANS_COPY_MEMCPY_MAX_BLOCKS", 16); }
size_t env_copy_memcpy_threshold_bytes() { return (size_t)posint("BLLM_KVTRANS_COPY_MEMCPY_BLOCK_THRESHOLD_BYTES", 256 * 1024); }
bool env_device_timestamps() { return anyint("BLLM_KVTRANS_DEVICE_TIMESTAMPS", 0) != 0; }
int env_copy_path() { return (int)anyint("BLLM_KVTRANS_COPY_PATH", 0); }

double env_kernel_copy_sm_usage() noexcept {
  std::lock_guard<std::mutex> g(g_mu);
  const char* env = "BLLM_KVTRANS_KERNEL_COPY_SM_USAGE";
  auto it = g_dbl_cache.find(env);
  if (it != g_dbl_cache.end()) return it->second;
  const char* v = getenv(env);
  echo(env, v, "1.0");
  double out = 1.0;
  if (v != nullptr) {
    double parsed = atof(v);
    if (parsed > 0.0 && parsed <= 1.0) out = parsed;
  }
  g_dbl_cache[env] = out;
  return out;
}

const struct sockaddr_in* env_send_done_addr() {
  std::lock_guard<std::mutex> g(g_mu);
  if (!g_send_done.parsed) {
    g_send_done.parsed = true;
    const char* v = getenv("BLLM_KVTRANS_SEND_DONE_ADDR");
    echo("BLLM_KVTRANS_SEND_DONE_ADDR", v, "NULL");
    if (v != nullptr) {
      std::string s(v);
      auto pos = s.rfind(':');
      if (pos != std::string::npos) {
        std::string ip = s.substr(0, pos);
        int port = atoi(s.c_str() + pos + 1);
        memset(&g_send_done.addr, 0, sizeof(g_send_done.addr));
        g_send_done.addr.sin_family = AF_INET;
        g_send_done.addr.sin_port = htons((uint16_t)port);
        if (port > 0 && inet_pton(AF_INET, ip.c_str(), &g_send_done.addr.sin_addr) == 1) g_send_done.valid = true;
      }
    }
  }
  return g_send_done.valid ? &g_send_done.addr : nullptr;
}

// "4096,8000;8192,1000;" -> {(4096, 8000), (8192, 1000)}
const std::vector<std::pair<uint64_t, int>>* env_reserve() {
  std::lock_guard<std::mutex> g(g_mu);
  if (!g_reserve_parsed) {
    g_reserve_parsed = true;
    const char* v = getenv("BLLM_KVTRANS_RESERVE");
    echo("BLLM_KVTRANS_RESERVE", v, "");
    if (v != nullptr) {
      std::string s(v);
      size_t start = 0;
      while (start < s.size()) {
        size_t end = s.find(';', start);
        if (end == std::string::npos) end = s.size();
        std::string item = s.substr(start, end - start);
        auto comma = item.find(',');
        if (comma != std::string::npos) {
          uint64_t size = strtoull(item.substr(0, comma).c_str(), nullptr, 10);
          int cnt = atoi(item.substr(comma + 1).c_str());
          if (size > 0 && cnt > 0) g_reserve.emplace_back(size, cnt);
        }
        start = end + 1;
      }
    }
  }
  return &g_reserve;
}

const char* env_nic_name() noexcept {
  std::lock_guard<std::mutex> g(g_mu);
  if (!g_nic_parsed) {
    g_nic_parsed = true;
    const char* v = getenv("BLADE_KVT_NIC_NAME");
    echo("BLADE_KVT_NIC_NAME", v, "");
    if (v != nullptr) g_nic = v;
  }
  return g_nic.empty() ? nullptr : g_nic.c_str();
}

std::string envcfg_dump() {
  std::lock_guard<std::mutex> g(g_mu);
  std::string out;
  for (const auto& kv : g_int_cache) out += kv.first + "=" + std::to_string(kv.second) + "\n";
  for (const auto& kv : g_dbl_cache) out += kv.first + "=" + std::to_string(kv.second) + "\n";
  return out.empty() ? "(no setting read yet)\n" : out;
}

void envcfg_reset_for_test() {
  std::lock_guard<std::mutex> g(g_mu);
  g_int_cache.clear();
  g_dbl_cache.clear();
  g_send_done = SendDoneAddr{};
  g_reserve.clear();
  g_reserve_parsed = false;
  g_nic.clear();
  g_nic_parsed = false;
  g_quiet = getenv("BLLM_KVTRANS_QUIET_ENV") != nullptr;
}

}  // namespace kvx
