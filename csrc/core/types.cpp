#include "core/types.h"

#include <sstream>

namespace kvx {

void rtassert_fail(const char* file, int line, const char* expr, const std::string& detail) {
  std::ostringstream ss;
  ss << "RTASSERT failed: " << expr;
  if (!detail.empty()) ss << " (" << detail << ")";
  ss << " at " << file << ":" << line;
  LOG(ERROR) << ss.str();
  throw RtAssertError(ss.str());
}

std::string TransferProtocol::to_string() const {
  switch (type) {
    case RDMA_DIRECT: return "rdma";
    case TCP: return "tcp";
    case NVLINK: return "nvlink";
    case SHM: return "shm";
    default: return "unknown";
  }
}

TransferProtocol TransferProtocol::from_string(const std::string& s) {
  if (s == "rdma") return TransferProtocol(RDMA_DIRECT);
  if (s == "tcp") return TransferProtocol(TCP);
  if (s == "nvlink") return TransferProtocol(NVLINK);
  if (s == "shm") return TransferProtocol(SHM);
  return TransferProtocol(UNKNOWN);
}

static std::string join_sizes(const std::vector<size_t>& v) {
  std::string out;
  for (size_t i = 0; i < v.size(); ++i) {
    if (i) out.push_back('|');
    out += std::to_string(v[i]);
  }
  return out;
}

static std::vector<size_t> split_sizes(const std::string& s) {
  std::vector<size_t> out;
  size_t start = 0;
  while (start <= s.size()) {
    size_t pos = s.find('|', start);
    if (pos == std::string::npos) pos = s.size();
    if (pos > start) out.push_back(std::stoul(s.substr(start, pos - start)));
    start = pos + 1;
  }
  return out;
}

static bool all_digits(const std::string& s) {
  if (s.empty()) return false;
  for (char c : s)
    if (c < '0' || c > '9') return false;
  return true;
}

std::string WorkerInfo::to_string() const {
  if (inst_id.size() > MAX_INSTANCE_NAME_LEN) throw std::runtime_error("invalid worker instance name, too large;");
  std::ostringstream ss;
  ss << inst_id << ',' << worker_id << ',' << engine_tp_size << ',' << worker_tp_rank << ','
     << join_sizes(block_sizes) << ',' << join_sizes(token_sizes) << ',' << layer_num_blocks << ',' << num_layers
     << ',' << static_cast<uint32_t>(transfer_protocols) << ',' << attn_kernel_blk_ntpb << ',' << indexer_blk_ntpb
     << ',' << attn_pack_size << ',' << kda_page_stride;
  if (!addr.empty()) {
    if (addr.size() > MAX_ADDRESS_LEN) throw std::runtime_error("invalid worker address, too large;");
    ss << ',' << addr;
  }
  if (!ext.empty()) {
    ss << ",x:";
    bool first = true;
    for (const auto& kv : ext) {
      if (!first) ss << ';';
      first = false;
      ss << kv.first << '=' << kv.second;
    }
  }
  return ss.str();
}

WorkerInfo WorkerInfo::from_string(const std::string& src) {
  std::vector<std::string> f;
  size_t start = 0;
  for (;;) {
    size_t pos = src.find(',', start);
    if (pos == std::string::npos) {
      f.emplace_back(src.substr(start));
      break;
    }
    f.emplace_back(src.substr(start, pos - start));
    start = pos + 1;
  }
  WorkerInfo w;
  if (!f.empty() && f.back().rfind("x:", 0) == 0) {
    const std::string body = f.back().substr(2);
    f.pop_back();
    size_t s0 = 0;
    while (s0 < body.size()) {
      size_t e = body.find(';', s0);
      if (e == std::string::npos) e = body.size();
      const std::string kv = body.substr(s0, e - s0);
      const size_t eq = kv.find('=');
      if (eq != std::string::npos) w.ext[kv.substr(0, eq)] = kv.substr(eq + 1);
      s0 = e + 1;
    }
  }
  // 11: legacy, no attn_pack_size, no addr.  12: {…, addr} or {…, attn_pack_size}.
  // 13: {…, attn_pack_size, addr} or {…, attn_pack_size, kda_page_stride}.  14: all three.
  if (f.size() < 11 || f.size() > 14) throw std::runtime_error("invalid worker info string;");
  w.inst_id = f[0];
  w.worker_id = static_cast<uint32_t>(std::stoul(f[1]));
  w.engine_tp_size = static_cast<uint32_t>(std::stoul(f[2]));
  w.worker_tp_rank = static_cast<uint32_t>(std::stoul(f[3]));
  w.block_sizes = split_sizes(f[4]);
  w.token_sizes = split_sizes(f[5]);
  w.layer_num_blocks = static_cast<uint32_t>(std::stoul(f[6]));
  w.num_layers = static_cast<uint32_t>(std::stoul(f[7]));
  w.transfer_protocols = static_cast<uint8_t>(std::stoul(f[8]));
  w.attn_kernel_blk_ntpb = static_cast<uint32_t>(std::stoul(f[9]));
  w.indexer_blk_ntpb = static_cast<uint32_t>(std::stoul(f[10]));
  w.attn_pack_size = 1;
  w.kda_page_stride = 0;
  if (f.size() == 12) {
    if (all_digits(f[11])) w.attn_pack_size = static_cast<uint32_t>(std::stoul(f[11]));
    else w.addr = f[11];
  } else if (f.size() == 13) {
    w.attn_pack_size = static_cast<uint32_t>(std::stoul(f[11]));
    if (all_digits(f[12])) w.kda_page_stride = std::stoull(f[12]);
    else w.addr = f[12];
  } else if (f.size() == 14) {
    w.attn_pack_size = static_cast<uint32_t>(std::stoul(f[11]));
    w.kda_page_stride = std::stoull(f[12]);
    w.addr = f[13];
  }
  if (w.attn_pack_size == 0) w.attn_pack_size = 1;
  return w;
}

int WorkerInfo::ext_int(const std::string& key, int def) const {
  auto it = ext.find(key);
  if (it == ext.end() || it->second.empty()) return def;
  try {
    return std::stoi(it->second);
  } catch (const std::exception&) {
    return def;
  }
}

std::string WorkerInfo::ext_str(const std::string& key, const std::string& def) const {
  auto it = ext.find(key);
  return it == ext.end() ? def : it->second;
}

std::string block_ids_to_string(const BlockIds& ids) {
  std::string out = "[";
  for (size_t i = 0; i < ids.size(); ++i) {
    out.push_back('[');
    for (size_t j = 0; j < ids[i].size(); ++j) {
      out += std::to_string(ids[i][j]);
      if (j + 1 < ids[i].size()) out.push_back(',');
    }
    out.push_back(']');
    if (i + 1 < ids.size()) out.push_back(',');
  }
  out.push_back(']');
  return out;
}

uint64_t new_id() {
  static std::atomic<uint64_t> next{20181218};
  return next.fetch_add(1, std::memory_order_relaxed);
}

}  // namespace kvx
