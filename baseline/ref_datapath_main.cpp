// Harness around the UNMODIFIED reference data path, for the reference arm of bench.py.
//
// The reference cannot be built as a package here (closed transport library), but the code that
// moves the bytes on one box can: its own ParseBlock generator for the FLASH / NHD cache shape
// (kvtransfer/src/parse_block_flash.cpp) produces the IpcBlocks, and its own copy kernels
// (kvtransfer/src/copy_kernels.{cu,cpp}) gather them GPU -> pinned host and scatter them pinned
// host -> GPU, exactly as its TCP channel does on both ends of the socket
// (kvtransfer/src/tcp_channel.cpp:520-560 sender, :230-262 receiver).  This file only drives
// those functions: it contains no copy of them.  The socket hop is left out, so the number is an
// upper bound on what the reference moves between two GPUs of one box.
//
// usage: ref_datapath <src_dev> <dst_dev> <layers> <tokens> <requests> <slots> <warmup> <steps>
// prints: ms_total bytes_per_step ok
#include <cuda_runtime.h>

#include <bitset>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <numeric>
#include <random>
#include <vector>

#include "copy_kernels.h"
#include "envcfg.h"
#include "parse_block_common.h"

using namespace blade_llm;

#define CK(x)                                                                          \
  do {                                                                                 \
    cudaError_t e_ = (x);                                                              \
    if (e_ != cudaSuccess) {                                                           \
      fprintf(stderr, "cuda error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); \
      return 3;                                                                        \
    }                                                                                  \
  } while (0)

int main(int argc, char** argv) {
  if (argc < 9) return 2;
  const int src_dev = atoi(argv[1]), dst_dev = atoi(argv[2]), L = atoi(argv[3]);
  const uint32_t tokens = atoi(argv[4]), n_req = atoi(argv[5]), slots = atoi(argv[6]);
  const int warmup = atoi(argv[7]), steps = atoi(argv[8]);
  const uint32_t ntpb = 16, heads = 8, dim = 128, esz = 2;
  const size_t token_bytes = 2ull * heads * dim * esz;             // K+V of one token in one layer
  const size_t block_bytes = token_bytes * ntpb;
  const uint32_t blocks_per_req = (tokens + ntpb - 1) / ntpb;
  const uint32_t n_blocks = 1 + blocks_per_req * n_req * slots;
  const size_t layer_bytes = block_bytes * n_blocks;

  WorkerInfo src, dst;
  for (WorkerInfo* w : {&src, &dst}) {
    w->inst_id = w == &src ? "P" : "D";
    w->worker_id = 0;
    w->engine_tp_size = 1;
    w->worker_tp_rank = 0;
    w->block_sizes = {block_bytes};
    w->token_sizes = {token_bytes};
    w->layer_num_blocks = n_blocks;
    w->attn_kernel_blk_ntpb = ntpb;
    w->attn_pack_size = 1;
    w->num_kv_heads = heads;
  }

  // random block tables per slot and request; IpcBlocks from the reference's own generator
  std::mt19937 rng(1234);
  std::vector<std::vector<IpcBlock>> slot_blocks(slots);
  std::vector<uint32_t> perm_s(n_blocks - 1), perm_d(n_blocks - 1);
  std::iota(perm_s.begin(), perm_s.end(), 1);
  std::iota(perm_d.begin(), perm_d.end(), 1);
  std::shuffle(perm_s.begin(), perm_s.end(), rng);
  std::shuffle(perm_d.begin(), perm_d.end(), rng);
  size_t cursor = 0;
  std::bitset<MAX_TP_SIZE> valid;
  valid.set(0);
  for (uint32_t s = 0; s < slots; ++s) {
    std::vector<std::vector<IpcBlock>> out;
    for (uint32_t r = 0; r < n_req; ++r) {
      BlockIds sb(1), db(1);
      for (uint32_t b = 0; b < blocks_per_req; ++b, ++cursor) {
        sb[0].push_back(perm_s[cursor]);
        db[0].push_back(perm_d[cursor]);
      }
      auto info = std::make_shared<RequestInfo>(dst.inst_id, dst.worker_id, "r" + std::to_string(s * n_req + r), sb, db);
      ReqSendTask task(info, 0, tokens, true);
      vllm_parse_block_send_p_eq_d(&src, &dst, valid, 1, 0, &task, out);
    }
    if (out.size() != 1) {
      fprintf(stderr, "unexpected tensor count %zu\n", out.size());
      return 4;
    }
    slot_blocks[s] = out[0];
  }
  size_t bytes_per_layer = 0;
  for (const auto& b : slot_blocks[0]) bytes_per_layer += b.length;

  // caches
  std::vector<char*> src_layers(L), dst_layers(L);
  CK(cudaSetDevice(src_dev));
  for (int l = 0; l < L; ++l) {
    CK(cudaMalloc(&src_layers[l], layer_bytes));
    CK(cudaMemset(src_layers[l], 0x11 + l, layer_bytes));
  }
  CK(cudaSetDevice(dst_dev));
  for (int l = 0; l < L; ++l) {
    CK(cudaMalloc(&dst_layers[l], layer_bytes));
    CK(cudaMemset(dst_layers[l], 0, layer_bytes));
  }
  // staging: two pinned buffers so that the gather of layer i+1 overlaps the scatter of layer i,
  // as the reference's sender and receiver do on the two ends of the connection
  const size_t max_desc = env_kernel_copy_max_block_num();
  char* stage[2];
  int64_t *host_meta[2][2], *dev_meta_src[2], *dev_meta_dst[2];
  for (int i = 0; i < 2; ++i) {
    CK(cudaHostAlloc(&stage[i], bytes_per_layer, cudaHostAllocPortable | cudaHostAllocMapped));
    for (int d = 0; d < 2; ++d) CK(cudaHostAlloc(&host_meta[i][d], 3 * sizeof(int64_t) * max_desc, cudaHostAllocPortable | cudaHostAllocMapped));
  }
  cudaStream_t d2h, h2d;
  CK(cudaSetDevice(src_dev));
  initialize_copy_method_profile(src_dev);
  CK(cudaStreamCreateWithFlags(&d2h, cudaStreamNonBlocking));
  for (int i = 0; i < 2; ++i) CK(cudaMalloc(&dev_meta_src[i], 3 * sizeof(int64_t) * max_desc));
  CK(cudaSetDevice(dst_dev));
  if (dst_dev != src_dev) initialize_copy_method_profile(dst_dev);
  CK(cudaStreamCreateWithFlags(&h2d, cudaStreamNonBlocking));
  for (int i = 0; i < 2; ++i) CK(cudaMalloc(&dev_meta_dst[i], 3 * sizeof(int64_t) * max_desc));

  // sender-side descriptor lists: dst_offset = GPU source offset (tcp_channel.cpp:538-543)
  std::vector<std::vector<IpcBlock>> gather_blocks(slots);
  for (uint32_t s = 0; s < slots; ++s)
    for (const auto& b : slot_blocks[s]) gather_blocks[s].emplace_back(0, b.src_offset, b.length);

  auto gather = [&](int l, uint32_t s) -> cudaError_t {
    cudaSetDevice(src_dev);
    return copy_handle_data_with_kernel(stage[l & 1], src_layers[l], gather_blocks[s], bytes_per_layer, CopyDirection::D2H,
                                        src_dev, d2h, dev_meta_src[l & 1], host_meta[l & 1][0]);
  };
  auto scatter = [&](int l, uint32_t s) -> cudaError_t {
    cudaSetDevice(dst_dev);
    return copy_handle_data_with_kernel(stage[l & 1], dst_layers[l], slot_blocks[s], bytes_per_layer, CopyDirection::H2D,
                                        dst_dev, h2d, dev_meta_dst[l & 1], host_meta[l & 1][1]);
  };
  auto step = [&](int it) -> int {
    const uint32_t s = it % slots;
    CK(gather(0, s));
    CK(cudaStreamSynchronize(d2h));
    for (int l = 0; l < L; ++l) {
      if (l + 1 < L) CK(gather(l + 1, s));
      CK(scatter(l, s));
      CK(cudaStreamSynchronize(h2d));
      CK(cudaStreamSynchronize(d2h));
    }
    return 0;
  };

  for (int i = 0; i < warmup; ++i)
    if (step(i)) return 5;
  cudaEvent_t e0, e1;
  CK(cudaSetDevice(src_dev));
  CK(cudaEventCreate(&e0));
  CK(cudaEventRecord(e0, d2h));
  for (int i = 0; i < steps; ++i)
    if (step(warmup + i)) return 5;
  CK(cudaSetDevice(dst_dev));
  CK(cudaEventCreate(&e1));
  CK(cudaEventRecord(e1, h2d));
  CK(cudaEventSynchronize(e1));
  float ms = 0;
  if (src_dev == dst_dev) {
    CK(cudaEventElapsedTime(&ms, e0, e1));
  } else {
    // events of two devices cannot be subtracted: the loop above ends with both streams idle, so
    // time the same region again against a second event on the source device
    cudaEvent_t e1s;
    CK(cudaSetDevice(src_dev));
    CK(cudaEventCreate(&e1s));
    CK(cudaEventRecord(e1s, d2h));
    CK(cudaEventSynchronize(e1s));
    CK(cudaEventElapsedTime(&ms, e0, e1s));
  }

  // verify the last slot that was moved, layer 0 and last
  int ok = 1;
  {
    const uint32_t s = (warmup + steps - 1) % slots;
    std::vector<char> a(block_bytes / 2), b(block_bytes / 2);
    const IpcBlock& blk = slot_blocks[s].front();
    for (int l : {0, L - 1}) {
      const size_t n = std::min<size_t>(blk.length, a.size());
      CK(cudaMemcpy(a.data(), src_layers[l] + blk.src_offset, n, cudaMemcpyDeviceToHost));
      CK(cudaMemcpy(b.data(), dst_layers[l] + blk.dst_offset, n, cudaMemcpyDeviceToHost));
      if (memcmp(a.data(), b.data(), n) != 0) ok = 0;
    }
  }
  printf("%.4f %zu %d\n", ms, bytes_per_layer * (size_t)L, ok);
  return 0;
}
