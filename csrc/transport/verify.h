// End-to-end check of a finished transfer (BLLM_KVTRANS_CRC=1).
//
// After a batch has landed and before its requests are reported, the sender sums a position-keyed
// checksum (kernels/kvt_checksum.cu) over the source ranges of its own cache, asks the destination's
// server to do the same over the destination ranges of its cache (CHECK_REQ), and fails the batch when the
// two numbers differ.  It is the role of the reference's CRC check on its RDMA channel (kvtransfer/src/
// rdma_channel.cpp:143-296, 845-852: local CRC over the written blocks, REMOTE_CRC_REQ, RTASSERT_EQ) with
// three differences: every transport is covered (the check sits in the send stub, above the channels); each
// side reads its own memory where it lives (a kernel for GPU caches, a loop for host caches), so no CPU
// mapping of device memory is needed; and the value is a 64-bit sum, not a CRC-32.
//
// Two forms.  Byte ranges (CHECK_REQ): source and destination cache of one layout and dtype, any shape, any
// transport.  Rows (CHECK_ATTN_REQ): a transfer of the fused attention kernel that changes the layout or moves a
// head window (GPU caches); each side walks its own block tables with its own strides and keys every byte by the
// logical coordinates of its row.  A transfer that changes the dtype (quantises) says so once and goes unchecked:
// its two sides differ by design.
//
// The per-(layer, tensor) sums are rotated by a layer- and tensor-dependent amount before they are added,
// so that data landing in the wrong layer or tensor changes the result.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "core/context.h"
#include "core/types.h"
#include "kernels/kvt_kernels.h"

namespace kvx {

struct CheckRange {
  uint64_t off, len;
};

// Sum over layers [layer_begin, layer_end) and tensors t of the ranges `per_tensor[t]` in this worker's
// cache.  Throws std::out_of_range for a range outside its tensor, std::runtime_error for a CUDA failure.
// Calls are serialised per process; the device path synchronises its own stream only.
uint64_t checksum_cache(Context* ctx, uint32_t layer_begin, uint32_t layer_end,
                        const std::vector<std::vector<CheckRange>>& per_tensor);

struct CheckOutcome {
  bool ok{false};
  uint64_t local{0}, remote{0};
  int64_t local_us{0}, remote_us{0};
};

// Sender side: `blocks[t]` are the batch's byte ranges of tensor t (source and destination offsets).
// Throws KVTransferException when the destination cannot be asked.
CheckOutcome verify_transfer(Context* ctx, const WorkerInfo& dst, uint32_t layer_begin, uint32_t layer_end,
                             const std::vector<std::vector<IpcBlock>>& blocks);

// Row form: one side of a transfer between attention caches (tensor 0 of every layer).
struct AttnCheck {
  KvtLayout layout{};
  uint32_t head0{0}, n_heads{0};
  std::vector<KvtCheckReq> reqs;      // `first` and `index` are filled by add()
  std::vector<uint32_t> pool;
  uint32_t total_tokens{0};
  // tokens [seen, seen + new_tokens) of a request whose block table on this side is `blocks`; `index` is the
  // request's number in the batch (the same on both sides)
  void add(const std::vector<uint32_t>& blocks, uint32_t seen, uint32_t new_tokens, uint32_t index);
};
uint64_t checksum_attn(Context* ctx, uint32_t layer_begin, uint32_t layer_end, const AttnCheck& side);
CheckOutcome verify_attn_transfer(Context* ctx, const WorkerInfo& dst, uint32_t layer_begin, uint32_t layer_end,
                                  const AttnCheck& src_side, const AttnCheck& dst_side);

// Server side: the whole response frame for a CHECK_REQ / CHECK_ATTN_REQ frame (`buf` starts at the RPC header).
std::string answer_check(Context* ctx, const char* buf, size_t len);
std::string answer_check_attn(Context* ctx, const char* buf, size_t len);

}  // namespace kvx
