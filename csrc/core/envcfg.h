// Environment configuration of the native engine.  Variable names, defaults and the
// `kvtenv: env=… val=… def=…` echo follow kvtransfer/src/envcfg.cpp:13-372; values are read
// once and cached.  `envcfg_reset_for_test()` drops the cache so unit tests can change them.
#pragma once
#include <netinet/in.h>

#include <cstddef>
#include <cstdint>
#include <string>
#include <utility>
#include <vector>

namespace kvx {

// Cache-shape ids (kvtransfer/include/envcfg.h:25-52).
constexpr int RAGGED_FLASH_CACHE_SHAPE = 1;
constexpr int FLASH_CACHE_SHAPE = 2;
constexpr int QWEN3_NEXT_FLASH_CACHE_SHAPE = 3;
constexpr int DPSK_V32_SPARSE_MLA_SHAPE = 4;
constexpr int FLASHINFER_CACHE_SHAPE = 5;
constexpr int TURBOQUANT_CACHE_SHAPE = 6;
constexpr int QWEN3_NEXT_FLASHINFER_CACHE_SHAPE = 7;
constexpr int KIMI_K3_MLA_CACHE_SHAPE = 8;

constexpr int SEND_DONE_HEAD_KIND = 1;
constexpr int SEND_SAVE_DONE_HEAD_KIND = 2;
constexpr size_t MAX_TP_SIZE = 16;

int env_heap_prof();
int env_send_parallel();
int env_ctx_tpsize();
int env_conn_tpsize();
int env_h2d_sync_tpsize();
int env_fsnaming_keepalive_interval_s();
int env_fsnaming_tolerate_interval_s();
int env_debug_tx_failrate();   // failure rate is (value - 1) percent
int env_debug_tx_delay_ms();
const struct sockaddr_in* env_send_done_addr();  // nullptr: send-done RPC disabled
int env_cache_shape();
int env_send_done_head_kind();
const std::vector<std::pair<uint64_t, int>>* env_reserve();
int env_rpc_timeout_s();
int env_crc();
int env_port_base();
int env_send_tpsize();
int env_txstub_cap();
int env_waitlayer_tpsize();
int env_shrink_tpsize();
int env_attn_kernel_blk_size();
size_t env_kernel_copy_max_block_num() noexcept;
double env_kernel_copy_sm_usage() noexcept;
bool env_bf162fp8_conversion() noexcept;
bool env_pad_last_attn_block() noexcept;
bool env_rdma_staged() noexcept;
const char* env_nic_name() noexcept;
// New in this engine: CTAs of the NVLink transfer kernel (0 = derive from SM usage),
// destination quantisation (0 none, 1 block-scaled e4m3), TMA on/off.
int env_nvlink_ctas();
int env_nvlink_streams();
int env_dst_mxfp8();
int env_use_tma();
// TMA tiles of the NVLink channel: order in shared memory (0 tokens outermost, 1 heads outermost, -1 = the
// destination's own order) and how they leave (0 tensor store, 1 one linear bulk store, -1 = linear when legal).
// 0: the NVLink channel plans hybrid / MLA / KDA shapes on the CPU and uploads byte ranges instead of walk ops.
int env_nvlink_walk();
int env_fanout_weak();    // multicast fan-out with weak stores (1) or relaxed system-scope stores (0)
int env_walk_threads();   // threads per CTA of the walk kernel (0: the kernel's default)
int env_walk_stages();    // bulk pipeline stages per CTA of the walk kernel (0: default)
// 0: the NVLink channel always pushes (kernels on the prefill GPU); default: it asks the destination for a pull session
// (kernels on the decode GPU, loads over NVLink) when the destination is another GPU and takes the bytes unconverted.
int env_nvlink_pull();
int env_tile_order();
int env_store_form();
// Host-staged copies (TCP / SHM transports): start-up measurement of copy kernel against copy
// engines, the static rule used without it, and a forced path (0 measured or static, 1 kernel, 2 memcpy).
bool env_copy_profile_enable();
size_t env_copy_memcpy_max_blocks();
size_t env_copy_memcpy_threshold_bytes();
int env_copy_path();
// NVLink channel: stamp the GPU timer at the start and the end of every batch and report DeviceUs in the flush line.
bool env_device_timestamps();
// How long a batch of a device transport may take to deliver its completion record before it is failed
// (default: the RPC timeout).
int env_completion_timeout_ms();

void envcfg_reset_for_test();
std::string envcfg_dump();   // every setting resolved so far, one key=value per line

}  // namespace kvx
