// C ABI of the sm_100a transfer kernels.
//
// Every launcher here is a plain `extern "C"` function so that the pybind module, the C++
// engine and ctypes callers all share one entry point.  Pointers are raw device (or
// peer-mapped / host-mapped) addresses; nothing in this header depends on torch.
//
// The kernels replace, in one pass, what the reference does in three places: the CPU
// ParseBlock offset generators (kvtransfer/src/parse_block_*.cpp), the gather/scatter copy
// kernels (kvtransfer/src/copy_kernels.cu:105-281) and the wire transfer in between
// (kvtransfer/src/tcp_channel.cpp:477-588).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Byte-stride description of one paged attention cache tensor (one layer, one rank).
// All cache shapes of the reference (kvtransfer/include/envcfg.h:25-52) reduce to this:
//   addr(block b, kv, slot t, head h) = base + b*block_stride + kv*kv_stride
//                                     + t*token_stride + h*head_stride
// For block-scaled fp8 pages the scale bytes (UE8M0, one per 32 values) sit in the same
// block at scale_base with their own strides.
typedef struct KvtLayout {
  int64_t block_stride;
  int64_t kv_stride;
  int64_t token_stride;
  int64_t head_stride;
  int64_t scale_base;          // byte offset of the scale region inside a block (fp8 pages)
  int64_t scale_kv_stride;
  int64_t scale_token_stride;
  int64_t scale_head_stride;
  uint32_t ntpb;               // token slots per block
  uint32_t num_heads;          // heads held by this rank
  uint32_t head_bytes;         // payload bytes of one (token, head) row
  uint32_t num_blocks;         // blocks in the tensor (bounds check)
  uint32_t kv_count;           // 2 for K+V caches, 1 for MLA latent / indexer caches
  uint32_t reserved;
} KvtLayout;

// One request (or one chunk of it) scheduled in this step.  Block ids live in a shared
// uint32 pool so a 64k-token request needs no per-block host descriptor.
typedef struct KvtReqDesc {
  uint32_t src_blk_off;        // index of this request's first src block id in the pool
  uint32_t dst_blk_off;        // index of this request's first dst block id in the pool
  uint32_t n_src_blocks;
  uint32_t n_dst_blocks;
  uint32_t seen_tokens;        // tokens already transferred by earlier chunks
  uint32_t new_tokens;         // tokens [seen, seen+new) move in this launch
  uint32_t flags;              // KVT_REQ_*
  uint32_t first_tile;         // exclusive prefix sum of tile counts (filled by the host)
} KvtReqDesc;

#define KVT_REQ_PAD_TAIL 1u    // zero dst slots [seen+new, end of last dst block)

enum KvtMode {
  KVT_MODE_COPY = 0,           // byte copy
  KVT_MODE_BF16_TO_MXFP8 = 1,  // bf16 -> e4m3 with one UE8M0 scale per 32 values
  KVT_MODE_MXFP8_TO_BF16 = 2,  // inverse
};

enum KvtStatus {
  KVT_OK = 0,
  KVT_ERR_BLOCK_RANGE = 1,     // a block id or block index was outside its table / tensor
  KVT_ERR_TMA_TIMEOUT = 2,     // a bounded mbarrier wait ran out
  KVT_ERR_BAD_ARGS = 3,
  KVT_ERR_FLAG_TIMEOUT = 4,    // a bounded wait on a completion flag ran out
};

typedef struct KvtAttnLaunch {
  const uint64_t* src_layers;  // device array, one base address per layer (local memory)
  const uint64_t* dst_layers;  // device array, one base address per layer (local / peer / host-mapped)
  const void* src_maps;        // device array of CUtensorMap per layer, or NULL (SIMT only)
  const void* dst_maps;
  KvtLayout src;
  KvtLayout dst;
  uint32_t layer_begin;
  uint32_t layer_end;
  const KvtReqDesc* reqs;      // device memory
  uint32_t n_reqs;
  uint32_t total_tiles;        // sum over requests of their tile count
  const uint32_t* block_ids;   // device memory pool
  uint32_t tile_tokens;        // tokens per tile; divides src.ntpb and dst.ntpb
  uint32_t src_head0;          // first source head moved
  uint32_t dst_head0;          // where it lands on the destination rank
  uint32_t n_heads;            // heads moved
  uint32_t mode;               // KvtMode
  uint32_t* status;            // device: [0] first error code, [1] detail
  uint32_t* done_counter;      // device, zero before launch; may be NULL with flag == NULL
  uint64_t* flag;              // completion word (device / peer / host-mapped) or NULL
  uint64_t flag_value;         // value stored to *flag by the last CTA after a system fence
  uint32_t simt_tile;          // SIMT path: 0 / 1 = a warp per tile (device destinations), 2 = a CTA per tile
                               // (mapped host destinations: longer contiguous PCIe writes)
  uint32_t dst_remote;         // 1: the destination is another GPU's memory.  The quantiser then stages its
                               // output in shared memory and sends it with bulk stores (256-byte NVLink
                               // packets); into local memory its own 16-byte stores are faster.
  // ---- TMA path: how a tile sits in shared memory and how it leaves ----
  uint32_t tile_order;         // 0: [slot][head][row] (maps from kvt_encode_tensor_map); 1: [head][slot][row] (maps
                               // encoded with token_inner = 1).  Both maps of a launch use the same order.
  uint32_t store_form;         // 0: tensor store through dst_maps; 1: one untiled bulk store per tile, legal when
                               // kvt_tile_is_flat(dst, n_heads, tile_tokens, tile_order): the tile is one contiguous
                               // run of the destination, which then crosses NVLink as one linear write
  uint32_t tma_stages;         // cap of the per-CTA pipeline depth (0: as many as shared memory allows, at most 8)
  uint32_t cache_hint;         // 1: L2 evict_first policy on the tile loads and stores (streamed once)
} KvtAttnLaunch;

// Tile count of one request for a given tile size (host helper, also used by tests).
uint32_t kvt_req_tiles(uint32_t seen, uint32_t new_tokens, uint32_t tile_tokens, uint32_t flags,
                       uint32_t dst_ntpb);

// Launch the fused transfer kernel.  grid_ctas <= 0 picks one CTA per SM.  use_tma != 0 moves
// full tiles with cp.async.bulk.tensor (needs src_maps/dst_maps and KVT_MODE_COPY).
// Returns a cudaError_t value.
int kvt_launch_p2d_attn(const KvtAttnLaunch* args, int grid_ctas, int threads, int use_tma,
                        void* stream);

// Encode one 5-D tensor map {head_bytes/4, heads, slots, blocks, kv} over a cache tensor with
// box {head_bytes/4, box_heads, box_tokens, 1, 1}.  `out` receives 128 bytes.  Returns 0 on
// success, a CUresult or -1 otherwise.  No multicast is ever used with these maps.
int kvt_encode_tensor_map(void* out, uint64_t base, const KvtLayout* layout, uint32_t box_heads,
                          uint32_t box_tokens);
// The same with the dimension order chosen: token_inner = 1 encodes {head_bytes/4, slots, heads, blocks, kv}
// with box {head_bytes/4, box_tokens, box_heads, 1, 1}, so that a tile lands in shared memory as
// [head][slot][row], the memory order of an HND page (KvtAttnLaunch::tile_order = 1).
int kvt_encode_tensor_map_ordered(void* out, uint64_t base, const KvtLayout* layout, uint32_t box_heads,
                                  uint32_t box_tokens, uint32_t token_inner);
// 1 when a tile of n_heads x tile_tokens rows, kept in that order, is one contiguous run of `layout`.
int kvt_tile_is_flat(const KvtLayout* layout, uint32_t n_heads, uint32_t tile_tokens, uint32_t token_inner);

// ---- block-relative strided segments (GDN / KDA / PLE recurrent state) -------------------
// One segment rule: for i in [0,count): copy len bytes from
//   src_block_base + src_off + i*src_stride  to  dst_block_base + dst_off + i*dst_stride.
typedef struct KvtSegRule {
  int64_t src_off;
  int64_t dst_off;
  int64_t src_stride;
  int64_t dst_stride;
  uint32_t len;
  uint32_t count;
} KvtSegRule;

typedef struct KvtStateLaunch {
  const uint64_t* src_layers;
  const uint64_t* dst_layers;
  uint32_t layer_begin, layer_end;
  int64_t src_block_stride;
  int64_t dst_block_stride;
  uint32_t src_num_blocks, dst_num_blocks;
  const uint32_t* src_blocks;  // device: one src block id per state page to move
  const uint32_t* dst_blocks;  // device: matching dst block ids
  uint32_t n_pages;
  const KvtSegRule* rules;     // device
  uint32_t n_rules;
  uint32_t* status;
  uint32_t* done_counter;
  uint64_t* flag;
  uint64_t flag_value;
} KvtStateLaunch;

int kvt_launch_p2d_state(const KvtStateLaunch* args, int grid_ctas, int threads, void* stream);

// ---- block-table walk for every other cache shape --------------------------------------------
// The hybrid, MLA and state-page shapes (kvtransfer/include/envcfg.h:25-52: 3, 4, 6, 7, 8) are moved by
// "walk ops".  One op is an affine rule over a range of positions (tokens, or whole pages) of one request:
//
//   for pos in [pos_lo, pos_hi), for i0 < inner[0].count, i1 < inner[1].count, i2 < inner[2].count:
//     side offset = table[pos / per_block] * block_stride + ((pos % per_block) / per_kb) * kb_stride
//                   + (pos % per_kb) * pos_stride + add + sum(i_k * inner[k].stride)
//     copy len bytes from the source offset to the destination offset (or write zeros: KVT_WALK_ZERO)
//
// with one table of block ids per side in a shared uint32 pool.  This is what the reference's ParseBlock
// functions expand on the CPU into one {src, dst, len} triple per piece (kvtransfer/src/parse_block_*.cpp);
// here the host writes a handful of ops per request, whatever its length, and the kernel does the
// expansion while it copies.  Positions are grouped in units of `run` (a divisor of both sides' kernel
// block), inside which both offsets are affine in pos; when pos_stride == len on both sides a unit is one
// contiguous piece.  Ops whose pieces are long and 16-byte aligned (KVT_WALK_BULK) go through the TMA
// engine in segments of KVT_WALK_SEG bytes, the others through the SIMT warps.
#define KVT_WALK_MAX_INNER 3
#define KVT_WALK_SEG 8192u
#define KVT_WALK_ZERO 1u         /* write zeros to the destination pieces (tail padding); no source */
#define KVT_WALK_BULK 2u         /* contiguous, 16-byte aligned pieces: moved by untiled bulk copies */
#define KVT_WALK_CONTIG 4u       /* pos_stride == len on both sides: the positions of a unit form one piece */
typedef struct KvtWalkLoop {
  uint32_t count;
  uint32_t reserved;
  int64_t src_stride;
  int64_t dst_stride;
} KvtWalkLoop;

typedef struct KvtWalkOp {
  uint32_t src_tbl, dst_tbl;             // first entry of each side's block table in the pool
  uint32_t n_src, n_dst;                 // table lengths (bounds)
  uint32_t pos_lo, pos_hi;
  uint32_t src_per_block, dst_per_block; // positions per block
  uint32_t src_per_kb, dst_per_kb;       // positions per kernel block (== per block when pages are not subdivided)
  int64_t src_block_stride, dst_block_stride;
  int64_t src_kb_stride, dst_kb_stride;
  int64_t src_pos_stride, dst_pos_stride;
  int64_t src_add, dst_add;
  uint32_t len;                          // bytes per position and inner iteration
  uint32_t tensor;                       // cache tensor of the layer (multi-tensor shapes)
  uint32_t flags;                        // KVT_WALK_*
  uint32_t n_inner;
  KvtWalkLoop inner[KVT_WALK_MAX_INNER]; // inner[n_inner - 1] varies fastest
  // filled by kvt_walk_finalize():
  uint32_t run;                          // positions per unit
  uint32_t inner_total;                  // product of the inner counts
  uint32_t segs;                         // KVT_WALK_BULK: segments per piece
  uint32_t reserved;
  uint64_t first_unit;                   // exclusive prefix sum of unit counts within the op's class (bulk / simt)
} KvtWalkOp;

// Completes run / inner_total / segs / flags of every op, orders the array as [bulk ops][simt ops][zero ops]
// and fills first_unit (counted within each of the three classes).  Returns the number of bulk ops; the
// counts and unit totals of the classes come back through the pointers.  Zero fills form a class of their own
// because they must land AFTER the copies: the reference pads a tail after it has copied the tokens, and in
// some geometries the padded range covers bytes the copies wrote; launch them behind the copies, on the same
// stream.  An op whose geometry is not usable (zero run, per_block not a multiple of per_kb, more than
// KVT_WALK_MAX_INNER loops) makes it return -1.
typedef struct KvtWalkCounts {
  uint32_t n_bulk, n_simt, n_zero, reserved;
  uint64_t bulk_units, simt_units, zero_units;
} KvtWalkCounts;
int kvt_walk_finalize(KvtWalkOp* ops, uint32_t n_ops, KvtWalkCounts* counts);

#define KVT_WALK_MAX_TENSORS 8
typedef struct KvtWalkLaunch {
  const uint64_t* src_ptrs;    // device: base address per [layer][tensor] (local memory)
  const uint64_t* dst_ptrs;    // device: the same for the destination (local / peer / host-mapped)
  uint32_t n_tensors;
  uint32_t layer_begin, layer_end;
  uint32_t shape;              // launch shape, 0 = default: threads per CTA in the low 16 bits (a multiple of 32, at
                               // least 64: one warp drives the bulk pipeline, the others are SIMT), pipeline stages above
  uint64_t src_cap[KVT_WALK_MAX_TENSORS];   // bytes of each tensor: every piece is checked against them
  uint64_t dst_cap[KVT_WALK_MAX_TENSORS];
  const KvtWalkOp* ops;        // device: [bulk ops][simt ops]
  uint32_t n_bulk_ops, n_simt_ops;
  uint64_t bulk_units, simt_units;
  const uint32_t* pool;        // device: block tables
  uint32_t pool_len;
  uint32_t* status;            // device: [0] first error code, [1] detail
} KvtWalkLaunch;
int kvt_launch_walk(const KvtWalkLaunch* args, int grid_ctas, void* stream);

// ---- IpcBlock list copy (descriptor-driven; TCP/shm staging and the generic fallback) -----
// Copies n triples {src_off, dst_off, len} (the 24-byte IpcBlock of the wire format,
// kvtransfer/include/channel.h:15-21) between two bases.
int kvt_launch_copy_blocks(uint64_t src_base, uint64_t dst_base, const uint64_t* triples,
                           uint32_t n, uint64_t src_capacity, uint64_t dst_capacity,
                           uint32_t* status, int grid_ctas, void* stream);

// Gather with the reference's unscaled cast (kvtransfer/src/copy_kernels.cu:369-481): descriptor
// {src_off, dst_off, n} reads n bf16 values (2n bytes) at src_off and writes n e4m3 bytes at dst_off,
// round to nearest even, saturating to +-448, NaN kept.  Used by the host-staged transports when
// BLLM_KVTRANS_BF162FP8_CONV is set (bf16 prefill cache, fp8 decode cache).
int kvt_launch_copy_blocks_cast(uint64_t src_base, uint64_t dst_base, const uint64_t* triples, uint32_t n,
                                uint64_t src_capacity, uint64_t dst_capacity, uint32_t* status, int grid_ctas,
                                void* stream);
// The same conversion of one value on the host (the CPU path of those transports, and the oracle).
uint8_t kvt_bf16_to_e4m3(uint16_t bf16_bits);

// The same copy over up to KVT_COPY_MAX_TENSORS tensor pairs in ONE launch: entry e moves descriptors
// [first[e], first[e] + count[e]) of `triples`, relative to src_base[e] / dst_base[e].  Entries may
// share a descriptor range: the tensors of one layer (MLA latent + indexer keys, hybrid groups) cost
// one launch instead of one each, and so do several layers whose pages use the same descriptors.
#define KVT_COPY_MAX_TENSORS 8
typedef struct KvtCopyMulti {
  uint64_t src_base[KVT_COPY_MAX_TENSORS];
  uint64_t dst_base[KVT_COPY_MAX_TENSORS];
  uint64_t src_cap[KVT_COPY_MAX_TENSORS];
  uint64_t dst_cap[KVT_COPY_MAX_TENSORS];
  uint32_t first[KVT_COPY_MAX_TENSORS];
  uint32_t count[KVT_COPY_MAX_TENSORS];
  uint32_t n_tensors;
  const uint64_t* triples;     // device
  uint32_t* status;            // device: [0] first error code, [1] descriptor index
} KvtCopyMulti;
int kvt_launch_copy_blocks_multi(const KvtCopyMulti* args, int grid_ctas, void* stream);
// The same, moved by the TMA engine: runs made of whole 16-byte words at 16-byte aligned addresses go
// through shared memory as untiled bulk copies of 8 KiB (one thread per CTA issues them, four in
// flight per CTA), the rest through the SIMT warps.  `rounds` = kvt_bulk_rounds(length of the first
// descriptor, length of the longest) maximised over the entries: 1 when the descriptors of an entry
// have one length (pages of a tensor).
uint32_t kvt_bulk_rounds(uint64_t first_len, uint64_t max_len);
int kvt_launch_copy_blocks_bulk(const KvtCopyMulti* args, uint32_t rounds, int grid_ctas, void* stream);

// ---- the same copy for callers that must not allocate --------------------------------------
// This entry point has no counterpart in the reference.  It exists for callers that cannot
// allocate at call time (a transfer issued in an engine's steady state with a fully sized
// pool, a recovery path that runs when the device is out of memory, a thread holding a lock the
// allocator takes): the descriptor array and the status words live in a fixed array inside the
// module's device image instead of memory the caller would have to allocate.  `host_triples`
// is HOST memory (n × {src_off, dst_off, len} u64); it is copied to the device on `stream`.
// When it is pinned memory the copy reads it when the stream reaches that point, not when the call
// returns: leave it untouched until the stream has passed the call (pageable memory is staged
// before the call returns).
// `host_status` (optional, 2 × u32: code, detail) receives the status words after the kernel, on
// `stream`; read it after synchronising the stream.  The call makes no allocation and frees
// nothing.  The first call on a device (with that device current) also looks up and caches the
// scratch address; make it before any stream capture begins.  First calls from several threads at
// once are safe (each publishes the same cached values).  One scratch array exists per device:
// calls on one device that overlap in time race on it.
// Returns 0, a positive cudaError_t, or one of the negative codes below.
#define KVT_NOALLOC_MAX_DESCS 4096u      /* descriptors per call; 96 KiB + 256 B of device image */
#define KVT_NOALLOC_ERR_TOO_MANY (-1)    /* n > KVT_NOALLOC_MAX_DESCS: rejected, nothing launched */
#define KVT_NOALLOC_ERR_BAD_ARGS (-2)    /* null descriptors / base, or device index out of range */
int kvt_copy_blocks_noalloc(uint64_t src_base, uint64_t dst_base, const uint64_t* host_triples,
                            uint32_t n, uint64_t src_capacity, uint64_t dst_capacity,
                            uint32_t* host_status, void* stream);

// ---- NVLS fan-out of replicated blocks --------------------------------------------------------
// Replicates byte range [block_off, block_off + block_len) of the listed source blocks, for layers
// [layer_begin, layer_end), from this GPU's memory into the listed destination blocks of every GPU
// bound to a multicast object (multimem.st through NVSwitch).  The source is any local memory: the
// member's own cache (in place: same tensors, same block ids; its copy is rewritten with the same
// bytes) or a landing buffer that a prefill GPU pushed into over CUDA-IPC peer memory.  mc_layers
// holds, per layer, the multicast address of the destination tensor.  Offsets, lengths and strides
// must be multiples of 16.  mc_flag (optional, multicast address of an 8-byte aligned word)
// receives flag_value with release semantics after the data.
typedef struct KvtMcFanout {
  const uint64_t* src_layers;  // device array: source base address per layer (this GPU's memory)
  const uint64_t* mc_layers;   // device array: multicast address of the destination tensor per layer
  uint32_t layer_begin, layer_end;
  int64_t src_block_stride;
  int64_t dst_block_stride;
  uint32_t src_num_blocks;     // bounds checks
  uint32_t dst_num_blocks;
  const uint32_t* src_blocks;  // device: source block id per block to replicate
  const uint32_t* dst_blocks;  // device: destination block id (the same on every GPU of the group)
  uint32_t n_blocks;
  uint32_t block_off;
  uint32_t block_len;
  uint32_t* status;            // device: [0] first error code, [1] detail
  uint32_t* done_counter;      // device, zero before launch (needed with mc_flag)
  uint64_t* mc_flag;
  uint64_t flag_value;
} KvtMcFanout;

int kvt_launch_mc_fanout(const KvtMcFanout* args, int grid_ctas, void* stream);

// The same replication driven by a walk plan: the member that received a request through walk ops
// (kvt_launch_walk, with `args` as launched there: its dst_ptrs are this GPU's cache) stores exactly
// the destination pieces of those ops - copies and zero fills - to the same offsets behind
// mc_ptrs[layer * n_tensors + tensor], the multicast addresses of the group's cache tensors.  The
// zero-fill class follows the two classes of `args` in the ops array.  Pieces must be made of whole
// 4-byte words (16-byte ones take the wide store); anything else reports KVT_ERR_BAD_ARGS.
int kvt_launch_walk_fanout(const KvtWalkLaunch* args, uint32_t n_zero_ops, uint64_t zero_units,
                           const uint64_t* mc_ptrs, int grid_ctas, void* stream);
// The sender's form: a GPU that is itself bound to the group's multicast object (so that it holds a mapping of
// it) stores the ops' SOURCE pieces, read from its own cache (args->src_ptrs), to the destination offsets behind
// mc_ptrs, and zeros for the zero-fill class.  No member receives the request first: the sender's link carries the
// bytes once and every member's link receives them once.  args->dst_ptrs is not used.
int kvt_launch_walk_multicast(const KvtWalkLaunch* args, uint32_t n_zero_ops, uint64_t zero_units,
                              const uint64_t* mc_ptrs, int grid_ctas, void* stream);

// ---- completion flags ---------------------------------------------------------------------
// Bounded device-side wait: returns through status[0]=KVT_ERR_FLAG_TIMEOUT when *flag has not
// reached `value` within timeout_ns.  Never spins without limit.
int kvt_launch_wait_flag(const uint64_t* flag, uint64_t value, uint64_t timeout_ns,
                         uint32_t* status, void* stream);
int kvt_launch_set_flag(uint64_t* flag, uint64_t value, void* stream);
// Device-side completion of a batch of launches.  `status` is the batch's status block in device memory
// (u32 code, u32 detail, u64 start stamp written by kvt_launch_stamp or zero); `record` is the device address
// of a KvtCompletion in mapped host memory.  Enqueue it on a stream ordered after the batch: when the stream
// gets there the kernel copies code, detail and stamps into the record, clears the status block and stores
// `seq` last (release, system scope).  The host polls record->seq: no stream synchronisation, no copy back.
typedef struct KvtCompletion {
  uint64_t seq;
  uint32_t status;
  uint32_t detail;
  uint64_t t_start_ns;
  uint64_t t_end_ns;
} KvtCompletion;
int kvt_launch_complete(uint32_t* status, KvtCompletion* record, uint64_t seq, void* stream);
// Writes the GPU's nanosecond timer (%globaltimer) to *slot (device or mapped host memory) when the
// stream reaches this point: device-side timestamps around a batch, comparable across the GPUs of a
// node, without CUDA events.
int kvt_launch_stamp(uint64_t* slot, void* stream);

// ---- end-to-end transfer check -------------------------------------------------------------
// Position-keyed 64-bit checksum of byte ranges of one tensor (kvt_checksum.cu): a piece is read as little-endian
// 32-bit words (the last padded with zero bytes) and word k with value w adds term(k, w), a 32-bit mix of both.
// Chunks are pieces cut to <= 64 KiB; index0 is the index of the chunk's first word in its piece.  One launch sums
// the same chunks over n_bases tensors of one shape (the layers of a cache): d_bases is a device array of their
// addresses and d_out[i] receives tensor i's sum.  The kernel ADDS to d_out (zero it first), skips a chunk outside
// [0, capacity) and reports it in d_status {KVT_ERR_BLOCK_RANGE, chunk number}.  grid_ctas is the total over all
// tensors.
typedef struct {
  uint64_t off;
  uint32_t len;
  uint32_t index0;
} KvtCheckChunk;
#define KVT_CHECK_CHUNK 65536u
int kvt_launch_checksum(const uint64_t* d_bases, uint32_t n_bases, uint64_t capacity, const KvtCheckChunk* d_chunks, uint32_t n,
                        uint64_t* d_out, uint32_t* d_status, int grid_ctas, void* stream);
uint64_t kvt_checksum_host(const void* data, uint64_t len, uint32_t index0);
// The same sum over the rows of an attention cache: for every request, token t in [seen, seen + new_tokens), K / V
// and head j in [0, n_heads), the head_bytes at
//   table[t / ntpb] * block_stride + kv * kv_stride + (t % ntpb) * token_stride + (head0 + j) * head_stride
// with word k of the row keyed by index
//   ((((index * 131 + t) * kv_count + kv) * n_heads + j) * ceil(head_bytes / 4) + k)        (32-bit arithmetic),
// which names the row by coordinates that do not depend on the layout.  `first` is the exclusive prefix sum of
// new_tokens over the requests; tables are [blk_off, blk_off + n_blocks) of the pool.
typedef struct {
  uint32_t blk_off, n_blocks, seen, new_tokens, first, index;
} KvtCheckReq;
int kvt_launch_checksum_attn(const uint64_t* d_bases, uint32_t n_bases, uint64_t capacity, const KvtLayout* layout, uint32_t head0,
                             uint32_t n_heads, const KvtCheckReq* d_reqs, uint32_t n_reqs, uint32_t total_tokens,
                             const uint32_t* d_pool, uint32_t pool_len, uint64_t* d_out, uint32_t* d_status, int grid_ctas,
                             void* stream);

// ---- peer memory / topology ---------------------------------------------------------------
int kvt_device_count(void);
int kvt_can_access_peer(int dev, int peer);
int kvt_enable_peer_access(int dev, int peer);              // idempotent
int kvt_p2p_attribute(int dev, int peer, int which);        // 0 perf rank, 1 access, 2 native atomics
int kvt_ipc_get_handle(uint64_t ptr, void* handle64, uint64_t* base, uint64_t* size);
int kvt_ipc_open_handle(const void* handle64, uint64_t* out_ptr);
int kvt_ipc_close(uint64_t ptr);
int kvt_malloc(uint64_t bytes, uint64_t* out_ptr);
int kvt_free(uint64_t ptr);
int kvt_host_alloc_mapped(uint64_t bytes, uint64_t* host_ptr, uint64_t* dev_ptr);
int kvt_host_free(uint64_t host_ptr);
int kvt_host_register(uint64_t host_ptr, uint64_t bytes, uint64_t* dev_ptr);
int kvt_host_unregister(uint64_t host_ptr);
int kvt_sm_count(int dev);
// Copy-engine copies by raw address (device, peer-mapped or pinned host memory on either side): one
// cudaMemcpyAsync, or one per {src_off, dst_off, len} triple of a host array.  They are the library
// baseline the transfer kernels are measured against (the reference's memcpy loop,
// kvtransfer/src/copy_kernels.cpp:267-294) and the bandwidth ceiling measured inside a benchmark run.
int kvt_memcpy_async(uint64_t dst, uint64_t src, uint64_t bytes, void* stream);
int kvt_memcpy_triples(uint64_t dst_base, uint64_t src_base, const uint64_t* host_triples, uint32_t n, void* stream);
const char* kvt_error_string(int err);

#ifdef __cplusplus
}
#endif
