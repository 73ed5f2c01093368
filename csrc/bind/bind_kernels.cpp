// pybind11 bindings of the kernel-level C ABI (csrc/kernels/kvt_kernels.h).
// Everything takes raw addresses (int) so that torch tensors, mapped host memory and
// peer-mapped IPC memory are handled alike:  tensor.data_ptr(), stream.cuda_stream.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "kernels/kvt_kernels.h"

namespace py = pybind11;

namespace kvx {

static void check_cuda(int err, const char* what) {
  if (err != 0) {
    throw std::runtime_error(std::string(what) + ": " + kvt_error_string(err) + " (" + std::to_string(err) + ")");
  }
}

// Host-side packing of a step's requests into the compact device plan: an array of
// KvtReqDesc followed by the uint32 block-id pool, in one buffer so that one copy uploads it.
struct PackedPlan {
  py::bytes blob;
  uint32_t n_reqs;
  uint32_t total_tiles;
  uint64_t block_ids_offset;  // byte offset of the pool inside blob
};

static py::tuple pack_plan(const std::vector<std::tuple<std::vector<uint32_t>, std::vector<uint32_t>, uint32_t,
                                                        uint32_t, uint32_t>>& reqs,
                           uint32_t tile_tokens, uint32_t dst_ntpb) {
  std::vector<KvtReqDesc> descs;
  std::vector<uint32_t> pool;
  descs.reserve(reqs.size());
  uint32_t tiles = 0;
  for (const auto& r : reqs) {
    const auto& sb = std::get<0>(r);
    const auto& db = std::get<1>(r);
    KvtReqDesc d{};
    d.src_blk_off = static_cast<uint32_t>(pool.size());
    pool.insert(pool.end(), sb.begin(), sb.end());
    d.dst_blk_off = static_cast<uint32_t>(pool.size());
    pool.insert(pool.end(), db.begin(), db.end());
    d.n_src_blocks = static_cast<uint32_t>(sb.size());
    d.n_dst_blocks = static_cast<uint32_t>(db.size());
    d.seen_tokens = std::get<2>(r);
    d.new_tokens = std::get<3>(r);
    d.flags = std::get<4>(r);
    d.first_tile = tiles;
    const uint32_t n = kvt_req_tiles(d.seen_tokens, d.new_tokens, tile_tokens, d.flags, dst_ntpb);
    if (n == 0) continue;
    tiles += n;
    descs.push_back(d);
  }
  const size_t desc_bytes = descs.size() * sizeof(KvtReqDesc);
  std::string blob(desc_bytes + pool.size() * sizeof(uint32_t), '\0');
  if (desc_bytes) std::memcpy(blob.data(), descs.data(), desc_bytes);
  if (!pool.empty()) std::memcpy(blob.data() + desc_bytes, pool.data(), pool.size() * sizeof(uint32_t));
  return py::make_tuple(py::bytes(blob), static_cast<uint32_t>(descs.size()), tiles,
                        static_cast<uint64_t>(desc_bytes));
}

void bind_kernels(py::module_& m) {
  py::class_<KvtLayout>(m, "KvtLayout")
      .def(py::init([]() { return KvtLayout{}; }))
      .def_readwrite("block_stride", &KvtLayout::block_stride)
      .def_readwrite("kv_stride", &KvtLayout::kv_stride)
      .def_readwrite("token_stride", &KvtLayout::token_stride)
      .def_readwrite("head_stride", &KvtLayout::head_stride)
      .def_readwrite("scale_base", &KvtLayout::scale_base)
      .def_readwrite("scale_kv_stride", &KvtLayout::scale_kv_stride)
      .def_readwrite("scale_token_stride", &KvtLayout::scale_token_stride)
      .def_readwrite("scale_head_stride", &KvtLayout::scale_head_stride)
      .def_readwrite("ntpb", &KvtLayout::ntpb)
      .def_readwrite("num_heads", &KvtLayout::num_heads)
      .def_readwrite("head_bytes", &KvtLayout::head_bytes)
      .def_readwrite("num_blocks", &KvtLayout::num_blocks)
      .def_readwrite("kv_count", &KvtLayout::kv_count);

  py::class_<KvtSegRule>(m, "KvtSegRule")
      .def(py::init([](int64_t so, int64_t dof, int64_t ss, int64_t ds, uint32_t len, uint32_t count) {
             return KvtSegRule{so, dof, ss, ds, len, count};
           }),
           py::arg("src_off"), py::arg("dst_off"), py::arg("src_stride"), py::arg("dst_stride"), py::arg("len"),
           py::arg("count"))
      .def_readwrite("src_off", &KvtSegRule::src_off)
      .def_readwrite("dst_off", &KvtSegRule::dst_off)
      .def_readwrite("src_stride", &KvtSegRule::src_stride)
      .def_readwrite("dst_stride", &KvtSegRule::dst_stride)
      .def_readwrite("len", &KvtSegRule::len)
      .def_readwrite("count", &KvtSegRule::count)
      .def("pack", [](const KvtSegRule& r) {
        return py::bytes(reinterpret_cast<const char*>(&r), sizeof(KvtSegRule));
      });

  m.attr("KVT_MODE_COPY") = static_cast<int>(KVT_MODE_COPY);
  m.attr("KVT_MODE_BF16_TO_MXFP8") = static_cast<int>(KVT_MODE_BF16_TO_MXFP8);
  m.attr("KVT_MODE_MXFP8_TO_BF16") = static_cast<int>(KVT_MODE_MXFP8_TO_BF16);
  m.attr("KVT_REQ_PAD_TAIL") = static_cast<int>(KVT_REQ_PAD_TAIL);
  m.attr("KVT_REQ_DESC_BYTES") = static_cast<int>(sizeof(KvtReqDesc));
  m.attr("KVT_SEG_RULE_BYTES") = static_cast<int>(sizeof(KvtSegRule));
  m.attr("KVT_TENSOR_MAP_BYTES") = 128;

  m.def("kvt_req_tiles", &kvt_req_tiles);
  m.def("kvt_pack_plan", &pack_plan, py::arg("reqs"), py::arg("tile_tokens"), py::arg("dst_ntpb"),
        "Pack [(src_blocks, dst_blocks, seen, new, flags)] into (blob, n_reqs, total_tiles, pool_offset).");

  m.def(
      "kvt_encode_tensor_map",
      [](uint64_t base, const KvtLayout& l, uint32_t box_heads, uint32_t box_tokens, uint32_t token_inner) {
        alignas(64) char buf[128];
        const int r = kvt_encode_tensor_map_ordered(buf, base, &l, box_heads, box_tokens, token_inner);
        if (r != 0) throw std::runtime_error("cuTensorMapEncodeTiled failed: " + std::to_string(r));
        return py::bytes(buf, 128);
      },
      py::arg("base"), py::arg("layout"), py::arg("box_heads"), py::arg("box_tokens"), py::arg("token_inner") = 0);
  m.def("kvt_tile_is_flat", [](const KvtLayout& l, uint32_t n_heads, uint32_t tile_tokens, uint32_t token_inner) {
    return kvt_tile_is_flat(&l, n_heads, tile_tokens, token_inner) != 0;
  });

  m.def(
      "kvt_launch_p2d_attn",
      [](uint64_t src_layers, uint64_t dst_layers, uint64_t src_maps, uint64_t dst_maps, const KvtLayout& src,
         const KvtLayout& dst, uint32_t layer_begin, uint32_t layer_end, uint64_t reqs, uint32_t n_reqs,
         uint32_t total_tiles, uint64_t block_ids, uint32_t tile_tokens, uint32_t src_head0, uint32_t dst_head0,
         uint32_t n_heads, uint32_t mode, uint64_t status, uint64_t done_counter, uint64_t flag,
         uint64_t flag_value, int grid, int threads, int use_tma, uint64_t stream, uint32_t simt_tile,
         uint32_t dst_remote, uint32_t tile_order, uint32_t store_form, uint32_t tma_stages, uint32_t cache_hint) {
        KvtAttnLaunch a{};
        a.simt_tile = simt_tile;
        a.dst_remote = dst_remote;
        a.tile_order = tile_order;
        a.store_form = store_form;
        a.tma_stages = tma_stages;
        a.cache_hint = cache_hint;
        a.src_layers = reinterpret_cast<const uint64_t*>(src_layers);
        a.dst_layers = reinterpret_cast<const uint64_t*>(dst_layers);
        a.src_maps = reinterpret_cast<const void*>(src_maps);
        a.dst_maps = reinterpret_cast<const void*>(dst_maps);
        a.src = src;
        a.dst = dst;
        a.layer_begin = layer_begin;
        a.layer_end = layer_end;
        a.reqs = reinterpret_cast<const KvtReqDesc*>(reqs);
        a.n_reqs = n_reqs;
        a.total_tiles = total_tiles;
        a.block_ids = reinterpret_cast<const uint32_t*>(block_ids);
        a.tile_tokens = tile_tokens;
        a.src_head0 = src_head0;
        a.dst_head0 = dst_head0;
        a.n_heads = n_heads;
        a.mode = mode;
        a.status = reinterpret_cast<uint32_t*>(status);
        a.done_counter = reinterpret_cast<uint32_t*>(done_counter);
        a.flag = reinterpret_cast<uint64_t*>(flag);
        a.flag_value = flag_value;
        check_cuda(kvt_launch_p2d_attn(&a, grid, threads, use_tma, reinterpret_cast<void*>(stream)),
                   "kvt_launch_p2d_attn");
      },
      py::arg("src_layers"), py::arg("dst_layers"), py::arg("src_maps"), py::arg("dst_maps"), py::arg("src"),
      py::arg("dst"), py::arg("layer_begin"), py::arg("layer_end"), py::arg("reqs"), py::arg("n_reqs"),
      py::arg("total_tiles"), py::arg("block_ids"), py::arg("tile_tokens"), py::arg("src_head0"),
      py::arg("dst_head0"), py::arg("n_heads"), py::arg("mode"), py::arg("status"), py::arg("done_counter"),
      py::arg("flag"), py::arg("flag_value"), py::arg("grid"), py::arg("threads"), py::arg("use_tma"),
      py::arg("stream"), py::arg("simt_tile") = 0, py::arg("dst_remote") = 0, py::arg("tile_order") = 0,
      py::arg("store_form") = 0, py::arg("tma_stages") = 0, py::arg("cache_hint") = 0);

  m.def(
      "kvt_launch_p2d_state",
      [](uint64_t src_layers, uint64_t dst_layers, uint32_t layer_begin, uint32_t layer_end,
         int64_t src_block_stride, int64_t dst_block_stride, uint32_t src_num_blocks, uint32_t dst_num_blocks,
         uint64_t src_blocks, uint64_t dst_blocks, uint32_t n_pages, uint64_t rules, uint32_t n_rules,
         uint64_t status, uint64_t done_counter, uint64_t flag, uint64_t flag_value, int grid, int threads,
         uint64_t stream) {
        KvtStateLaunch a{};
        a.src_layers = reinterpret_cast<const uint64_t*>(src_layers);
        a.dst_layers = reinterpret_cast<const uint64_t*>(dst_layers);
        a.layer_begin = layer_begin;
        a.layer_end = layer_end;
        a.src_block_stride = src_block_stride;
        a.dst_block_stride = dst_block_stride;
        a.src_num_blocks = src_num_blocks;
        a.dst_num_blocks = dst_num_blocks;
        a.src_blocks = reinterpret_cast<const uint32_t*>(src_blocks);
        a.dst_blocks = reinterpret_cast<const uint32_t*>(dst_blocks);
        a.n_pages = n_pages;
        a.rules = reinterpret_cast<const KvtSegRule*>(rules);
        a.n_rules = n_rules;
        a.status = reinterpret_cast<uint32_t*>(status);
        a.done_counter = reinterpret_cast<uint32_t*>(done_counter);
        a.flag = reinterpret_cast<uint64_t*>(flag);
        a.flag_value = flag_value;
        check_cuda(kvt_launch_p2d_state(&a, grid, threads, reinterpret_cast<void*>(stream)), "kvt_launch_p2d_state");
      },
      py::arg("src_layers"), py::arg("dst_layers"), py::arg("layer_begin"), py::arg("layer_end"),
      py::arg("src_block_stride"), py::arg("dst_block_stride"), py::arg("src_num_blocks"),
      py::arg("dst_num_blocks"), py::arg("src_blocks"), py::arg("dst_blocks"), py::arg("n_pages"),
      py::arg("rules"), py::arg("n_rules"), py::arg("status"), py::arg("done_counter"), py::arg("flag"),
      py::arg("flag_value"), py::arg("grid"), py::arg("threads"), py::arg("stream"));

  m.def(
      "kvt_launch_copy_blocks",
      [](uint64_t src_base, uint64_t dst_base, uint64_t triples, uint32_t n, uint64_t src_cap, uint64_t dst_cap,
         uint64_t status, int grid, uint64_t stream) {
        check_cuda(kvt_launch_copy_blocks(src_base, dst_base, reinterpret_cast<const uint64_t*>(triples), n,
                                          src_cap, dst_cap, reinterpret_cast<uint32_t*>(status), grid,
                                          reinterpret_cast<void*>(stream)),
                   "kvt_launch_copy_blocks");
      },
      py::arg("src_base"), py::arg("dst_base"), py::arg("triples"), py::arg("n"), py::arg("src_capacity"),
      py::arg("dst_capacity"), py::arg("status"), py::arg("grid"), py::arg("stream"));

  m.def(
      "kvt_launch_copy_blocks_multi",
      [](const std::vector<uint64_t>& src_bases, const std::vector<uint64_t>& dst_bases,
         const std::vector<uint64_t>& src_caps, const std::vector<uint64_t>& dst_caps, const std::vector<uint32_t>& first,
         const std::vector<uint32_t>& count, uint64_t triples, uint64_t status, int grid, uint64_t stream,
         uint32_t bulk_rounds) {
        const size_t nt = src_bases.size();
        if (nt == 0 || nt > KVT_COPY_MAX_TENSORS || dst_bases.size() != nt || src_caps.size() != nt ||
            dst_caps.size() != nt || first.size() != nt || count.size() != nt)
          throw std::invalid_argument("kvt_launch_copy_blocks_multi: 1..8 entries, every list of that length");
        KvtCopyMulti a{};
        for (size_t t = 0; t < nt; ++t) {
          a.src_base[t] = src_bases[t];
          a.dst_base[t] = dst_bases[t];
          a.src_cap[t] = src_caps[t];
          a.dst_cap[t] = dst_caps[t];
          a.first[t] = first[t];
          a.count[t] = count[t];
        }
        a.n_tensors = static_cast<uint32_t>(nt);
        a.triples = reinterpret_cast<const uint64_t*>(triples);
        a.status = reinterpret_cast<uint32_t*>(status);
        if (bulk_rounds > 0) {
          check_cuda(kvt_launch_copy_blocks_bulk(&a, bulk_rounds, grid, reinterpret_cast<void*>(stream)),
                     "kvt_launch_copy_blocks_bulk");
        } else {
          check_cuda(kvt_launch_copy_blocks_multi(&a, grid, reinterpret_cast<void*>(stream)), "kvt_launch_copy_blocks_multi");
        }
      },
      py::arg("src_bases"), py::arg("dst_bases"), py::arg("src_caps"), py::arg("dst_caps"), py::arg("first"),
      py::arg("count"), py::arg("triples"), py::arg("status"), py::arg("grid"), py::arg("stream"),
      py::arg("bulk_rounds") = 0);
  m.def("kvt_bulk_rounds", &kvt_bulk_rounds, py::arg("first_len"), py::arg("max_len"));

  m.def(
      "kvt_launch_mc_fanout",
      [](uint64_t src_layers, uint64_t mc_layers, uint32_t layer_begin, uint32_t layer_end, int64_t src_block_stride,
         int64_t dst_block_stride, uint32_t src_num_blocks, uint32_t dst_num_blocks, uint64_t src_blocks,
         uint64_t dst_blocks, uint32_t n_blocks, uint32_t block_off, uint32_t block_len, uint64_t status,
         uint64_t done_counter, uint64_t mc_flag, uint64_t flag_value, int grid, uint64_t stream) {
        KvtMcFanout a{};
        a.src_layers = reinterpret_cast<const uint64_t*>(src_layers);
        a.mc_layers = reinterpret_cast<const uint64_t*>(mc_layers);
        a.layer_begin = layer_begin;
        a.layer_end = layer_end;
        a.src_block_stride = src_block_stride;
        a.dst_block_stride = dst_block_stride;
        a.src_num_blocks = src_num_blocks;
        a.dst_num_blocks = dst_num_blocks;
        a.src_blocks = reinterpret_cast<const uint32_t*>(src_blocks);
        a.dst_blocks = reinterpret_cast<const uint32_t*>(dst_blocks);
        a.n_blocks = n_blocks;
        a.block_off = block_off;
        a.block_len = block_len;
        a.status = reinterpret_cast<uint32_t*>(status);
        a.done_counter = reinterpret_cast<uint32_t*>(done_counter);
        a.mc_flag = reinterpret_cast<uint64_t*>(mc_flag);
        a.flag_value = flag_value;
        check_cuda(kvt_launch_mc_fanout(&a, grid, reinterpret_cast<void*>(stream)), "kvt_launch_mc_fanout");
      },
      py::arg("src_layers"), py::arg("mc_layers"), py::arg("layer_begin"), py::arg("layer_end"),
      py::arg("src_block_stride"), py::arg("dst_block_stride"), py::arg("src_num_blocks"), py::arg("dst_num_blocks"),
      py::arg("src_blocks"), py::arg("dst_blocks"), py::arg("n_blocks"), py::arg("block_off"), py::arg("block_len"),
      py::arg("status"), py::arg("done_counter"), py::arg("mc_flag"), py::arg("flag_value"), py::arg("grid"),
      py::arg("stream"));

  m.def("kvt_launch_copy_blocks_cast",
        [](uint64_t src_base, uint64_t dst_base, uint64_t triples, uint32_t n, uint64_t src_cap, uint64_t dst_cap,
           uint64_t status, int grid, uint64_t stream) {
          check_cuda(kvt_launch_copy_blocks_cast(src_base, dst_base, reinterpret_cast<const uint64_t*>(triples), n, src_cap,
                                                 dst_cap, reinterpret_cast<uint32_t*>(status), grid,
                                                 reinterpret_cast<void*>(stream)),
                     "kvt_launch_copy_blocks_cast");
        },
        py::arg("src_base"), py::arg("dst_base"), py::arg("triples"), py::arg("n"), py::arg("src_capacity"),
        py::arg("dst_capacity"), py::arg("status"), py::arg("grid"), py::arg("stream"));
  // end-to-end transfer check: the CPU function, and the kernel over device arrays of {off u64, len u32, index0 u32}
  m.def("kvt_checksum_host", [](py::buffer data, uint32_t index0) {
    const py::buffer_info bi = data.request();
    return kvt_checksum_host(bi.ptr, static_cast<uint64_t>(bi.size) * static_cast<uint64_t>(bi.itemsize), index0);
  }, py::arg("data"), py::arg("index0") = 0);
  m.def("kvt_launch_checksum",
        [](uint64_t bases, uint32_t n_bases, uint64_t capacity, uint64_t chunks, uint32_t n, uint64_t out, uint64_t status,
           int grid, uint64_t stream) {
          check_cuda(kvt_launch_checksum(reinterpret_cast<const uint64_t*>(bases), n_bases, capacity,
                                         reinterpret_cast<const KvtCheckChunk*>(chunks), n, reinterpret_cast<uint64_t*>(out),
                                         reinterpret_cast<uint32_t*>(status), grid, reinterpret_cast<void*>(stream)),
                     "kvt_launch_checksum");
        },
        py::arg("bases"), py::arg("n_bases"), py::arg("capacity"), py::arg("chunks"), py::arg("n"), py::arg("out"),
        py::arg("status"), py::arg("grid"), py::arg("stream"));
  // the row form: device arrays of {blk_off, n_blocks, seen, new_tokens, first, index} (u32 x 6) and of block ids
  m.def("kvt_launch_checksum_attn",
        [](uint64_t bases, uint32_t n_bases, uint64_t capacity, const KvtLayout& layout, uint32_t head0, uint32_t n_heads,
           uint64_t reqs, uint32_t n_reqs, uint32_t total_tokens, uint64_t pool, uint32_t pool_len, uint64_t out, uint64_t status,
           int grid, uint64_t stream) {
          check_cuda(kvt_launch_checksum_attn(reinterpret_cast<const uint64_t*>(bases), n_bases, capacity, &layout, head0, n_heads,
                                              reinterpret_cast<const KvtCheckReq*>(reqs), n_reqs, total_tokens,
                                              reinterpret_cast<const uint32_t*>(pool), pool_len, reinterpret_cast<uint64_t*>(out),
                                              reinterpret_cast<uint32_t*>(status), grid, reinterpret_cast<void*>(stream)),
                     "kvt_launch_checksum_attn");
        },
        py::arg("bases"), py::arg("n_bases"), py::arg("capacity"), py::arg("layout"), py::arg("head0"), py::arg("n_heads"),
        py::arg("reqs"),
        py::arg("n_reqs"), py::arg("total_tokens"), py::arg("pool"), py::arg("pool_len"), py::arg("out"), py::arg("status"),
        py::arg("grid"), py::arg("stream"));
  m.def("kvt_bf16_to_e4m3", [](uint16_t bits) { return static_cast<int>(kvt_bf16_to_e4m3(bits)); });

  m.def("kvt_launch_wait_flag", [](uint64_t flag, uint64_t value, uint64_t timeout_ns, uint64_t status,
                                   uint64_t stream) {
    check_cuda(kvt_launch_wait_flag(reinterpret_cast<const uint64_t*>(flag), value, timeout_ns,
                                    reinterpret_cast<uint32_t*>(status), reinterpret_cast<void*>(stream)),
               "kvt_launch_wait_flag");
  });
  m.def("kvt_launch_set_flag", [](uint64_t flag, uint64_t value, uint64_t stream) {
    check_cuda(kvt_launch_set_flag(reinterpret_cast<uint64_t*>(flag), value, reinterpret_cast<void*>(stream)),
               "kvt_launch_set_flag");
  });

  m.def("kvt_device_count", &kvt_device_count);
  m.def("kvt_can_access_peer", &kvt_can_access_peer);
  m.def("kvt_enable_peer_access",
        [](int dev, int peer) { check_cuda(kvt_enable_peer_access(dev, peer), "cudaDeviceEnablePeerAccess"); });
  m.def("kvt_p2p_attribute", &kvt_p2p_attribute);
  m.def("kvt_sm_count", &kvt_sm_count);
  m.def("kvt_ipc_get_handle", [](uint64_t ptr) {
    char h[64];
    uint64_t base = 0, size = 0;
    check_cuda(kvt_ipc_get_handle(ptr, h, &base, &size), "cudaIpcGetMemHandle");
    return py::make_tuple(py::bytes(h, 64), base, size);
  });
  m.def("kvt_ipc_open_handle", [](const std::string& h) {
    if (h.size() != 64) throw std::runtime_error("IPC handle must be 64 bytes");
    uint64_t p = 0;
    check_cuda(kvt_ipc_open_handle(h.data(), &p), "cudaIpcOpenMemHandle");
    return p;
  });
  m.def("kvt_ipc_close", [](uint64_t p) { check_cuda(kvt_ipc_close(p), "cudaIpcCloseMemHandle"); });
  m.def("kvt_malloc", [](uint64_t bytes) {
    uint64_t p = 0;
    check_cuda(kvt_malloc(bytes, &p), "cudaMalloc");
    return p;
  });
  m.def("kvt_free", [](uint64_t p) { check_cuda(kvt_free(p), "cudaFree"); });
  m.def("kvt_host_alloc_mapped", [](uint64_t bytes) {
    uint64_t h = 0, d = 0;
    check_cuda(kvt_host_alloc_mapped(bytes, &h, &d), "cudaHostAlloc");
    return py::make_tuple(h, d);
  });
  m.def("kvt_host_free", [](uint64_t p) { check_cuda(kvt_host_free(p), "cudaFreeHost"); });
  m.def("kvt_host_register", [](uint64_t p, uint64_t bytes) {
    uint64_t d = 0;
    check_cuda(kvt_host_register(p, bytes, &d), "cudaHostRegister");
    return d;
  });
  m.def("kvt_memcpy_async", [](uint64_t dst, uint64_t src, uint64_t bytes, uint64_t stream) {
    check_cuda(kvt_memcpy_async(dst, src, bytes, reinterpret_cast<void*>(stream)), "cudaMemcpyAsync");
  });
  m.def("kvt_memcpy_triples", [](uint64_t dst_base, uint64_t src_base, py::buffer triples, uint64_t stream) {
    const py::buffer_info bi = triples.request();
    if (bi.itemsize != 8 || bi.size % 3 != 0) throw std::invalid_argument("triples: a contiguous array of u64, 3 per copy");
    py::gil_scoped_release nogil;
    check_cuda(kvt_memcpy_triples(dst_base, src_base, static_cast<const uint64_t*>(bi.ptr),
                                  static_cast<uint32_t>(bi.size / 3), reinterpret_cast<void*>(stream)),
               "cudaMemcpyAsync");
  }, py::arg("dst_base"), py::arg("src_base"), py::arg("triples"), py::arg("stream"));
  m.def("kvt_host_unregister", [](uint64_t p) { check_cuda(kvt_host_unregister(p), "cudaHostUnregister"); });
}

}  // namespace kvx
