// Python binding of the shared host-DRAM block store.  Keys cross the boundary as one bytes
// object of concatenated 16-byte keys.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <string.h>

#include <memory>

#include "store/kvstore.h"

namespace py = pybind11;

namespace kvx {

namespace {
std::vector<StoreKey> unpack_keys(const py::bytes& b) {
  const std::string s = b;
  if (s.size() % 16 != 0) throw std::invalid_argument("keys must be a multiple of 16 bytes");
  std::vector<StoreKey> out(s.size() / 16);
  for (size_t i = 0; i < out.size(); ++i) {
    memcpy(&out[i].hi, s.data() + 16 * i, 8);
    memcpy(&out[i].lo, s.data() + 16 * i + 8, 8);
  }
  return out;
}

StoreKey one_key(const py::bytes& b) {
  auto v = unpack_keys(b);
  if (v.size() != 1) throw std::invalid_argument("expected exactly one 16-byte key");
  return v[0];
}
}  // namespace

void bind_store(py::module_& m) {
  py::class_<KvStore, std::unique_ptr<KvStore>>(m, "KvStore")
      .def_static(
          "open",
          [](const std::string& name, uint64_t slot_bytes, uint32_t n_slots, int mode, const std::string& tag) {
            return std::unique_ptr<KvStore>(KvStore::open(name, slot_bytes, n_slots, mode, tag));
          },
          py::arg("name"), py::arg("slot_bytes"), py::arg("n_slots"), py::arg("mode"), py::arg("format_tag") = "")
      .def_static("unlink", &KvStore::unlink)
      .def("lookup_prefix",
           [](KvStore& s, const py::bytes& keys) {
             auto k = unpack_keys(keys);
             py::gil_scoped_release nogil;
             return s.lookup_prefix(k);
           })
      .def("reserve",
           [](KvStore& s, const py::bytes& key, int64_t ttl_ms) {
             const StoreKey k = one_key(key);
             uint32_t slot = 0;
             ReserveResult r;
             {
               py::gil_scoped_release nogil;
               r = s.reserve(k, ttl_ms, &slot);
             }
             return py::make_tuple((int)r, r == ReserveResult::kNew ? (int64_t)slot : (int64_t)-1);
           },
           py::arg("key"), py::arg("ttl_ms") = 0)
      .def("seal", [](KvStore& s, const py::bytes& key) { return s.seal(one_key(key)); })
      .def("discard", [](KvStore& s, const py::bytes& key) { return s.discard(one_key(key)); })
      .def("pin_prefix",
           [](KvStore& s, const py::bytes& keys) {
             auto k = unpack_keys(keys);
             py::gil_scoped_release nogil;
             return s.pin_prefix(k);
           })
      .def("unpin",
           [](KvStore& s, const py::bytes& keys) {
             auto k = unpack_keys(keys);
             py::gil_scoped_release nogil;
             s.unpin(k);
           })
      .def("reap_dead_writers", &KvStore::reap_dead_writers)
      .def("reap_dead_readers", &KvStore::reap_dead_readers)
      .def("clear", &KvStore::clear)
      .def("advance_clock_for_test", &KvStore::advance_clock_for_test)
      .def("stats",
           [](KvStore& s) {
             const StoreStats st = s.stats();
             py::dict d;
             d["n_slots"] = st.n_slots;
             d["slot_bytes"] = st.slot_bytes;
             d["used"] = st.used;
             d["sealed"] = st.sealed;
             d["writing"] = st.writing;
             d["pinned"] = st.pinned;
             d["hits"] = st.hits;
             d["misses"] = st.misses;
             d["evictions"] = st.evictions;
             d["expired"] = st.expired;
             d["reserve_fail"] = st.reserve_fail;
             d["discards"] = st.discards;
             return d;
           })
      .def_property_readonly("data_ptr", [](KvStore& s) { return reinterpret_cast<uint64_t>(s.data()); })
      .def_property_readonly("data_bytes", &KvStore::data_bytes)
      .def_property_readonly("slot_bytes", &KvStore::slot_bytes)
      .def_property_readonly("n_slots", &KvStore::n_slots)
      .def_property_readonly("name", &KvStore::name);
  m.attr("STORE_RESERVE_NEW") = (int)ReserveResult::kNew;
  m.attr("STORE_RESERVE_EXISTS") = (int)ReserveResult::kExists;
  m.attr("STORE_RESERVE_BUSY") = (int)ReserveResult::kBusy;
  m.attr("STORE_RESERVE_FULL") = (int)ReserveResult::kFull;
}

}  // namespace kvx
