// Host-DRAM KV block store shared by every rank (and process) of a node.
//
// The reference has no store of its own: its "kvs" backends are adapters to external
// services (blade_kvt/hybrid_connector/kvsbackend.py:111-514 for Vineyard,
// mooncake_kvsbackend.py:172-634 for Mooncake).  This is the in-repo equivalent of what those
// services provide to the connector: a block-hash index, TTL, seal / discard, and a data arena
// the GPU can gather into and scatter out of directly.
//
// One POSIX shared-memory segment holds everything:
//
//   [Header | Entry table (open addressing) | free-slot stack | slot data ...]
//
// A *slot* is a fixed-size page: all layers of one KV block of one TP rank.  An *entry* maps a
// 128-bit key (chained hash of the block's tokens, salted with rank / model) to a slot and goes
//   EMPTY -> WRITING (reserve) -> SEALED (seal) -> EMPTY (evict / expire / discard).
// Readers pin sealed entries while a load is in flight; pinned and WRITING entries are never
// evicted.  All index operations take one process-shared robust mutex; data copies happen
// outside it (a slot's bytes are owned by its writer until seal, immutable afterwards).
// The data area is page-aligned so that each process can register it with CUDA
// (cudaHostRegister) and let kernels read / write it in place.
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

namespace kvx {

struct StoreKey {
  uint64_t hi = 0, lo = 0;
  bool operator==(const StoreKey& o) const { return hi == o.hi && lo == o.lo; }
};

enum class ReserveResult : int {
  kNew = 0,      // slot reserved for this writer
  kExists = 1,   // already sealed: nothing to write
  kBusy = 2,     // another writer holds it
  kFull = 3,     // no slot could be freed (everything pinned or being written)
};

struct StoreStats {
  uint64_t n_slots, slot_bytes, used, sealed, writing, pinned;
  uint64_t hits, misses, evictions, expired, reserve_fail, discards;
};

class KvStore {
 public:
  // kAttach: the segment must exist.  kCreate: an existing segment of that name is replaced.
  // kAttachOrCreate: the first opener creates it, everyone else attaches (engines of one node
  // sharing a store).  `format_tag` describes the slot format (layout id, sizes); attaching
  // with a different tag, slot size or slot count fails.
  enum OpenMode : int { kAttach = 0, kCreate = 1, kAttachOrCreate = 2 };
  static KvStore* open(const std::string& name, uint64_t slot_bytes, uint32_t n_slots, int mode,
                       const std::string& format_tag);
  static void unlink(const std::string& name);
  ~KvStore();

  // Number of leading keys that are sealed and not expired (refreshes their LRU stamp).
  uint32_t lookup_prefix(const std::vector<StoreKey>& keys);
  ReserveResult reserve(const StoreKey& key, int64_t ttl_ms, uint32_t* slot);
  bool seal(const StoreKey& key);              // WRITING (owned by this process) -> SEALED
  bool discard(const StoreKey& key);           // drops a WRITING entry of this process, or an unpinned sealed one
  // Pins the leading sealed keys and returns their slots; stops at the first miss.
  std::vector<uint32_t> pin_prefix(const std::vector<StoreKey>& keys);
  void unpin(const std::vector<StoreKey>& keys);
  // Drops WRITING entries whose writer process no longer exists; returns how many.
  uint32_t reap_dead_writers();
  // Releases the pins of reader processes that no longer exist (a reader that died between
  // pin_prefix and unpin would otherwise make its slots unevictable); returns how many pins.
  uint32_t reap_dead_readers();
  // Drops every entry that no reader has pinned; returns how many pinned entries stayed.
  uint32_t clear();

  StoreStats stats();
  uint8_t* data() const { return data_; }
  uint64_t data_bytes() const;
  uint64_t slot_bytes() const;
  uint32_t n_slots() const;
  const std::string& name() const { return name_; }
  // Test hook: shifts this handle's notion of "now" (TTL expiry) by `ms`.
  void advance_clock_for_test(int64_t ms) { clock_skew_ns_ += ms * 1000000; }

 private:
  KvStore() = default;
  struct Header;
  struct Entry;
  struct Guard;
  Entry* find(const StoreKey& key, bool for_insert);
  void free_entry(Entry* e);
  bool evict_one(int64_t now);
  void lru_unlink(uint32_t slot);
  void lru_push_front(uint32_t slot);
  void touch(Entry* e);
  int64_t now_ns() const;

  std::string name_;
  void* map_ = nullptr;
  uint64_t map_bytes_ = 0;
  Header* hdr_ = nullptr;
  Entry* table_ = nullptr;
  uint32_t* free_ = nullptr;
  uint32_t* lru_prev_ = nullptr;      // per slot: neighbours in the recency list of sealed entries
  uint32_t* lru_next_ = nullptr;
  uint32_t* slot_bucket_ = nullptr;   // per slot: table bucket of the entry that owns it
  uint8_t* data_ = nullptr;
  int64_t clock_skew_ns_ = 0;
};

}  // namespace kvx
