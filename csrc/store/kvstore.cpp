#include "store/kvstore.h"

#include <errno.h>
#include <fcntl.h>
#include <pthread.h>
#include <signal.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <stdexcept>

namespace kvx {

namespace {
constexpr uint64_t kMagic = 0x4b5653544f524533ull;  // "KVSTORE3"
constexpr uint32_t kEmpty = 0, kWriting = 1, kSealed = 2;
constexpr uint64_t kPage = 4096;

uint64_t round_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

std::string shm_name(const std::string& name) { return name.empty() || name[0] != '/' ? "/" + name : name; }
}  // namespace

struct KvStore::Header {
  uint64_t magic;
  uint64_t slot_bytes;
  uint32_t n_slots;
  uint32_t table_cap;  // power of two
  uint64_t table_off, free_off, data_off, total_bytes;
  char format_tag[128];
  pthread_mutex_t mu;
  uint32_t n_free;
  uint32_t n_entries;
  uint64_t clock;  // LRU stamp source
  uint32_t lru_head, lru_tail;  // slots of the most / least recently used SEALED entries (kNoSlot: empty list)
  uint64_t hits, misses, evictions, expired, reserve_fail, discards;
};

constexpr uint32_t kPinOwners = 4;
constexpr uint32_t kNoSlot = 0xffffffffu;

struct KvStore::Entry {
  uint64_t hi, lo;
  uint32_t slot;
  uint32_t state;
  uint32_t pins;       // all pins on the entry, whoever holds them
  uint32_t owner_pid;
  int64_t expire_ns;  // 0 = never
  uint64_t last_use;
  // Who holds the pins, so that a reader that died can be released: up to kPinOwners processes
  // are tracked per entry; pins of further processes count in `pins` only and stay until unpinned.
  uint32_t pin_pid[kPinOwners];
  uint32_t pin_cnt[kPinOwners];
};

// Takes the process-shared mutex; a holder that died leaves it recoverable (robust mutex).
struct KvStore::Guard {
  explicit Guard(Header* h) : h_(h) {
    const int rc = pthread_mutex_lock(&h_->mu);
    if (rc == EOWNERDEAD) pthread_mutex_consistent(&h_->mu);
  }
  ~Guard() { pthread_mutex_unlock(&h_->mu); }
  Header* h_;
};

int64_t KvStore::now_ns() const {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (int64_t)ts.tv_sec * 1000000000ll + ts.tv_nsec + clock_skew_ns_;
}

KvStore* KvStore::open(const std::string& name, uint64_t slot_bytes, uint32_t n_slots, int mode,
                       const std::string& format_tag) {
  bool create = mode == kCreate;
  if (slot_bytes == 0 || n_slots == 0) throw std::invalid_argument("KvStore: slot_bytes and n_slots must be > 0");
  if (format_tag.size() >= sizeof(Header::format_tag)) throw std::invalid_argument("KvStore: format tag too long");
  const std::string sname = shm_name(name);
  uint32_t cap = 16;
  while (cap < 2 * n_slots) cap <<= 1;
  const uint64_t table_off = round_up(sizeof(Header), 64);
  const uint64_t free_off = table_off + (uint64_t)cap * sizeof(Entry);
  // after the free list, three arrays indexed by slot: the recency list's links and the bucket that owns the slot
  const uint64_t links_off = free_off + (uint64_t)n_slots * 4;
  const uint64_t data_off = round_up(links_off + (uint64_t)n_slots * 12, kPage);
  const uint64_t total = data_off + round_up(slot_bytes * n_slots, kPage);

  int fd;
  if (mode == kAttachOrCreate) {
    // whoever wins the exclusive create initialises the segment; everyone else attaches
    fd = shm_open(sname.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd < 0 && errno == EEXIST) return open(name, slot_bytes, n_slots, kAttach, format_tag);
    if (fd < 0) throw std::runtime_error("KvStore: shm_open(create) failed: " + std::string(strerror(errno)));
    create = true;
  } else if (create) {
    shm_unlink(sname.c_str());
    fd = shm_open(sname.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd < 0) throw std::runtime_error("KvStore: shm_open(create) failed: " + std::string(strerror(errno)));
  }
  if (create) {
    if (ftruncate(fd, (off_t)total) != 0) {
      const int e = errno;
      close(fd);
      shm_unlink(sname.c_str());
      throw std::runtime_error("KvStore: ftruncate failed: " + std::string(strerror(e)));
    }
  } else {
    fd = shm_open(sname.c_str(), O_RDWR, 0600);
    if (fd < 0) throw std::runtime_error("KvStore: no such store '" + name + "': " + strerror(errno));
    // the creator may still be sizing the segment: give it a moment
    struct stat st {};
    for (int spin = 0; spin < 500; ++spin) {
      if (fstat(fd, &st) == 0 && st.st_size != 0) break;
      usleep(10000);
    }
    if ((uint64_t)st.st_size != total) {
      close(fd);
      throw std::runtime_error("KvStore: store '" + name + "' has a different geometry");
    }
  }
  void* map = mmap(nullptr, total, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (map == MAP_FAILED) throw std::runtime_error("KvStore: mmap failed: " + std::string(strerror(errno)));

  KvStore* s = new KvStore();
  s->name_ = name;
  s->map_ = map;
  s->map_bytes_ = total;
  s->hdr_ = reinterpret_cast<Header*>(map);
  s->table_ = reinterpret_cast<Entry*>(reinterpret_cast<uint8_t*>(map) + table_off);
  s->free_ = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(map) + free_off);
  s->lru_prev_ = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(map) + links_off);
  s->lru_next_ = s->lru_prev_ + n_slots;
  s->slot_bucket_ = s->lru_next_ + n_slots;
  s->data_ = reinterpret_cast<uint8_t*>(map) + data_off;
  Header* h = s->hdr_;
  if (create) {
    memset(h, 0, sizeof(Header));  // ftruncate'd pages are zero: the table starts EMPTY
    h->slot_bytes = slot_bytes;
    h->n_slots = n_slots;
    h->table_cap = cap;
    h->table_off = table_off;
    h->free_off = free_off;
    h->data_off = data_off;
    h->total_bytes = total;
    strncpy(h->format_tag, format_tag.c_str(), sizeof(h->format_tag) - 1);
    pthread_mutexattr_t at;
    pthread_mutexattr_init(&at);
    pthread_mutexattr_setpshared(&at, PTHREAD_PROCESS_SHARED);
    pthread_mutexattr_setrobust(&at, PTHREAD_MUTEX_ROBUST);
    pthread_mutex_init(&h->mu, &at);
    pthread_mutexattr_destroy(&at);
    for (uint32_t i = 0; i < n_slots; ++i) s->free_[i] = n_slots - 1 - i;  // pop order 0, 1, 2, ...
    h->n_free = n_slots;
    h->lru_head = h->lru_tail = kNoSlot;
    __atomic_store_n(&h->magic, kMagic, __ATOMIC_RELEASE);
  } else {
    for (int spin = 0; spin < 500 && __atomic_load_n(&h->magic, __ATOMIC_ACQUIRE) != kMagic; ++spin) usleep(10000);
    if (__atomic_load_n(&h->magic, __ATOMIC_ACQUIRE) != kMagic || h->slot_bytes != slot_bytes ||
        h->n_slots != n_slots || format_tag != h->format_tag) {
      const std::string have = h->format_tag;
      delete s;
      throw std::runtime_error("KvStore: store '" + name + "' was created with another format ('" + have +
                               "' vs '" + format_tag + "')");
    }
  }
  return s;
}

void KvStore::unlink(const std::string& name) { shm_unlink(shm_name(name).c_str()); }

KvStore::~KvStore() {
  if (map_ != nullptr) munmap(map_, map_bytes_);
}

uint64_t KvStore::data_bytes() const { return hdr_->slot_bytes * hdr_->n_slots; }
uint64_t KvStore::slot_bytes() const { return hdr_->slot_bytes; }
uint32_t KvStore::n_slots() const { return hdr_->n_slots; }

// Linear probing.  for_insert: returns the entry of the key if present, else the first empty
// bucket of its probe sequence.  Lookup: the entry or nullptr.
KvStore::Entry* KvStore::find(const StoreKey& key, bool for_insert) {
  const uint32_t mask = hdr_->table_cap - 1;
  uint32_t i = (uint32_t)(key.lo ^ (key.hi * 0x9e3779b97f4a7c15ull)) & mask;
  for (uint32_t n = 0; n <= mask; ++n, i = (i + 1) & mask) {
    Entry* e = &table_[i];
    if (e->state == kEmpty) return for_insert ? e : nullptr;
    if (e->hi == key.hi && e->lo == key.lo) return e;
  }
  return nullptr;
}

// Removes an entry and closes the gap in its probe run (backward-shift deletion), so that the
// table needs no tombstones.
void KvStore::lru_unlink(uint32_t slot) {
  const uint32_t p = lru_prev_[slot], n = lru_next_[slot];
  if (p != kNoSlot) lru_next_[p] = n; else hdr_->lru_head = n;
  if (n != kNoSlot) lru_prev_[n] = p; else hdr_->lru_tail = p;
  lru_prev_[slot] = lru_next_[slot] = kNoSlot;
}

void KvStore::lru_push_front(uint32_t slot) {
  lru_prev_[slot] = kNoSlot;
  lru_next_[slot] = hdr_->lru_head;
  if (hdr_->lru_head != kNoSlot) lru_prev_[hdr_->lru_head] = slot; else hdr_->lru_tail = slot;
  hdr_->lru_head = slot;
}

// A sealed entry was used: it becomes the most recent one.
void KvStore::touch(Entry* e) {
  e->last_use = ++hdr_->clock;
  if (e->state == kSealed && hdr_->lru_head != e->slot) {
    lru_unlink(e->slot);
    lru_push_front(e->slot);
  }
}

void KvStore::free_entry(Entry* e) {
  if (e->state == kSealed) lru_unlink(e->slot);
  free_[hdr_->n_free++] = e->slot;
  hdr_->n_entries--;
  const uint32_t mask = hdr_->table_cap - 1;
  uint32_t hole = (uint32_t)(e - table_);
  table_[hole].state = kEmpty;
  uint32_t j = hole;
  for (;;) {
    j = (j + 1) & mask;
    Entry* c = &table_[j];
    if (c->state == kEmpty) break;
    const uint32_t home = (uint32_t)(c->lo ^ (c->hi * 0x9e3779b97f4a7c15ull)) & mask;
    // c may move into the hole iff its home bucket is not inside (hole, j] cyclically
    const bool between = hole <= j ? (home > hole && home <= j) : (home > hole || home <= j);
    if (!between) {
      table_[hole] = *c;
      slot_bucket_[c->slot] = hole;     // the list finds an entry through its slot
      c->state = kEmpty;
      hole = j;
    }
  }
}

// Frees one unpinned sealed entry.  The recency list is walked from its old end: the first unpinned entry is
// the victim, unless one of the next few is past its lease, which then goes first.  A handful of list steps
// whatever the size of the store (the table is never scanned).
bool KvStore::evict_one(int64_t now) {
  constexpr int kLookahead = 32;
  Entry* victim = nullptr;
  bool victim_expired = false;
  int seen = 0;
  for (uint32_t s = hdr_->lru_tail; s != kNoSlot; s = lru_prev_[s]) {
    Entry* e = &table_[slot_bucket_[s]];
    if (e->state != kSealed || e->slot != s || e->pins != 0) continue;   // pinned: a reader is copying from it
    if (e->expire_ns != 0 && e->expire_ns <= now) {
      victim = e;
      victim_expired = true;
      break;
    }
    if (victim == nullptr) victim = e;
    if (++seen >= kLookahead) break;
  }
  if (victim == nullptr) return false;
  if (victim_expired)
    hdr_->expired++;
  else
    hdr_->evictions++;
  free_entry(victim);
  return true;
}

uint32_t KvStore::lookup_prefix(const std::vector<StoreKey>& keys) {
  Guard g(hdr_);
  const int64_t now = now_ns();
  uint32_t n = 0;
  for (const StoreKey& k : keys) {
    Entry* e = find(k, false);
    if (e != nullptr && e->state == kSealed && e->expire_ns != 0 && e->expire_ns <= now && e->pins == 0) {
      hdr_->expired++;
      free_entry(e);
      e = nullptr;
    }
    if (e == nullptr || e->state != kSealed) {
      hdr_->misses++;
      break;
    }
    touch(e);
    hdr_->hits++;
    ++n;
  }
  return n;
}

ReserveResult KvStore::reserve(const StoreKey& key, int64_t ttl_ms, uint32_t* slot) {
  Guard g(hdr_);
  const int64_t now = now_ns();
  Entry* e = find(key, false);
  if (e != nullptr) {
    if (e->state == kSealed) {
      if (e->expire_ns != 0 && e->expire_ns <= now && e->pins == 0) {
        hdr_->expired++;
        free_entry(e);
      } else {
        touch(e);
        if (ttl_ms > 0 && e->expire_ns != 0) e->expire_ns = now + ttl_ms * 1000000;  // a re-save renews the lease
        return ReserveResult::kExists;
      }
    } else {
      return ReserveResult::kBusy;
    }
  }
  if (hdr_->n_free == 0 && !evict_one(now)) {
    hdr_->reserve_fail++;
    return ReserveResult::kFull;
  }
  e = find(key, true);
  if (e == nullptr || e->state != kEmpty) {  // cannot happen with cap >= 2 * n_slots
    hdr_->reserve_fail++;
    return ReserveResult::kFull;
  }
  e->hi = key.hi;
  e->lo = key.lo;
  e->slot = free_[--hdr_->n_free];
  e->state = kWriting;
  e->pins = 0;
  memset(e->pin_pid, 0, sizeof(e->pin_pid));
  memset(e->pin_cnt, 0, sizeof(e->pin_cnt));
  e->owner_pid = (uint32_t)getpid();
  e->expire_ns = ttl_ms > 0 ? now + ttl_ms * 1000000 : 0;
  e->last_use = ++hdr_->clock;
  slot_bucket_[e->slot] = (uint32_t)(e - table_);
  lru_prev_[e->slot] = lru_next_[e->slot] = kNoSlot;      // joins the recency list when it is sealed
  hdr_->n_entries++;
  *slot = e->slot;
  return ReserveResult::kNew;
}

bool KvStore::seal(const StoreKey& key) {
  Guard g(hdr_);
  Entry* e = find(key, false);
  if (e == nullptr || e->state != kWriting || e->owner_pid != (uint32_t)getpid()) return false;
  e->state = kSealed;
  e->last_use = ++hdr_->clock;
  lru_push_front(e->slot);
  return true;
}

bool KvStore::discard(const StoreKey& key) {
  Guard g(hdr_);
  Entry* e = find(key, false);
  if (e == nullptr) return false;
  if (e->state == kWriting && e->owner_pid != (uint32_t)getpid()) return false;
  if (e->state == kSealed && e->pins != 0) return false;
  hdr_->discards++;
  free_entry(e);
  return true;
}

std::vector<uint32_t> KvStore::pin_prefix(const std::vector<StoreKey>& keys) {
  Guard g(hdr_);
  const int64_t now = now_ns();
  const uint32_t me = (uint32_t)getpid();
  std::vector<uint32_t> out;
  for (const StoreKey& k : keys) {
    Entry* e = find(k, false);
    if (e == nullptr || e->state != kSealed) break;
    if (e->expire_ns != 0 && e->expire_ns <= now && e->pins == 0) break;
    e->pins++;
    for (uint32_t r = 0, spare = kPinOwners; r <= kPinOwners; ++r) {
      if (r == kPinOwners) {     // not yet listed: take a spare record if there is one
        if (spare < kPinOwners) {
          e->pin_pid[spare] = me;
          e->pin_cnt[spare] = 1;
        }
        break;
      }
      if (e->pin_cnt[r] != 0 && e->pin_pid[r] == me) {
        e->pin_cnt[r]++;
        break;
      }
      if (e->pin_cnt[r] == 0 && spare == kPinOwners) spare = r;
    }
    touch(e);
    out.push_back(e->slot);
  }
  return out;
}

void KvStore::unpin(const std::vector<StoreKey>& keys) {
  Guard g(hdr_);
  const uint32_t me = (uint32_t)getpid();
  for (const StoreKey& k : keys) {
    Entry* e = find(k, false);
    if (e == nullptr || e->state != kSealed || e->pins == 0) continue;
    e->pins--;
    for (uint32_t r = 0; r < kPinOwners; ++r) {
      if (e->pin_cnt[r] != 0 && e->pin_pid[r] == me) {
        e->pin_cnt[r]--;
        break;
      }
    }
  }
}

uint32_t KvStore::reap_dead_readers() {
  Guard g(hdr_);
  uint32_t n = 0;
  for (uint32_t i = 0; i < hdr_->table_cap; ++i) {
    Entry* e = &table_[i];
    if (e->state != kSealed || e->pins == 0) continue;
    for (uint32_t r = 0; r < kPinOwners; ++r) {
      if (e->pin_cnt[r] == 0 || e->pin_pid[r] == (uint32_t)getpid()) continue;
      if (kill((pid_t)e->pin_pid[r], 0) != 0 && errno == ESRCH) {
        const uint32_t c = e->pin_cnt[r] < e->pins ? e->pin_cnt[r] : e->pins;
        e->pins -= c;
        e->pin_cnt[r] = 0;
        n += c;
      }
    }
  }
  return n;
}

uint32_t KvStore::reap_dead_writers() {
  Guard g(hdr_);
  uint32_t n = 0;
  for (uint32_t i = 0; i < hdr_->table_cap;) {
    Entry* e = &table_[i];
    if (e->state == kWriting && e->owner_pid != (uint32_t)getpid() && kill((pid_t)e->owner_pid, 0) != 0 &&
        errno == ESRCH) {
      free_entry(e);  // may shift another entry into bucket i: look at i again
      ++n;
      continue;
    }
    ++i;
  }
  return n;
}

uint32_t KvStore::clear() {
  Guard g(hdr_);
  uint32_t kept = 0;
  for (uint32_t i = 0; i < hdr_->table_cap; ++i)
    if (table_[i].state == kSealed && table_[i].pins != 0) ++kept;
  if (kept == 0) {
    memset(table_, 0, (size_t)hdr_->table_cap * sizeof(Entry));
    for (uint32_t i = 0; i < hdr_->n_slots; ++i) free_[i] = hdr_->n_slots - 1 - i;
    hdr_->n_free = hdr_->n_slots;
    hdr_->n_entries = 0;
    hdr_->lru_head = hdr_->lru_tail = kNoSlot;
    return 0;
  }
  // a reader is still copying out of a pinned slot: drop everything else, entry by entry
  for (uint32_t i = 0; i < hdr_->table_cap;) {
    Entry* e = &table_[i];
    if (e->state != kEmpty && !(e->state == kSealed && e->pins != 0)) {
      free_entry(e);  // may shift another entry into bucket i: look at i again
      continue;
    }
    ++i;
  }
  return kept;
}

StoreStats KvStore::stats() {
  Guard g(hdr_);
  StoreStats s{};
  s.n_slots = hdr_->n_slots;
  s.slot_bytes = hdr_->slot_bytes;
  s.used = hdr_->n_slots - hdr_->n_free;
  for (uint32_t i = 0; i < hdr_->table_cap; ++i) {
    const Entry& e = table_[i];
    if (e.state == kSealed) s.sealed++;
    if (e.state == kWriting) s.writing++;
    if (e.state == kSealed && e.pins > 0) s.pinned++;
  }
  s.hits = hdr_->hits;
  s.misses = hdr_->misses;
  s.evictions = hdr_->evictions;
  s.expired = hdr_->expired;
  s.reserve_fail = hdr_->reserve_fail;
  s.discards = hdr_->discards;
  return s;
}

}  // namespace kvx
