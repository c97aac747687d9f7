// Step-descriptor ring between the tensor-parallel ranks of one node: a single-producer, multi-consumer
// broadcast ring in POSIX shared memory.
//
// The leader rank (the one that runs the scheduler and the HTTP front end) pushes one variable-length message per
// engine call; every follower rank pops every message in order and makes the same call on its own engine, so the
// ranks launch the same kernels in the same order and meet in the kernels' own collectives. The ring never touches
// the GPU or NCCL: a message costs one memcpy and one release store, and a follower that spins on the sequence word
// sees it within a cache-line transfer.
//
// Layout: [Header][data bytes, capacity a power of two]. `head` counts bytes ever written; each reader owns a
// `tail[r]` that counts bytes it has consumed. A message is [u32 length][payload][pad to 8]. The producer blocks
// (bounded by its timeout) while the slowest reader is more than capacity behind. A `closed` flag ends all waits.
//
// Reference counterpart: the host-side command channel between the TP engines (crates/engine/src/parallel/tp.rs,
// TpEngine::run mirrors each step to the second rank); there it is an in-process channel between two threads.
#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <fcntl.h>
#include <new>
#include <sys/mman.h>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>

#define API extern "C" __attribute__((visibility("default")))

namespace {

constexpr uint32_t RING_MAGIC = 0x4F574C52u;   // "OWLR"
constexpr int MAX_READERS = 15;

struct alignas(64) Cursor {
  std::atomic<uint64_t> v;
  char pad[56];
};

struct Header {
  uint32_t magic;
  uint32_t n_readers;
  uint64_t capacity;                 // bytes of the data area (power of two)
  std::atomic<uint32_t> closed;
  std::atomic<uint32_t> attached;    // readers that have opened the ring (diagnostics)
  char pad[40];
  Cursor head;
  Cursor tail[MAX_READERS];
};

struct Ring {
  Header* h;
  uint8_t* data;
  size_t map_bytes;
  int reader;          // -1: producer
  char name[96];
  bool owner;
};

inline uint64_t now_us() {
  return (uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(
             std::chrono::steady_clock::now().time_since_epoch()).count();
}

// Spin briefly, then yield, then sleep: a follower that waits for the next decode step is usually served within
// microseconds, one that waits for the next request may wait seconds.
inline void backoff(uint32_t& spins) {
  ++spins;
  if (spins < 2000) {
#if defined(__x86_64__)
    __builtin_ia32_pause();
#endif
  } else if (spins < 4000) {
    std::this_thread::yield();
  } else {
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

void copy_in(Ring* r, uint64_t pos, const void* src, size_t n) {
  const uint64_t cap = r->h->capacity, off = pos & (cap - 1);
  const size_t first = n < cap - off ? n : (size_t)(cap - off);
  memcpy(r->data + off, src, first);
  if (first < n) memcpy(r->data, (const uint8_t*)src + first, n - first);
}
void copy_out(Ring* r, uint64_t pos, void* dst, size_t n) {
  const uint64_t cap = r->h->capacity, off = pos & (cap - 1);
  const size_t first = n < cap - off ? n : (size_t)(cap - off);
  memcpy(dst, r->data + off, first);
  if (first < n) memcpy((uint8_t*)dst + first, r->data, n - first);
}

Ring* map_ring(const char* name, int fd, size_t bytes, int reader, bool owner) {
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) return nullptr;
  Ring* r = new (std::nothrow) Ring();
  if (!r) { munmap(p, bytes); return nullptr; }
  r->h = reinterpret_cast<Header*>(p);
  r->data = reinterpret_cast<uint8_t*>(p) + sizeof(Header);
  r->map_bytes = bytes;
  r->reader = reader;
  r->owner = owner;
  strncpy(r->name, name, sizeof(r->name) - 1);
  return r;
}

}  // namespace

// Producer side: creates (or replaces) the named ring. capacity is rounded up to a power of two (>= 4096).
API void* owl_ring_create(const char* name, uint64_t capacity, int n_readers) {
  if (!name || n_readers < 1 || n_readers > MAX_READERS) return nullptr;
  uint64_t cap = 4096;
  while (cap < capacity) cap <<= 1;
  shm_unlink(name);
  int fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd < 0) return nullptr;
  const size_t bytes = sizeof(Header) + cap;
  if (ftruncate(fd, (off_t)bytes) != 0) { close(fd); shm_unlink(name); return nullptr; }
  Ring* r = map_ring(name, fd, bytes, -1, true);
  if (!r) { shm_unlink(name); return nullptr; }
  Header* h = r->h;
  h->n_readers = (uint32_t)n_readers;
  h->capacity = cap;
  h->closed.store(0);
  h->attached.store(0);
  h->head.v.store(0);
  for (int i = 0; i < MAX_READERS; ++i) h->tail[i].v.store(0);
  std::atomic_thread_fence(std::memory_order_release);
  h->magic = RING_MAGIC;            // last: readers wait for it
  return r;
}

// Consumer side: opens the named ring as reader `reader` (0-based), waiting up to timeout_ms for the producer to create it.
API void* owl_ring_open(const char* name, int reader, int timeout_ms) {
  if (!name || reader < 0 || reader >= MAX_READERS) return nullptr;
  const uint64_t t0 = now_us();
  for (;;) {
    int fd = shm_open(name, O_RDWR, 0600);
    if (fd >= 0) {
      struct stat st;
      if (fstat(fd, &st) == 0 && (size_t)st.st_size > sizeof(Header)) {
        Ring* r = map_ring(name, fd, (size_t)st.st_size, reader, false);
        if (r) {
          std::atomic_thread_fence(std::memory_order_acquire);
          if (r->h->magic == RING_MAGIC && (uint32_t)reader < r->h->n_readers &&
              sizeof(Header) + r->h->capacity == r->map_bytes) {
            r->h->attached.fetch_add(1);
            return r;
          }
          munmap(r->h, r->map_bytes);
          delete r;
        }
      } else {
        close(fd);
      }
    }
    if (now_us() - t0 > (uint64_t)timeout_ms * 1000ull) return nullptr;
    std::this_thread::sleep_for(std::chrono::milliseconds(2));
  }
}

// 0 ok, -1 bad argument / message larger than the ring, -2 timed out (a reader fell behind), -3 closed.
API int owl_ring_push(void* ring, const void* msg, uint32_t len, int timeout_ms) {
  Ring* r = reinterpret_cast<Ring*>(ring);
  if (!r || r->reader != -1 || (!msg && len)) return -1;
  Header* h = r->h;
  const uint64_t need = ((uint64_t)len + 4 + 7) & ~7ull;
  if (need > h->capacity) return -1;
  const uint64_t head = h->head.v.load(std::memory_order_relaxed);
  const uint64_t t0 = now_us();
  uint32_t spins = 0;
  for (;;) {
    if (h->closed.load(std::memory_order_acquire)) return -3;
    uint64_t slowest = head;
    for (uint32_t i = 0; i < h->n_readers; ++i) {
      const uint64_t t = h->tail[i].v.load(std::memory_order_acquire);
      if (t < slowest) slowest = t;
    }
    if (head + need - slowest <= h->capacity) break;
    if (timeout_ms >= 0 && now_us() - t0 > (uint64_t)timeout_ms * 1000ull) return -2;
    backoff(spins);
  }
  copy_in(r, head, &len, 4);
  if (len) copy_in(r, head + 4, msg, len);
  h->head.v.store(head + need, std::memory_order_release);
  return 0;
}

// Returns the message length (>= 0) and copies it into buf; -1 bad argument, -2 timed out, -3 closed and drained,
// -4 buf too small (the message stays queued; *need receives its length).
API int64_t owl_ring_pop(void* ring, void* buf, uint32_t cap, int timeout_ms, uint32_t* need) {
  Ring* r = reinterpret_cast<Ring*>(ring);
  if (!r || r->reader < 0 || (!buf && cap)) return -1;
  Header* h = r->h;
  Cursor& mine = h->tail[r->reader];
  const uint64_t tail = mine.v.load(std::memory_order_relaxed);
  const uint64_t t0 = now_us();
  uint32_t spins = 0;
  while (h->head.v.load(std::memory_order_acquire) == tail) {
    if (h->closed.load(std::memory_order_acquire)) return -3;
    if (timeout_ms >= 0 && now_us() - t0 > (uint64_t)timeout_ms * 1000ull) return -2;
    backoff(spins);
  }
  uint32_t len = 0;
  copy_out(r, tail, &len, 4);
  if (need) *need = len;
  if (len > cap) return -4;
  if (len) copy_out(r, tail + 4, buf, len);
  mine.v.store(tail + (((uint64_t)len + 4 + 7) & ~7ull), std::memory_order_release);
  return (int64_t)len;
}

// Bytes queued for the slowest reader (producer) or for this reader (consumer).
API uint64_t owl_ring_backlog(void* ring) {
  Ring* r = reinterpret_cast<Ring*>(ring);
  if (!r) return 0;
  Header* h = r->h;
  const uint64_t head = h->head.v.load(std::memory_order_acquire);
  if (r->reader >= 0) return head - h->tail[r->reader].v.load(std::memory_order_acquire);
  uint64_t slowest = head;
  for (uint32_t i = 0; i < h->n_readers; ++i) {
    const uint64_t t = h->tail[i].v.load(std::memory_order_acquire);
    if (t < slowest) slowest = t;
  }
  return head - slowest;
}

API int owl_ring_attached(void* ring) {
  Ring* r = reinterpret_cast<Ring*>(ring);
  return r ? (int)r->h->attached.load() : -1;
}

// Marks the ring closed: pending pops drain what is queued and then return -3; pushes return -3.
API void owl_ring_close(void* ring) {
  Ring* r = reinterpret_cast<Ring*>(ring);
  if (r) r->h->closed.store(1, std::memory_order_release);
}

// Unmaps; the creator also unlinks the name.
API void owl_ring_free(void* ring) {
  Ring* r = reinterpret_cast<Ring*>(ring);
  if (!r) return;
  if (r->owner) shm_unlink(r->name);
  munmap(r->h, r->map_bytes);
  delete r;
}
