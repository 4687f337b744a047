// Host-side native I/O (no device code): a parallel safetensors writer / reader and a shared-memory message ring.
//
// * Safetensors: the reference saves checkpoints through `save_pretrained` on rank 0, one tensor after another
//   (openrlhf/utils/deepspeed/deepspeed.py:560-640). Here the Python side lays out the header, and the data section is
//   written / read with one pwrite / pread stream per thread, straight from / into the tensors' (pinned) host memory.
// * Ring: single-producer / single-consumer byte-message queue in POSIX shared memory for the controller <-> worker
//   runtime (payloads are copied once into the ring and once out, no pickling of tensor bytes). It takes the place of
//   Ray's object store for same-node transfers (openrlhf/trainer/ray/launcher.py:226-373 passes everything through
//   ray.put / ray.get). Every wait has a deadline.
#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <fcntl.h>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>
#include <vector>

namespace {

bool pwrite_all(int fd, const char* p, long long n, long long off) {
  while (n > 0) {
    const ssize_t w = pwrite(fd, p, (size_t)std::min<long long>(n, 1ll << 30), off);
    if (w < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    p += w; n -= w; off += w;
  }
  return true;
}

bool pread_all(int fd, char* p, long long n, long long off) {
  while (n > 0) {
    const ssize_t r = pread(fd, p, (size_t)std::min<long long>(n, 1ll << 30), off);
    if (r < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    if (r == 0) return false;   // short file
    p += r; n -= r; off += r;
  }
  return true;
}

// Work is cut into 64 MiB pieces handed out round-robin, so that one huge tensor is also written by all threads.
struct Piece { int tensor; long long off, len; };

std::vector<Piece> make_pieces(int n, const long long* sizes) {
  std::vector<Piece> v;
  const long long chunk = 64ll << 20;
  for (int i = 0; i < n; ++i)
    for (long long o = 0; o < sizes[i]; o += chunk) v.push_back({i, o, std::min(chunk, sizes[i] - o)});
  return v;
}

}  // namespace

// File = u64 header length | header (JSON, caller-padded) | data. offsets[i] is tensor i's offset inside the data
// section. Returns 0, or -1 (open), -2 (write), -3 (close / sync).
extern "C" int b200_st_write(const char* path, const char* header, long long header_len, int n,
                             const void* const* ptrs, const long long* sizes, const long long* offsets, int threads,
                             int do_fsync) {
  const int fd = open(path, O_CREAT | O_TRUNC | O_WRONLY, 0644);
  if (fd < 0) return -1;
  const uint64_t hl = (uint64_t)header_len;
  bool ok = pwrite_all(fd, reinterpret_cast<const char*>(&hl), 8, 0) && pwrite_all(fd, header, header_len, 8);
  const long long data0 = 8 + header_len;
  const std::vector<Piece> pieces = make_pieces(n, sizes);
  std::atomic<bool> good(ok);
  threads = std::max(1, std::min<int>(threads, (int)pieces.size()));
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t)
    pool.emplace_back([&, t]() {
      for (size_t i = t; i < pieces.size() && good.load(); i += threads) {
        const Piece& p = pieces[i];
        if (!pwrite_all(fd, static_cast<const char*>(ptrs[p.tensor]) + p.off, p.len, data0 + offsets[p.tensor] + p.off))
          good.store(false);
      }
    });
  for (auto& th : pool) th.join();
  if (!good.load()) {
    close(fd);
    return -2;
  }
  if (do_fsync && fsync(fd) != 0) {
    close(fd);
    return -3;
  }
  return close(fd) == 0 ? 0 : -3;
}

// Reads n byte ranges of the data section (which starts at data_start) into dst_ptrs.
extern "C" int b200_st_read(const char* path, long long data_start, int n, void* const* dst_ptrs, const long long* sizes,
                            const long long* offsets, int threads) {
  const int fd = open(path, O_RDONLY);
  if (fd < 0) return -1;
  const std::vector<Piece> pieces = make_pieces(n, sizes);
  std::atomic<bool> good(true);
  threads = std::max(1, std::min<int>(threads, (int)pieces.size()));
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t)
    pool.emplace_back([&, t]() {
      for (size_t i = t; i < pieces.size() && good.load(); i += threads) {
        const Piece& p = pieces[i];
        if (!pread_all(fd, static_cast<char*>(dst_ptrs[p.tensor]) + p.off, p.len, data_start + offsets[p.tensor] + p.off))
          good.store(false);
      }
    });
  for (auto& th : pool) th.join();
  close(fd);
  return good.load() ? 0 : -2;
}

// ---------------------------------------------------------------------------------------------- shared-memory ring
namespace {

struct RingHeader {
  uint64_t magic;
  uint64_t capacity;                       // bytes of the data area (power of two not required)
  alignas(64) std::atomic<uint64_t> head;  // total bytes written
  alignas(64) std::atomic<uint64_t> tail;  // total bytes read
  alignas(64) std::atomic<uint32_t> closed;
};

struct Ring {
  RingHeader* h;
  char* data;
  size_t map_bytes;
  std::string name;
  bool owner;
};

constexpr uint64_t RING_MAGIC = 0x62323030726e6731ull;

void ring_copy_in(Ring* r, uint64_t pos, const char* src, uint64_t n) {
  if (n == 0) return;   // an empty part may come with a null pointer
  const uint64_t cap = r->h->capacity, o = pos % cap;
  const uint64_t first = std::min(n, cap - o);
  memcpy(r->data + o, src, first);
  if (n > first) memcpy(r->data, src + first, n - first);
}

void ring_copy_out(Ring* r, uint64_t pos, char* dst, uint64_t n) {
  if (n == 0) return;
  const uint64_t cap = r->h->capacity, o = pos % cap;
  const uint64_t first = std::min(n, cap - o);
  memcpy(dst, r->data + o, first);
  if (n > first) memcpy(dst + first, r->data, n - first);
}

bool wait_until(const std::chrono::steady_clock::time_point& deadline, int& spins) {
  if (++spins < 200) {
    std::this_thread::yield();
  } else {
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
  return std::chrono::steady_clock::now() < deadline;
}

}  // namespace

extern "C" void* b200_ring_open(const char* name, long long capacity, int create) {
  const int fd = shm_open(name, create ? (O_CREAT | O_EXCL | O_RDWR) : O_RDWR, 0600);
  if (fd < 0) return nullptr;
  size_t bytes = sizeof(RingHeader) + (size_t)capacity;
  if (create) {
    if (ftruncate(fd, (off_t)bytes) != 0) {
      close(fd);
      shm_unlink(name);
      return nullptr;
    }
  } else {
    struct stat st;
    if (fstat(fd, &st) != 0 || (size_t)st.st_size < sizeof(RingHeader)) {
      close(fd);
      return nullptr;
    }
    bytes = (size_t)st.st_size;
  }
  void* m = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (m == MAP_FAILED) return nullptr;
  Ring* r = new Ring{static_cast<RingHeader*>(m), static_cast<char*>(m) + sizeof(RingHeader), bytes, name, create != 0};
  if (create) {
    r->h->capacity = (uint64_t)capacity;
    r->h->head.store(0);
    r->h->tail.store(0);
    r->h->closed.store(0);
    std::atomic_thread_fence(std::memory_order_release);
    r->h->magic = RING_MAGIC;
  } else if (r->h->magic != RING_MAGIC) {
    munmap(m, bytes);
    delete r;
    return nullptr;
  }
  return r;
}

// Message = u64 length + payload given as `parts` byte ranges (so a small pickled header and raw tensor bytes go out
// as one message without an intermediate copy). Returns 0, -1 timeout, -2 closed, -3 message larger than the ring.
extern "C" int b200_ring_send(void* handle, int parts, const void* const* ptrs, const long long* lens, int timeout_ms) {
  Ring* r = static_cast<Ring*>(handle);
  uint64_t total = 0;
  for (int i = 0; i < parts; ++i) total += (uint64_t)lens[i];
  const uint64_t need = total + 8;
  if (need > r->h->capacity) return -3;
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  int spins = 0;
  uint64_t head = r->h->head.load(std::memory_order_relaxed);
  while (r->h->capacity - (head - r->h->tail.load(std::memory_order_acquire)) < need) {
    if (r->h->closed.load()) return -2;
    if (!wait_until(deadline, spins)) return -1;
  }
  ring_copy_in(r, head, reinterpret_cast<const char*>(&total), 8);
  uint64_t pos = head + 8;
  for (int i = 0; i < parts; ++i) {
    ring_copy_in(r, pos, static_cast<const char*>(ptrs[i]), (uint64_t)lens[i]);
    pos += (uint64_t)lens[i];
  }
  r->h->head.store(pos, std::memory_order_release);
  return 0;
}

// Length of the next message (waits for one): >= 0, or -1 timeout, -2 closed and drained.
extern "C" long long b200_ring_peek(void* handle, int timeout_ms) {
  Ring* r = static_cast<Ring*>(handle);
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  int spins = 0;
  const uint64_t tail = r->h->tail.load(std::memory_order_relaxed);
  while (r->h->head.load(std::memory_order_acquire) - tail < 8) {
    if (r->h->closed.load()) return -2;
    if (!wait_until(deadline, spins)) return -1;
  }
  uint64_t len = 0;
  ring_copy_out(r, tail, reinterpret_cast<char*>(&len), 8);
  return (long long)len;
}

// Copies the next message (whose length b200_ring_peek returned) into dst and releases its space.
extern "C" int b200_ring_recv(void* handle, void* dst, long long len) {
  Ring* r = static_cast<Ring*>(handle);
  const uint64_t tail = r->h->tail.load(std::memory_order_relaxed);
  if (r->h->head.load(std::memory_order_acquire) - tail < 8 + (uint64_t)len) return -1;
  ring_copy_out(r, tail + 8, static_cast<char*>(dst), (uint64_t)len);
  r->h->tail.store(tail + 8 + (uint64_t)len, std::memory_order_release);
  return 0;
}

extern "C" long long b200_ring_capacity(void* handle) { return (long long)static_cast<Ring*>(handle)->h->capacity; }

extern "C" void b200_ring_close(void* handle, int mark_closed) {
  Ring* r = static_cast<Ring*>(handle);
  if (mark_closed) r->h->closed.store(1);
  const bool owner = r->owner;
  const std::string name = r->name;
  munmap(r->h, r->map_bytes);
  if (owner) shm_unlink(name.c_str());
  delete r;
}
