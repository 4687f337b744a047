// Driver for the sanitizer builds of the host-only native code (csrc/host_io.cu compiled as C++):
// a producer / consumer pair over the shared-memory ring and a parallel safetensors write / read round trip.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <unistd.h>
#include <vector>

extern "C" {
void* b200_ring_open(const char* name, long long capacity, int create);
int b200_ring_send(void* handle, int parts, const void* const* ptrs, const long long* lens, int timeout_ms);
long long b200_ring_peek(void* handle, int timeout_ms);
int b200_ring_recv(void* handle, void* dst, long long len);
void b200_ring_close(void* handle, int mark_closed);
int b200_st_write(const char* path, const char* header, long long header_len, int n, const void* const* ptrs,
                  const long long* sizes, const long long* offsets, int threads, int do_fsync);
int b200_st_read(const char* path, long long data_start, int n, void* const* dst_ptrs, const long long* sizes,
                 const long long* offsets, int threads);
}

static int fail(const char* what) {
  std::fprintf(stderr, "FAILED: %s\n", what);
  return 1;
}

int main() {
  // ---- ring: small capacity so that messages wrap and the producer has to wait for space
  const std::string name = "/b200_san_" + std::to_string((long)getpid());
  void* prod = b200_ring_open(name.c_str(), 1 << 16, 1);
  if (!prod) return fail("ring create");
  void* cons = b200_ring_open(name.c_str(), 0, 0);
  if (!cons) return fail("ring attach");
  const int N = 3000;
  std::thread producer([&]() {
    std::vector<unsigned char> a, b;
    for (int i = 0; i < N; ++i) {
      a.assign(1 + (i * 37) % 5000, (unsigned char)(i & 0xff));
      b.assign((i * 11) % 3000, (unsigned char)((i >> 3) & 0xff));
      const void* ptrs[2] = {a.data(), b.data()};
      const long long lens[2] = {(long long)a.size(), (long long)b.size()};
      if (b200_ring_send(prod, 2, ptrs, lens, 20000) != 0) std::abort();
    }
  });
  std::vector<unsigned char> buf;
  for (int i = 0; i < N; ++i) {
    const long long len = b200_ring_peek(cons, 20000);
    const long long want = 1 + (i * 37) % 5000 + (i * 11) % 3000;
    if (len != want) return fail("ring length");
    buf.resize((size_t)len);
    if (b200_ring_recv(cons, buf.data(), len) != 0) return fail("ring recv");
    if (buf[0] != (unsigned char)(i & 0xff)) return fail("ring payload");
    if ((i * 11) % 3000 && buf[(size_t)len - 1] != (unsigned char)((i >> 3) & 0xff)) return fail("ring payload tail");
  }
  producer.join();
  if (b200_ring_peek(cons, 10) != -1) return fail("ring should be empty");
  b200_ring_close(cons, 0);
  b200_ring_close(prod, 1);

  // ---- safetensors-style file: header + three byte ranges written by 4 threads, read back by 3
  std::vector<std::vector<unsigned char>> t = {std::vector<unsigned char>(70 << 20), std::vector<unsigned char>(12345),
                                               std::vector<unsigned char>(1)};
  for (size_t k = 0; k < t.size(); ++k)
    for (size_t i = 0; i < t[k].size(); i += 4099) t[k][i] = (unsigned char)(i * 31 + k);
  const char header[] = "{\"fake\":1}      ";
  const void* ptrs[3] = {t[0].data(), t[1].data(), t[2].data()};
  const long long sizes[3] = {(long long)t[0].size(), (long long)t[1].size(), (long long)t[2].size()};
  const long long offs[3] = {0, sizes[0], sizes[0] + sizes[1]};
  const std::string path = "/tmp/b200_san_" + std::to_string((long)getpid()) + ".bin";
  if (b200_st_write(path.c_str(), header, 16, 3, ptrs, sizes, offs, 4, 0) != 0) return fail("st write");
  std::vector<std::vector<unsigned char>> r = {std::vector<unsigned char>(t[0].size()),
                                               std::vector<unsigned char>(t[1].size()), std::vector<unsigned char>(1)};
  void* dst[3] = {r[0].data(), r[1].data(), r[2].data()};
  if (b200_st_read(path.c_str(), 8 + 16, 3, dst, sizes, offs, 3) != 0) return fail("st read");
  for (size_t k = 0; k < t.size(); ++k)
    if (std::memcmp(t[k].data(), r[k].data(), t[k].size()) != 0) return fail("st round trip");
  std::remove(path.c_str());
  std::puts("SANITIZER_DRIVER_OK");
  return 0;
}
