// Safetensors reader: header index, mmap'd payload, parallel copy into caller buffers (pinned
// host memory for the upload path) with optional SHA-256 verification per tensor.
// Plays the role of the reference's weights reader (crates/orinfer-engine/src/weights.rs,
// weights/read.rs: safetensors index, mmap/pread, optional SHA-256, tensor sources for the
// asynchronous upload) and of its N reader threads (backend/cuda/weight_upload.rs:1-330).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstring>
#include <map>
#include <string>
#include <thread>
#include <vector>

#include "core_api.h"

namespace {

// ---------------------------------------------------------------- SHA-256 (FIPS 180-4)
struct Sha256 {
  uint32_t h[8];
  uint8_t buf[64];
  uint64_t len = 0;
  size_t fill = 0;
  Sha256() {
    static const uint32_t init[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a,
                                     0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
    std::memcpy(h, init, sizeof(h));
  }
  static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void block(const uint8_t* p) {
    static const uint32_t K[64] = {
        0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4,
        0xab1c5ed5, 0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe,
        0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f,
        0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7,
        0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc,
        0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85, 0xa2bfe8a1, 0xa81a664b,
        0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116,
        0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
        0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7,
        0xc67178f2};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = (uint32_t(p[4 * i]) << 24) | (uint32_t(p[4 * i + 1]) << 16) |
             (uint32_t(p[4 * i + 2]) << 8) | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t t1 = hh + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) +
                          K[i] + w[i];
      const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
      hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
  }
  void update(const uint8_t* p, size_t n) {
    len += n;
    if (fill) {
      const size_t take = std::min(n, 64 - fill);
      std::memcpy(buf + fill, p, take);
      fill += take; p += take; n -= take;
      if (fill == 64) { block(buf); fill = 0; }
    }
    for (; n >= 64; p += 64, n -= 64) block(p);
    if (n) { std::memcpy(buf, p, n); fill = n; }
  }
  std::string hex() {
    const uint64_t bits = len * 8;
    uint8_t pad[72] = {0x80};
    const size_t padlen = (fill < 56 ? 56 - fill : 120 - fill);
    uint8_t tail[8];
    for (int i = 0; i < 8; ++i) tail[i] = uint8_t(bits >> (56 - 8 * i));
    update(pad, padlen);
    len -= padlen;
    update(tail, 8);
    static const char* digits = "0123456789abcdef";
    std::string out;
    for (int i = 0; i < 8; ++i)
      for (int s = 28; s >= 0; s -= 4) out.push_back(digits[(h[i] >> s) & 15]);
    return out;
  }
};

// ---------------------------------------------------------------- header scanner
struct Tensor {
  std::string name, dtype;
  std::vector<long long> shape;
  long long begin = 0, end = 0;
};

struct File {
  int fd = -1;
  const uint8_t* map = nullptr;
  size_t size = 0, data0 = 0;
  std::vector<Tensor> tensors;
  std::map<std::string, std::string> metadata;
  std::string error;
};

struct Scanner {
  const char* p;
  const char* e;
  bool ok = true;
  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) {
    ws();
    if (p < e && *p == c) { ++p; return true; }
    return false;
  }
  std::string str() {
    std::string out;
    ws();
    if (p >= e || *p != '"') { ok = false; return out; }
    ++p;
    while (p < e && *p != '"') {
      if (*p == '\\' && p + 1 < e) {
        ++p;
        switch (*p) {
          case 'n': out.push_back('\n'); break;
          case 't': out.push_back('\t'); break;
          case 'u': out.push_back('?'); p += 4; break;     // names in checkpoints are ASCII
          default: out.push_back(*p);
        }
        ++p;
      } else {
        out.push_back(*p++);
      }
    }
    if (p >= e) ok = false; else ++p;
    return out;
  }
  long long num() {
    ws();
    long long v = 0;
    bool any = false;
    while (p < e && *p >= '0' && *p <= '9') { v = v * 10 + (*p++ - '0'); any = true; }
    if (!any) ok = false;
    return v;
  }
  std::vector<long long> nums() {
    std::vector<long long> out;
    if (!eat('[')) { ok = false; return out; }
    if (eat(']')) return out;
    do out.push_back(num()); while (ok && eat(','));
    if (!eat(']')) ok = false;
    return out;
  }
};

bool parse_header(File* f, const char* text, size_t n) {
  Scanner s{text, text + n};
  if (!s.eat('{')) return false;
  if (s.eat('}')) return true;
  do {
    const std::string name = s.str();
    if (!s.ok || !s.eat(':') || !s.eat('{')) return false;
    if (name == "__metadata__") {
      if (!s.eat('}')) {
        do {
          const std::string k = s.str();
          if (!s.eat(':')) return false;
          f->metadata[k] = s.str();
        } while (s.ok && s.eat(','));
        if (!s.eat('}')) return false;
      }
      continue;
    }
    Tensor t;
    t.name = name;
    do {
      const std::string key = s.str();
      if (!s.eat(':')) return false;
      if (key == "dtype") t.dtype = s.str();
      else if (key == "shape") t.shape = s.nums();
      else if (key == "data_offsets") {
        const auto o = s.nums();
        if (o.size() != 2) return false;
        t.begin = o[0];
        t.end = o[1];
      } else return false;
    } while (s.ok && s.eat(','));
    if (!s.eat('}')) return false;
    f->tensors.push_back(std::move(t));
  } while (s.ok && s.eat(','));
  return s.ok && s.eat('}');
}

}  // namespace

extern "C" {

// Opens and indexes a .safetensors file; nullptr on failure (see orinfer_st_error).
static thread_local std::string g_st_error;
const char* orinfer_st_error(void) { return g_st_error.c_str(); }

void* orinfer_st_open(const char* path) {
  File* f = new File();
  auto bail = [&](const std::string& why) -> void* {
    g_st_error = why;
    if (f->map) munmap(const_cast<uint8_t*>(f->map), f->size);
    if (f->fd >= 0) close(f->fd);
    delete f;
    return nullptr;
  };
  f->fd = open(path, O_RDONLY);
  if (f->fd < 0) return bail("cannot open file");
  struct stat st;
  if (fstat(f->fd, &st) != 0 || st.st_size < 8) return bail("file too small");
  f->size = static_cast<size_t>(st.st_size);
  void* m = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
  if (m == MAP_FAILED) return bail("mmap failed");
  f->map = static_cast<const uint8_t*>(m);
  uint64_t hlen = 0;
  std::memcpy(&hlen, f->map, 8);
  if (hlen > f->size - 8) return bail("header length exceeds the file");
  f->data0 = 8 + static_cast<size_t>(hlen);
  if (!parse_header(f, reinterpret_cast<const char*>(f->map + 8), static_cast<size_t>(hlen)))
    return bail("malformed safetensors header");
  for (const Tensor& t : f->tensors)
    if (t.begin < 0 || t.end < t.begin || f->data0 + static_cast<size_t>(t.end) > f->size)
      return bail("tensor extent outside the file: " + t.name);
  return f;
}

void orinfer_st_close(void* h) {
  File* f = static_cast<File*>(h);
  if (!f) return;
  if (f->map) munmap(const_cast<uint8_t*>(f->map), f->size);
  if (f->fd >= 0) close(f->fd);
  delete f;
}

int orinfer_st_count(void* h) { return static_cast<int>(static_cast<File*>(h)->tensors.size()); }

// name (<= cap chars), dtype (<= 8 chars), shape (<= 8 dims); returns the byte size or -1.
long long orinfer_st_info(void* h, int index, char* name, int cap, char* dtype, long long* shape,
                          int* ndim) {
  File* f = static_cast<File*>(h);
  if (index < 0 || index >= static_cast<int>(f->tensors.size())) return -1;
  const Tensor& t = f->tensors[index];
  if (static_cast<int>(t.name.size()) >= cap || t.shape.size() > 8 || t.dtype.size() > 7) return -1;
  std::strcpy(name, t.name.c_str());
  std::strcpy(dtype, t.dtype.c_str());
  *ndim = static_cast<int>(t.shape.size());
  for (size_t i = 0; i < t.shape.size(); ++i) shape[i] = t.shape[i];
  return t.end - t.begin;
}

// Value of a __metadata__ key into out (<= cap chars); returns its length or -1.
int orinfer_st_metadata(void* h, const char* key, char* out, int cap) {
  File* f = static_cast<File*>(h);
  auto it = f->metadata.find(key);
  if (it == f->metadata.end() || static_cast<int>(it->second.size()) >= cap) return -1;
  std::strcpy(out, it->second.c_str());
  return static_cast<int>(it->second.size());
}

// Copies tensors indices[0..n) into dst[i] with `workers` threads (largest first).  When
// digests != nullptr, digests[i] is a 64-char hex SHA-256 that tensor i must match (or
// nullptr to skip).  Returns 0, or 1 + the position of the first tensor that failed.
int orinfer_st_read(void* h, const int* indices, void* const* dst, int n, int workers,
                    const char* const* digests) {
  File* f = static_cast<File*>(h);
  std::vector<int> order(n);
  for (int i = 0; i < n; ++i) order[i] = i;
  std::sort(order.begin(), order.end(), [&](int a, int b) {
    const Tensor& ta = f->tensors[indices[a]];
    const Tensor& tb = f->tensors[indices[b]];
    return ta.end - ta.begin > tb.end - tb.begin;
  });
  std::atomic<int> next{0};
  std::atomic<int> failed{0};
  auto run = [&]() {
    for (;;) {
      const int j = next.fetch_add(1);
      if (j >= n || failed.load()) return;
      const int i = order[j];
      const Tensor& t = f->tensors[indices[i]];
      const uint8_t* src = f->map + f->data0 + t.begin;
      const size_t bytes = static_cast<size_t>(t.end - t.begin);
      if (bytes) std::memcpy(dst[i], src, bytes);  // an empty tensor may come with a null dst
      if (digests && digests[i]) {
        Sha256 sha;
        if (bytes) sha.update(static_cast<const uint8_t*>(dst[i]), bytes);
        if (sha.hex() != digests[i]) {
          int expected = 0;
          failed.compare_exchange_strong(expected, i + 1);
        }
      }
    }
  };
  workers = std::max(1, std::min(workers, 32));
  std::vector<std::thread> pool;
  for (int w = 1; w < workers; ++w) pool.emplace_back(run);
  run();
  for (auto& t : pool) t.join();
  return failed.load();
}

// SHA-256 of a byte range as 64 hex chars + NUL into out65.
void orinfer_sha256_hex(const void* data, long long bytes, char* out65) {
  Sha256 sha;
  sha.update(static_cast<const uint8_t*>(data), static_cast<size_t>(bytes));
  std::strcpy(out65, sha.hex().c_str());
}

}  // extern "C"
