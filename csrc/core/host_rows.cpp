// Conditional-memory support on the host: n-gram addressing of table rows, per-rank row
// shards and unique-row gather plans, and immutable INT8 row stores read through mmap with a
// bounded four-way row cache or a RAM-resident copy.
//
// Behaviour follows the reference's crates/orinfer-model-sdk/src/conditional_memory.rs
// (hash layout, explicit committed history, media barriers) and
// crates/orinfer-engine/src/host_rows.rs + host_rows/{cache,resident}.rs (ceil-divided
// shards, unique rows grouped by owner with a restore map, 4-way bounded cache, release of a
// resident table in 128 MiB pieces).  The tables are PLE / Engram style memories that are too
// large or too cold for HBM; a decode step needs a few dozen rows of them.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

thread_local std::string g_rows_error;
int fail(const std::string& m) {
  g_rows_error = m;
  return -1;
}

// ------------------------------------------------------------------ n-gram hasher
struct HashLayer {
  int64_t rows;
  int64_t mult[4];
  std::vector<int64_t> primes;   // heads * 3: order-2, order-3, order-4 buckets
  std::vector<int64_t> offsets;  // first table row of each bucket
};
struct Hasher {
  std::vector<uint32_t> token_map;
  uint32_t pad;
  std::vector<uint8_t> barrier;  // per token id
  int heads;
  std::vector<HashLayer> layers;
};

inline int64_t wrap_mul(int64_t a, int64_t b) {
  return static_cast<int64_t>(static_cast<uint64_t>(a) * static_cast<uint64_t>(b));
}
inline int64_t floor_mod(int64_t a, int64_t p) {
  const int64_t r = a % p;
  return r < 0 ? r + p : r;
}

// ------------------------------------------------------------------ row cache
constexpr int kWays = 4;
struct RowCache {
  size_t width = 0;
  std::vector<uint64_t> tags, ages;
  std::vector<uint8_t> data;
  uint64_t clock = 0;

  static size_t slots_for(size_t width, size_t budget) {
    const size_t overhead = 4096;
    if (budget <= overhead) return 0;
    return (budget - overhead) / (width + 16) / kWays * kWays;
  }
  size_t set_of(uint64_t row) const {
    row = (row ^ (row >> 30)) * 0xbf58476d1ce4e5b9ull;   // splitmix64 finaliser
    row = (row ^ (row >> 27)) * 0x94d049bb133111ebull;
    row ^= row >> 31;
    return static_cast<size_t>(row % (tags.size() / kWays)) * kWays;
  }
  const uint8_t* get(uint64_t row) {
    const size_t first = set_of(row);
    for (size_t s = first; s < first + kWays; ++s)
      if (tags[s] == row) {
        ages[s] = ++clock;
        return data.data() + s * width;
      }
    return nullptr;
  }
  void put(uint64_t row, const uint8_t* bytes) {
    const size_t first = set_of(row);
    size_t victim = first;
    for (size_t s = first; s < first + kWays; ++s) {
      if (tags[s] == UINT64_MAX) { victim = s; break; }
      if (ages[s] < ages[victim]) victim = s;
    }
    tags[victim] = row;
    ages[victim] = ++clock;
    std::memcpy(data.data() + victim * width, bytes, width);
  }
};

// ------------------------------------------------------------------ row store
constexpr size_t kReleaseChunk = size_t(128) << 20;

struct RowStore {
  int fd = -1;
  const uint8_t* map = nullptr;
  size_t map_bytes = 0;
  size_t data_offset = 0;
  size_t row_bytes = 0;
  uint64_t first = 0, rows = 0;      // global row range held by this file
  std::vector<uint8_t> resident;      // optional RAM copy (pread, not page cache)
  bool has_cache = false;
  RowCache cache;
  std::mutex mu;
  uint64_t hits = 0, misses = 0, gathered_rows = 0, gathered_bytes = 0;

  ~RowStore() {
    if (map) munmap(const_cast<uint8_t*>(map), map_bytes);
    if (fd >= 0) close(fd);
    release_resident();
  }
  void release_resident() {
    // give a very large table back piecewise so no single call stalls for seconds
    uint8_t* base = resident.data();
    const size_t page = static_cast<size_t>(sysconf(_SC_PAGESIZE));
    for (size_t off = 0; off < resident.size(); off += kReleaseChunk) {
      uintptr_t lo = (reinterpret_cast<uintptr_t>(base + off) + page - 1) / page * page;
      uintptr_t hi = reinterpret_cast<uintptr_t>(base + std::min(resident.size(), off + kReleaseChunk))
                     / page * page;
      if (hi > lo) madvise(reinterpret_cast<void*>(lo), hi - lo, MADV_DONTNEED);
    }
    std::vector<uint8_t>().swap(resident);
  }
  const uint8_t* source(uint64_t local) const {
    return (resident.empty() ? map + data_offset : resident.data()) + local * row_bytes;
  }
};

}  // namespace

extern "C" {

const char* orinfer_rows_error(void) { return g_rows_error.c_str(); }

// ---- n-gram hasher -------------------------------------------------------------------
// layers: for each layer `rows`, 4 multipliers, heads*3 primes, flattened as int64.
void* orinfer_ngram_create(const uint32_t* token_map, int vocab, uint32_t pad_token,
                           const uint32_t* barriers, int n_barriers, int heads,
                           const int64_t* layer_data, int n_layers) {
  if (vocab <= 0 || pad_token >= static_cast<uint32_t>(vocab) || heads <= 0 || heads > 64 ||
      n_layers <= 0 || n_layers > 64) {
    fail("invalid conditional-memory hash layout");
    return nullptr;
  }
  auto* h = new Hasher;
  h->token_map.assign(token_map, token_map + vocab);
  h->pad = pad_token;
  h->heads = heads;
  h->barrier.assign(vocab, 0);
  for (int i = 0; i < n_barriers; ++i) {
    if (barriers[i] >= static_cast<uint32_t>(vocab)) {
      delete h;
      fail("barrier token outside the tokenizer");
      return nullptr;
    }
    h->barrier[barriers[i]] = 1;
  }
  const int stride = 5 + heads * 3;
  for (int l = 0; l < n_layers; ++l) {
    const int64_t* d = layer_data + static_cast<size_t>(l) * stride;
    HashLayer layer;
    layer.rows = d[0];
    bool ok = layer.rows > 0;
    for (int k = 0; k < 4; ++k) {
      layer.mult[k] = d[1 + k];
      ok = ok && layer.mult[k] > 0 && (layer.mult[k] & 1);
    }
    int64_t offset = 0;
    for (int b = 0; b < heads * 3 && ok; ++b) {
      const int64_t p = d[5 + b];
      ok = p >= 2 && !__builtin_add_overflow(offset, p, &offset);
      layer.primes.push_back(p);
      layer.offsets.push_back(offset - p);
    }
    if (!ok || offset != layer.rows) {
      delete h;
      fail("invalid conditional-memory layer geometry (bucket sizes must sum to the table rows)");
      return nullptr;
    }
    h->layers.push_back(std::move(layer));
  }
  return h;
}

void orinfer_ngram_destroy(void* handle) { delete static_cast<Hasher*>(handle); }

int orinfer_ngram_width(void* handle) {
  auto* h = static_cast<Hasher*>(handle);
  return static_cast<int>(h->layers.size()) * h->heads * 3;
}

// out[token][layer][order][head]; valid[token] = 0 for barrier (media) tokens, whose row is
// zero.  `history` is the committed tokens before `tokens[0]` (only its last 3 matter), so
// chunked prefill and speculative roll-back give the same addresses as one pass.
int orinfer_ngram_hash(void* handle, const uint32_t* history, int n_history,
                       const uint32_t* tokens, int n, int64_t* out, uint8_t* valid) {
  auto* h = static_cast<Hasher*>(handle);
  const uint32_t vocab = static_cast<uint32_t>(h->token_map.size());
  for (int i = 0; i < n; ++i)
    if (tokens[i] >= vocab) return fail("token outside the tokenizer");
  for (int i = std::max(0, n_history - 3); i < n_history; ++i)
    if (history[i] >= vocab) return fail("history token outside the tokenizer");
  const int width = orinfer_ngram_width(handle);
  std::fill(out, out + static_cast<size_t>(n) * width, int64_t(0));
  const int64_t pad = h->token_map[h->pad];
  for (int row = 0; row < n; ++row) {
    valid[row] = 0;
    if (h->barrier[tokens[row]]) continue;
    valid[row] = 1;
    int64_t window[4] = {pad, pad, pad, pad};
    for (int shift = 0; shift < 4; ++shift) {
      uint32_t raw;
      if (shift <= row) {
        raw = tokens[row - shift];
      } else {
        const int back = shift - row;          // 1 = last committed token
        if (back > n_history) break;
        raw = history[n_history - back];
      }
      if (h->barrier[raw]) break;              // never look across a media boundary
      window[shift] = h->token_map[raw];
    }
    int64_t* dst = out + static_cast<size_t>(row) * width;
    for (size_t l = 0; l < h->layers.size(); ++l) {
      const HashLayer& layer = h->layers[l];
      int64_t rolling = wrap_mul(window[0], layer.mult[0]);
      for (int shift = 1; shift < 4; ++shift) {
        rolling ^= wrap_mul(window[shift], layer.mult[shift]);
        for (int head = 0; head < h->heads; ++head) {
          const int bucket = (shift - 1) * h->heads + head;
          dst[l * h->heads * 3 + bucket] =
              floor_mod(rolling, layer.primes[bucket]) + layer.offsets[bucket];
        }
      }
    }
  }
  return 0;
}

// ---- shards and gather plans ---------------------------------------------------------
int orinfer_row_shard(uint64_t rows, int ranks, int rank, uint64_t* first, uint64_t* count) {
  if (rows == 0 || ranks <= 0 || rank < 0 || rank >= ranks) return fail("invalid row shard topology");
  const uint64_t span = (rows + ranks - 1) / ranks;
  *first = std::min(rows, span * static_cast<uint64_t>(rank));
  *count = std::min(span, rows - *first);
  return 0;
}

// Unique rows grouped by owning rank (in first-seen order inside a rank).  rows_out gets
// the unique rows (capacity n), restore[i] = position in rows_out of query i, starts has
// ranks + 1 entries.  Returns the number of unique rows.
int orinfer_row_plan(const int64_t* ids, int n, uint64_t table_rows, int ranks, int max_queries,
                     uint64_t* rows_out, int32_t* restore, int32_t* starts) {
  if (n < 0 || n > max_queries || ranks <= 0 || ranks > 1024 || table_rows == 0)
    return fail("invalid host-row plan dimensions or query budget");
  const uint64_t span = (table_rows + ranks - 1) / ranks;
  std::unordered_map<uint64_t, int> slot_of;
  slot_of.reserve(n * 2 + 1);
  std::vector<uint64_t> unique;
  std::vector<int> original(n), counts(ranks, 0);
  for (int i = 0; i < n; ++i) {
    if (ids[i] < 0 || static_cast<uint64_t>(ids[i]) >= table_rows)
      return fail("conditional-memory row outside the table");
    const uint64_t row = static_cast<uint64_t>(ids[i]);
    auto it = slot_of.find(row);
    if (it == slot_of.end()) {
      it = slot_of.emplace(row, static_cast<int>(unique.size())).first;
      unique.push_back(row);
      ++counts[row / span];
    }
    original[i] = it->second;
  }
  starts[0] = 0;
  for (int r = 0; r < ranks; ++r) starts[r + 1] = starts[r] + counts[r];
  std::vector<int> cursor(starts, starts + ranks), position(unique.size());
  for (size_t s = 0; s < unique.size(); ++s) {
    const int p = cursor[unique[s] / span]++;
    rows_out[p] = unique[s];
    position[s] = p;
  }
  for (int i = 0; i < n; ++i) restore[i] = position[original[i]];
  return static_cast<int>(unique.size());
}

// ---- INT8 row store --------------------------------------------------------------------
// A file of `rows` rows of `row_bytes` bytes starting at `data_offset`; it holds the global
// rows [first_row, first_row + rows).
void* orinfer_rows_open(const char* path, uint64_t data_offset, uint64_t row_bytes,
                        uint64_t first_row, uint64_t rows) {
  if (row_bytes == 0 || rows == 0) {
    fail("empty row store");
    return nullptr;
  }
  uint64_t extent;
  if (__builtin_mul_overflow(rows, row_bytes, &extent) ||
      __builtin_add_overflow(extent, data_offset, &extent)) {
    fail("row store extent overflow");
    return nullptr;
  }
  const int fd = open(path, O_RDONLY | O_CLOEXEC);
  if (fd < 0) {
    fail(std::string("cannot open ") + path);
    return nullptr;
  }
  struct stat st;
  if (fstat(fd, &st) != 0 || static_cast<uint64_t>(st.st_size) < extent) {
    close(fd);
    fail(std::string(path) + ": file is shorter than its declared rows");
    return nullptr;
  }
  void* m = mmap(nullptr, st.st_size, PROT_READ, MAP_SHARED, fd, 0);
  if (m == MAP_FAILED) {
    close(fd);
    fail(std::string("cannot map ") + path);
    return nullptr;
  }
  madvise(m, st.st_size, MADV_RANDOM);
  auto* s = new RowStore;
  s->fd = fd;
  s->map = static_cast<const uint8_t*>(m);
  s->map_bytes = st.st_size;
  s->data_offset = data_offset;
  s->row_bytes = row_bytes;
  s->first = first_row;
  s->rows = rows;
  return s;
}

void orinfer_rows_close(void* handle) { delete static_cast<RowStore*>(handle); }

// Bounded cache of hot rows; returns the number of slots (0 = budget too small, no cache).
long long orinfer_rows_enable_cache(void* handle, uint64_t budget_bytes) {
  auto* s = static_cast<RowStore*>(handle);
  std::lock_guard<std::mutex> lock(s->mu);
  const size_t slots = RowCache::slots_for(s->row_bytes, budget_bytes);
  if (slots == 0) return 0;
  try {
    s->cache.width = s->row_bytes;
    s->cache.tags.assign(slots, UINT64_MAX);
    s->cache.ages.assign(slots, 0);
    s->cache.data.assign(slots * s->row_bytes, 0);
  } catch (const std::bad_alloc&) {
    s->cache = RowCache();
    return fail("host row cache allocation failed");
  }
  s->has_cache = true;
  return static_cast<long long>(slots);
}

// Copy the whole table into RAM (refused above `budget_bytes`); the cache is dropped.
int orinfer_rows_make_resident(void* handle, uint64_t budget_bytes) {
  auto* s = static_cast<RowStore*>(handle);
  std::lock_guard<std::mutex> lock(s->mu);
  const uint64_t need = s->rows * s->row_bytes;
  if (need > budget_bytes) return fail("resident row table exceeds its memory budget");
  try {
    s->resident.resize(need);
  } catch (const std::bad_alloc&) {
    return fail("resident row table allocation failed");
  }
  size_t done = 0;
  while (done < need) {
    const ssize_t got = pread(s->fd, s->resident.data() + done,
                              std::min<size_t>(need - done, size_t(64) << 20),
                              s->data_offset + done);
    if (got <= 0) {
      s->release_resident();
      return fail("short read while loading a resident row table");
    }
    done += got;
  }
  s->has_cache = false;
  s->cache = RowCache();
  return 0;
}

int orinfer_rows_is_resident(void* handle) {
  return !static_cast<RowStore*>(handle)->resident.empty();
}

// Gather global rows `ids[0..n)` into `out` (n * row_bytes, refused above max_bytes).
int orinfer_rows_gather(void* handle, const uint64_t* ids, int n, uint8_t* out,
                        uint64_t max_bytes) {
  auto* s = static_cast<RowStore*>(handle);
  if (n < 0 || static_cast<uint64_t>(n) * s->row_bytes > max_bytes)
    return fail("host row gather exceeds its byte budget");
  for (int i = 0; i < n; ++i)
    if (ids[i] < s->first || ids[i] - s->first >= s->rows)
      return fail("row is outside this host shard");
  std::lock_guard<std::mutex> lock(s->mu);
  for (int i = 0; i < n; ++i) {
    uint8_t* dst = out + static_cast<size_t>(i) * s->row_bytes;
    const uint64_t local = ids[i] - s->first;
    if (s->has_cache) {
      if (const uint8_t* hit = s->cache.get(ids[i])) {
        std::memcpy(dst, hit, s->row_bytes);
        ++s->hits;
        continue;
      }
      ++s->misses;
      std::memcpy(dst, s->source(local), s->row_bytes);
      s->cache.put(ids[i], dst);
    } else {
      std::memcpy(dst, s->source(local), s->row_bytes);
    }
  }
  s->gathered_rows += n;
  s->gathered_bytes += static_cast<uint64_t>(n) * s->row_bytes;
  return 0;
}

// out: hits, misses, gathered rows, gathered bytes, cache slots, resident bytes
void orinfer_rows_stats(void* handle, uint64_t out[6]) {
  auto* s = static_cast<RowStore*>(handle);
  std::lock_guard<std::mutex> lock(s->mu);
  out[0] = s->hits;
  out[1] = s->misses;
  out[2] = s->gathered_rows;
  out[3] = s->gathered_bytes;
  out[4] = s->has_cache ? s->cache.tags.size() : 0;
  out[5] = s->resident.size();
}

}  // extern "C"
