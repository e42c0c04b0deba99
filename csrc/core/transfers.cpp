// Host-side planning of uploads: a bounded ring of pinned staging memory and the packing of
// many small input writes into few contiguous DMA ranges.
//
// Two rules are taken from the reference's transfer layers
// (crates/orinfer-engine/src/backend/cuda/transfers.rs:1-200: bounded pinned slabs, uploads in
// stream order, the caller's buffer is free as soon as the call returns;
// backend/ascend/runtime/input_transfer.rs and host_transfer.rs: disjoint input views are
// packed into contiguous DMAs without reordering overlapping writes, and pageable bytes never
// back a DMA that is still in flight):
//   1. every upload is first copied into pinned memory owned by the ring, so the caller's
//      (pageable) buffer can be reused at once and is never the source of an active DMA;
//   2. staging space is reclaimed strictly in submission order, when the stream has passed the
//      copy that read it (the owner reports completed tickets).
// This file holds only the bookkeeping; the pinned allocation and the copies belong to the
// caller (PyTorch pinned tensors and cudaMemcpyAsync in the engine).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <vector>

namespace {

struct Ticket {
  uint64_t id;
  uint64_t offset, bytes;   // region of the ring, never wrapping (a wrap wastes the tail)
  uint64_t waste;           // tail bytes skipped before this region
};

struct Ring {
  uint64_t capacity, alignment;
  uint64_t head = 0;        // next free offset
  uint64_t used = 0;        // bytes held by live tickets, including wasted tails
  uint64_t next_id = 1;
  std::deque<Ticket> live;  // submission order
  uint64_t peak = 0, refused = 0;
};

struct Write {
  uint64_t offset, bytes;
};

}  // namespace

extern "C" {

void* orinfer_ring_create(uint64_t capacity, uint64_t alignment) {
  if (capacity == 0 || alignment == 0 || (alignment & (alignment - 1)) || capacity % alignment)
    return nullptr;
  auto* r = new Ring;
  r->capacity = capacity;
  r->alignment = alignment;
  return r;
}

void orinfer_ring_destroy(void* h) { delete static_cast<Ring*>(h); }

// Reserve `bytes` of staging space.  Returns a ticket id (> 0) and its offset, 0 when the
// ring cannot hold the request right now (the caller waits for the stream and retires
// tickets), -1 when the request can never fit.
int64_t orinfer_ring_acquire(void* h, uint64_t bytes, uint64_t* offset) {
  auto* r = static_cast<Ring*>(h);
  const uint64_t need = (std::max<uint64_t>(bytes, 1) + r->alignment - 1) / r->alignment * r->alignment;
  if (need > r->capacity) return -1;
  uint64_t at = r->head, waste = 0;
  if (at + need > r->capacity) {      // not enough room before the end: start over at 0
    waste = r->capacity - at;
    at = 0;
  }
  if (r->used + waste + need > r->capacity) {
    ++r->refused;
    return 0;
  }
  // live regions form one circular interval of length `used` that ends at `head`, so the
  // check above is all that keeps a new region off the ones still in flight
  Ticket t{r->next_id++, at, need, waste};
  r->live.push_back(t);
  r->used += waste + need;
  r->head = (at + need) % r->capacity;
  r->peak = std::max(r->peak, r->used);
  *offset = at;
  return static_cast<int64_t>(t.id);
}

// The stream has passed every copy up to and including ticket `id`: free them, in order.
// Returns the number of tickets retired; retiring out of order is refused (-1).
int orinfer_ring_retire_through(void* h, uint64_t id) {
  auto* r = static_cast<Ring*>(h);
  if (r->live.empty() || id < r->live.front().id) return 0;
  if (id > r->live.back().id) return -1;
  int n = 0;
  while (!r->live.empty() && r->live.front().id <= id) {
    r->used -= r->live.front().bytes + r->live.front().waste;
    r->live.pop_front();
    ++n;
  }
  if (r->live.empty()) r->head = 0, r->used = 0;   // an empty ring starts over, unfragmented
  return n;
}

// out: capacity, used, live tickets, peak used, refused acquisitions
void orinfer_ring_stats(void* h, uint64_t out[5]) {
  auto* r = static_cast<Ring*>(h);
  out[0] = r->capacity;
  out[1] = r->used;
  out[2] = r->live.size();
  out[3] = r->peak;
  out[4] = r->refused;
}

// ---- input packing -----------------------------------------------------------------------
// `n` writes (dst offset, length, source pointer) into an input block of `block_bytes` are
// applied to the staging image `stage` in the given order (so where two writes overlap the
// later one wins, as it would if each were its own copy) and the touched bytes are returned as
// disjoint ranges sorted by offset; ranges closer than `merge_gap` bytes are joined, trading a
// few untouched bytes for one DMA instead of two.  The bytes of a joined gap are taken from the
// staging image, which therefore has to mirror the device block (it does when every upload
// goes through it).  Returns the number of ranges, or -1 for a write outside the block.
int orinfer_pack_inputs(uint8_t* stage, uint64_t block_bytes, const uint64_t* offsets,
                        const uint64_t* lengths, const uint8_t* const* sources, int n,
                        uint64_t merge_gap, uint64_t* range_offsets, uint64_t* range_lengths,
                        int max_ranges) {
  std::vector<Write> dirty;
  dirty.reserve(n);
  for (int i = 0; i < n; ++i) {
    if (offsets[i] > block_bytes || lengths[i] > block_bytes - offsets[i]) return -1;
    if (lengths[i] == 0) continue;
    std::memcpy(stage + offsets[i], sources[i], lengths[i]);
    dirty.push_back({offsets[i], lengths[i]});
  }
  std::sort(dirty.begin(), dirty.end(),
            [](const Write& a, const Write& b) { return a.offset < b.offset; });
  int count = 0;
  for (const Write& w : dirty) {
    if (count && w.offset <= range_offsets[count - 1] + range_lengths[count - 1] + merge_gap) {
      const uint64_t end = std::max(range_offsets[count - 1] + range_lengths[count - 1],
                                    w.offset + w.bytes);
      range_lengths[count - 1] = end - range_offsets[count - 1];
      continue;
    }
    if (count == max_ranges) return -1;
    range_offsets[count] = w.offset;
    range_lengths[count] = w.bytes;
    ++count;
  }
  return count;
}

}  // extern "C"
