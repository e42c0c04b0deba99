// Graph registry: which launch geometries have a captured CUDA graph, per rank, and the rule
// that keeps the ranks' graphs identical.
//
// A captured graph records the collective and peer-memory work of its step.  If one rank
// replays a graph while another runs the same step directly (because it evicted the graph, or
// its capture failed), the two issue different sequences of collectives.  So graph use is
// decided for all ranks at once:
//
//   * every rank *probes* its own pool for the geometry (hit / miss, no side effect);
//   * the votes are combined; if every rank hits, all replay;
//   * if any rank misses, the ranks that hit invalidate their graph (it is handed back for
//     destruction and the entry's epoch is bumped, so a capture still in flight cannot be
//     committed), and all ranks capture again in the same step (or all run directly while
//     the geometry is still on trial).
//
// One registry object serves one process.  It may hold the pools of several ranks (threads of
// one process driving several GPUs) or one pool (one process per GPU, votes exchanged by the
// caller).  Pools are LRU with a fixed capacity; a geometry is captured at its `threshold`-th
// use, so one-off geometries never pay a capture.  The first error is sticky: every later
// call reports it, and the engine above fails closed.
//
// Counterpart of the reference's per-device graph-callback registry and its all-rank
// probe-then-recapture rule (crates/orinfer-engine/native/ascend/hccl_graph_registry.cc,
// crates/orinfer-engine/src/backend/ascend/graph.rs).
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <list>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace {

enum Decision : int { RUN_DIRECT = 0, CAPTURE = 1, REPLAY = 2 };
enum Error : int { OK = 0, E_ARG = -1, E_STICKY = -2, E_TIMEOUT = -3, E_STALE = -4 };

struct Entry {
  uint64_t key = 0;
  long long graph = -1;       // caller's handle; -1 while on trial
  int uses = 0;
  int epoch = 0;              // bumped whenever a held graph is invalidated
};

struct Pool {
  std::list<Entry> lru;       // front = most recently used
  std::unordered_map<uint64_t, std::list<Entry>::iterator> index;
};

struct Vote {
  uint64_t key = 0;
  int arrived = 0;
  int misses = 0;
  int generation = 0;         // completed votes
  int decision = RUN_DIRECT;
  int epoch = 0;
};

struct Registry {
  int world, capacity, threshold;
  std::mutex mu;
  std::condition_variable cv;
  std::vector<Pool> pools;
  Vote vote;
  int error = OK, error_rank = -1;
  long long hits = 0, captures = 0, recaptures = 0, evictions = 0;
};

Entry* find(Pool& p, uint64_t key) {
  auto it = p.index.find(key);
  return it == p.index.end() ? nullptr : &*it->second;
}

void touch(Pool& p, uint64_t key) {
  auto it = p.index.find(key);
  if (it != p.index.end()) p.lru.splice(p.lru.begin(), p.lru, it->second);
}

// Makes room for one more entry; returns the evicted graph handle or -1.
long long make_room(Registry& r, Pool& p) {
  long long freed = -1;
  while (static_cast<int>(p.lru.size()) >= r.capacity) {
    Entry& victim = p.lru.back();
    if (victim.graph >= 0) {
      freed = victim.graph;
      ++r.evictions;
    }
    p.index.erase(victim.key);
    p.lru.pop_back();
    if (freed >= 0) break;     // hand back one graph per call; trial entries go silently
  }
  return freed;
}

bool fail(Registry& r, int code, int rank) {
  if (r.error == OK) {
    r.error = code;
    r.error_rank = rank;
  }
  r.cv.notify_all();
  return false;
}

}  // namespace

extern "C" {

void* orinfer_greg_create(int world, int capacity, int threshold) {
  if (world < 1 || world > 64 || capacity < 1 || threshold < 1) return nullptr;
  auto* r = new Registry();
  r->world = world;
  r->capacity = capacity;
  r->threshold = threshold;
  r->pools.resize(world);
  return r;
}

void orinfer_greg_destroy(void* h) { delete static_cast<Registry*>(h); }

// 1 when `rank` holds a captured graph of the current epoch for `key`, else 0; negative on
// error.  No side effect.
int orinfer_greg_probe(void* h, int rank, uint64_t key) {
  auto* r = static_cast<Registry*>(h);
  if (!r || rank < 0 || rank >= r->world) return E_ARG;
  std::lock_guard<std::mutex> lock(r->mu);
  if (r->error != OK) return E_STICKY;
  Entry* e = find(r->pools[rank], key);
  return e && e->graph >= 0 ? 1 : 0;
}

// Applies a combined vote to `rank`'s pool and returns the decision for this use of `key`:
// REPLAY (graph handle in *graph), CAPTURE (capture now and `commit`), or RUN_DIRECT (still
// on trial).  `all_hit` = every rank's probe returned 1.  When a held graph is invalidated or
// an entry is evicted to make room, its handle is returned in *release (else -1) and the
// caller destroys it.  *epoch is the epoch a following commit must carry.
int orinfer_greg_decide(void* h, int rank, uint64_t key, int all_hit, long long* graph,
                        long long* release, int* epoch) {
  auto* r = static_cast<Registry*>(h);
  if (!r || rank < 0 || rank >= r->world || !graph || !release || !epoch) return E_ARG;
  std::lock_guard<std::mutex> lock(r->mu);
  if (r->error != OK) return E_STICKY;
  Pool& p = r->pools[rank];
  *graph = *release = -1;
  Entry* e = find(p, key);
  if (all_hit) {
    if (!e || e->graph < 0) {                            // the vote contradicts this pool
      fail(*r, E_STALE, rank);
      return E_STALE;
    }
    touch(p, key);
    ++e->uses;
    *graph = e->graph;
    *epoch = e->epoch;
    ++r->hits;
    return REPLAY;
  }
  // some rank missed: a graph held here is no longer usable
  if (e && e->graph >= 0) {
    *release = e->graph;
    e->graph = -1;
    ++e->epoch;                                          // a capture in flight is now stale
    ++r->recaptures;
  }
  if (!e) {
    const long long freed = make_room(*r, p);
    if (*release < 0) *release = freed;
    p.lru.push_front(Entry{key, -1, 0, 0});
    p.index[key] = p.lru.begin();
    e = &p.lru.front();
  } else {
    touch(p, key);
  }
  ++e->uses;
  *epoch = e->epoch;
  return e->uses >= r->threshold ? CAPTURE : RUN_DIRECT;
}

// Follower form of `decide`: applies the decision the leading rank took for this use of `key`
// (every rank executes a step once whether it replays, captures or runs directly, so a rank
// may fall back to a direct run without disturbing its peers).  Returns the decision this
// rank can carry out: the leader's, or RUN_DIRECT with *missed = 1 when REPLAY was asked for
// and this pool holds no graph; the caller reports the miss so that the leader evicts the
// geometry and every rank captures it again.
int orinfer_greg_follow(void* h, int rank, uint64_t key, int decision, long long* graph,
                        long long* release, int* epoch, int* missed) {
  auto* r = static_cast<Registry*>(h);
  if (!r || rank < 0 || rank >= r->world || !graph || !release || !epoch || !missed ||
      decision < RUN_DIRECT || decision > REPLAY)
    return E_ARG;
  std::lock_guard<std::mutex> lock(r->mu);
  if (r->error != OK) return E_STICKY;
  Pool& p = r->pools[rank];
  *graph = *release = -1;
  *missed = 0;
  Entry* e = find(p, key);
  if (decision == REPLAY) {
    if (e && e->graph >= 0) {
      touch(p, key);
      ++e->uses;
      *graph = e->graph;
      *epoch = e->epoch;
      ++r->hits;
      return REPLAY;
    }
    *missed = 1;
    decision = RUN_DIRECT;
  }
  if (e && e->graph >= 0) {                    // the leader no longer holds it: neither do we
    *release = e->graph;
    e->graph = -1;
    ++e->epoch;
    ++r->recaptures;
  }
  if (!e) {
    const long long freed = make_room(*r, p);
    if (*release < 0) *release = freed;
    p.lru.push_front(Entry{key, -1, 0, 0});
    p.index[key] = p.lru.begin();
    e = &p.lru.front();
  } else {
    touch(p, key);
  }
  ++e->uses;
  *epoch = e->epoch;
  return decision;
}

// Stores the graph captured for `key` at `epoch`.  A commit that carries an old epoch (a
// recapture was forced in between) is refused with E_STALE and the caller destroys the graph.
int orinfer_greg_commit(void* h, int rank, uint64_t key, long long graph, int epoch) {
  auto* r = static_cast<Registry*>(h);
  if (!r || rank < 0 || rank >= r->world || graph < 0) return E_ARG;
  std::lock_guard<std::mutex> lock(r->mu);
  if (r->error != OK) return E_STICKY;
  Entry* e = find(r->pools[rank], key);
  if (!e || e->graph >= 0 || epoch != e->epoch) return E_STALE;
  e->graph = graph;
  ++r->captures;
  return OK;
}

// Drops `key` from `rank`'s pool (e.g. its capture failed); the held handle, if any, is
// returned for destruction.  The next vote on this geometry then sees a miss.
long long orinfer_greg_evict(void* h, int rank, uint64_t key) {
  auto* r = static_cast<Registry*>(h);
  if (!r || rank < 0 || rank >= r->world) return E_ARG;
  std::lock_guard<std::mutex> lock(r->mu);
  Pool& p = r->pools[rank];
  auto it = p.index.find(key);
  if (it == p.index.end()) return -1;
  const long long g = it->second->graph;
  p.lru.erase(it->second);
  p.index.erase(it);
  if (g >= 0) ++r->evictions;
  return g;
}

// Drops every entry of `rank`; writes up to `cap` held handles to `out`, returns their count.
int orinfer_greg_clear(void* h, int rank, long long* out, int cap) {
  auto* r = static_cast<Registry*>(h);
  if (!r || rank < 0 || rank >= r->world) return E_ARG;
  std::lock_guard<std::mutex> lock(r->mu);
  Pool& p = r->pools[rank];
  int n = 0;
  for (const Entry& e : p.lru)
    if (e.graph >= 0 && n < cap && out) out[n++] = e.graph;
  p.lru.clear();
  p.index.clear();
  return n;
}

// Several ranks in one process: each rank thread calls this with its own probe result; the
// call returns when all `world` ranks have voted on the same key (1 = all hit, 0 = some
// missed) or fails closed: a different key from some rank, or a rank that does not arrive
// within `timeout_ms`, is a sticky error for everybody.
int orinfer_greg_vote(void* h, int rank, uint64_t key, int hit, int timeout_ms) {
  auto* r = static_cast<Registry*>(h);
  if (!r || rank < 0 || rank >= r->world) return E_ARG;
  std::unique_lock<std::mutex> lock(r->mu);
  if (r->error != OK) return E_STICKY;
  Vote& v = r->vote;
  if (v.arrived == 0) {
    v.key = key;
    v.misses = 0;
  } else if (v.key != key) {
    fail(*r, E_STALE, rank);
    return E_STALE;
  }
  if (!hit) ++v.misses;
  const int my_generation = v.generation;
  if (++v.arrived == r->world) {
    v.decision = v.misses == 0 ? 1 : 0;
    v.arrived = 0;
    ++v.generation;
    r->cv.notify_all();
    return v.decision;
  }
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  while (v.generation == my_generation && r->error == OK) {
    if (r->cv.wait_until(lock, deadline) == std::cv_status::timeout &&
        v.generation == my_generation) {
      fail(*r, E_TIMEOUT, rank);
      return E_TIMEOUT;
    }
  }
  if (v.generation == my_generation) return E_STICKY;
  return v.decision;
}

void orinfer_greg_fail(void* h, int rank, int code) {
  auto* r = static_cast<Registry*>(h);
  if (!r) return;
  std::lock_guard<std::mutex> lock(r->mu);
  fail(*r, code < 0 ? code : E_STICKY, rank);
}

// 0 while healthy, else the first error; *rank = who raised it.
int orinfer_greg_status(void* h, int* rank) {
  auto* r = static_cast<Registry*>(h);
  if (!r) return E_ARG;
  std::lock_guard<std::mutex> lock(r->mu);
  if (rank) *rank = r->error_rank;
  return r->error;
}

// out[0..5] = hits, captures, forced recaptures, evictions, entries of rank 0, graphs of rank 0
void orinfer_greg_stats(void* h, long long* out) {
  auto* r = static_cast<Registry*>(h);
  if (!r || !out) return;
  std::lock_guard<std::mutex> lock(r->mu);
  out[0] = r->hits;
  out[1] = r->captures;
  out[2] = r->recaptures;
  out[3] = r->evictions;
  out[4] = static_cast<long long>(r->pools[0].lru.size());
  long long g = 0;
  for (const Entry& e : r->pools[0].lru) g += e.graph >= 0;
  out[5] = g;
}

}  // extern "C"
