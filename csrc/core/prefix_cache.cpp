// Radix prefix cache over token ids at KV-page granularity.
//
// Every node stands for one full page (page_tokens token ids) below its parent, so a
// root-to-node path is a cached prompt prefix and the node's page id says where its
// KV lives.  Requests that match a path borrow those pages read-only; the cache
// holds one reference of its own on each indexed page.  Eviction removes leaves that
// no request is using, lowest utility first, where
//     utility = saved replay distance (tokens up to the node) * (1 + hits) / age
// so long, popular and recent prefixes survive (the reference ranks victims by saved
// replay distance x hits over freed bytes x age: crates/orinfer-engine/src/prefix.rs:207-511).
// A second tier keeps evicted pages' contents in host memory under its own budget
// (crates/orinfer-engine/src/prefix/tiered.rs:8-111): the node stays in the tree with
// page = -1 and a host handle until it is restored or dropped.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <unordered_map>
#include <vector>

#include "core_api.h"

namespace {

struct Node {
  int32_t id = 0;
  Node* parent = nullptr;
  std::vector<uint32_t> tokens;            // exactly page_tokens ids
  uint64_t media = 0;                      // hash of media spans overlapping this page
  int32_t page = -1;                       // device page, -1 when only on host
  int64_t host_handle = -1;                // host-tier slot, -1 when none
  int32_t users = 0;                       // live requests borrowing this node
  uint64_t hits = 0;
  uint64_t last_use = 0;
  int32_t depth = 0;                       // pages from the root, this one included
  std::multimap<uint64_t, Node*> children; // keyed by content hash
};

uint64_t hash_tokens(const uint32_t* t, int n, uint64_t media) {
  uint64_t h = 0xcbf29ce484222325ull ^ media;
  for (int i = 0; i < n; ++i) {
    h ^= t[i];
    h *= 0x100000001b3ull;
    h ^= h >> 29;
  }
  return h;
}

struct Cache {
  int page_tokens;
  Node root;
  std::unordered_map<int32_t, std::unique_ptr<Node>> nodes;
  int32_t next_id = 1;
  uint64_t clock = 0;
  // statistics
  uint64_t lookups = 0, hit_tokens = 0, miss_tokens = 0, inserted = 0, evicted = 0, offloaded = 0,
           restored = 0;
  int32_t device_pages = 0, host_pages = 0;

  Node* child(Node* parent, const uint32_t* t, uint64_t media) {
    const uint64_t h = hash_tokens(t, page_tokens, media);
    auto range = parent->children.equal_range(h);
    for (auto it = range.first; it != range.second; ++it) {
      Node* c = it->second;
      if (c->media == media && std::memcmp(c->tokens.data(), t, sizeof(uint32_t) * page_tokens) == 0)
        return c;
    }
    return nullptr;
  }

  void unlink(Node* n) {
    const uint64_t h = hash_tokens(n->tokens.data(), page_tokens, n->media);
    auto range = n->parent->children.equal_range(h);
    for (auto it = range.first; it != range.second; ++it)
      if (it->second == n) {
        n->parent->children.erase(it);
        break;
      }
    nodes.erase(n->id);
  }
};

double utility(const Cache& c, const Node& n) {
  const double age = static_cast<double>(c.clock - n.last_use) + 1.0;
  return static_cast<double>(n.depth) * c.page_tokens * (1.0 + static_cast<double>(n.hits)) / age;
}

}  // namespace

extern "C" {

void* orinfer_prefix_create(int page_tokens) {
  if (page_tokens <= 0) return nullptr;
  Cache* c = new Cache();
  c->page_tokens = page_tokens;
  return c;
}

void orinfer_prefix_destroy(void* handle) { delete static_cast<Cache*>(handle); }

// Longest cached prefix of tokens[0..n).  Writes node ids and device pages (page -1 =
// host-resident, must be restored before use) for up to max_out pages; returns the
// number of matched pages.  When `acquire` is set, every returned node gains a user.
// `limit_tokens` caps the match (a prompt must keep >= 1 token to run through the model).
int orinfer_prefix_match(void* handle, const uint32_t* tokens, int n, const uint64_t* media,
                         int limit_tokens, int acquire, int32_t* node_ids, int32_t* pages,
                         int max_out) {
  Cache* c = static_cast<Cache*>(handle);
  ++c->lookups;
  ++c->clock;
  Node* cur = &c->root;
  int matched = 0;
  const int usable = std::min(n, limit_tokens);
  while ((matched + 1) * c->page_tokens <= usable && matched < max_out) {
    Node* next = c->child(cur, tokens + static_cast<size_t>(matched) * c->page_tokens,
                          media ? media[matched] : 0);
    if (!next || (next->page < 0 && next->host_handle < 0)) break;
    node_ids[matched] = next->id;
    pages[matched] = next->page;
    if (acquire) {
      ++next->users;
      ++next->hits;
      next->last_use = c->clock;
    }
    cur = next;
    ++matched;
  }
  c->hit_tokens += static_cast<uint64_t>(matched) * c->page_tokens;
  c->miss_tokens += static_cast<uint64_t>(n - matched * c->page_tokens);
  return matched;
}

// Index the full pages of a prompt: pages[i] holds tokens[i*P .. (i+1)*P).  For each page
// adopted[i] = 1 when the cache newly indexed that page (the caller must add a pool
// reference for it), 0 when an equal node already existed.  Returns pages walked.
int orinfer_prefix_insert(void* handle, const uint32_t* tokens, int n, const uint64_t* media,
                          const int32_t* pages, int n_pages, int32_t* adopted,
                          int32_t* node_ids) {
  Cache* c = static_cast<Cache*>(handle);
  ++c->clock;
  Node* cur = &c->root;
  const int full = std::min(n / c->page_tokens, n_pages);
  for (int i = 0; i < full; ++i) {
    const uint32_t* t = tokens + static_cast<size_t>(i) * c->page_tokens;
    const uint64_t m = media ? media[i] : 0;
    Node* next = c->child(cur, t, m);
    adopted[i] = 0;
    if (!next) {
      auto node = std::make_unique<Node>();
      node->id = c->next_id++;
      node->parent = cur;
      node->tokens.assign(t, t + c->page_tokens);
      node->media = m;
      node->page = pages[i];
      node->depth = cur->depth + 1;
      node->last_use = c->clock;
      next = node.get();
      cur->children.emplace(hash_tokens(t, c->page_tokens, m), next);
      c->nodes.emplace(next->id, std::move(node));
      adopted[i] = 1;
      ++c->inserted;
      ++c->device_pages;
    } else if (next->page < 0 && pages[i] >= 0) {
      // A host-only node regains a device copy computed by this request.
      next->page = pages[i];
      adopted[i] = 1;
      ++c->device_pages;
    }
    next->last_use = c->clock;
    if (node_ids) node_ids[i] = next->id;
    cur = next;
  }
  return full;
}

void orinfer_prefix_release(void* handle, const int32_t* node_ids, int n) {
  Cache* c = static_cast<Cache*>(handle);
  for (int i = 0; i < n; ++i) {
    auto it = c->nodes.find(node_ids[i]);
    if (it != c->nodes.end() && it->second->users > 0) --it->second->users;
  }
}

// Release of a match that was never used (the request could not be admitted and will match
// again on its next attempt): the users go, and so do the hits the match counted, so that a
// request waiting for pages does not inflate the utility of its prefix with every retry.
void orinfer_prefix_abandon(void* handle, const int32_t* node_ids, int n) {
  Cache* c = static_cast<Cache*>(handle);
  for (int i = 0; i < n; ++i) {
    auto it = c->nodes.find(node_ids[i]);
    if (it == c->nodes.end()) continue;
    if (it->second->users > 0) --it->second->users;
    if (it->second->hits > 0) --it->second->hits;
  }
}

// Choose up to `want` evictable device pages (leaf-first, no users), lowest utility
// first.  With to_host != 0 the nodes stay indexed as host-resident (the caller copies
// the page out and later reports the host handle); otherwise they are removed.
// Writes (node id, page) pairs; returns the count.
int orinfer_prefix_evict(void* handle, int want, int to_host, int32_t* node_ids, int32_t* pages) {
  Cache* c = static_cast<Cache*>(handle);
  int done = 0;
  while (done < want) {
    Node* victim = nullptr;
    double best = 0.0;
    for (auto& kv : c->nodes) {
      Node* n = kv.second.get();
      if (n->page < 0 || n->users > 0) continue;
      bool blocked = false;
      for (auto& ch : n->children)
        if (!to_host || ch.second->page >= 0 || ch.second->users > 0) blocked = true;
      if (blocked) continue;
      const double u = utility(*c, *n);
      if (!victim || u < best) {
        victim = n;
        best = u;
      }
    }
    if (!victim) break;
    node_ids[done] = victim->id;
    pages[done] = victim->page;
    ++done;
    --c->device_pages;
    ++c->evicted;
    if (to_host) {
      victim->page = -1;            // stays indexed; caller reports its host handle next
      ++c->offloaded;
    } else {
      c->unlink(victim);            // a true leaf: nothing below it
    }
  }
  return done;
}

int orinfer_prefix_set_host(void* handle, int32_t node_id, int64_t host_handle) {
  Cache* c = static_cast<Cache*>(handle);
  auto it = c->nodes.find(node_id);
  if (it == c->nodes.end()) return -1;
  if (it->second->host_handle < 0 && host_handle >= 0) ++c->host_pages;
  if (it->second->host_handle >= 0 && host_handle < 0) --c->host_pages;
  it->second->host_handle = host_handle;
  return 0;
}

int64_t orinfer_prefix_host_handle(void* handle, int32_t node_id) {
  Cache* c = static_cast<Cache*>(handle);
  auto it = c->nodes.find(node_id);
  return it == c->nodes.end() ? -1 : it->second->host_handle;
}

int orinfer_prefix_restore(void* handle, int32_t node_id, int32_t page) {
  Cache* c = static_cast<Cache*>(handle);
  auto it = c->nodes.find(node_id);
  if (it == c->nodes.end() || it->second->page >= 0) return -1;
  it->second->page = page;
  ++c->device_pages;
  ++c->restored;
  return 0;
}

// Drop host-only leaves (lowest utility first) to free host slots; returns handles freed.
int orinfer_prefix_drop_host(void* handle, int want, int64_t* handles) {
  Cache* c = static_cast<Cache*>(handle);
  int done = 0;
  while (done < want) {
    Node* victim = nullptr;
    double best = 0.0;
    for (auto& kv : c->nodes) {
      Node* n = kv.second.get();
      if (n->page >= 0 || n->host_handle < 0 || n->users > 0 || !n->children.empty()) continue;
      const double u = utility(*c, *n);
      if (!victim || u < best) {
        victim = n;
        best = u;
      }
    }
    if (!victim) break;
    handles[done++] = victim->host_handle;
    --c->host_pages;
    c->unlink(victim);
  }
  return done;
}

void orinfer_prefix_stats(void* handle, uint64_t out[10]) {
  Cache* c = static_cast<Cache*>(handle);
  out[0] = c->lookups;
  out[1] = c->hit_tokens;
  out[2] = c->miss_tokens;
  out[3] = c->inserted;
  out[4] = c->evicted;
  out[5] = c->offloaded;
  out[6] = c->restored;
  out[7] = static_cast<uint64_t>(c->device_pages);
  out[8] = static_cast<uint64_t>(c->host_pages);
  out[9] = static_cast<uint64_t>(c->nodes.size());
}

}  // extern "C"
