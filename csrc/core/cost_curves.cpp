// Bounded cost curves of real packets: measured step times keyed by the packet's family
// (execution domain, power-of-two buckets of context, decode rows and decode context), its
// prompt-token count and its execution path (direct launches, graph replay, shared graph).
// 256 cells at most, least recently used evicted.  Estimates prefer the exact cell, then
// another path of the same shape, then interpolation between the nearest measured token
// counts of the family, then the cold prior (tokens / cold rate).  The scheduler uses them
// to size prefill chunks against its budget and to price admissions.
// Behavioural contract: crates/orinfer-engine/src/scheduler/prefill.rs:5-130 of the reference
// (bounded cells, first sample after a set-up excluded, hot cost transferred between paths
// as a prior, x1.25 conservative cold transfer).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <map>
#include <tuple>

#include "core_api.h"

namespace {

struct Ewma {
  double mean = 0, dev = 0;
  uint64_t n = 0;
  void observe(double v) {
    if (n == 0) {
      mean = v;
    } else {
      dev = dev * 0.8 + std::fabs(v - mean) * 0.2;
      mean = mean * 0.8 + v * 0.2;
    }
    ++n;
  }
  double upper() const { return mean + 2 * dev; }
};

uint32_t bucket(uint32_t n) {
  uint32_t b = 1;
  while (b < std::max(n, 1u)) b <<= 1;
  return b;
}

using Family = std::tuple<int, uint32_t, uint32_t, uint32_t>;   // domain, ctx, rows, decode ctx
using Key = std::tuple<Family, uint32_t, int>;                   // family, tokens, path

struct Cell {
  Ewma time;
  uint64_t last = 0;
  bool primed = false;          // a sample taken together with a set-up (capture) came first
};

struct Curves {
  std::map<Key, Cell> cells;
  std::map<std::pair<Family, uint32_t>, int> mode;
  uint64_t clock = 0;
  double cold_token_s;
};

Family family(const OrinferWork& w) {
  return Family(w.domain, bucket(w.context), w.decode_rows ? bucket(w.decode_rows) : 0,
                bucket(w.decode_context));
}

bool measured(const Curves& c, const Family& f, uint32_t tokens, int path, double* mean,
              double* upper, uint64_t* n) {
  auto it = c.cells.find(Key(f, tokens, path));
  if (it == c.cells.end() || it->second.time.n == 0) return false;
  *mean = it->second.time.mean;
  *upper = it->second.time.upper();
  *n = it->second.time.n;
  return true;
}

}  // namespace

extern "C" {

void* orinfer_costs_create(double cold_tokens_per_s) {
  if (!(cold_tokens_per_s > 0) || !std::isfinite(cold_tokens_per_s)) return nullptr;
  Curves* c = new Curves();
  c->cold_token_s = 1.0 / cold_tokens_per_s;
  return c;
}
void orinfer_costs_destroy(void* h) { delete static_cast<Curves*>(h); }
int orinfer_costs_cells(void* h) { return static_cast<int>(static_cast<Curves*>(h)->cells.size()); }

// path: 0 direct, 1 graph replay, 2 shared graph.  setup_s > 0 marks a step that also paid a
// capture / load; only the first such sample of a cell is kept (as a primer).
void orinfer_costs_observe(void* h, const OrinferWork* w, int path, double seconds,
                           double setup_s) {
  Curves* c = static_cast<Curves*>(h);
  if (!std::isfinite(seconds) || seconds <= 0 || !std::isfinite(setup_s) || setup_s < 0 ||
      w->tokens + w->decode_rows == 0)
    return;
  const Family f = family(*w);
  const Key key(f, w->tokens, path);
  ++c->clock;
  if (!c->cells.count(key) && c->cells.size() >= 256) {
    auto old = std::min_element(c->cells.begin(), c->cells.end(), [](auto& a, auto& b) {
      return a.second.last < b.second.last;
    });
    c->cells.erase(old);
  }
  c->mode[{f, w->tokens}] = path;
  Cell& cell = c->cells[key];
  cell.last = c->clock;
  if (setup_s == 0) {
    if (cell.primed) {              // drop the primer once a clean sample exists
      cell.time = Ewma();
      cell.primed = false;
    }
    cell.time.observe(seconds);
  } else if (cell.time.n == 0) {
    cell.time.observe(seconds);
    cell.primed = true;
  }
}

// out: seconds, upper_s, samples, path.  path < 0 asks for the family's last used path.
void orinfer_costs_estimate(void* h, const OrinferWork* w, int path, double out[4]) {
  const Curves* c = static_cast<const Curves*>(h);
  out[0] = out[1] = out[2] = 0;
  const Family f = family(*w);
  if (path < 0) {
    auto m = c->mode.find({f, w->tokens});
    path = m == c->mode.end() ? 0 : m->second;
  }
  out[3] = path;
  if (w->tokens + w->decode_rows == 0) return;
  double mean, upper;
  uint64_t n;
  if (measured(*c, f, w->tokens, path, &mean, &upper, &n)) {
    out[0] = mean; out[1] = upper; out[2] = static_cast<double>(n);
    return;
  }
  for (int other = 0; other < 3; ++other)       // hot cost of another path as a prior
    if (other != path && measured(*c, f, w->tokens, other, &mean, &upper, &n)) {
      const double k = other == 0 && path != 0 ? 1.0 : 1.25;
      out[0] = mean * k; out[1] = upper * k;
      return;
    }
  // nearest measured token counts of the family on this path: interpolate / extrapolate
  bool lo_ok = false, hi_ok = false;
  uint32_t lo_t = 0, hi_t = 0;
  double lo_m = 0, lo_u = 0, hi_m = 0, hi_u = 0;
  for (const auto& kv : c->cells) {
    if (std::get<0>(kv.first) != f || std::get<2>(kv.first) != path || kv.second.time.n == 0)
      continue;
    const uint32_t t = std::get<1>(kv.first);
    if (t < w->tokens && (!lo_ok || t > lo_t)) {
      lo_ok = true; lo_t = t; lo_m = kv.second.time.mean; lo_u = kv.second.time.upper();
    }
    if (t > w->tokens && (!hi_ok || t < hi_t)) {
      hi_ok = true; hi_t = t; hi_m = kv.second.time.mean; hi_u = kv.second.time.upper();
    }
  }
  if (lo_ok && hi_ok) {
    const double a = static_cast<double>(w->tokens - lo_t) / (hi_t - lo_t);
    out[0] = lo_m + a * (hi_m - lo_m);
    out[1] = lo_u + a * (hi_u - lo_u);
  } else if (lo_ok && lo_t > 0) {
    const double k = static_cast<double>(w->tokens) / lo_t;   // linear in tokens beyond the data
    out[0] = lo_m * k; out[1] = lo_u * k;
  } else if (hi_ok) {
    out[0] = hi_m; out[1] = hi_u;                             // a smaller packet costs no more
  } else {
    out[0] = out[1] = (w->tokens + w->decode_rows) * c->cold_token_s;
  }
}

// Largest chunk (multiple of `quantum`, <= limit) whose upper estimate fits budget_s.
int orinfer_costs_fit_tokens(void* h, const OrinferWork* w, int path, double budget_s, int limit,
                             int quantum) {
  OrinferWork probe = *w;
  int best = 0;
  for (int t = quantum; t <= limit; t += quantum) {
    probe.tokens = static_cast<uint32_t>(t);
    double out[4];
    orinfer_costs_estimate(h, &probe, path, out);
    if (out[1] > budget_s) break;
    best = t;
  }
  return best > 0 ? best : std::min(quantum, limit);
}

}  // extern "C"
