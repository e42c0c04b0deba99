// Adaptive multi-token-prediction control and request-local prompt lookup, host only.
//
// Acceptance keeps one conditional acceptance probability per draft position (prior 0.7),
// updated only at positions that were actually tested, with an order-independent batch
// update; the expected yield of w-1 drafts is 1 + sum of prefix survivals.  select() scores
// every legal verification width by (mean cost - fixed) / expected tokens against the plain
// decode baseline x 0.98, lets uncalibrated or stale candidates spend a bounded loss
// budget, and never picks a plan whose upper cost exceeds the slack.
// Behavioural contract: crates/orinfer-engine/src/mtp/adaptive.rs:6-8,11-65,68-101,178-326
// and runtime/requests/prompt_lookup.rs:12-110 of the reference.
#include <algorithm>
#include <array>
#include <cmath>
#include <cstdint>
#include <deque>
#include <map>
#include <vector>

#include "core_api.h"

namespace {

constexpr int MAX_DRAFTS = 31;
constexpr int REFRESH_AFTER = 512;
constexpr int HOT_SAMPLES = 3;
constexpr int CALIBRATION_ROUNDS = HOT_SAMPLES + 1;

struct Acceptance {
  double probability[MAX_DRAFTS];
  uint64_t samples[MAX_DRAFTS];
  Acceptance() {
    for (int i = 0; i < MAX_DRAFTS; ++i) {
      probability[i] = 0.7;
      samples[i] = 0;
    }
  }
  double rate(int pos, double prior) const {
    return (pos < MAX_DRAFTS && samples[pos] > 0) ? probability[pos] : prior;
  }
};

// ---- prompt lookup
constexpr int KEY = 4, CONTEXT = 8, SAMPLED_CONTEXT = 7, WINDOW = 8192, COOLDOWN = 16;
using Key = std::array<uint32_t, KEY>;

struct PromptLookup {
  std::map<Key, std::deque<size_t>> index;
  std::deque<std::pair<Key, size_t>> order;
  size_t indexed = 0, misses = 0, cooldown = 0;

  void extend(const uint32_t* h, size_t n) {
    if (n < KEY) return;
    size_t first = std::max(indexed, n > WINDOW ? n - WINDOW : 0);
    for (size_t start = first; start + KEY <= n; ++start) {
      Key k;
      std::copy(h + start, h + start + KEY, k.begin());
      index[k].push_back(start);
      order.emplace_back(k, start);
      while (order.size() > WINDOW) {
        auto old = order.front();
        order.pop_front();
        auto it = index.find(old.first);
        it->second.pop_front();
        if (it->second.empty()) index.erase(it);
      }
    }
    indexed = n - KEY + 1;
  }

  long find(const uint32_t* h, size_t n, size_t count, size_t minimum) const {
    if (n < KEY || count == 0 || n < cooldown) return -1;
    Key k;
    std::copy(h + n - KEY, h + n, k.begin());
    auto it = index.find(k);
    if (it == index.end()) return -1;
    long best = -1;
    size_t longest = KEY - 1;
    int looked = 0;
    for (auto p = it->second.rbegin(); p != it->second.rend() && looked < 64; ++p, ++looked) {
      const size_t end = *p + KEY;
      if (end + count > n) continue;
      size_t matched = KEY;
      while (matched < CONTEXT && matched < end && h[end - matched - 1] == h[n - matched - 1])
        ++matched;
      if (matched > longest) {
        longest = matched;
        best = static_cast<long>(end);
      }
      if (longest == CONTEXT) break;
    }
    return longest >= minimum ? best : -1;
  }
};

}  // namespace

extern "C" {

// ---- acceptance statistics
void* orinfer_acceptance_create(void) { return new Acceptance(); }
void orinfer_acceptance_destroy(void* h) { delete static_cast<Acceptance*>(h); }

// counts: n pairs (proposed, accepted) of one packet.
void orinfer_acceptance_observe(void* h, const int* proposed, const int* accepted, int n) {
  Acceptance* a = static_cast<Acceptance*>(h);
  for (int j = 0; j < MAX_DRAFTS; ++j) {
    int attempts = 0, passed = 0;
    for (int i = 0; i < n; ++i) {
      if (proposed[i] > j && accepted[i] >= j) ++attempts;
      if (proposed[i] > j && accepted[i] > j) ++passed;
    }
    if (!attempts) continue;
    const double value = static_cast<double>(passed) / attempts;
    const double decay = std::pow(0.8, static_cast<double>(attempts));
    a->probability[j] = a->probability[j] * decay + value * (1.0 - decay);
    a->samples[j] += attempts;
  }
}

double orinfer_acceptance_rate(void* h, int position, double prior) {
  return static_cast<Acceptance*>(h)->rate(position, prior);
}

// Expected committed tokens of a round with `drafts` proposals: 1 + sum prefix survival.
double orinfer_acceptance_expected(void* h, int drafts) {
  const Acceptance* a = static_cast<Acceptance*>(h);
  double total = 1.0, prefix = 1.0;
  for (int i = 0; i < std::min(drafts, MAX_DRAFTS); ++i) {
    prefix *= a->rate(i, 0.7);
    total += prefix;
  }
  return total;
}

double orinfer_mtp_progress(const double* yields, int n, int batch, int latency) {
  double acc = 0;
  for (int i = 0; i < n; ++i) acc += latency ? 1.0 / yields[i] : yields[i];
  return latency ? static_cast<double>(batch) * batch / acc : acc;
}

// Places `budget` draft rows of one verification packet on `n` requests.  Request r accepts
// each of its drafts with probability rate[r] given that the one before was accepted, so its
// j-th draft is worth rate[r]^j committed tokens: rows go one at a time to the request whose
// next draft is worth most (optimal for this separable, concave gain), never more than cap[r]
// per request, and not at all once the next draft is worth less than `floor`.  Ties go to the
// request with fewer rows, then the lower index, so equal requests get equal shares.  Returns
// the rows placed.  Role of the reference's per-request draft selection under a
// verification-row budget (models/deepseek_v41/provider/dspark.rs:55-100, dspark/policy.rs).
int orinfer_mtp_allocate(const double* rate, const int* cap, int n, int budget, double floor,
                         int* counts) {
  if (n <= 0) return 0;
  std::vector<double> next(n);
  for (int r = 0; r < n; ++r) {
    counts[r] = 0;
    const double a = std::min(std::max(rate[r], 0.0), 1.0);
    next[r] = cap[r] > 0 ? a : -1.0;
  }
  int placed = 0;
  while (placed < budget) {
    int best = -1;
    for (int r = 0; r < n; ++r) {
      if (next[r] < 0.0 || next[r] < floor) continue;
      if (best < 0 || next[r] > next[best] + 1e-12 ||
          (std::fabs(next[r] - next[best]) <= 1e-12 && counts[r] < counts[best]))
        best = r;
    }
    if (best < 0) break;
    ++counts[best];
    ++placed;
    const double a = std::min(std::max(rate[best], 0.0), 1.0);
    next[best] = counts[best] < cap[best] ? next[best] * a : -1.0;
  }
  return placed;
}

// Returns the chosen candidate id or -1 (plain decode); flags: bit0 exploring, bit1 calibrating.
int orinfer_mtp_select(const OrinferMtpSelection* in, const OrinferMtpCandidate* cands, int n,
                       int* flags) {
  *flags = 0;
  const double normal = in->normal_s, fixed_s = in->fixed_s, slack = in->slack_s;
  const int batch = in->batch;
  if (batch == 0 || !std::isfinite(normal) || normal <= 0 || !std::isfinite(fixed_s) ||
      normal <= fixed_s || std::isnan(slack) || slack <= 0 || std::isnan(in->available_s) ||
      std::isnan(in->calibration_s) || in->calibration_s == -INFINITY ||
      (in->normal_last >= 0 && in->calls - in->normal_last >= REFRESH_AFTER))
    return -1;
  const double baseline = (normal - fixed_s) / batch;
  int best_id = -1;
  double best_score = baseline * 0.98;
  bool have_probe = false;
  int probe_id = -1, probe_cal = 0;
  long probe_rank0 = 0, probe_rank1 = 0;
  for (int i = 0; i < n; ++i) {
    const OrinferMtpCandidate& c = cands[i];
    if (c.width < 2 || !std::isfinite(c.expected_tokens) || c.expected_tokens < batch ||
        !std::isfinite(c.maximum_tokens) || c.maximum_tokens < batch)
      continue;
    const double available = c.samples < HOT_SAMPLES ? in->calibration_s : in->available_s;
    const double horizon = std::min(std::max(c.remaining_tokens / c.expected_tokens, 1.0), 3.0);
    const double hot = c.mean_s;
    const double mean = hot + c.transition_s / horizon;
    const double upper = c.upper_s + c.transition_s;
    if (!std::isfinite(mean) || mean <= 0 || !std::isfinite(upper) || upper <= 0 || upper > slack)
      continue;
    const int missing = c.samples < HOT_SAMPLES ? CALIBRATION_ROUNDS - c.samples : 0;
    if (c.remaining_tokens < static_cast<long long>(batch) * std::max(c.width + missing - 1, 0))
      continue;
    const double score = (mean - fixed_s) / c.expected_tokens;
    const bool review =
        c.review_acceptance && (hot - fixed_s) / c.maximum_tokens < baseline * 0.98;
    const double reserved = review ? batch : c.expected_tokens;
    const double loss = std::max(upper - fixed_s - baseline * reserved, 0.0);
    if (c.samples >= HOT_SAMPLES && score < best_score &&
        (!c.review_acceptance || in->allow_exploration) && (c.warm_ready || loss <= available)) {
      best_id = c.id;
      best_score = score;
    }
    const bool stale = c.last >= 0 && in->calls - c.last >= REFRESH_AFTER;
    const double recoverable =
        review ? (baseline - (hot - fixed_s) / c.maximum_tokens) * c.remaining_tokens -
                     c.transition_s
               : baseline * c.remaining_tokens * (1.0 - batch / c.expected_tokens);
    if (in->allow_exploration && (missing > 0 || stale || review) && loss <= available &&
        loss <= recoverable) {
      const long r0 = (missing == 0 && !review) ? 1 : 0;
      const long r1 = (missing > 0 || review) ? c.width : c.last;
      if (!have_probe || r0 < probe_rank0 || (r0 == probe_rank0 && r1 < probe_rank1)) {
        have_probe = true;
        probe_id = c.id;
        probe_cal = missing > 0;
        probe_rank0 = r0;
        probe_rank1 = r1;
      }
    }
  }
  if (have_probe) {
    *flags = 1 | (probe_cal ? 2 : 0);
    return probe_id;
  }
  return best_id;
}

// ---- prompt lookup
void* orinfer_lookup_create(void) { return new PromptLookup(); }
void orinfer_lookup_destroy(void* h) { delete static_cast<PromptLookup*>(h); }

// Index the committed history and propose `count` tokens copied from the continuation of
// the best earlier match (>= minimum context: 4 greedy, 7 when sampling).  Returns count or 0.
int orinfer_lookup_propose(void* h, const uint32_t* history, int n, int count, int confident,
                           uint32_t* out) {
  PromptLookup* p = static_cast<PromptLookup*>(h);
  if (n < KEY || count <= 0) return 0;
  p->extend(history, static_cast<size_t>(n));
  const long end = p->find(history, n, count, confident ? SAMPLED_CONTEXT : KEY);
  if (end < 0) return 0;
  for (int i = 0; i < count; ++i) out[i] = history[end + i];
  return count;
}

void orinfer_lookup_observe(void* h, int accepted, int proposed, int progress) {
  PromptLookup* p = static_cast<PromptLookup*>(h);
  if (accepted * 2 >= proposed) {
    p->misses = 0;
  } else if (++p->misses >= 2) {
    p->cooldown = static_cast<size_t>(progress) + COOLDOWN;
    p->misses = 0;
  }
}

}  // extern "C"
