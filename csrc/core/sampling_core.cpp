// Host sampling law and counter RNG (bit-exact determinism contract).
//
// Draws are keyed by (seed, stream, committed position), never by batch slot, graph
// replay count or packet shape, so a request produces the same tokens whatever it is
// batched with.  The law: processed scores in f64 (repetition / presence / frequency
// penalties, logit bias, grammar mask) -> order by (score desc, id asc) -> optional
// top-k -> weights exp((s - max)/T) -> nucleus cut at total * top_p -> normalise ->
// inverse-CDF draw.  Speculative verification uses exact rejection sampling with
// separate counter streams for proposals, acceptance tests and corrections.
// Behavioural contract: crates/orinfer-engine/src/sampling.rs:17-51,56-130,141-206,
// 260-299 and crates/orinfer-engine/src/mtp.rs:10-22,24-39,48-97 of the reference.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <string>
#include <vector>

#include "core_api.h"

namespace {

uint64_t splitmix64(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

struct Entry {
  uint32_t id;
  double score;
};

inline bool before(const Entry& a, const Entry& b) {
  // total order: higher score first (with -0.0 < +0.0 as in IEEE totalOrder), then lower id
  if (a.score != b.score) return a.score > b.score;
  const bool na = std::signbit(a.score), nb = std::signbit(b.score);
  if (na != nb) return nb;
  return a.id < b.id;
}

thread_local std::string g_error;

int fail(const char* message) {
  g_error = message;
  return -1;
}

struct Law {
  std::vector<Entry> ordered;   // (id, probability), descending
};

int validate(const OrinferSamplingOptions& o) {
  auto in = [](double v, double lo, double hi) { return v >= lo && v <= hi; };
  if (!in(o.temperature, 0.0, 2.0)) return fail("temperature: Invalid sampling value");
  if (!in(o.top_p, 0.0, 1.0) || o.top_p == 0.0) return fail("top_p: Invalid sampling value");
  if (!in(o.presence_penalty, -2.0, 2.0)) return fail("presence_penalty: Invalid sampling value");
  if (!in(o.frequency_penalty, -2.0, 2.0))
    return fail("frequency_penalty: Invalid sampling value");
  if (!std::isfinite(o.repetition_penalty) || o.repetition_penalty <= 0.0)
    return fail("repetition_penalty: Expected positive finite value");
  if (o.top_logprobs > 20) return fail("top_logprobs: Expected 0-20");
  for (int i = 0; i < o.bias_count; ++i)
    if (!in(o.bias_values[i], -100.0, 100.0)) return fail("logit_bias: Bias outside -100..100");
  return 0;
}

bool processes_scores(const OrinferSamplingOptions& o) {
  return o.presence_penalty != 0.0 || o.frequency_penalty != 0.0 ||
         o.repetition_penalty != 1.0 || o.bias_count > 0;
}

// Processed scores of the unmasked tokens.
int processed(const float* logits, int vocab, const uint32_t* history, int history_len,
              const OrinferSamplingOptions& o, const uint32_t* mask, std::vector<Entry>* out) {
  if (vocab <= 0) return fail("Invalid sampling logits");
  for (int i = 0; i < vocab; ++i)
    if (!std::isfinite(logits[i])) return fail("Invalid sampling logits");
  std::vector<uint32_t> counts;
  const bool penalise =
      o.repetition_penalty != 1.0 || o.presence_penalty != 0.0 || o.frequency_penalty != 0.0;
  if (penalise) {
    counts.assign(vocab, 0);
    for (int i = 0; i < history_len; ++i)
      if (history[i] < static_cast<uint32_t>(vocab)) ++counts[history[i]];
  }
  std::vector<double> bias;
  if (o.bias_count > 0) {
    bias.assign(vocab, 0.0);
    for (int i = 0; i < o.bias_count; ++i)
      if (o.bias_ids[i] < static_cast<uint32_t>(vocab)) bias[o.bias_ids[i]] = o.bias_values[i];
  }
  out->clear();
  out->reserve(vocab);
  for (int i = 0; i < vocab; ++i) {
    if (mask && !(mask[i / 32] & (1u << (i % 32)))) continue;
    double s = static_cast<double>(logits[i]);
    if (processes_scores(o)) {
      const uint32_t c = penalise ? counts[i] : 0;
      if (c > 0) {
        s = s < 0.0 ? s * o.repetition_penalty : s / o.repetition_penalty;
        s -= o.presence_penalty;
      }
      s -= o.frequency_penalty * static_cast<double>(c);
      if (!bias.empty()) s += bias[i];
      if (!std::isfinite(s)) return fail("Nonfinite processed sampling logits");
    } else {
      s += 0.0;
    }
    out->push_back({static_cast<uint32_t>(i), s});
  }
  if (out->empty()) return fail("Grammar permits no tokens");
  return 0;
}

// Turns processed scores into the normalised, truncated law.
void make_law(std::vector<Entry>& scores, const OrinferSamplingOptions& o, Law* law) {
  if (o.temperature == 0.0) {
    const Entry best = *std::min_element(scores.begin(), scores.end(), before);
    law->ordered = {{best.id, 1.0}};
    return;
  }
  if (o.top_k > 0 && static_cast<size_t>(o.top_k) < scores.size()) {
    std::nth_element(scores.begin(), scores.begin() + o.top_k, scores.end(), before);
    scores.resize(o.top_k);
  } else {
    // Weights below exp(-38) vanish when added to a descending sum that starts at 1;
    // dropping them first does not change any retained probability.
    double mx = -std::numeric_limits<double>::infinity();
    for (const Entry& e : scores) mx = std::max(mx, e.score);
    const double cut = mx - 38.0 * o.temperature;
    scores.erase(std::remove_if(scores.begin(), scores.end(),
                                [cut](const Entry& e) { return e.score < cut; }),
                 scores.end());
  }
  std::sort(scores.begin(), scores.end(), before);
  const double mx = scores[0].score;
  double total = 0.0;
  for (Entry& e : scores) {
    e.score = std::exp((e.score - mx) / o.temperature);
    total += e.score;
  }
  const double threshold = total * o.top_p;
  double mass = 0.0;
  size_t keep = scores.size();
  for (size_t i = 0; i < scores.size(); ++i) {
    mass += scores[i].score;
    if (mass >= threshold) {
      keep = i + 1;
      break;
    }
  }
  scores.resize(keep);
  for (Entry& e : scores) e.score /= mass;
  law->ordered.swap(scores);
}

int draw_law(const Law& law, double uniform, uint32_t* token) {
  if (!std::isfinite(uniform) || uniform < 0.0 || uniform >= 1.0)
    return fail("Sampling uniform outside [0,1)");
  double mass = 0.0;
  for (const Entry& e : law.ordered) {
    mass += e.score;
    if (uniform < mass) {
      *token = e.id;
      return 0;
    }
  }
  for (auto it = law.ordered.rbegin(); it != law.ordered.rend(); ++it)
    if (it->score > 0.0) {
      *token = it->id;
      return 0;
    }
  return fail("Empty sampling distribution");
}

double probability(const Law& law, uint32_t token) {
  for (const Entry& e : law.ordered)
    if (e.id == token) return e.score;
  return 0.0;
}

int build_law(const float* logits, int vocab, const uint32_t* history, int history_len,
              const OrinferSamplingOptions& o, const uint32_t* mask, Law* law) {
  std::vector<Entry> scores;
  if (processed(logits, vocab, history, history_len, o, mask, &scores)) return -1;
  make_law(scores, o, law);
  return 0;
}

}  // namespace

extern "C" {

const char* orinfer_core_last_error(void) { return g_error.c_str(); }

uint64_t orinfer_splitmix64(uint64_t x) { return splitmix64(x); }

double orinfer_counter_uniform(uint64_t seed, uint64_t stream, uint64_t step) {
  const uint64_t bits = splitmix64(splitmix64(seed ^ stream) ^ step) >> 11;
  return static_cast<double>(bits) * (1.0 / 9007199254740992.0);
}

void orinfer_categorical_key(uint64_t seed, uint64_t step, uint32_t out[2]) {
  const uint64_t key = splitmix64(splitmix64(seed) ^ step);
  out[0] = static_cast<uint32_t>(key);
  out[1] = static_cast<uint32_t>(key >> 32);
}

void orinfer_philox2x32_10(uint32_t c0, uint32_t c1, uint32_t key, uint32_t out[2]) {
  for (int round = 0; round < 10; ++round) {
    const uint64_t product = static_cast<uint64_t>(c0) * 0xd256d193ull;
    const uint32_t hi = static_cast<uint32_t>(product >> 32), lo = static_cast<uint32_t>(product);
    c0 = hi ^ key ^ c1;
    c1 = lo;
    key += 0x9e3779b9u;
  }
  out[0] = c0;
  out[1] = c1;
}

uint64_t orinfer_round_step(uint64_t round, uint64_t position) {
  return ((round + 1) << 32) | (position & 0xffffffffull);
}

int orinfer_sampling_validate(const OrinferSamplingOptions* o) { return validate(*o); }

int orinfer_sampling_is_greedy(const OrinferSamplingOptions* o) {
  return o->temperature == 0.0 && !processes_scores(*o);
}

int orinfer_sampling_device_categorical(const OrinferSamplingOptions* o) {
  const bool untruncated = (o->temperature == 0.0 || (o->temperature >= 1e-5 && o->temperature <= 2.0)) &&
                           o->top_p == 1.0 && o->top_k == 0 && !processes_scores(*o);
  return o->temperature > 0.0 && untruncated && o->top_logprobs < 0;
}

int orinfer_sample(const float* logits, int vocab, const uint32_t* history, int history_len,
                   const OrinferSamplingOptions* o, const uint32_t* mask, double uniform,
                   uint32_t* token) {
  if (validate(*o)) return -1;
  Law law;
  if (build_law(logits, vocab, history, history_len, *o, mask, &law)) return -1;
  return draw_law(law, uniform, token);
}

// Writes the retained support (ids, probabilities) in draw order; returns its size
// (or -1).  `capacity` bounds the copy, the true size is still returned.
int orinfer_sampling_law(const float* logits, int vocab, const uint32_t* history, int history_len,
                         const OrinferSamplingOptions* o, const uint32_t* mask, uint32_t* ids,
                         double* probs, int capacity) {
  if (validate(*o)) return -1;
  Law law;
  if (build_law(logits, vocab, history, history_len, *o, mask, &law)) return -1;
  const int n = static_cast<int>(law.ordered.size());
  for (int i = 0; i < n && i < capacity; ++i) {
    ids[i] = law.ordered[i].id;
    probs[i] = law.ordered[i].score;
  }
  return n;
}

// Log-probabilities after penalties / bias / mask and before top-k / top-p
// (temperature applied when > 0).  Fills the chosen token's value and the top `top_n`.
int orinfer_logprobs(const float* logits, int vocab, const uint32_t* history, int history_len,
                     const OrinferSamplingOptions* o, const uint32_t* mask, uint32_t chosen,
                     int top_n, double* chosen_logprob, uint32_t* top_ids, double* top_logprobs) {
  std::vector<Entry> scores;
  if (processed(logits, vocab, history, history_len, *o, mask, &scores)) return -1;
  const double t = o->temperature > 0.0 ? o->temperature : 1.0;
  double mx = -std::numeric_limits<double>::infinity();
  for (const Entry& e : scores) mx = std::max(mx, e.score);
  double total = 0.0;
  for (const Entry& e : scores) total += std::exp((e.score - mx) / t);
  const double lse = mx / t + std::log(total);
  *chosen_logprob = -std::numeric_limits<double>::infinity();
  for (const Entry& e : scores)
    if (e.id == chosen) *chosen_logprob = e.score / t - lse;
  const int n = std::min<int>(top_n, static_cast<int>(scores.size()));
  if (n > 0) {
    std::partial_sort(scores.begin(), scores.begin() + n, scores.end(), before);
    for (int i = 0; i < n; ++i) {
      top_ids[i] = scores[i].id;
      top_logprobs[i] = scores[i].score / t - lse;
    }
  }
  return n;
}

int orinfer_greedy_commit(const uint32_t* drafts, int n_drafts, const uint32_t* target,
                          int n_target, uint32_t* committed) {
  if (n_target != n_drafts + 1 || n_target <= 0)
    return fail("MTP verification must include one target token beyond drafts");
  int accepted = 0;
  while (accepted < n_drafts && drafts[accepted] == target[accepted]) ++accepted;
  for (int i = 0; i < accepted; ++i) committed[i] = drafts[i];
  committed[accepted] = target[accepted];
  return accepted + 1;
}

// Exact rejection sampling.  Draft laws are either point masses (draft_probs == null,
// greedy proposer) or dense probability rows [n_drafts, vocab].  Returns the number
// of committed tokens (accepted drafts + one correction or bonus token).
int orinfer_sampled_commit(const uint32_t* drafts, int n_drafts, const double* draft_probs,
                           const float* target_logits, int vocab, const uint32_t* history,
                           int history_len, const OrinferSamplingOptions* o, uint64_t step,
                           uint32_t* committed) {
  if (validate(*o)) return -1;
  if (vocab <= 0) return fail("Invalid MTP verification logits extent");
  std::vector<uint32_t> hist(history, history + history_len);
  int count = 0;
  for (int i = 0; i < n_drafts; ++i) {
    Law p;
    if (build_law(target_logits + static_cast<size_t>(i) * vocab, vocab, hist.data(),
                  static_cast<int>(hist.size()), *o, nullptr, &p))
      return -1;
    const uint32_t x = drafts[i];
    if (x >= static_cast<uint32_t>(vocab)) return fail("Proposal token exceeds vocabulary");
    const double* q = draft_probs ? draft_probs + static_cast<size_t>(i) * vocab : nullptr;
    const double qx = q ? q[x] : 1.0;
    if (!(qx > 0.0)) return fail("MTP proposal outside its draft distribution");
    const double u = orinfer_counter_uniform(o->seed, 0x4d545002ull, step + i);
    if (u < std::min(1.0, probability(p, x) / qx)) {
      committed[count++] = x;
      hist.push_back(x);
      continue;
    }
    // residual law proportional to (p - q)+, in ascending token order
    std::vector<Entry> res;
    for (const Entry& e : p.ordered) {
      const double qv = q ? q[e.id] : (e.id == x ? 1.0 : 0.0);
      const double r = std::max(e.score - qv, 0.0);
      if (r > 0.0) res.push_back({e.id, r});
    }
    std::sort(res.begin(), res.end(), [](const Entry& a, const Entry& b) { return a.id < b.id; });
    double total = 0.0;
    for (const Entry& e : res) total += e.score;
    if (!std::isfinite(total) || total <= 0.0)
      return fail("Rejected proposal has no residual mass");
    Law r;
    for (Entry& e : res) e.score /= total;
    r.ordered.swap(res);
    uint32_t tok;
    if (draw_law(r, orinfer_counter_uniform(o->seed, 0x4d545003ull, step + i), &tok)) return -1;
    committed[count++] = tok;
    return count;
  }
  Law p;
  if (build_law(target_logits + static_cast<size_t>(n_drafts) * vocab, vocab, hist.data(),
                static_cast<int>(hist.size()), *o, nullptr, &p))
    return -1;
  uint32_t tok;
  if (draw_law(p, orinfer_counter_uniform(o->seed, 0, step + n_drafts), &tok)) return -1;
  committed[count++] = tok;
  return count;
}

}  // extern "C"
