// Scheduler policy math (pure functions + small estimators), host only.
//
// Queue ordering: cost / (1 + age/2) with a hard oldest-first promotion after 30 s;
// throughput ranking groups requests by expected remaining output length; Estimate is an
// EWMA plus a rolling positive-residual P95 allowance; Timing discards its first-use sample
// (graph capture / lazy module load); prefill credits are replenished in whole quanta;
// decode bursts are bounded by wall time.  Behavioural contract:
// crates/orinfer-engine/src/scheduler.rs:143-179,183-218,222-252,256-327,332-364,369-448.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>

#include "core_api.h"

namespace {

double cost_s(const OrinferWaiting& w) {
  return std::max(w.remaining_s + w.restore_s + w.startup_s, 0.001);
}

// total order of doubles as IEEE totalOrder restricted to non-NaN inputs
int cmp(double a, double b) { return a < b ? -1 : (a > b ? 1 : 0); }

int waiting_order(const OrinferWaiting& a, const OrinferWaiting& b) {
  const bool old_a = a.age_s >= 30.0, old_b = b.age_s >= 30.0;
  if (old_a != old_b) return old_a ? -1 : 1;
  if (old_a) return cmp(b.age_s, a.age_s);
  const int c = cmp(cost_s(a) / (1.0 + a.age_s / 2.0), cost_s(b) / (1.0 + b.age_s / 2.0));
  return c != 0 ? c : cmp(b.age_s, a.age_s);
}

struct Estimate {
  double mean = 0, error = 0;
  uint64_t samples = 0;
  double residuals[32] = {0};
  uint64_t cursor = 0;

  void observe(double s) {
    if (!std::isfinite(s) || s <= 0) return;
    if (samples == 0) {
      mean = s;
    } else {
      residuals[cursor % 32] = std::max(s - mean, 0.0);
      ++cursor;
      error = error * 0.8 + std::fabs(s - mean) * 0.2;
      mean = mean * 0.8 + s * 0.2;
    }
    ++samples;
  }
  double upper() const {
    const uint64_t count = std::min<uint64_t>(cursor, 32);
    double pct = 0;
    if (count) {
      double v[32];
      std::memcpy(v, residuals, sizeof(v));
      std::sort(v, v + count);
      const uint64_t idx = (count * 95 + 99) / 100;
      pct = v[idx ? idx - 1 : 0];
    }
    return mean + std::max(2 * error, pct);
  }
};

struct Timing {
  Estimate time;
  uint64_t trials = 0;
  void observe(double s) {
    if (trials == 1) time = Estimate();      // the first use may have captured a graph
    time.observe(s);
    ++trials;
  }
  uint64_t samples() const { return trials <= 1 ? 0 : time.samples; }
};

struct OutputLengths {
  uint64_t count[64] = {0};
  double ratio[64] = {0};
};

int ilog2(uint64_t v) {
  int r = 0;
  while (v >>= 1) ++r;
  return r;
}

}  // namespace

extern "C" {

int orinfer_select_waiting(const OrinferWaiting* reqs, int n) {
  if (n <= 0) return -1;
  int best = 0;
  for (int i = 1; i < n; ++i)
    if (waiting_order(reqs[i], reqs[best]) < 0) best = i;
  return best;
}

void orinfer_rank_throughput_waiting(const OrinferWaiting* reqs, const double* expected, int n,
                                     int has_cohort, double cohort_remaining, int* order) {
  std::vector<int> idx(n);
  std::iota(idx.begin(), idx.end(), 0);
  auto mismatch = [&](int i) {
    if (!has_cohort) return 0.0;
    return std::fabs(std::log(std::max(expected[i], 1.0) / std::max(cohort_remaining, 1.0)));
  };
  std::sort(idx.begin(), idx.end(), [&](int a, int b) {
    const bool old_a = reqs[a].age_s >= 30.0, old_b = reqs[b].age_s >= 30.0;
    if (old_a != old_b) return old_a;
    int c;
    if (old_a) {
      c = cmp(reqs[b].age_s, reqs[a].age_s);
    } else {
      c = cmp(mismatch(a), mismatch(b));
      if (!c) c = cmp(expected[b], expected[a]);
      if (!c) c = cmp(cost_s(reqs[a]), cost_s(reqs[b]));
    }
    return c != 0 ? c < 0 : a < b;
  });
  for (int i = 0; i < n; ++i) order[i] = idx[i];
}

void orinfer_replenish(double* credits, int n, double quantum_s) {
  double highest = -INFINITY;
  for (int i = 0; i < n; ++i) highest = std::max(highest, credits[i]);
  if (highest <= 0 && std::isfinite(highest)) {
    const double refill = (std::floor(-highest / quantum_s) + 1.0) * quantum_s;
    for (int i = 0; i < n; ++i) credits[i] += refill;
  }
}

double orinfer_prefill_window(double slack_s, double decode_s, double ceiling_ms) {
  return std::min(std::max(slack_s - decode_s, 0.0), ceiling_ms / 1000.0);
}

int orinfer_joint_prefill_worthwhile(int loses_large_tile, int measured, double joint_s,
                                     double native_s) {
  return (!loses_large_tile || measured) && joint_s < native_s * 0.95;
}

double orinfer_decode_quantum_s(double prefill_s, double prefill_budget_ms, double tpot_ms) {
  return std::min(prefill_s, std::min(prefill_budget_ms / 1000.0, tpot_ms / 1000.0));
}

int orinfer_admission_should_yield(int has_decoders, int admitted, double elapsed_s,
                                   int batchable_start) {
  if (!batchable_start)
    return has_decoders ? elapsed_s >= 0.010 : (admitted >= 8 || elapsed_s >= 0.200);
  const int count = has_decoders ? 8 : 32;
  const double seconds = has_decoders ? 0.100 : 3.0;
  return admitted >= count || elapsed_s >= seconds;
}

// MemTotal / MemAvailable (kB) -> usable bytes = available - total/16, or -1 when invalid.
long long orinfer_usable_host_bytes(long long total_kb, long long available_kb) {
  if (total_kb <= 0 || available_kb < 0 || available_kb > total_kb) return -1;
  const long long total = total_kb * 1024, avail = available_kb * 1024;
  return std::max(avail - total / 16, 0LL);
}

// ---- Estimate / Timing handles
void* orinfer_timing_create(void) { return new Timing(); }
void orinfer_timing_destroy(void* h) { delete static_cast<Timing*>(h); }
void orinfer_timing_observe(void* h, double seconds) { static_cast<Timing*>(h)->observe(seconds); }
double orinfer_timing_mean(void* h) { return static_cast<Timing*>(h)->time.mean; }
double orinfer_timing_upper(void* h) { return static_cast<Timing*>(h)->time.upper(); }
long long orinfer_timing_samples(void* h) {
  return static_cast<long long>(static_cast<Timing*>(h)->samples());
}

// ---- online output-length estimator (per power-of-two input bin, exponential forgetting)
void* orinfer_lengths_create(void) { return new OutputLengths(); }
void orinfer_lengths_destroy(void* h) { delete static_cast<OutputLengths*>(h); }
void orinfer_lengths_observe(void* h, long long input, long long output) {
  if (input <= 0 || output <= 0) return;
  OutputLengths* o = static_cast<OutputLengths*>(h);
  const int bin = ilog2(static_cast<uint64_t>(input));
  const double r = static_cast<double>(output) / static_cast<double>(input);
  o->ratio[bin] = o->count[bin] == 0 ? r : o->ratio[bin] * 0.95 + r * 0.05;
  ++o->count[bin];
}
double orinfer_lengths_estimate(void* h, long long input, long long limit) {
  OutputLengths* o = static_cast<OutputLengths*>(h);
  const int key = ilog2(static_cast<uint64_t>(std::max<long long>(input, 1)));
  double ratio = 1.0;
  int best = 1 << 30;
  for (int i = 0; i < 64; ++i)
    if (o->count[i] > 0 && std::abs(i - key) < best) {
      best = std::abs(i - key);
      ratio = o->ratio[i];
    }
  return std::min(std::max(static_cast<double>(input) * ratio, 1.0), static_cast<double>(limit));
}

// ---- error taxonomy (crates/orinfer-engine/src/error.rs:6-97): request and capacity
// errors fail one request; out-of-memory, device and invariant errors are fatal.
int orinfer_error_is_fatal(int kind) {
  switch (kind) {
    case 0:  // Request
    case 1:  // Capacity
      return 0;
    default:  // OutOfMemory, Cuda, Nccl/Peer, Invariant
      return 1;
  }
}

}  // extern "C"
