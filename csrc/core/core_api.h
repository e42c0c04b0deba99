// C ABI of liborinfer_core.so: the host-side policy core (no CUDA dependency).
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct OrinferSamplingOptions {
  double temperature;
  double top_p;
  int32_t top_k;
  double presence_penalty;
  double frequency_penalty;
  double repetition_penalty;
  uint64_t seed;
  int32_t bias_count;
  const uint32_t* bias_ids;
  const double* bias_values;
  int32_t top_logprobs;          // < 0 = not requested
} OrinferSamplingOptions;

const char* orinfer_core_last_error(void);

// ---- sampling law / counter RNG
uint64_t orinfer_splitmix64(uint64_t x);
double orinfer_counter_uniform(uint64_t seed, uint64_t stream, uint64_t step);
void orinfer_categorical_key(uint64_t seed, uint64_t step, uint32_t out[2]);
void orinfer_philox2x32_10(uint32_t c0, uint32_t c1, uint32_t key, uint32_t out[2]);
uint64_t orinfer_round_step(uint64_t round, uint64_t position);
int orinfer_sampling_validate(const OrinferSamplingOptions* o);
int orinfer_sampling_is_greedy(const OrinferSamplingOptions* o);
int orinfer_sampling_device_categorical(const OrinferSamplingOptions* o);
int orinfer_sample(const float* logits, int vocab, const uint32_t* history, int history_len,
                   const OrinferSamplingOptions* o, const uint32_t* mask, double uniform,
                   uint32_t* token);
int orinfer_sampling_law(const float* logits, int vocab, const uint32_t* history, int history_len,
                         const OrinferSamplingOptions* o, const uint32_t* mask, uint32_t* ids,
                         double* probs, int capacity);
int orinfer_logprobs(const float* logits, int vocab, const uint32_t* history, int history_len,
                     const OrinferSamplingOptions* o, const uint32_t* mask, uint32_t chosen,
                     int top_n, double* chosen_logprob, uint32_t* top_ids, double* top_logprobs);
int orinfer_greedy_commit(const uint32_t* drafts, int n_drafts, const uint32_t* target,
                          int n_target, uint32_t* committed);
int orinfer_sampled_commit(const uint32_t* drafts, int n_drafts, const double* draft_probs,
                           const float* target_logits, int vocab, const uint32_t* history,
                           int history_len, const OrinferSamplingOptions* o, uint64_t step,
                           uint32_t* committed);

// ---- scheduler policy
typedef struct OrinferWaiting {
  double age_s, remaining_s, restore_s, startup_s;
  long long remaining_tokens;
} OrinferWaiting;
int orinfer_select_waiting(const OrinferWaiting* reqs, int n);
void orinfer_rank_throughput_waiting(const OrinferWaiting* reqs, const double* expected, int n,
                                     int has_cohort, double cohort_remaining, int* order);
void orinfer_replenish(double* credits, int n, double quantum_s);
double orinfer_prefill_window(double slack_s, double decode_s, double ceiling_ms);
int orinfer_joint_prefill_worthwhile(int loses_large_tile, int measured, double joint_s,
                                     double native_s);
double orinfer_decode_quantum_s(double prefill_s, double prefill_budget_ms, double tpot_ms);
int orinfer_admission_should_yield(int has_decoders, int admitted, double elapsed_s,
                                   int batchable_start);
long long orinfer_usable_host_bytes(long long total_kb, long long available_kb);
void* orinfer_timing_create(void);
void orinfer_timing_destroy(void* h);
void orinfer_timing_observe(void* h, double seconds);
double orinfer_timing_mean(void* h);
double orinfer_timing_upper(void* h);
long long orinfer_timing_samples(void* h);
void* orinfer_lengths_create(void);
void orinfer_lengths_destroy(void* h);
void orinfer_lengths_observe(void* h, long long input, long long output);
double orinfer_lengths_estimate(void* h, long long input, long long limit);
int orinfer_error_is_fatal(int kind);

// ---- adaptive MTP control and prompt lookup
typedef struct OrinferMtpCandidate {
  int id, width;
  double expected_tokens, maximum_tokens;
  long long remaining_tokens;
  double mean_s, upper_s, transition_s;
  int warm_ready, review_acceptance, samples;
  long long last;                 // call index of the last use, -1 = never
} OrinferMtpCandidate;
typedef struct OrinferMtpSelection {
  double normal_s, fixed_s;
  int batch;
  double slack_s, available_s, calibration_s;
  int allow_exploration;
  long long calls, normal_last;   // normal_last -1 = never
} OrinferMtpSelection;
void* orinfer_acceptance_create(void);
void orinfer_acceptance_destroy(void* h);
void orinfer_acceptance_observe(void* h, const int* proposed, const int* accepted, int n);
double orinfer_acceptance_rate(void* h, int position, double prior);
double orinfer_acceptance_expected(void* h, int drafts);
double orinfer_mtp_progress(const double* yields, int n, int batch, int latency);
int orinfer_mtp_allocate(const double* rate, const int* cap, int n, int budget, double floor,
                         int* counts);
int orinfer_mtp_select(const OrinferMtpSelection* in, const OrinferMtpCandidate* cands, int n,
                       int* flags);
void* orinfer_lookup_create(void);
void orinfer_lookup_destroy(void* h);
int orinfer_lookup_propose(void* h, const uint32_t* history, int n, int count, int confident,
                           uint32_t* out);
void orinfer_lookup_observe(void* h, int accepted, int proposed, int progress);

// ---- radix prefix cache (page granular)
void* orinfer_prefix_create(int page_tokens);
void orinfer_prefix_destroy(void* handle);
int orinfer_prefix_match(void* handle, const uint32_t* tokens, int n, const uint64_t* media,
                         int limit_tokens, int acquire, int32_t* node_ids, int32_t* pages,
                         int max_out);
int orinfer_prefix_insert(void* handle, const uint32_t* tokens, int n, const uint64_t* media,
                          const int32_t* pages, int n_pages, int32_t* adopted, int32_t* node_ids);
void orinfer_prefix_release(void* handle, const int32_t* node_ids, int n);
void orinfer_prefix_abandon(void* handle, const int32_t* node_ids, int n);
int orinfer_prefix_evict(void* handle, int want, int to_host, int32_t* node_ids, int32_t* pages);
int orinfer_prefix_set_host(void* handle, int32_t node_id, int64_t host_handle);
int64_t orinfer_prefix_host_handle(void* handle, int32_t node_id);
int orinfer_prefix_restore(void* handle, int32_t node_id, int32_t page);
int orinfer_prefix_drop_host(void* handle, int want, int64_t* handles);
void orinfer_prefix_stats(void* handle, uint64_t out[10]);

// ---- cost curves (cost_curves.cpp)
typedef struct OrinferWork {
  uint32_t tokens;          // prompt tokens in the packet
  uint32_t context;         // longest context among its prompt chunks
  uint32_t decode_rows;     // decode rows riding along
  uint32_t decode_context;  // longest context among them
  int domain;               // execution family (model / parallel layout); curves never mix
} OrinferWork;

#ifdef __cplusplus
}
#endif
