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

// ---- radix prefix cache (page granular)
void* orinfer_prefix_create(int page_tokens);
void orinfer_prefix_destroy(void* handle);
int orinfer_prefix_match(void* handle, const uint32_t* tokens, int n, const uint64_t* media,
                         int limit_tokens, int acquire, int32_t* node_ids, int32_t* pages,
                         int max_out);
int orinfer_prefix_insert(void* handle, const uint32_t* tokens, int n, const uint64_t* media,
                          const int32_t* pages, int n_pages, int32_t* adopted, int32_t* node_ids);
void orinfer_prefix_release(void* handle, const int32_t* node_ids, int n);
int orinfer_prefix_evict(void* handle, int want, int to_host, int32_t* node_ids, int32_t* pages);
int orinfer_prefix_set_host(void* handle, int32_t node_id, int64_t host_handle);
int64_t orinfer_prefix_host_handle(void* handle, int32_t node_id);
int orinfer_prefix_restore(void* handle, int32_t node_id, int32_t page);
int orinfer_prefix_drop_host(void* handle, int want, int64_t* handles);
void orinfer_prefix_stats(void* handle, uint64_t out[10]);

#ifdef __cplusplus
}
#endif
