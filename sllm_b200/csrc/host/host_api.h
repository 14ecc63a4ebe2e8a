/* C ABI of the host runtime library (libsllm_b200_host.so): no CUDA dependency.
 * Handles are small positive integers; functions that return a handle or a count return a negated
 * status code on failure, all others return a status code (0 = ok).
 */
#pragma once
#include <stdint.h>

#define SLLM_HOST_EXPORT extern "C" __attribute__((visibility("default")))

enum SllmHostStatus {
  SLLM_HOST_OK = 0,
  SLLM_HOST_INVALID = 1,
  SLLM_HOST_NOT_FOUND = 2,
  SLLM_HOST_OUT_OF_PAGES = 3,
  SLLM_HOST_LIMIT = 4,
  SLLM_HOST_PARSE_ERROR = 5,
  SLLM_HOST_BUSY = 6,
  SLLM_SAMPLE_NAN = 7,     /* a logit is NaN: *token holds its index */
  SLLM_SAMPLE_EMPTY = 8,   /* no token is left to choose from */
};

/* page_pool.cpp */
SLLM_HOST_EXPORT int sllm_kv_pool_create(int num_pages, int page_size);
SLLM_HOST_EXPORT int sllm_kv_pool_destroy(int h);
SLLM_HOST_EXPORT int sllm_kv_pool_stats(int h, long long* out4);
SLLM_HOST_EXPORT int sllm_kv_pool_inject_alloc_failure(int h, int fail_after_calls);
SLLM_HOST_EXPORT int sllm_kv_page_refcount(int h, int page);
SLLM_HOST_EXPORT int sllm_kv_seq_new(int h);
SLLM_HOST_EXPORT int sllm_kv_seq_free(int h, int seq);
SLLM_HOST_EXPORT int sllm_kv_seq_reserve(int h, int seq, long long new_len);
SLLM_HOST_EXPORT int sllm_kv_seq_commit(int h, int seq, long long new_len);
SLLM_HOST_EXPORT int sllm_kv_seq_truncate(int h, int seq, long long len);
SLLM_HOST_EXPORT long long sllm_kv_seq_length(int h, int seq);
SLLM_HOST_EXPORT int sllm_kv_seq_pages(int h, int seq, int* out, int cap);
SLLM_HOST_EXPORT int sllm_kv_seq_fork(int h, int seq, long long prefix_len, int* copy_pair);
SLLM_HOST_EXPORT int sllm_kv_seq_make_tail_private(int h, int seq, int* copy_pair);
SLLM_HOST_EXPORT int sllm_kv_fill_block_table(int h, const int* seqs, int n, int* table, int max_blocks);

/* grammar.cpp */
SLLM_HOST_EXPORT int sllm_grammar_create(const char* gbnf, const char* root, char* err, int err_cap);
SLLM_HOST_EXPORT int sllm_grammar_destroy(int h);
SLLM_HOST_EXPORT int sllm_grammar_set_vocab(int h, int n_tokens, const unsigned char* blob, const unsigned int* offsets);
SLLM_HOST_EXPORT int sllm_grammar_state_new(int h);
SLLM_HOST_EXPORT int sllm_grammar_state_clone(int s);
SLLM_HOST_EXPORT int sllm_grammar_state_free(int s);
SLLM_HOST_EXPORT int sllm_grammar_mask(int s, unsigned char* out_mask, int n);
SLLM_HOST_EXPORT int sllm_grammar_accept(int s, int token);
SLLM_HOST_EXPORT int sllm_grammar_accept_bytes(int s, const unsigned char* bytes, int n);
SLLM_HOST_EXPORT int sllm_grammar_is_complete(int s);
SLLM_HOST_EXPORT int sllm_grammar_stats(int h, long long* out3);

/* sampler.cpp: the host sampler chain over one row of logits (stage order and arithmetic: see the file). */
typedef struct SllmSamplerConfig {
  double temperature, top_p, min_p, typical_p;   /* temperature <= 0: greedy over the processed logits */
  double presence_penalty, frequency_penalty, repeat_penalty;
  double dyn_range, dyn_exponent;                /* used when dynamic_temperature != 0 */
  double dry_multiplier, dry_base;
  double xtc_probability, xtc_threshold;
  double mirostat_tau, mirostat_eta;
  const int* bias_tokens;                        /* n_bias (token, value) pairs */
  const float* bias_values;
  const int* dry_breakers;                       /* single-token sequence breakers */
  int n_bias, n_dry_breakers;
  int top_k;                                     /* 0: off */
  int repeat_last_n;
  int dynamic_temperature;
  int ignore_eos_token;                          /* < 0: off */
  int dry, dry_allowed_length, dry_last_n;
  int xtc, xtc_min_keep;
  int mirostat;                                  /* 0 off, 1, 2 */
  int return_logprobs, top_logprobs;
} SllmSamplerConfig;

typedef struct SllmSamplerState {
  uint64_t rng_state;                            /* SplitMix64: the state after k draws is seed + k * gamma */
  long long draws;
  double mu;                                     /* Mirostat */
} SllmSamplerState;

/* history: accepted tokens, oldest first; count_tokens / count_values: occurrences per distinct token.
 * top_ids / top_logprobs: room for cfg->top_logprobs entries (may be null when that is 0). */
SLLM_HOST_EXPORT int sllm_host_sample(const float* logits, int vocab, const unsigned char* valid_mask,
                                      const SllmSamplerConfig* cfg, SllmSamplerState* state, const int* history,
                                      int n_history, const int* count_tokens, const int* count_values, int n_counts,
                                      int* token, double* logprob, int* top_ids, double* top_logprobs, int* n_top);
SLLM_HOST_EXPORT int sllm_host_sampler_abi(int* out, int cap);
