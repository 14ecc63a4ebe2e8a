// Host sampler chain: one row of fp32 logits -> one token, in the fixed stage order
//   LogitBias -> LegacyPenalty (presence / frequency) -> RepeatPenalty -> DryPenalty -> GrammarMask -> IgnoreEos ->
//   Temperature (static or entropy-driven) -> TopK -> MinP -> Typical -> TopP -> Xtc -> Mirostat (1 / 2) -> draw,
// with optional log-probabilities of the chosen token and of the most likely ones, and a SplitMix64 stream whose state
// is owned by the caller.  This is the per-token critical path of every request the device selector cannot take
// (typical sampling, DRY, XTC, Mirostat, dynamic temperature, repeat penalty, top-logprobs) over vocabularies of 128 K
// and more; the Python form of the same chain (engine/sampling.py) stays as the oracle the tests compare against.
//
// Arithmetic follows the oracle: penalties in fp32, everything from the softmax on in fp64, candidates ordered by
// descending scaled logit with ties to the lower token id.
// (Reference: crates/sllm-core/src/sampling.rs:364-468 selection, :646-661 stage order, :228-319 the random stream.)
#include "host_api.h"

#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <limits>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

constexpr uint64_t kGamma = 0x9E3779B97F4A7C15ull;

inline uint64_t mix64(uint64_t v) {
  v = (v ^ (v >> 30)) * 0xBF58476D1CE4E5B9ull;
  v = (v ^ (v >> 27)) * 0x94D049BB133111EBull;
  return v ^ (v >> 31);
}

inline double next_unit(SllmSamplerState* st) {
  st->rng_state += kGamma;
  st->draws += 1;
  return static_cast<double>(mix64(st->rng_state) >> 11) * (1.0 / 9007199254740992.0);
}

struct Cand {
  double s;   // scaled logit
  int id;
};

inline bool cand_before(const Cand& a, const Cand& b) { return a.s > b.s || (a.s == b.s && a.id < b.id); }

// Descending by scaled logit, ties by ascending id: a stable LSD radix sort over the fp32 bit patterns (the scaled
// logits are fp32 values) of candidates that arrive in ascending id order.  A comparison sort of 128 K entries costs
// more than every other stage of the chain together.
void sort_candidates(std::vector<Cand>& cand, const std::vector<float>& s32) {
  const size_t n = cand.size();
  std::vector<uint32_t> key(n), key2(n);
  std::vector<uint32_t> idx(n), idx2(n);
  for (size_t i = 0; i < n; ++i) {
    uint32_t b;
    static_assert(sizeof(float) == 4, "fp32");
    __builtin_memcpy(&b, &s32[i], 4);
    const uint32_t asc = (b & 0x80000000u) ? ~b : (b | 0x80000000u);   // ascending order of the float values
    key[i] = ~asc;                                                      // descending
    idx[i] = static_cast<uint32_t>(i);
  }
  for (int pass = 0; pass < 4; ++pass) {
    size_t count[257] = {0};
    const int sh = 8 * pass;
    for (size_t i = 0; i < n; ++i) ++count[((key[i] >> sh) & 0xffu) + 1];
    for (int b = 0; b < 256; ++b) count[b + 1] += count[b];
    for (size_t i = 0; i < n; ++i) {
      const size_t d = count[(key[i] >> sh) & 0xffu]++;
      key2[d] = key[i];
      idx2[d] = idx[i];
    }
    key.swap(key2);
    idx.swap(idx2);
  }
  std::vector<Cand> out(n);
  for (size_t i = 0; i < n; ++i) out[i] = cand[idx[i]];
  cand.swap(out);
}

// first index i with cum[i] >= x (side = left) or cum[i] > x (side = right) over the running sum of p
inline int search_cumsum(const std::vector<double>& p, double x, bool right) {
  double c = 0.0;
  const int n = static_cast<int>(p.size());
  for (int i = 0; i < n; ++i) {
    c += p[i];
    if (right ? c > x : c >= x) return i;
  }
  return n;
}

inline void renorm(std::vector<double>& p) {
  double t = 0.0;
  for (double v : p) t += v;
  for (double& v : p) v /= t;
}

}  // namespace

SLLM_HOST_EXPORT int sllm_host_sample(const float* logits, int vocab, const unsigned char* valid_mask,
                                      const SllmSamplerConfig* c, SllmSamplerState* st, const int* history, int n_history,
                                      const int* count_tokens, const int* count_values, int n_counts, int* token,
                                      double* logprob, int* top_ids, double* top_logprobs, int* n_top) {
  if (!logits || vocab <= 0 || !c || !st || !token || n_history < 0 || n_counts < 0 || (n_history && !history) ||
      (n_counts && (!count_tokens || !count_values)))
    return SLLM_HOST_INVALID;
  if (n_top) *n_top = 0;
  for (int i = 0; i < vocab; ++i)
    if (logits[i] != logits[i]) {
      *token = i;
      return SLLM_SAMPLE_NAN;
    }
  std::vector<float> lg(logits, logits + vocab);
  // ---- LogitBias, LegacyPenalty, RepeatPenalty, DryPenalty (fp32)
  for (int i = 0; i < c->n_bias; ++i) {
    const int t = c->bias_tokens[i];
    if (t >= 0 && t < vocab) lg[t] += c->bias_values[i];
  }
  if (n_counts && (c->frequency_penalty != 0.0 || c->presence_penalty != 0.0)) {
    const float fp = static_cast<float>(c->frequency_penalty), pp = static_cast<float>(c->presence_penalty);
    for (int i = 0; i < n_counts; ++i) {
      const int t = count_tokens[i];
      if (t >= 0 && t < vocab) {
        const float prod = static_cast<float>(count_values[i]) * fp;
        const float d = prod + pp;
        lg[t] -= d;
      }
    }
  }
  if (c->repeat_penalty != 1.0 && c->repeat_last_n > 0 && n_history > 0) {
    const float rp = static_cast<float>(c->repeat_penalty);
    const int from = std::max(0, n_history - c->repeat_last_n);
    std::unordered_set<int> seen;
    for (int i = from; i < n_history; ++i) {
      const int t = history[i];
      if (t < 0 || t >= vocab || !seen.insert(t).second) continue;
      lg[t] = lg[t] > 0.f ? lg[t] / rp : lg[t] * rp;
    }
  }
  if (c->dry && c->dry_multiplier > 0.0 && n_history > 0) {
    const int from = c->dry_last_n > 0 ? std::max(0, n_history - c->dry_last_n) : 0;
    const int* h = history + from;
    const int n = n_history - from;
    if (n >= 2) {
      std::unordered_set<int> breakers(c->dry_breakers, c->dry_breakers + c->n_dry_breakers);
      const int last = h[n - 1];
      std::unordered_map<int, int> best;   // token that would extend a repetition -> longest match length
      if (!breakers.count(last)) {
        for (int i = 0; i < n - 1; ++i) {
          if (h[i] != last) continue;
          int len = 1;
          while (i - len >= 0 && len < n - 1 && h[i - len] == h[n - 1 - len] && !breakers.count(h[i - len])) ++len;
          int& b = best[h[i + 1]];
          if (len > b) b = len;
        }
      }
      for (const auto& kv : best) {
        if (kv.second >= c->dry_allowed_length && kv.first >= 0 && kv.first < vocab)
          lg[kv.first] -= static_cast<float>(c->dry_multiplier * std::pow(c->dry_base, kv.second - c->dry_allowed_length));
      }
    }
  }
  // ---- GrammarMask, IgnoreEos
  const float ninf = -std::numeric_limits<float>::infinity();
  if (valid_mask)
    for (int i = 0; i < vocab; ++i)
      if (!valid_mask[i]) lg[i] = ninf;
  if (c->ignore_eos_token >= 0 && c->ignore_eos_token < vocab) lg[c->ignore_eos_token] = ninf;
  std::vector<int> ids;
  ids.reserve(vocab);
  for (int i = 0; i < vocab; ++i)
    if (lg[i] != ninf) ids.push_back(i);
  if (ids.empty()) return SLLM_SAMPLE_EMPTY;

  // log-probabilities of the processed distribution (before temperature), ascending token id
  const bool want_lp = c->return_logprobs || c->top_logprobs > 0;
  std::vector<double> base_lp;
  if (want_lp) {
    double zmax = -std::numeric_limits<double>::infinity();
    for (int id : ids) zmax = std::max(zmax, static_cast<double>(lg[id]));
    double sum = 0.0;
    for (int id : ids) sum += std::exp(static_cast<double>(lg[id]) - zmax);
    const double lse = zmax + std::log(sum);
    base_lp.resize(ids.size());
    for (size_t i = 0; i < ids.size(); ++i) base_lp[i] = static_cast<double>(lg[ids[i]]) - lse;
  }
  auto finish = [&](int tok) {
    *token = tok;
    if (want_lp) {
      const size_t pos = std::lower_bound(ids.begin(), ids.end(), tok) - ids.begin();
      if (logprob) *logprob = base_lp[pos];
      if (c->top_logprobs > 0 && top_ids && top_logprobs && n_top) {
        std::vector<int> o(ids.size());
        for (size_t i = 0; i < o.size(); ++i) o[i] = static_cast<int>(i);
        const int k = std::min<int>(c->top_logprobs, static_cast<int>(o.size()));
        std::partial_sort(o.begin(), o.begin() + k, o.end(), [&](int a, int b) {
          return base_lp[a] > base_lp[b] || (base_lp[a] == base_lp[b] && ids[a] < ids[b]);
        });
        for (int i = 0; i < k; ++i) {
          top_ids[i] = ids[o[i]];
          top_logprobs[i] = base_lp[o[i]];
        }
        *n_top = k;
      }
    }
    return SLLM_HOST_OK;
  };

  // ---- greedy over the processed logits
  if (!(c->temperature > 0.0) && !c->mirostat) {
    int best = ids[0];
    for (int id : ids)
      if (lg[id] > lg[best]) best = id;
    return finish(best);
  }
  // ---- Temperature
  double temp = c->temperature > 0.0 ? c->temperature : 1.0;
  if (c->dynamic_temperature && c->temperature > 0.0) {
    double zmax = -std::numeric_limits<double>::infinity();
    for (int id : ids) zmax = std::max(zmax, static_cast<double>(lg[id]));
    std::vector<double> pr(ids.size());
    double sum = 0.0;
    for (size_t i = 0; i < ids.size(); ++i) sum += (pr[i] = std::exp(static_cast<double>(lg[ids[i]]) - zmax));
    double ent = 0.0;
    for (double& v : pr) {
      v /= sum;
      if (v > 0.0) ent -= v * std::log(v);
    }
    const double max_ent = ids.size() > 1 ? std::log(static_cast<double>(ids.size())) : 1.0;
    const double t0 = c->temperature;
    const double lo = std::max(0.0, t0 - c->dyn_range), hi = t0 + c->dyn_range;
    temp = max_ent > 0.0 ? lo + (hi - lo) * std::pow(ent / max_ent, c->dyn_exponent) : t0;
    temp = std::max(temp, 1e-6);
  }
  const float t32 = static_cast<float>(temp);
  std::vector<Cand> cand(ids.size());
  std::vector<float> s32(ids.size());
  bool any_pos_inf = false;
  for (size_t i = 0; i < ids.size(); ++i) {
    float s = lg[ids[i]] / t32;
    if (s == 0.f) s = 0.f;                         // -0 and +0 compare equal: one bit pattern for the radix sort
    s32[i] = s;
    cand[i] = {static_cast<double>(s), ids[i]};
    any_pos_inf |= (s == std::numeric_limits<float>::infinity());
  }
  if (any_pos_inf) {
    std::vector<int> inf_ids;
    for (const Cand& x : cand)
      if (x.s == std::numeric_limits<double>::infinity()) inf_ids.push_back(x.id);   // ascending id = sorted order
    const double u = next_unit(st);
    const size_t k = std::min(static_cast<size_t>(u * static_cast<double>(inf_ids.size())), inf_ids.size() - 1);
    return finish(inf_ids[k]);
  }
  // ---- TopK (the sort is the cost of the chain at 128 K entries: only the part that can matter is ordered)
  size_t n = cand.size();
  if (c->top_k > 0 && static_cast<size_t>(c->top_k) < n) {
    std::partial_sort(cand.begin(), cand.begin() + c->top_k, cand.end(), cand_before);
    n = static_cast<size_t>(c->top_k);
    cand.resize(n);
  } else {
    sort_candidates(cand, s32);
  }
  std::vector<double> prob(n);
  {
    double sum = 0.0;
    for (size_t i = 0; i < n; ++i) sum += (prob[i] = std::exp(cand[i].s - cand[0].s));
    for (double& v : prob) v /= sum;
  }
  std::vector<int> cid(n);
  for (size_t i = 0; i < n; ++i) cid[i] = cand[i].id;
  auto keep_where = [&](const std::vector<char>& keep) {
    size_t w = 0;
    for (size_t i = 0; i < cid.size(); ++i)
      if (keep[i]) {
        cid[w] = cid[i];
        prob[w] = prob[i];
        ++w;
      }
    cid.resize(w);
    prob.resize(w);
  };
  // ---- MinP
  if (c->min_p > 0.0) {
    const double thr = c->min_p * prob[0];
    std::vector<char> keep(cid.size());
    for (size_t i = 0; i < cid.size(); ++i) keep[i] = prob[i] >= thr;
    keep_where(keep);
    renorm(prob);
  }
  // ---- Typical
  if (c->typical_p < 1.0 && cid.size() > 1) {
    const size_t m = cid.size();
    std::vector<double> logp(m), dev(m);
    double ent = 0.0;
    for (size_t i = 0; i < m; ++i) {
      logp[i] = std::log(std::max(prob[i], 1e-300));
      ent -= prob[i] * logp[i];
    }
    for (size_t i = 0; i < m; ++i) dev[i] = std::fabs(-logp[i] - ent);
    // (deviation, index) pairs sorted by value: a sort of indices through a comparator that loads dev[] misses the
    // cache on every comparison and took 300 ms at 128 K entries
    std::vector<std::pair<double, int>> o(m);
    for (size_t i = 0; i < m; ++i) o[i] = {dev[i], static_cast<int>(i)};
    std::sort(o.begin(), o.end());
    double cum = 0.0;
    size_t k = m;
    for (size_t i = 0; i < m; ++i) {
      cum += prob[o[i].second];
      if (cum >= c->typical_p) {
        k = i + 1;
        break;
      }
    }
    k = std::max<size_t>(1, std::min(k, m));
    std::vector<char> keep(m, 0);
    for (size_t i = 0; i < k; ++i) keep[o[i].second] = 1;
    keep_where(keep);
    renorm(prob);
  }
  // ---- TopP
  if (c->top_p < 1.0) {
    size_t k = static_cast<size_t>(search_cumsum(prob, c->top_p, false)) + 1;
    k = std::max<size_t>(1, std::min(k, cid.size()));
    cid.resize(k);
    prob.resize(k);
  }
  // ---- Xtc
  if (c->xtc && cid.size() > 1) {
    if (next_unit(st) < c->xtc_probability) {
      double sum = 0.0;
      for (double v : prob) sum += v;
      std::vector<int> above;
      for (size_t i = 0; i < cid.size(); ++i)
        if (prob[i] / sum >= c->xtc_threshold) above.push_back(static_cast<int>(i));
      if (above.size() >= 2 && cid.size() - (above.size() - 1) >= static_cast<size_t>(c->xtc_min_keep)) {
        std::vector<char> keep(cid.size(), 1);
        for (size_t i = 0; i + 1 < above.size(); ++i) keep[above[i]] = 0;   // all but the least likely of them
        keep_where(keep);
      }
    }
  }
  // ---- Mirostat
  if (c->mirostat) {
    renorm(prob);
    if (c->mirostat == 1) {
      const int m = static_cast<int>(prob.size());
      const int mtop = std::min(100, m - 1);
      double s_hat = 1.0;
      if (mtop >= 1) {
        double tb = 0.0, tt = 0.0;
        for (int i = 0; i < mtop; ++i) {
          const double t = std::log(static_cast<double>(i + 2) / static_cast<double>(i + 1));
          const double b = std::log(std::max(prob[i], 1e-300) / std::max(prob[i + 1], 1e-300));
          tb += t * b;
          tt += t * t;
        }
        s_hat = tt > 0.0 ? tb / tt : 1.0;
      }
      const double eps = s_hat - 1.0;
      double k = static_cast<double>(m);
      if (std::fabs(eps) > 1e-9)
        k = std::pow((eps * std::pow(2.0, st->mu)) / (1.0 - std::pow(static_cast<double>(m), -eps)), 1.0 / s_hat);
      // round half to even, as the oracle's round()
      const double kr = std::nearbyint(k);
      const int ki = (kr != kr) ? 1 : static_cast<int>(std::min<double>(std::max<double>(kr, 1.0), static_cast<double>(m)));
      cid.resize(ki);
      prob.resize(ki);
      renorm(prob);
    } else {
      std::vector<char> keep(cid.size());
      bool any = false;
      for (size_t i = 0; i < cid.size(); ++i) {
        keep[i] = -std::log2(std::max(prob[i], 1e-300)) <= st->mu;
        any |= keep[i] != 0;
      }
      if (!any) keep[0] = 1;
      keep_where(keep);
      renorm(prob);
    }
    const double thr = next_unit(st);
    int i = search_cumsum(prob, thr, true);
    i = std::min<int>(i, static_cast<int>(cid.size()) - 1);
    const double observed = -std::log2(std::max(prob[i], 1e-300));
    st->mu -= c->mirostat_eta * (observed - c->mirostat_tau);
    return finish(cid[i]);
  }
  // ---- draw
  double retained = 0.0;
  for (double v : prob) retained += v;
  const double thr = next_unit(st) * retained;
  int i = search_cumsum(prob, thr, true);
  i = std::min<int>(i, static_cast<int>(cid.size()) - 1);
  return finish(cid[i]);
}

// Layout of the two structs the Python bindings mirror by hand: sizes and the offsets of fields spread over the struct.
SLLM_HOST_EXPORT int sllm_host_sampler_abi(int* out, int cap) {
  const int v[] = {static_cast<int>(sizeof(SllmSamplerConfig)),
                   static_cast<int>(offsetof(SllmSamplerConfig, repeat_penalty)),
                   static_cast<int>(offsetof(SllmSamplerConfig, mirostat_eta)),
                   static_cast<int>(offsetof(SllmSamplerConfig, bias_tokens)),
                   static_cast<int>(offsetof(SllmSamplerConfig, dry_breakers)),
                   static_cast<int>(offsetof(SllmSamplerConfig, n_bias)),
                   static_cast<int>(offsetof(SllmSamplerConfig, ignore_eos_token)),
                   static_cast<int>(offsetof(SllmSamplerConfig, mirostat)),
                   static_cast<int>(offsetof(SllmSamplerConfig, top_logprobs)),
                   static_cast<int>(sizeof(SllmSamplerState)),
                   static_cast<int>(offsetof(SllmSamplerState, draws)),
                   static_cast<int>(offsetof(SllmSamplerState, mu))};
  const int n = static_cast<int>(sizeof(v) / sizeof(v[0]));
  if (!out || cap < n) return -SLLM_HOST_INVALID;
  for (int i = 0; i < n; ++i) out[i] = v[i];
  return n;
}
