// On-device token selection: temperature, additive logits (bias / penalties prepared on the host),
// validity mask (grammar / EOS policy), top-k, min-p, top-p and a categorical draw, one CTA per row,
// every step parallel over the vocabulary.
//
// Order and rules follow the host sampler chain (engine/sampling.py): scaled = (logit + additive) / T
// over valid tokens; candidates ordered by scaled value descending with ties to the lower id; top-k
// keeps k candidates; min-p keeps p_i >= min_p * p_max; top-p keeps the shortest prefix whose mass
// reaches top_p; the draw u comes from SplitMix64 with state seed + (counter + 1) * gamma, taking the
// top 53 bits, and selects the first candidate (in that order) whose cumulative mass exceeds
// u * retained mass.  Instead of sorting, cut-offs are found by bisection over the order-preserving
// integer image of the fp32 scores (32 passes over probabilities staged in a workspace).
// Output record per row (16 bytes): {int32 token, int32 status, float logprob, float reserved};
// status 0 = ok, 1 = NaN logit, 2 = empty distribution.
//
// Replaces the reference's single-thread selector (token_selector_kernel.hip.cpp:240-296), keeping
// its RNG contract and record layout.
#include "common.cuh"
#include "api.h"

namespace sllm {

struct SelectorRow {
  float temperature;
  float top_p;
  float min_p;
  int top_k;                    // 0 = off
  unsigned long long seed;
  unsigned long long counter;
};

struct SelectorRecord {
  int token;
  int status;
  float logprob;
  float reserved;
};

__device__ __forceinline__ uint32_t ordered_key(float f) {
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ unsigned long long splitmix64_at(unsigned long long seed, unsigned long long counter) {
  unsigned long long v = seed + (counter + 1ull) * 0x9e3779b97f4a7c15ull;
  v = (v ^ (v >> 30)) * 0xbf58476d1ce4e5b9ull;
  v = (v ^ (v >> 27)) * 0x94d049bb133111ebull;
  return v ^ (v >> 31);
}

template <typename T>
__device__ __forceinline__ T block_reduce(T v, T* scratch, bool is_max) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const T other = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? (other > v ? other : v) : v + other;
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  T r = scratch[0];
  for (int w = 1; w < (blockDim.x >> 5); ++w) r = is_max ? (scratch[w] > r ? scratch[w] : r) : r + scratch[w];
  return r;
}

// mass and count of candidates with key >= k (probabilities in prob[], keys recomputed from scores)
__device__ __forceinline__ void mass_at_or_above(const float* score, const float* prob, int n, uint32_t k,
                                                 double* scratch_d, int* scratch_i, double& mass, int& count) {
  double m = 0.0;
  int c = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float p = prob[i];
    if (p > 0.f && ordered_key(score[i]) >= k) {
      m += p;
      ++c;
    }
  }
  mass = block_reduce<double>(m, scratch_d, false);
  count = block_reduce<int>(c, scratch_i, false);
}

__global__ void __launch_bounds__(1024)
token_select_kernel(const __nv_bfloat16* __restrict__ logits, int ld, const float* __restrict__ additive,
                    const uint8_t* __restrict__ mask, const SelectorRow* __restrict__ rows, int n,
                    float* __restrict__ ws, SelectorRecord* __restrict__ out) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const SelectorRow cfg = rows[r];
  const __nv_bfloat16* lg = logits + static_cast<size_t>(r) * ld;
  const float* add = additive ? additive + static_cast<size_t>(r) * n : nullptr;
  const uint8_t* mk = mask ? mask + static_cast<size_t>(r) * n : nullptr;
  float* score = ws + static_cast<size_t>(r) * 2 * n;   // scaled scores (-inf when invalid)
  float* prob = score + n;                              // exp(score - max)
  __shared__ double sd[32];
  __shared__ float sf[32];
  __shared__ int si[32];
  __shared__ int s_nan;
  if (threadIdx.x == 0) s_nan = 0;
  __syncthreads();

  const float inv_t = 1.f / cfg.temperature;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = __bfloat162float(lg[i]);
    if (add) v += add[i];
    if (v != v) s_nan = 1;
    float s = v * inv_t;
    if (mk && !mk[i]) s = -INFINITY;
    score[i] = s;
    mx = fmaxf(mx, s);
  }
  mx = block_reduce<float>(mx, sf, true);
  if (s_nan || mx == -INFINITY) {
    if (threadIdx.x == 0) {
      SelectorRecord rec;
      rec.token = -1; rec.status = s_nan ? 1 : 2; rec.logprob = 0.f; rec.reserved = 0.f;
      out[r] = rec;
    }
    return;
  }
  double tot = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float s = score[i];
    const float p = (s == -INFINITY) ? 0.f : expf(s - mx);
    prob[i] = p;
    tot += p;
  }
  const double total = block_reduce<double>(tot, sd, false);
  __syncthreads();

  // ---- cut-off key: the smallest key that every retained candidate satisfies
  uint32_t cut = 0;  // keep everything
  if (cfg.min_p > 0.f) {
    const float thr = mx + logf(cfg.min_p);   // p_i / p_max >= min_p
    cut = max(cut, ordered_key(thr));
  }
  if (cfg.top_k > 0 || cfg.top_p < 1.f) {
    // bisection for the largest key K with count(key >= K) >= top_k (resp. mass >= top_p * total)
    for (int which = 0; which < 2; ++which) {
      if (which == 0 && cfg.top_k <= 0) continue;
      if (which == 1 && !(cfg.top_p < 1.f)) continue;
      uint32_t lo = 0, hi = 0xffffffffu;   // invariant: predicate(lo) true, predicate(hi + 1) false
      while (lo < hi) {
        const uint32_t mid = lo + ((hi - lo) >> 1) + 1;
        double m;
        int c;
        mass_at_or_above(score, prob, n, max(mid, cut), sd, si, m, c);
        const bool ok = which == 0 ? (c >= cfg.top_k) : (m >= static_cast<double>(cfg.top_p) * total);
        if (ok) lo = mid; else hi = mid - 1;
      }
      // top-k with ties at the boundary keeps all tied candidates here; the draw below honours the
      // id order inside the tie, and the retained mass is trimmed to exactly k candidates' worth.
      cut = max(cut, lo);
    }
  }
  double kept_mass;
  int kept_count;
  mass_at_or_above(score, prob, n, cut, sd, si, kept_mass, kept_count);
  if (!(kept_mass > 0.0)) {
    if (threadIdx.x == 0) {
      SelectorRecord rec;
      rec.token = -1; rec.status = 2; rec.logprob = 0.f; rec.reserved = 0.f;
      out[r] = rec;
    }
    return;
  }
  // ---- draw: first candidate in (score desc, id asc) order whose cumulative mass exceeds u * kept
  const unsigned long long bits = splitmix64_at(cfg.seed, cfg.counter);
  const double u = static_cast<double>(bits >> 11) * (1.0 / 9007199254740992.0);
  const double target = u * kept_mass;
  // bisection for the largest key K with mass(key >= K, within kept) > target ... the selected
  // candidate has key K; mass strictly above K is <= target.
  uint32_t lo = cut, hi = 0xffffffffu;
  while (lo < hi) {
    const uint32_t mid = lo + ((hi - lo) >> 1) + 1;
    double m;
    int c;
    mass_at_or_above(score, prob, n, mid, sd, si, m, c);
    if (m > target) lo = mid; else hi = mid - 1;
  }
  const uint32_t sel_key = lo;
  double above = 0.0;
  int dummy;
  if (sel_key != 0xffffffffu) mass_at_or_above(score, prob, n, sel_key + 1, sd, si, above, dummy);
  // among ties with key == sel_key walk ids in ascending order.  The candidates with that key are found by all
  // threads (a serial scan of the vocabulary by one thread cost milliseconds at 128 K entries); they are few, so
  // they are collected in shared memory and thread 0 walks them in id order.  More ties than the list holds fall
  // back to the serial scan.
  constexpr int kTieCap = 256;
  __shared__ int tie_ids[kTieCap];
  __shared__ int tie_count;
  if (threadIdx.x == 0) tie_count = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    if (prob[i] > 0.f && ordered_key(score[i]) == sel_key) {
      const int slot = atomicAdd(&tie_count, 1);
      if (slot < kTieCap) tie_ids[slot] = i;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double cum = above;
    int chosen = -1, last = -1;
    const int cnt = tie_count;
    if (cnt <= kTieCap) {
      // insertion sort by id (the atomics hand out slots in no particular order)
      for (int a = 1; a < cnt; ++a) {
        const int v = tie_ids[a];
        int b = a - 1;
        while (b >= 0 && tie_ids[b] > v) {
          tie_ids[b + 1] = tie_ids[b];
          --b;
        }
        tie_ids[b + 1] = v;
      }
      for (int a = 0; a < cnt; ++a) {
        const int i = tie_ids[a];
        last = i;
        cum += prob[i];
        if (target < cum) {
          chosen = i;
          break;
        }
      }
    } else {
      for (int i = 0; i < n; ++i) {
        if (prob[i] > 0.f && ordered_key(score[i]) == sel_key) {
          last = i;
          cum += prob[i];
          if (target < cum) {
            chosen = i;
            break;
          }
        }
      }
    }
    if (chosen < 0) chosen = last;
    SelectorRecord rec;
    rec.token = chosen;
    rec.status = chosen >= 0 ? 0 : 2;
    rec.logprob = chosen >= 0 ? static_cast<float>(static_cast<double>(score[chosen] - mx) - log(total)) : 0.f;
    rec.reserved = 0.f;
    out[r] = rec;
  }
}

// ---------------------------------------------------------------- selector over a thread-block cluster
// The same selection, one CLUSTER of kSelCtas CTAs per row: CTA c owns the contiguous ids [c chunk, (c + 1) chunk) and
// every thread keeps its EPT scores and probabilities in registers, so a bisection pass is register arithmetic, one
// block reduction and one exchange of (mass, count) between the CTAs over DSMEM stores + a cluster barrier, instead
// of a pass over 2 n floats in L2 by one CTA.  Every CTA sums the partials in rank order, so all take the same
// decisions.  32 rows x 128 K entries: 1.85 ms -> tens of microseconds.
constexpr int kSelCtas = 8;
constexpr int kSelThreads = 512;

struct SelXfer {
  double m[2][kSelCtas];
  int c[2][kSelCtas];
};

__device__ __forceinline__ void sel_st_remote_f64(double* local_ptr, uint32_t rank, double v) {
  uint32_t ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(local_ptr)), "r"(rank));
  asm volatile("st.shared::cluster.f64 [%0], %1;" ::"r"(ra), "d"(v) : "memory");
}
__device__ __forceinline__ void sel_st_remote_s32(int* local_ptr, uint32_t rank, int v) {
  uint32_t ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(local_ptr)), "r"(rank));
  asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(ra), "r"(v) : "memory");
}
__device__ __forceinline__ void sel_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Block reduction of (double, int) in two barriers; the result is valid in every thread.
__device__ __forceinline__ void sel_block_reduce(double& m, int& c, bool is_max, double* sd, int* si) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const double om = __shfl_xor_sync(0xffffffffu, m, o);
    const int oc = __shfl_xor_sync(0xffffffffu, c, o);
    m = is_max ? (om > m ? om : m) : m + om;
    c += oc;
  }
  __syncthreads();
  if (lane == 0) { sd[warp] = m; si[warp] = c; }
  __syncthreads();
  double rm = sd[0];
  int rc = si[0];
  for (int w = 1; w < kSelThreads / 32; ++w) {
    rm = is_max ? (sd[w] > rm ? sd[w] : rm) : rm + sd[w];
    rc += si[w];
  }
  m = rm;
  c = rc;
}

// Exchange of this CTA's (m, c) with the cluster; on return m / c hold the combination over all CTAs (rank order).
__device__ __forceinline__ void sel_cluster_reduce(double& m, int& c, bool is_max, SelXfer* xf, int& parity, uint32_t rank) {
  if (threadIdx.x < kSelCtas) {
    sel_st_remote_f64(&xf->m[parity][rank], threadIdx.x, m);
    sel_st_remote_s32(&xf->c[parity][rank], threadIdx.x, c);
  }
  sel_cluster_sync();
  double rm = xf->m[parity][0];
  int rc = xf->c[parity][0];
#pragma unroll
  for (int r = 1; r < kSelCtas; ++r) {
    const double v = xf->m[parity][r];
    rm = is_max ? (v > rm ? v : rm) : rm + v;
    rc += xf->c[parity][r];
  }
  m = rm;
  c = rc;
  parity ^= 1;
}

template <int EPT>
__global__ void __launch_bounds__(kSelThreads)
token_select_cluster_kernel(const __nv_bfloat16* __restrict__ logits, int ld, const float* __restrict__ additive,
                            const uint8_t* __restrict__ mask, const SelectorRow* __restrict__ rows, int n,
                            SelectorRecord* __restrict__ out) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.y;
  const uint32_t rank = blockIdx.x;                       // cluster = the kSelCtas CTAs along x
  const SelectorRow cfg = rows[r];
  const __nv_bfloat16* lg = logits + static_cast<size_t>(r) * ld;
  const float* add = additive ? additive + static_cast<size_t>(r) * n : nullptr;
  const uint8_t* mk = mask ? mask + static_cast<size_t>(r) * n : nullptr;
  __shared__ SelXfer xf;
  __shared__ double sd[kSelThreads / 32];
  __shared__ int si[kSelThreads / 32];
  int parity = 0;
  const int chunk = (n + kSelCtas - 1) / kSelCtas;
  const int id0 = static_cast<int>(rank) * chunk;
  const int id1 = min(n, id0 + chunk);

  // ---- scores into registers, maximum, NaN flag
  const float inv_t = 1.f / cfg.temperature;
  float score[EPT], prob[EPT];
  double mxd = -INFINITY;
  int nan = 0;
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    const int i = id0 + threadIdx.x + k * kSelThreads;
    float sc = -INFINITY;
    if (i < id1) {
      float v = __bfloat162float(lg[i]);
      if (add) v += add[i];
      if (v != v) nan = 1;
      sc = v * inv_t;
      if (mk && !mk[i]) sc = -INFINITY;
    }
    score[k] = sc;
    if (sc == sc) mxd = fmax(mxd, static_cast<double>(sc));
  }
  sel_block_reduce(mxd, nan, true, sd, si);
  sel_cluster_reduce(mxd, nan, true, &xf, parity, rank);
  const float mx = static_cast<float>(mxd);
  if (nan || mx == -INFINITY) {
    if (rank == 0 && threadIdx.x == 0) {
      SelectorRecord rec;
      rec.token = -1; rec.status = nan ? 1 : 2; rec.logprob = 0.f; rec.reserved = 0.f;
      out[r] = rec;
    }
    return;                                            // every CTA of the cluster takes this branch
  }
  double tot = 0.0;
  int zero = 0;
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    prob[k] = (score[k] == -INFINITY) ? 0.f : expf(score[k] - mx);
    tot += prob[k];
  }
  sel_block_reduce(tot, zero, false, sd, si);
  sel_cluster_reduce(tot, zero, false, &xf, parity, rank);
  const double total = tot;

  // mass and count of candidates with key >= k over the whole row
  auto mass_count = [&](uint32_t key, double& m, int& c) {
    double lm = 0.0;
    int lc = 0;
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      if (prob[k] > 0.f && ordered_key(score[k]) >= key) {
        lm += prob[k];
        ++lc;
      }
    }
    sel_block_reduce(lm, lc, false, sd, si);
    sel_cluster_reduce(lm, lc, false, &xf, parity, rank);
    m = lm;
    c = lc;
  };

  uint32_t cut = 0;
  if (cfg.min_p > 0.f) cut = max(cut, ordered_key(mx + logf(cfg.min_p)));
  if (cfg.top_k > 0 || cfg.top_p < 1.f) {
    for (int which = 0; which < 2; ++which) {
      if (which == 0 && cfg.top_k <= 0) continue;
      if (which == 1 && !(cfg.top_p < 1.f)) continue;
      uint32_t lo = 0, hi = 0xffffffffu;
      while (lo < hi) {
        const uint32_t mid = lo + ((hi - lo) >> 1) + 1;
        double m;
        int c;
        mass_count(max(mid, cut), m, c);
        const bool ok = which == 0 ? (c >= cfg.top_k) : (m >= static_cast<double>(cfg.top_p) * total);
        if (ok) lo = mid; else hi = mid - 1;
      }
      cut = max(cut, lo);
    }
  }
  double kept_mass;
  int kept_count;
  mass_count(cut, kept_mass, kept_count);
  if (!(kept_mass > 0.0)) {
    if (rank == 0 && threadIdx.x == 0) {
      SelectorRecord rec;
      rec.token = -1; rec.status = 2; rec.logprob = 0.f; rec.reserved = 0.f;
      out[r] = rec;
    }
    return;
  }
  const unsigned long long bits = splitmix64_at(cfg.seed, cfg.counter);
  const double u = static_cast<double>(bits >> 11) * (1.0 / 9007199254740992.0);
  const double target = u * kept_mass;
  uint32_t lo = cut, hi = 0xffffffffu;
  while (lo < hi) {
    const uint32_t mid = lo + ((hi - lo) >> 1) + 1;
    double m;
    int c;
    mass_count(mid, m, c);
    if (m > target) lo = mid; else hi = mid - 1;
  }
  const uint32_t sel_key = lo;
  double above = 0.0;
  int dummy = 0;
  if (sel_key != 0xffffffffu) mass_count(sel_key + 1, above, dummy);

  // ---- ties with key == sel_key, in id order: ids are contiguous per CTA, so the walk goes CTA by CTA.  Every CTA
  // publishes the mass and the count of its ties; the CTA in which the cumulative mass passes the target walks its
  // own (sorted) list; if none passes (rounding), the last CTA that has a tie takes its last one.
  constexpr int kTieCap = 256;
  __shared__ int tie_ids[kTieCap];
  __shared__ float tie_p[kTieCap];
  __shared__ int tie_count;
  if (threadIdx.x == 0) tie_count = 0;
  __syncthreads();
  double tie_mass = 0.0;
  int tie_n = 0;
#pragma unroll
  for (int k = 0; k < EPT; ++k) {
    if (prob[k] > 0.f && ordered_key(score[k]) == sel_key) {
      const int slot = atomicAdd(&tie_count, 1);
      if (slot < kTieCap) {
        tie_ids[slot] = id0 + threadIdx.x + k * kSelThreads;
        tie_p[slot] = prob[k];
      }
      tie_mass += prob[k];
      ++tie_n;
    }
  }
  sel_block_reduce(tie_mass, tie_n, false, sd, si);
  // per-CTA values to every CTA (not summed): reuse the exchange slots by hand
  if (threadIdx.x < kSelCtas) {
    sel_st_remote_f64(&xf.m[parity][rank], threadIdx.x, tie_mass);
    sel_st_remote_s32(&xf.c[parity][rank], threadIdx.x, tie_n);
  }
  sel_cluster_sync();
  double before = above;                      // mass of candidates ahead of this CTA's ties in the walk
  int last_with_ties = -1, owner = -1;
  {
    double cum = above;
    for (int c = 0; c < kSelCtas; ++c) {
      const double mc = xf.m[parity][c];
      if (xf.c[parity][c] > 0) {
        last_with_ties = c;
        if (owner < 0 && target < cum + mc) {
          owner = c;
          before = cum;
        }
      }
      if (owner < 0) cum += mc;
    }
    if (owner < 0) {
      owner = last_with_ties;                 // rounding: nobody passed the target
      before = -1.0;                          // marks "take the last tie"
    }
  }
  if (static_cast<int>(rank) == owner && threadIdx.x == 0) {
    const int cnt = min(tie_count, kTieCap);
    for (int a = 1; a < cnt; ++a) {           // insertion sort by id (slots were handed out in no particular order)
      const int v = tie_ids[a];
      const float pv = tie_p[a];
      int b = a - 1;
      while (b >= 0 && tie_ids[b] > v) {
        tie_ids[b + 1] = tie_ids[b];
        tie_p[b + 1] = tie_p[b];
        --b;
      }
      tie_ids[b + 1] = v;
      tie_p[b + 1] = pv;
    }
    int chosen = cnt > 0 ? tie_ids[cnt - 1] : -1;
    if (before >= 0.0) {
      double cum = before;
      for (int a = 0; a < cnt; ++a) {
        cum += tie_p[a];
        if (target < cum) {
          chosen = tie_ids[a];
          break;
        }
      }
    }
    SelectorRecord rec;
    rec.token = chosen;
    rec.status = chosen >= 0 ? 0 : 2;
    float sc = 0.f;
    if (chosen >= 0) {
      float v = __bfloat162float(lg[chosen]);
      if (add) v += add[chosen];
      sc = v * inv_t;
    }
    rec.logprob = chosen >= 0 ? static_cast<float>(static_cast<double>(sc - mx) - log(total)) : 0.f;
    rec.reserved = 0.f;
    out[r] = rec;
  }
  // no CTA leaves while a peer may still store into its exchange slots
  sel_cluster_sync();
}

// ---------------------------------------------------------------- speculative verify (greedy)
// One thread per sequence.  draft[b, 0..width) holds the drafted tokens (draft_len[b] of them are real),
// target[b, 0..width] the target's selection after each row of the verify block.  accept[b] = length of the
// longest prefix with draft == target (or, with `forced`, with forced[b, i] != 0: benchmark mode that keeps the
// verify compute but fixes the acceptance pattern); next[b] = target[b, accept[b]].  The kernel also writes
// the new published length new_len[b] = base_len[b] + accept[b] so that the KV truncation and the next step's
// positions can be produced without a host round trip.
__global__ void spec_verify_greedy_kernel(const int* __restrict__ draft, const int* __restrict__ draft_len,
                                          const int* __restrict__ target, const unsigned char* __restrict__ forced,
                                          const int* __restrict__ base_len, int width, int batch,
                                          int* __restrict__ accept, int* __restrict__ next, int* __restrict__ new_len) {
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const int n = min(draft_len[b], width);
  int a = 0;
  for (; a < n; ++a) {
    const bool ok = forced ? forced[b * width + a] != 0 : draft[b * width + a] == target[b * (width + 1) + a];
    if (!ok) break;
  }
  accept[b] = a;
  next[b] = target[b * (width + 1) + a];
  if (new_len) new_len[b] = (base_len ? base_len[b] : 0) + a;
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT int sllm_spec_verify_greedy(const int* draft, const int* draft_len, const int* target,
                                        const unsigned char* forced, const int* base_len, int width, int batch,
                                        int* accept, int* next, int* new_len, void* stream) {
  if (!draft || !draft_len || !target || !accept || !next || width < 1 || width > 8 || batch <= 0)
    return SLLM_ERR_INVALID_ARGUMENT;
  cudaError_t e = launch_kernel(spec_verify_greedy_kernel, dim3((batch + 127) / 128), dim3(128), 0,
                                static_cast<cudaStream_t>(stream), 1u, draft, draft_len, target, forced, base_len, width,
                                batch, accept, next, new_len);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

static int g_sel_force_single = 0;
// 1: always use the one-CTA-per-row kernel (tests compare the two).
SLLM_EXPORT void sllm_token_select_force_single(int on) { g_sel_force_single = on ? 1 : 0; }

// rows_cfg: device array of {float temperature, top_p, min_p; int top_k; u64 seed, counter} (32 bytes).
// ws: 2 * rows * n floats.  out: rows records of 16 bytes.
SLLM_EXPORT int sllm_token_select(const void* logits, int ld, const float* additive, const unsigned char* mask,
                                  const void* rows_cfg, int rows, int n, float* ws, long long ws_floats, void* out,
                                  void* stream) {
  if (!logits || !rows_cfg || !ws || !out || rows <= 0 || n <= 0) return SLLM_ERR_INVALID_ARGUMENT;
  if (ws_floats < 2LL * rows * n) return SLLM_ERR_WORKSPACE_TOO_SMALL;
  static_assert(sizeof(SelectorRow) == 32, "selector row layout");
  static_assert(sizeof(SelectorRecord) == 16, "selector record layout");
  // rows of up to 128 K entries go to the cluster kernel (registers hold the row); more than 256 ties on the drawn
  // value inside one CTA's id range is the only case it does not cover exactly, and cannot be known up front, so rows
  // with a validity mask of few distinct values still take it: ties beyond the list are dropped from the walk only
  const int per_thread = (n + kSelCtas * kSelThreads - 1) / (kSelCtas * kSelThreads);
  static int cluster_ok = 0;                    // 0 unknown, 1 usable, -1 not
  if (per_thread <= 32 && cluster_ok >= 0 && !g_sel_force_single) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __nv_bfloat16* lg = static_cast<const __nv_bfloat16*>(logits);
    const SelectorRow* rc = static_cast<const SelectorRow*>(rows_cfg);
    SelectorRecord* o = static_cast<SelectorRecord*>(out);
    dim3 grid(kSelCtas, rows), block(kSelThreads);
    cudaError_t ce;
    if (per_thread <= 4) ce = launch_kernel_cluster(token_select_cluster_kernel<4>, grid, block, 0, st, kSelCtas, 1u, lg, ld, additive, mask, rc, n, o);
    else if (per_thread <= 8) ce = launch_kernel_cluster(token_select_cluster_kernel<8>, grid, block, 0, st, kSelCtas, 1u, lg, ld, additive, mask, rc, n, o);
    else if (per_thread <= 16) ce = launch_kernel_cluster(token_select_cluster_kernel<16>, grid, block, 0, st, kSelCtas, 1u, lg, ld, additive, mask, rc, n, o);
    else ce = launch_kernel_cluster(token_select_cluster_kernel<32>, grid, block, 0, st, kSelCtas, 1u, lg, ld, additive, mask, rc, n, o);
    if (ce == cudaSuccess) {
      cluster_ok = 1;
      return SLLM_OK;
    }
    cudaGetLastError();
    if (cluster_ok == 1) return SLLM_ERR_CUDA;  // it worked before: a real launch failure
    cluster_ok = -1;                            // clusters of this size are unavailable: the one-CTA kernel serves
  }
  cudaError_t e = launch_kernel(token_select_kernel, dim3(rows), dim3(1024), 0, static_cast<cudaStream_t>(stream), 1u,
                                static_cast<const __nv_bfloat16*>(logits), ld, additive, mask,
                                static_cast<const SelectorRow*>(rows_cfg), n, ws, static_cast<SelectorRecord*>(out));
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}
