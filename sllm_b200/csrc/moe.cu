// Mixture-of-experts routing and token movement.
//
//   moe_route        router logits [T, E] -> top-k experts per token and their weights (softmax over the k
//                    selected logits, or the selected entries of the softmax over all experts);
//   moe_permute      groups the T x k assignments by expert: tok_off[E_local + 1], perm_src[P] (source token of
//                    each permuted row), perm_dst[T, k] (row of each assignment, -1 when the expert is not local),
//                    perm_w[P] (routing weight of each permuted row);
//   moe_gather       X_perm[p, :] = X[perm_src[p], :];
//   moe_combine      Y[t, :] = residual[t, :] + sum_j Y_perm[perm_dst[t, j], :]  (weights were applied by the
//                    expert GEMM epilogue);
//   moe_combine_allreduce   expert-parallel combine fused with the cross-rank reduction: every rank adds up its
//                    local experts' rows for a token block, stores the partial block straight into every peer's
//                    receive slot over NVLink, raises a flag per (block, source rank), waits (bounded) for the
//                    peers' flags and sums the partials in rank order, so all ranks hold bit-identical results.
//                    Activations are replicated across the expert-parallel ranks (they leave the attention
//                    all-reduce that way), so dispatch moves no data: each rank gathers the tokens routed to its
//                    own experts from its local copy.
//
// Reference counterparts: reference_sparse_moe_route (crates/sllm-core/src/moe.rs:229), the routing / expert
// kernels of native/hip/src/moe_expert_kernel.hip.cpp (one request at a time, no expert parallelism).
#include "common.cuh"
#include "api.h"

namespace sllm {

constexpr int kMaxTopK = 8;
constexpr int kMaxExperts = 256;

// One warp per token.  Ties go to the lower expert index; NaN logits count as -inf.
__global__ void moe_route_kernel(const __nv_bfloat16* __restrict__ logits, int ld, int tokens, int experts, int top_k,
                                 int softmax_all, int* __restrict__ out_idx, float* __restrict__ out_w) {
  pdl_wait();
  pdl_trigger();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  float v[kMaxExperts / 32];
#pragma unroll
  for (int i = 0; i < kMaxExperts / 32; ++i) {
    const int e = i * 32 + lane;
    float x = e < experts ? __bfloat162float(logits[static_cast<size_t>(warp) * ld + e]) : -INFINITY;
    v[i] = (x == x) ? x : -INFINITY;
  }
  float denom_all = 0.f, mx_all = -INFINITY;
  if (softmax_all) {
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i) mx_all = fmaxf(mx_all, v[i]);
    mx_all = warp_max(mx_all);
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i) denom_all += (v[i] == -INFINITY) ? 0.f : __expf(v[i] - mx_all);
    denom_all = warp_sum(denom_all);
  }
  float sel_v[kMaxTopK];
  int sel_i[kMaxTopK];
  for (int j = 0; j < top_k; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i) {
      const int e = i * 32 + lane;
      if (v[i] > best || (v[i] == best && e < bi && v[i] != -INFINITY)) {
        best = v[i];
        bi = e;
      }
    }
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
      }
    }
    if (bi == 0x7fffffff) bi = j;     // fewer finite logits than k: fall back to distinct low indices
    sel_v[j] = best;
    sel_i[j] = bi;
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i)
      if (i * 32 + lane == bi) v[i] = -INFINITY;
  }
  if (lane == 0) {
    float w[kMaxTopK];
    float sum = 0.f;
    const float m0 = softmax_all ? mx_all : sel_v[0];
    for (int j = 0; j < top_k; ++j) {
      w[j] = sel_v[j] == -INFINITY ? 0.f : __expf(sel_v[j] - m0);
      sum += w[j];
    }
    // mode 0: softmax over the selected logits; mode 1: probabilities of the softmax over all experts
    const float inv = softmax_all ? (denom_all > 0.f ? 1.f / denom_all : 0.f) : (sum > 0.f ? 1.f / sum : 0.f);
    for (int j = 0; j < top_k; ++j) {
      out_idx[warp * top_k + j] = sel_i[j];
      out_w[warp * top_k + j] = sum > 0.f ? w[j] * inv : 1.f / top_k;
    }
  }
}

// Single CTA of kPermuteThreads threads.  Counts per local expert in shared memory, exclusive scan, then a stable
// placement chunk by chunk: inside a chunk of one assignment per thread, lanes that share an expert find each
// other with match.any and rank themselves by lane, each warp's count per expert is scanned over the warps in
// order, and the running cursor of the expert advances by the chunk's total.  Assignments therefore keep their
// index order inside an expert (the layout is deterministic) at O(assignments / threads) steps instead of one
// serial walk per expert.
constexpr int kPermuteThreads = 1024;
constexpr int kPermuteWarps = kPermuteThreads / 32;

__global__ void __launch_bounds__(kPermuteThreads)
moe_permute_kernel(const int* __restrict__ idx, const float* __restrict__ w, int tokens, int top_k, int e_lo, int e_hi,
                   int* __restrict__ tok_off, int* __restrict__ perm_src, int* __restrict__ perm_dst,
                   float* __restrict__ perm_w) {
  pdl_wait();
  pdl_trigger();
  __shared__ int cursor[kMaxExperts + 1];
  __shared__ int wcount[kPermuteWarps * kMaxExperts];   // [warp][local expert] counts, then start offsets, of a chunk
  const int n_local = e_hi - e_lo;
  const int total = tokens * top_k;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i <= n_local; i += blockDim.x) cursor[i] = 0;
  __syncthreads();
  for (int a = threadIdx.x; a < total; a += blockDim.x) {
    const int e = idx[a];
    if (e >= e_lo && e < e_hi) atomicAdd(&cursor[e - e_lo], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < n_local; ++e) {
      const int c = cursor[e];
      cursor[e] = run;
      tok_off[e] = run;
      run += c;
    }
    cursor[n_local] = run;
    tok_off[n_local] = run;
  }
  for (int base = 0; base < total; base += kPermuteThreads) {
    for (int i = threadIdx.x; i < kPermuteWarps * n_local; i += blockDim.x) wcount[i] = 0;
    __syncthreads();                                   // also orders the scan above / the previous chunk's reads
    const int a = base + threadIdx.x;
    int e = -1;
    if (a < total) {
      e = idx[a] - e_lo;
      if (e < 0 || e >= n_local) e = -1;
    }
    // lanes without a local expert get a key of their own, so they match nobody
    const unsigned peers = __match_any_sync(0xffffffffu, e >= 0 ? e : (0x40000000 | lane));
    const int rank = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && rank == 0) wcount[warp * n_local + e] = __popc(peers);
    __syncthreads();
    for (int x = threadIdx.x; x < n_local; x += blockDim.x) {
      int run = cursor[x];
      for (int wv = 0; wv < kPermuteWarps; ++wv) {
        const int c = wcount[wv * n_local + x];
        wcount[wv * n_local + x] = run;
        run += c;
      }
      cursor[x] = run;
    }
    __syncthreads();
    if (e >= 0) {
      const int pos = wcount[warp * n_local + e] + rank;
      perm_src[pos] = a / top_k;
      perm_w[pos] = w[a];
      perm_dst[a] = pos;
    } else if (a < total) {
      perm_dst[a] = -1;
    }
    __syncthreads();
  }
}

// Shared expert of the Qwen3.5 MoE layer: y[t, :] = a[t, :] + sigmoid(gate[t * ld_gate]) * b[t, :] (the always-on
// expert's output joins the routed sum under a per-token sigmoid gate; reference:
// native/hip/src/moe_expert_kernel.hip.cpp:134-174 computes the gate, :176 applies it in the combine).
__global__ void moe_shared_add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                      const __nv_bfloat16* __restrict__ gate, int ld_gate, __nv_bfloat16* __restrict__ y,
                                      int d) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const float g = 1.f / (1.f + __expf(-__bfloat162float(gate[static_cast<size_t>(t) * ld_gate])));
  const uint4* pa = reinterpret_cast<const uint4*>(a + static_cast<size_t>(t) * d);
  const uint4* pb = reinterpret_cast<const uint4*>(b + static_cast<size_t>(t) * d);
  uint4* py = reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * d);
  for (int i = threadIdx.x; i < d / 8; i += blockDim.x) {
    const uint4 va = pa[i], vb = pb[i];
    const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&va);
    const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&vb);
    uint4 o;
    __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 fa = __bfloat1622float2(ha[j]), fb = __bfloat1622float2(hb[j]);
      ho[j] = __floats2bfloat162_rn(fa.x + g * fb.x, fa.y + g * fb.y);
    }
    py[i] = o;
  }
}

__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const int* __restrict__ perm_src,
                                  const int* __restrict__ tok_off, int n_local, __nv_bfloat16* __restrict__ xp, int d) {
  pdl_wait();
  pdl_trigger();
  const int p = blockIdx.x;
  if (p >= tok_off[n_local]) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(perm_src[p]) * ldx);
  uint4* dst = reinterpret_cast<uint4*>(xp + static_cast<size_t>(p) * d);
  for (int i = threadIdx.x; i < d / 8; i += blockDim.x) dst[i] = src[i];
}

__device__ __forceinline__ void add8(float (&acc)[8], const uint4 v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&acc)[8]) {
  uint4 o;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  return o;
}

// One CTA per token: sum of the (local) expert rows in slot order, plus the residual.
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ yp, const int* __restrict__ perm_dst, int top_k,
                                   const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ y, int d) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < d / 8; i += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      const int p = perm_dst[t * top_k + j];
      if (p >= 0) add8(acc, reinterpret_cast<const uint4*>(yp + static_cast<size_t>(p) * d)[i]);
    }
    if (residual) add8(acc, reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * d)[i]);
    reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * d)[i] = pack8(acc);
  }
}

struct EpPeers {
  int world, rank;
  __nv_bfloat16* recv[8];   // recv[p]: rank p's receive area [2 parities][world][max_tokens * d] as mapped here
  uint32_t* flags[8];       // flags[p]: rank p's flags [world][max_blocks]
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// grid.x = token blocks of `rows_per_block` tokens.  cap = max_tokens * d elements per (parity, source) slot.
__global__ void moe_combine_allreduce_kernel(EpPeers pe, const __nv_bfloat16* __restrict__ yp,
                                             const int* __restrict__ perm_dst, int top_k,
                                             const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ y,
                                             int tokens, int d, int rows_per_block, long long cap, int max_blocks,
                                             uint32_t* __restrict__ epoch, int* status) {
  pdl_wait();
  pdl_trigger();
  __shared__ uint32_t s_e;
  __shared__ int s_ok;
  const int b = blockIdx.x;
  if (threadIdx.x == 0) {
    s_e = epoch[b] + 1;
    epoch[b] = s_e;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t e = s_e;
  const long long par = static_cast<long long>(e & 1) * pe.world * cap;
  const int t0 = b * rows_per_block;
  const int t1 = min(tokens, t0 + rows_per_block);
  const int vec = d / 8;
  // 1. local partial rows -> every rank's slot [parity][my rank] (own slot included)
  for (int i = threadIdx.x; i < (t1 - t0) * vec; i += blockDim.x) {
    const int t = t0 + i / vec, c = i % vec;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      const int p = perm_dst[t * top_k + j];
      if (p >= 0) add8(acc, reinterpret_cast<const uint4*>(yp + static_cast<size_t>(p) * d)[c]);
    }
    const uint4 o = pack8(acc);
    const long long off = par + static_cast<long long>(pe.rank) * cap + static_cast<long long>(t) * d + c * 8;
    for (int p = 0; p < pe.world; ++p) *reinterpret_cast<uint4*>(pe.recv[p] + off) = o;
  }
  __threadfence_system();
  __syncthreads();
  // 2. flags: one per (block, source rank) at every destination; then wait for all sources (bounded)
  if (threadIdx.x < pe.world) {
    st_release_sys(pe.flags[threadIdx.x] + pe.rank * max_blocks + b, e);
    const uint32_t* mine = pe.flags[pe.rank] + threadIdx.x * max_blocks + b;
    uint32_t spins = 0;
    long long tstart = 0;
    while (static_cast<int32_t>(ld_acquire_sys_(mine) - e) < 0) {
      ++spins;
      if (spins == 1024) tstart = clock64();
      if (spins > 1024 && (spins & 63) == 0 && clock64() - tstart > kWaitLimitCycles) {
        if (status) atomicCAS(status, 0, SLLM_DEV_TIMEOUT_PEER_FLAG);
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (!s_ok) return;
  // 3. sum the partials in rank order (+ residual)
  const __nv_bfloat16* base = pe.recv[pe.rank] + par;
  for (int i = threadIdx.x; i < (t1 - t0) * vec; i += blockDim.x) {
    const int t = t0 + i / vec, c = i % vec;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < pe.world; ++r)
      add8(acc, __ldcg(reinterpret_cast<const uint4*>(base + static_cast<long long>(r) * cap + static_cast<long long>(t) * d) + c));
    if (residual) add8(acc, reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * d)[c]);
    reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * d)[c] = pack8(acc);
  }
}

// ------------------------------------------------------------------------------------------------ owner combine
// Expert parallelism with token owners.  Rank r owns the tokens [r tpr, (r + 1) tpr).  The down-projection GEMM of
// every rank stores each routed row (route weight applied) straight into the OWNER's receive slot (token, j) over
// NVLink - slot j of a token belongs to the j-th expert of its top-k list, written by the one rank that holds that
// expert - so a rank sends only the rows its experts produced, once, to one peer.  Then:
//   signal  (1 CTA)  after the GEMM: system fence, "my rows have landed" flag at every peer
//   reduce  owners wait for all ranks' flags (bounded), sum their tokens' k slots in slot order (+ residual) and
//           store the finished row into every rank's gather buffer; the last CTA raises "my tokens are out"
//   finish  waits for all ranks' gather flags (bounded) and copies the gathered rows out
// Per step a rank sends (rows its experts produced) + (world - 1) tpr rows, instead of (world - 1) T rows when every
// rank pushed a full partial to every peer.  Slots and gather rows alternate between two parities per call.
// No counterpart in the reference, which has no multi-GPU path (its fused single-GPU pair is
// native/hip/src/moe_expert_kernel.hip.cpp:88 gate/up + SiLU and :176 down + route weight + combine).
struct EpOwner {
  int world, rank;
  __nv_bfloat16* recv[8];     // recv[p]: rank p's slots [2][tpr_cap * top_k_cap * d]
  __nv_bfloat16* gath[8];     // gath[p]: rank p's gather buffer [2][max_tokens * d]
  uint32_t* flags[8];         // flags[p]: rank p's flags [2][world]: rows landed / tokens out, per source rank
  long long recv_cap, gath_cap;   // elements per parity
};

__global__ void moe_owner_plan_kernel(EpOwner pe, const int* __restrict__ perm_dst, int tokens, int top_k, int d, int tpr,
                                      const uint32_t* __restrict__ epoch, long long* __restrict__ row_ptr) {
  pdl_wait();
  pdl_trigger();
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= tokens * top_k) return;
  const int p = perm_dst[a];
  if (p < 0) return;                       // another rank holds that expert
  const int t = a / top_k, j = a - t * top_k;
  const int owner = t / tpr, tl = t - owner * tpr;
  const uint32_t e = epoch[0] + 1;         // the call in progress; the signal kernel publishes it
  row_ptr[p] = reinterpret_cast<long long>(pe.recv[owner] + static_cast<long long>(e & 1) * pe.recv_cap +
                                           (static_cast<long long>(tl) * top_k + j) * d);
}

__global__ void moe_owner_signal_kernel(EpOwner pe, uint32_t* epoch) {
  pdl_wait();
  pdl_trigger();
  const uint32_t e = epoch[0] + 1;
  __threadfence_system();
  if (threadIdx.x < pe.world) st_release_sys(pe.flags[threadIdx.x] + pe.rank, e);
  __syncthreads();
  if (threadIdx.x == 0) epoch[0] = e;
}

// Bounded wait of thread `src` (< world) for flag word `kind * world + src` of this rank; false when it gave up.
__device__ __forceinline__ bool owner_wait(const EpOwner& pe, int kind, int src, uint32_t e, int* status) {
  const uint32_t* f = pe.flags[pe.rank] + kind * pe.world + src;
  uint32_t spins = 0;
  long long tstart = 0;
  while (static_cast<int32_t>(ld_acquire_sys_(f) - e) < 0) {
    ++spins;
    if (spins == 1024) tstart = clock64();
    if (spins > 1024 && (spins & 63) == 0 && clock64() - tstart > kWaitLimitCycles) {
      if (status) atomicCAS(status, 0, SLLM_DEV_TIMEOUT_PEER_FLAG);
      return false;
    }
  }
  return true;
}

__global__ void moe_owner_reduce_kernel(EpOwner pe, int top_k, const __nv_bfloat16* __restrict__ residual, int tokens,
                                        int d, int tpr, int rows_per_block, const uint32_t* __restrict__ epoch,
                                        int* counter, int* status) {
  pdl_wait();
  pdl_trigger();
  __shared__ int s_ok;
  const uint32_t e = epoch[0];
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < pe.world && !owner_wait(pe, 0, threadIdx.x, e, status)) s_ok = 0;
  __syncthreads();
  const int t_lo = pe.rank * tpr;
  const int t_hi = min(tokens, t_lo + tpr);
  const int t0 = t_lo + blockIdx.x * rows_per_block;
  const int t1 = min(t_hi, t0 + rows_per_block);
  const int vec = d / 8;
  if (s_ok && t0 < t1) {
    const __nv_bfloat16* slots = pe.recv[pe.rank] + static_cast<long long>(e & 1) * pe.recv_cap;
    const long long goff = static_cast<long long>(e & 1) * pe.gath_cap;
    for (int i = threadIdx.x; i < (t1 - t0) * vec; i += blockDim.x) {
      const int t = t0 + i / vec, c = i % vec;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      const __nv_bfloat16* row = slots + static_cast<long long>(t - t_lo) * top_k * d;
      for (int j = 0; j < top_k; ++j) add8(acc, __ldcg(reinterpret_cast<const uint4*>(row + static_cast<long long>(j) * d) + c));
      if (residual) add8(acc, reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * d)[c]);
      const uint4 o = pack8(acc);
      for (int p = 0; p < pe.world; ++p)
        *reinterpret_cast<uint4*>(pe.gath[p] + goff + static_cast<long long>(t) * d + c * 8) = o;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(counter, 1);
    s_ok = (prev == static_cast<int>(gridDim.x) - 1) ? 2 : 0;
    if (s_ok == 2) *counter = 0;
  }
  __syncthreads();
  // the last CTA of this rank: every row of its tokens is on its way to every peer
  if (s_ok == 2) {
    __threadfence_system();
    if (threadIdx.x < pe.world) st_release_sys(pe.flags[threadIdx.x] + pe.world + pe.rank, e);
  }
}

__global__ void moe_owner_finish_kernel(EpOwner pe, __nv_bfloat16* __restrict__ y, int tokens, int d, int rows_per_block,
                                        const uint32_t* __restrict__ epoch, int* status) {
  pdl_wait();
  pdl_trigger();
  __shared__ int s_ok;
  const uint32_t e = epoch[0];
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < pe.world && !owner_wait(pe, 1, threadIdx.x, e, status)) s_ok = 0;
  __syncthreads();
  if (!s_ok) return;
  const int t0 = blockIdx.x * rows_per_block, t1 = min(tokens, t0 + rows_per_block);
  const int vec = d / 8;
  const uint4* src = reinterpret_cast<const uint4*>(pe.gath[pe.rank] + static_cast<long long>(e & 1) * pe.gath_cap);
  for (int i = threadIdx.x; i < (t1 - t0) * vec; i += blockDim.x)
    reinterpret_cast<uint4*>(y)[static_cast<size_t>(t0) * vec + i] = __ldcg(src + static_cast<size_t>(t0) * vec + i);
}

}  // namespace sllm

using namespace sllm;

static int owner_desc(EpOwner* pe, void* const* recv, void* const* gath, void* const* flags, int world, int rank,
                      long long recv_cap, long long gath_cap) {
  if (!recv || !gath || !flags || world < 1 || world > 8 || rank < 0 || rank >= world || recv_cap <= 0 || gath_cap <= 0)
    return SLLM_ERR_INVALID_ARGUMENT;
  pe->world = world; pe->rank = rank; pe->recv_cap = recv_cap; pe->gath_cap = gath_cap;
  for (int i = 0; i < world; ++i) {
    if (!recv[i] || !gath[i] || !flags[i]) return SLLM_ERR_INVALID_ARGUMENT;
    pe->recv[i] = static_cast<__nv_bfloat16*>(recv[i]);
    pe->gath[i] = static_cast<__nv_bfloat16*>(gath[i]);
    pe->flags[i] = static_cast<uint32_t*>(flags[i]);
  }
  return SLLM_OK;
}

// Step 1 of the owner combine: destination address of every local permuted row (perm_dst from sllm_moe_permute) in
// its token owner's receive slots, for the scatter epilogue of the down-projection GEMM (sllm_gemm_w4_scatter).
// tpr = tokens per rank (ceil(tokens / world)); epoch: one device word, zero before the first call.
SLLM_EXPORT int sllm_moe_owner_plan(void* const* recv, void* const* gath, void* const* flags, int world, int rank,
                                    long long recv_cap, long long gath_cap, const int* perm_dst, int tokens, int top_k, int d,
                                    int tpr, const void* epoch, long long* row_ptr, void* stream) {
  EpOwner pe;
  const int rc = owner_desc(&pe, recv, gath, flags, world, rank, recv_cap, gath_cap);
  if (rc != SLLM_OK) return rc;
  if (!perm_dst || !epoch || !row_ptr || tokens <= 0 || top_k <= 0 || d <= 0 || (d % 8) || tpr <= 0 ||
      static_cast<long long>(tpr) * world < tokens || static_cast<long long>(tpr) * top_k * d > recv_cap ||
      static_cast<long long>(tokens) * d > gath_cap)
    return SLLM_ERR_INVALID_ARGUMENT;
  const int n = tokens * top_k;
  cudaError_t e = launch_kernel(moe_owner_plan_kernel, dim3((n + 255) / 256), dim3(256), 0, static_cast<cudaStream_t>(stream), 1u,
                                pe, perm_dst, tokens, top_k, d, tpr, static_cast<const uint32_t*>(epoch), row_ptr);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

// Steps 2-4, launched after the scatter GEMM on the same stream: signal, reduce + gather, finish (see above).
// y: bf16 [tokens, d] result on this rank; counter: one zeroed device int.
SLLM_EXPORT int sllm_moe_owner_combine(void* const* recv, void* const* gath, void* const* flags, int world, int rank,
                                       long long recv_cap, long long gath_cap, int top_k, const void* residual, void* y,
                                       int tokens, int d, int tpr, int rows_per_block, void* epoch, int* counter, int* status,
                                       void* stream) {
  EpOwner pe;
  const int rc = owner_desc(&pe, recv, gath, flags, world, rank, recv_cap, gath_cap);
  if (rc != SLLM_OK) return rc;
  if (!y || !epoch || !counter || tokens <= 0 || top_k <= 0 || d <= 0 || (d % 8) || tpr <= 0 || rows_per_block <= 0 ||
      static_cast<long long>(tpr) * world < tokens)
    return SLLM_ERR_INVALID_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (launch_kernel(moe_owner_signal_kernel, dim3(1), dim3(32), 0, st, 1u, pe, static_cast<uint32_t*>(epoch)) != cudaSuccess)
    return SLLM_ERR_CUDA;
  const int own_blocks = (tpr + rows_per_block - 1) / rows_per_block;
  if (launch_kernel(moe_owner_reduce_kernel, dim3(own_blocks), dim3(256), 0, st, 1u, pe, top_k,
                    static_cast<const __nv_bfloat16*>(residual), tokens, d, tpr, rows_per_block,
                    static_cast<const uint32_t*>(epoch), counter, status) != cudaSuccess)
    return SLLM_ERR_CUDA;
  const int blocks = (tokens + rows_per_block - 1) / rows_per_block;
  if (launch_kernel(moe_owner_finish_kernel, dim3(blocks), dim3(256), 0, st, 1u, pe, static_cast<__nv_bfloat16*>(y), tokens, d,
                    rows_per_block, static_cast<const uint32_t*>(epoch), status) != cudaSuccess)
    return SLLM_ERR_CUDA;
  return SLLM_OK;
}

SLLM_EXPORT int sllm_moe_route(const void* logits, int ld, int tokens, int experts, int top_k, int softmax_all,
                               int* out_idx, float* out_w, void* stream) {
  if (!logits || !out_idx || !out_w || tokens <= 0 || experts <= 0 || experts > kMaxExperts || top_k <= 0 ||
      top_k > kMaxTopK || top_k > experts)
    return SLLM_ERR_INVALID_ARGUMENT;
  cudaError_t e = launch_kernel(moe_route_kernel, dim3((tokens + 3) / 4), dim3(128), 0, static_cast<cudaStream_t>(stream),
                                1u, static_cast<const __nv_bfloat16*>(logits), ld, tokens, experts, top_k, softmax_all,
                                out_idx, out_w);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

SLLM_EXPORT int sllm_moe_permute(const int* idx, const float* w, int tokens, int top_k, int e_lo, int e_hi, int* tok_off,
                                 int* perm_src, int* perm_dst, float* perm_w, void* stream) {
  if (!idx || !w || !tok_off || !perm_src || !perm_dst || !perm_w || tokens <= 0 || top_k <= 0 || e_lo < 0 ||
      e_hi <= e_lo || e_hi - e_lo > kMaxExperts)
    return SLLM_ERR_INVALID_ARGUMENT;
  if (static_cast<long long>(tokens) * top_k > (1LL << 30)) return SLLM_ERR_UNSUPPORTED_SHAPE;
  cudaError_t e = launch_kernel(moe_permute_kernel, dim3(1), dim3(kPermuteThreads), 0, static_cast<cudaStream_t>(stream), 1u,
                                idx, w, tokens, top_k, e_lo, e_hi, tok_off, perm_src, perm_dst, perm_w);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

// y = a + sigmoid(gate[t * ld_gate]) * b over [tokens, d] bf16 rows (y may alias a); d a multiple of 8.
SLLM_EXPORT int sllm_moe_shared_add(const void* a, const void* b, const void* gate, int ld_gate, void* y, int tokens, int d,
                                    void* stream) {
  if (!a || !b || !gate || !y || tokens <= 0 || d <= 0 || (d % 8) || ld_gate <= 0) return SLLM_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(y)) & 15)
    return SLLM_ERR_ALIGNMENT;
  cudaError_t e = launch_kernel(moe_shared_add_kernel, dim3(tokens), dim3(128), 0, static_cast<cudaStream_t>(stream), 1u,
                                static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b),
                                static_cast<const __nv_bfloat16*>(gate), ld_gate, static_cast<__nv_bfloat16*>(y), d);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

SLLM_EXPORT int sllm_moe_gather(const void* x, int ldx, const int* perm_src, const int* tok_off, int n_local, void* xp,
                                int d, int max_rows, void* stream) {
  if (!x || !perm_src || !tok_off || !xp || d <= 0 || (d % 8) || (ldx % 8) || max_rows <= 0) return SLLM_ERR_INVALID_ARGUMENT;
  cudaError_t e = launch_kernel(moe_gather_kernel, dim3(max_rows), dim3(128), 0, static_cast<cudaStream_t>(stream), 1u,
                                static_cast<const __nv_bfloat16*>(x), ldx, perm_src, tok_off, n_local,
                                static_cast<__nv_bfloat16*>(xp), d);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

SLLM_EXPORT int sllm_moe_combine(const void* yp, const int* perm_dst, int top_k, const void* residual, void* y, int tokens,
                                 int d, void* stream) {
  if (!yp || !perm_dst || !y || tokens <= 0 || d <= 0 || (d % 8) || top_k <= 0) return SLLM_ERR_INVALID_ARGUMENT;
  cudaError_t e = launch_kernel(moe_combine_kernel, dim3(tokens), dim3(128), 0, static_cast<cudaStream_t>(stream), 1u,
                                static_cast<const __nv_bfloat16*>(yp), perm_dst, top_k,
                                static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(y), d);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

// recv / flags: arrays of `world` peer pointers (this rank's own included); cap_elems = max_tokens * d.
SLLM_EXPORT int sllm_moe_combine_allreduce(const void* const* recv, const void* const* flags, int world, int rank,
                                           const void* yp, const int* perm_dst, int top_k, const void* residual, void* y,
                                           int tokens, int d, int rows_per_block, long long cap_elems, int max_blocks,
                                           void* epoch, int* status, void* stream) {
  if (!recv || !flags || world < 2 || world > 8 || rank < 0 || rank >= world || !yp || !perm_dst || !y || !epoch ||
      tokens <= 0 || d <= 0 || (d % 8) || rows_per_block <= 0)
    return SLLM_ERR_INVALID_ARGUMENT;
  const int blocks = (tokens + rows_per_block - 1) / rows_per_block;
  if (blocks > max_blocks || static_cast<long long>(tokens) * d > cap_elems) return SLLM_ERR_WORKSPACE_TOO_SMALL;
  EpPeers pe;
  pe.world = world;
  pe.rank = rank;
  for (int i = 0; i < world; ++i) {
    pe.recv[i] = static_cast<__nv_bfloat16*>(const_cast<void*>(recv[i]));
    pe.flags[i] = static_cast<uint32_t*>(const_cast<void*>(flags[i]));
  }
  cudaError_t e = launch_kernel(moe_combine_allreduce_kernel, dim3(blocks), dim3(256), 0,
                                static_cast<cudaStream_t>(stream), 1u, pe, static_cast<const __nv_bfloat16*>(yp), perm_dst,
                                top_k, static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(y), tokens, d,
                                rows_per_block, cap_elems, max_blocks, static_cast<uint32_t*>(epoch), status);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}
