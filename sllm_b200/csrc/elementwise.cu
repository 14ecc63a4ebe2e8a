// Memory-bound kernels of the decoder layer: embedding gather, RMSNorm (+ FP8 1x128 output
// quantisation), gated activations (+ quantisation), stand-alone activation quantisation, RoPE fused
// with the quantising KV-page append, residual/elementwise helpers and row argmax.
//
// FP8 activation format produced here and consumed by the block-scaled GEMM: E4M3FN values [M, K]
// plus one fp32 scale per (row, 128-wide K block) stored K-block-major: scale[kb * ld + row], with
// scale = amax / 448 (1.0 when the block is all zero), NaN -> 0x7f, +-Inf saturating to +-448.
//
// Counterparts in the reference: rmsnorm_kernel.hip.cpp:67, elementwise_kernel.hip.cpp:40-147,
// embedding_kernel.hip.cpp:4, rotary_kernel.hip.cpp:40, kv_state_kernel.hip.cpp:161-335,
// matmul_kernel.hip.cpp:210-247 (activation quantisation), argmax_kernel.hip.cpp:37.
#include "common.cuh"
#include "api.h"
#include "noalloc.h"
#include <mutex>

namespace sllm {

constexpr float kE4M3Max = 448.f;

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float gelu_tanh(float x) {
  const float c = 0.7978845608028654f;
  return 0.5f * x * (1.f + tanhf(c * (x + 0.044715f * x * x * x)));
}

// Quantise 8 values held by each of 16 consecutive lanes (one 128-element block) and store them.
// `store` = false for lanes that only take part in the shuffle (pointers are then never dereferenced;
// no pointer to a local dummy is ever formed, which the compiler would fold into a dead store).
__device__ __forceinline__ void quant_block128_store(const float (&v)[8], uint8_t* dst8, float* scale_dst,
                                                     bool store, bool lane_writes_scale) {
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float a = fabsf(v[j]);
    if (a == a && a <= 3.0e38f) amax = fmaxf(amax, a);  // NaN / Inf do not set the scale
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = amax > 0.f ? amax / kE4M3Max : 1.f;
  uint32_t lo = 0, hi = 0;  // true division keeps the bytes identical to the host quantiser
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    lo |= static_cast<uint32_t>(f32_to_e4m3(__fdiv_rn(v[j], scale))) << (8 * j);
    hi |= static_cast<uint32_t>(f32_to_e4m3(__fdiv_rn(v[j + 4], scale))) << (8 * j);
  }
  if (store) {
    *reinterpret_cast<uint2*>(dst8) = make_uint2(lo, hi);
    if (lane_writes_scale) *scale_dst = scale;
  }
}

__device__ __forceinline__ void load8_bf16(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __bfloat162float(h[j].x);
    v[2 * j + 1] = __bfloat162float(h[j].y);
  }
}
__device__ __forceinline__ void store8_bf16(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 out;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
  for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
  *reinterpret_cast<uint4*>(p) = out;
}

// ---------------------------------------------------------------- embedding
__global__ void embedding_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ ids,
                                 __nv_bfloat16* __restrict__ out, int d, int vocab, float scale) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const __nv_bfloat16* src = table + static_cast<size_t>(id) * d;
  __nv_bfloat16* dst = out + static_cast<size_t>(t) * d;
  for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8) {
    if (scale == 1.f) {
      *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
    } else {
      float v[8];
      load8_bf16(src + i, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] *= scale;
      store8_bf16(dst + i, v);
    }
  }
}

// ---------------------------------------------------------------- RMSNorm (+ quant)
// One CTA per row.  offset_one selects the (1 + w) scale convention, otherwise the weight is the scale.
template <bool kQuant>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
               __nv_bfloat16* __restrict__ y_bf16, uint8_t* __restrict__ y_fp8, float* __restrict__ y_scale,
               int ld_scale, int d, float eps, int offset_one) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float row[];  // d floats
  __shared__ float red[8];
  const int r = blockIdx.x;
  const __nv_bfloat16* xr = x + static_cast<size_t>(r) * d;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < d; i += blockDim.x * 8) {
    float v[8];
    load8_bf16(xr + i, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      row[i + j] = v[j];
      ss += v[j] * v[j];
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += (i < (blockDim.x >> 5)) ? red[i] : 0.f;
  const float inv = rsqrtf(tot / d + eps);
  // Uniform trip count per CTA so that the 16-lane quantisation shuffles always see a full warp.
  for (int i0 = 0; i0 < d; i0 += blockDim.x * 8) {
    const int i = i0 + threadIdx.x * 8;
    const bool in_range = i < d;
    float wv[8], v[8];
    if (in_range) {
      load8_bf16(w + i, wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float g = offset_one ? 1.f + wv[j] : wv[j];
        // The normalised value is rounded to bf16 before any further use, as the unfused sequence
        // norm -> bf16 tensor -> quantise would do.
        v[j] = __bfloat162float(__float2bfloat16_rn(row[i + j] * inv * g));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
    if (kQuant) {
      quant_block128_store(v, y_fp8 + static_cast<size_t>(r) * d + i,
                           y_scale + static_cast<size_t>(i >> 7) * ld_scale + r, in_range, (threadIdx.x & 15) == 0);
    } else if (in_range) {
      store8_bf16(y_bf16 + static_cast<size_t>(r) * d + i, v);
    }
  }
}

// ---------------------------------------------------------------- gated activation (+ quant)
// in: [M, 2*I] with the gate in columns [0, I) and up in [I, 2I).  act: 0 SiLU, 1 GELU(tanh).
template <bool kQuant>
__global__ void __launch_bounds__(256)
gated_act_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ y_bf16,
                 uint8_t* __restrict__ y_fp8, float* __restrict__ y_scale, int ld_scale, int inter, int act) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  // All lanes of a 16-lane group run the quantisation shuffle; out-of-range lanes contribute zeros.
  float g[8], u[8], v[8];
  const bool in_range = i < inter;
  if (in_range) {
    load8_bf16(in + static_cast<size_t>(r) * 2 * inter + i, g);
    load8_bf16(in + static_cast<size_t>(r) * 2 * inter + inter + i, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = act == 0 ? silu(g[j]) : gelu_tanh(g[j]);
      v[j] = __bfloat162float(__float2bfloat16_rn(__bfloat162float(__float2bfloat16_rn(a)) * u[j]));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
  }
  if (kQuant) {
    quant_block128_store(v, y_fp8 + static_cast<size_t>(r) * inter + i,
                         y_scale + static_cast<size_t>(i >> 7) * ld_scale + r, in_range, (threadIdx.x & 15) == 0);
  } else if (in_range) {
    store8_bf16(y_bf16 + static_cast<size_t>(r) * inter + i, v);
  }
}

// ---------------------------------------------------------------- stand-alone 1x128 quantisation
__global__ void __launch_bounds__(256)
quant_fp8_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ y, float* __restrict__ scale,
                 int ld_scale, int k) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const int i = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  float v[8];
  const bool in_range = i < k;
  if (in_range) {
    load8_bf16(x + static_cast<size_t>(r) * k + i, v);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
  }
  quant_block128_store(v, y + static_cast<size_t>(r) * k + i, scale + static_cast<size_t>(i >> 7) * ld_scale + r,
                       in_range, (threadIdx.x & 15) == 0);
}

// ---------------------------------------------------------------- RoPE + KV page append
// qkv: [T, (hq + 2*hkv) * hd] bf16.  One CTA per (token, head): q and k heads are rotated in place, k heads
// are also written to the K pages, v heads are copied to the V pages; pages are bf16 or E4M3
// with one fp32 scale per (token, head) = amax / 448.
// Split-half ("NeoX") rotation over the first rotary_dim channels:
//   out[i] = x[i] cos - x[i + r/2] sin,  out[i + r/2] = x[i + r/2] cos + x[i] sin,  angle = pos * theta^(-2i/r)
struct RopeKvParams {
  __nv_bfloat16* qkv;
  const int* positions;    // [T]
  const int* seq_index;    // [T] row of block_table owning each token
  const int* block_table;  // [num_seqs, max_blocks]
  int max_blocks;
  void* k_pages;           // [num_pages, hkv, page, hd]
  void* v_pages;
  float* k_scale;          // [num_pages, hkv, page] (fp8 only)
  float* v_scale;
  int hq, hkv, hd, rotary_dim, page_size, kv_fp8;
  float theta;
  float k_static_scale, v_static_scale;  // > 0: static fp8 scales instead of per token-head amax
  const float* inv_freq;   // optional [rotary_dim / 2] precomputed frequencies (scaled RoPE variants)
  // multi-axis rotary positions (vision-language prompts): [3, tokens] = temporal, height, width index of every
  // token; rotary pair j turns with axis 0 for j < sec_t, axis 1 for j < sec_t + sec_h, axis 2 otherwise.
  // Null: every pair turns with positions[t].  The page slot always comes from positions[t].
  const int* rope_pos3;
  int tokens, sec_t, sec_h;
  // 0: channel i pairs with i + rotary_dim / 2, frequencies theta^(-2 i / rotary_dim).  > 0 ("proportional" layout of
  // partially rotated wide heads): channel i < rotary_dim / 2 pairs with i + pair_offset (= head_dim / 2) and the
  // frequencies are theta^(-2 i / head_dim); the channels between stay as they are.
  int pair_offset;
};

__global__ void __launch_bounds__(128) rope_kv_append_kernel(const RopeKvParams p) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int h = blockIdx.y;  // 0..hq-1 q, hq..hq+hkv-1 k, then v
  const int hd = p.hd;
  __shared__ float vals[512];
  __shared__ float rot[512];
  __shared__ float red[4];
  __nv_bfloat16* src = p.qkv + (static_cast<size_t>(t) * (p.hq + 2 * p.hkv) + h) * hd;
  const int pos = p.positions[t];
  const bool is_v = h >= p.hq + p.hkv;
  const bool is_q = h < p.hq;
  const int half = p.rotary_dim >> 1;
  const int poff = p.pair_offset > 0 ? p.pair_offset : half;      // distance between the two channels of a pair
  const int fdim = p.pair_offset > 0 ? hd : p.rotary_dim;         // denominator of the frequency exponent
  for (int i = threadIdx.x; i < hd; i += blockDim.x) vals[i] = __bfloat162float(src[i]);
  __syncthreads();
  float amax = 0.f;
  for (int i = threadIdx.x; i < hd; i += blockDim.x) {
    float o = vals[i];
    if (!is_v && (i < half || (i >= poff && i < poff + half))) {
      const int fi = i < half ? i : i - poff;
      const float freq = p.inv_freq ? p.inv_freq[fi] : powf(p.theta, -2.f * fi / fdim);
      int rp = pos;
      if (p.rope_pos3) {
        const int axis = fi < p.sec_t ? 0 : (fi < p.sec_t + p.sec_h ? 1 : 2);
        rp = p.rope_pos3[static_cast<size_t>(axis) * p.tokens + t];
      }
      float sn, cs;
      sincosf(rp * freq, &sn, &cs);
      const float a = vals[fi], b = vals[fi + poff];
      o = i < half ? a * cs - b * sn : b * cs + a * sn;
    }
    o = __bfloat162float(__float2bfloat16_rn(o));
    rot[i] = o;
    const float ao = fabsf(o);
    if (ao == ao && ao <= 3.0e38f) amax = fmaxf(amax, ao);
    if (!is_v) src[i] = __float2bfloat16_rn(o);  // q and k are rotated in place as well
  }
  if (is_q) return;  // uniform per CTA
  const int kvh = is_v ? h - p.hq - p.hkv : h - p.hq;
  const int blk = p.block_table[static_cast<size_t>(p.seq_index[t]) * p.max_blocks + pos / p.page_size];
  const size_t slot = (static_cast<size_t>(blk) * p.hkv + kvh) * p.page_size + pos % p.page_size;   // head-major pages
  if (!p.kv_fp8) {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(is_v ? p.v_pages : p.k_pages) + slot * hd;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) dst[i] = __float2bfloat16_rn(rot[i]);
    return;
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  if (p.kv_fp8 == 2) {
    // ---- NVFP4 row: outer = amax / (448 * 6) (1 for an all-zero row), an E4M3 scale per 16 channels relative to it,
    // E2M1 codes relative to the decoded block scale (reference: kv_state_kernel.hip.cpp:240-290)
    const float outer = amax > 0.f ? amax / (kE4M3Max * 6.f) : 1.f;
    uint8_t* dst = static_cast<uint8_t*>(is_v ? p.v_pages : p.k_pages) + slot * nvfp4_row_bytes(hd);
    for (int b = threadIdx.x; b < hd / 16; b += blockDim.x) {
      float bmax = 0.f;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float a = fabsf(rot[16 * b + j]);
        if (a == a && a <= 3.0e38f) bmax = fmaxf(bmax, a);
        else if (a > 3.0e38f) bmax = 3.0e38f;               // an infinity saturates the block
      }
      const uint8_t sb = f32_to_e4m3(__fdiv_rn(bmax / 6.f, outer));
      const float bs = e4m3_to_f32(sb) * outer;
      dst[hd / 2 + b] = sb;
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        uint32_t lo = 0u, hi = 0u;
        if (bs > 0.f) {
          lo = f32_to_e2m1(__fdiv_rn(fminf(fmaxf(rot[16 * b + j], -3.0e38f), 3.0e38f), bs));
          hi = f32_to_e2m1(__fdiv_rn(fminf(fmaxf(rot[16 * b + j + 1], -3.0e38f), 3.0e38f), bs));
        }
        dst[8 * b + j / 2] = static_cast<uint8_t>(lo | (hi << 4));
      }
    }
    if (threadIdx.x == 0) (is_v ? p.v_scale : p.k_scale)[slot] = outer;
    return;
  }
  const float st = is_v ? p.v_static_scale : p.k_static_scale;
  const float scale = st > 0.f ? st : (amax > 0.f ? amax / kE4M3Max : 1.f);
  uint8_t* dst = static_cast<uint8_t*>(is_v ? p.v_pages : p.k_pages) + slot * hd;
  for (int i = threadIdx.x; i < hd; i += blockDim.x) dst[i] = f32_to_e4m3(__fdiv_rn(rot[i], scale));
  if (threadIdx.x == 0 && st <= 0.f) {
    float* sd = (is_v ? p.v_scale : p.k_scale) + slot;
    *sd = scale;
  }
}

// ---------------------------------------------------------------- elementwise helpers
// op: 0 add, 1 scalar_mul, 2 sigmoid_mul (a * sigmoid(b)), 3 tanh_softcap (s * tanh(a / s)),
//     4 broadcast_add (a[r, :] + b[:]), 5 copy
__global__ void elementwise_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                   __nv_bfloat16* __restrict__ y, long long n, int d, int op, float s) {
  pdl_wait();
  pdl_trigger();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float av = __bfloat162float(a[i]);
  float r;
  switch (op) {
    case 0: r = av + __bfloat162float(b[i]); break;
    case 1: r = av * s; break;
    case 2: {
      const float g = 1.f / (1.f + __expf(-__bfloat162float(b[i])));
      r = av * __bfloat162float(__float2bfloat16_rn(g));
      break;
    }
    case 3: r = s * tanhf(av / s); break;
    case 4: r = av + __bfloat162float(b[i % d]); break;
    default: r = av; break;
  }
  y[i] = __float2bfloat16_rn(r);
}

// ---------------------------------------------------------------- row argmax
// NaN anywhere in the row -> -1; ties -> lowest index.  index_offset lets vocabulary shards report
// global ids; out_val (optional) receives the winning value for cross-rank merges.
// grid = (rows, chunks): every CTA scans one slice with 16-byte loads and publishes a partial
// (value, index, nan) record; the CTA that arrives last for a row (counter) merges the records.
struct ArgmaxPartial {
  float val;
  int idx;
  int nan;
  int pad;
};

__device__ __forceinline__ void argmax_take(float& best, int& bi, float v, int i) {
  if (v > best || (v == best && i < bi)) {
    best = v;
    bi = i;
  }
}

__global__ void __launch_bounds__(256)
argmax_kernel(const __nv_bfloat16* __restrict__ logits, int* __restrict__ out_idx, float* __restrict__ out_val,
              int n, int ld, int index_offset, int chunk, ArgmaxPartial* partials, int* counters) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const int c0 = blockIdx.y * chunk;
  int c1 = c0 + chunk;
  if (c1 > n) c1 = n;
  const __nv_bfloat16* row = logits + static_cast<size_t>(r) * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  int nan = 0;
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(row) & 15) == 0) && ((c0 & 7) == 0);
  int i = c0 + threadIdx.x * 8;
  if (vec_ok) {
    for (; i + 8 <= c1; i += blockDim.x * 8) {
      float v[8];
      load8_bf16(row + i, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (v[j] != v[j]) nan = 1;
        argmax_take(best, bi, v[j], i + j);
      }
    }
    // ragged tail of the slice (fewer than 8 elements), handled by one thread
    const int tail0 = c0 + ((c1 - c0) & ~7);
    if (threadIdx.x == 0) {
      for (int t = tail0; t < c1; ++t) {
        const float v = __bfloat162float(row[t]);
        if (v != v) nan = 1;
        argmax_take(best, bi, v, t);
      }
    }
  } else {
    for (int t = c0 + threadIdx.x; t < c1; t += blockDim.x) {
      const float v = __bfloat162float(row[t]);
      if (v != v) nan = 1;
      argmax_take(best, bi, v, t);
    }
  }
  __shared__ float sv[8];
  __shared__ int si[8];
  __shared__ int snan;
  __shared__ int s_last;
  if (threadIdx.x == 0) snan = 0;
  __syncthreads();
  if (nan) snan = 1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_take(best, bi, ov, oi);
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = best;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w) argmax_take(best, bi, sv[w], si[w]);
    const int chunks = gridDim.y;
    ArgmaxPartial rec;
    rec.val = best; rec.idx = bi; rec.nan = snan; rec.pad = 0;
    int last = 1;
    if (chunks > 1) {
      partials[static_cast<size_t>(r) * chunks + blockIdx.y] = rec;
      __threadfence();
      const int old = atomicAdd(&counters[r], 1);
      last = old == chunks - 1;
      if (last) {
        counters[r] = 0;
        __threadfence();
        best = -INFINITY; bi = 0x7fffffff; snan = 0;
        for (int c = 0; c < chunks; ++c) {
          const ArgmaxPartial* pr = partials + static_cast<size_t>(r) * chunks + c;
          const float v = __ldcg(&pr->val);
          const int ix = __ldcg(&pr->idx);
          if (__ldcg(&pr->nan)) snan = 1;
          argmax_take(best, bi, v, ix);
        }
      }
    }
    if (last) {
      if (snan) {
        out_idx[r] = -1;
        if (out_val) out_val[r] = NAN;
      } else {
        out_idx[r] = (bi == 0x7fffffff ? 0 : bi) + index_offset;
        if (out_val) out_val[r] = best;
      }
    }
  }
}

}  // namespace sllm

using namespace sllm;

static inline int check_launch() { return cudaGetLastError() == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA; }

SLLM_EXPORT int sllm_embedding(const void* table, const int* ids, void* out, int tokens, int d, int vocab,
                               float scale, void* stream) {
  if (!table || !ids || !out || tokens <= 0 || d <= 0 || (d % 8)) return SLLM_ERR_INVALID_ARGUMENT;
  launch_kernel(embedding_kernel, dim3(tokens), dim3(128), 0, static_cast<cudaStream_t>(stream), 1u, 
      static_cast<const __nv_bfloat16*>(table), ids, static_cast<__nv_bfloat16*>(out), d, vocab, scale);
  return check_launch();
}

SLLM_EXPORT int sllm_rmsnorm(const void* x, const void* w, void* y_bf16, void* y_fp8, float* y_scale, int ld_scale,
                             int rows, int d, float eps, int offset_one, void* stream) {
  if (!x || !w || rows <= 0 || d <= 0 || (d % 8)) return SLLM_ERR_INVALID_ARGUMENT;
  if (d > 16384) return SLLM_ERR_LIMIT;
  const size_t smem = static_cast<size_t>(d) * sizeof(float);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (y_fp8) {
    if (!y_scale || (d % 128)) return SLLM_ERR_INVALID_ARGUMENT;
    static bool cfg = false;
    if (!cfg) {
      cudaFuncSetAttribute(rmsnorm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
      cfg = true;
    }
    launch_kernel(rmsnorm_kernel<true>, dim3(rows), dim3(256), smem, st, 1u, static_cast<const __nv_bfloat16*>(x),
                                                  static_cast<const __nv_bfloat16*>(w), nullptr,
                                                  static_cast<uint8_t*>(y_fp8), y_scale, ld_scale, d, eps, offset_one);
  } else {
    if (!y_bf16) return SLLM_ERR_INVALID_ARGUMENT;
    static bool cfg = false;
    if (!cfg) {
      cudaFuncSetAttribute(rmsnorm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536);
      cfg = true;
    }
    launch_kernel(rmsnorm_kernel<false>, dim3(rows), dim3(256), smem, st, 1u, static_cast<const __nv_bfloat16*>(x),
                                                   static_cast<const __nv_bfloat16*>(w),
                                                   static_cast<__nv_bfloat16*>(y_bf16), nullptr, nullptr, 0, d, eps,
                                                   offset_one);
  }
  return check_launch();
}

SLLM_EXPORT int sllm_gated_act(const void* in, void* y_bf16, void* y_fp8, float* y_scale, int ld_scale, int rows,
                               int inter, int act, void* stream) {
  if (!in || rows <= 0 || inter <= 0 || (inter % 8)) return SLLM_ERR_INVALID_ARGUMENT;
  dim3 grid(rows, (inter / 8 + 255) / 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (y_fp8) {
    if (!y_scale) return SLLM_ERR_INVALID_ARGUMENT;
    launch_kernel(gated_act_kernel<true>, dim3(grid), dim3(256), 0, st, 1u, static_cast<const __nv_bfloat16*>(in), nullptr,
                                                 static_cast<uint8_t*>(y_fp8), y_scale, ld_scale, inter, act);
  } else {
    if (!y_bf16) return SLLM_ERR_INVALID_ARGUMENT;
    launch_kernel(gated_act_kernel<false>, dim3(grid), dim3(256), 0, st, 1u, static_cast<const __nv_bfloat16*>(in),
                                                  static_cast<__nv_bfloat16*>(y_bf16), nullptr, nullptr, 0, inter, act);
  }
  return check_launch();
}

SLLM_EXPORT int sllm_quant_fp8_1x128(const void* x, void* y, float* scale, int ld_scale, int rows, int k,
                                     void* stream) {
  if (!x || !y || !scale || rows <= 0 || k <= 0 || (k % 8)) return SLLM_ERR_INVALID_ARGUMENT;
  dim3 grid(rows, (k / 8 + 255) / 256);
  launch_kernel(quant_fp8_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), 1u, 
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(y), scale, ld_scale, k);
  return check_launch();
}

static int rope_kv_append_impl(void* qkv, const int* positions, const int* seq_index, const int* block_table,
                               int max_blocks, void* k_pages, void* v_pages, float* k_scale, float* v_scale,
                               int tokens, int hq, int hkv, int hd, int rotary_dim, int page_size, int kv_fp8,
                               float theta, float k_static_scale, float v_static_scale, const float* inv_freq,
                               const int* rope_pos3, int sec_t, int sec_h, void* stream, int pair_offset = 0) {
  if (!qkv || !positions || !seq_index || !block_table || !k_pages || !v_pages || tokens <= 0)
    return SLLM_ERR_INVALID_ARGUMENT;
  if (pair_offset < 0 || (pair_offset > 0 && (pair_offset < rotary_dim / 2 || pair_offset + rotary_dim / 2 > hd)))
    return SLLM_ERR_INVALID_ARGUMENT;
  if (hd > 512 || (rotary_dim & 1) || rotary_dim > hd || page_size <= 0) return SLLM_ERR_UNSUPPORTED_SHAPE;
  if (kv_fp8 && k_static_scale <= 0.f && (!k_scale || !v_scale)) return SLLM_ERR_INVALID_ARGUMENT;
  if (kv_fp8 == 2 && ((hd & 15) || !k_scale || !v_scale)) return SLLM_ERR_INVALID_ARGUMENT;   // NVFP4 rows: outer scale planes
  if (kv_fp8 < 0 || kv_fp8 > 2) return SLLM_ERR_INVALID_ARGUMENT;
  if (rope_pos3 && (sec_t < 0 || sec_h < 0 || sec_t + sec_h > rotary_dim / 2)) return SLLM_ERR_INVALID_ARGUMENT;
  RopeKvParams p;
  p.qkv = static_cast<__nv_bfloat16*>(qkv);
  p.positions = positions; p.seq_index = seq_index; p.block_table = block_table; p.max_blocks = max_blocks;
  p.k_pages = k_pages; p.v_pages = v_pages; p.k_scale = k_scale; p.v_scale = v_scale;
  p.hq = hq; p.hkv = hkv; p.hd = hd; p.rotary_dim = rotary_dim; p.page_size = page_size; p.kv_fp8 = kv_fp8;
  p.theta = theta; p.k_static_scale = k_static_scale; p.v_static_scale = v_static_scale; p.inv_freq = inv_freq;
  p.rope_pos3 = rope_pos3; p.tokens = tokens; p.sec_t = sec_t; p.sec_h = sec_h; p.pair_offset = pair_offset;
  dim3 grid(tokens, hq + 2 * hkv);
  launch_kernel(rope_kv_append_kernel, dim3(grid), dim3(128), 0, static_cast<cudaStream_t>(stream), 1u, p);
  return check_launch();
}

SLLM_EXPORT int sllm_rope_kv_append(void* qkv, const int* positions, const int* seq_index, const int* block_table,
                                    int max_blocks, void* k_pages, void* v_pages, float* k_scale, float* v_scale,
                                    int tokens, int hq, int hkv, int hd, int rotary_dim, int page_size, int kv_fp8,
                                    float theta, float k_static_scale, float v_static_scale, const float* inv_freq,
                                    void* stream) {
  return rope_kv_append_impl(qkv, positions, seq_index, block_table, max_blocks, k_pages, v_pages, k_scale, v_scale,
                             tokens, hq, hkv, hd, rotary_dim, page_size, kv_fp8, theta, k_static_scale, v_static_scale,
                             inv_freq, nullptr, 0, 0, stream);
}

// The same with the "proportional" pair layout of partially rotated wide heads (see RopeKvParams::pair_offset;
// reference: SplitHalfRotaryContract, crates/sllm-core/src/op.rs:805-811).
SLLM_EXPORT int sllm_rope_kv_append_paired(void* qkv, const int* positions, const int* seq_index, const int* block_table,
                                           int max_blocks, void* k_pages, void* v_pages, float* k_scale, float* v_scale,
                                           int tokens, int hq, int hkv, int hd, int rotary_dim, int page_size, int kv_fp8,
                                           float theta, float k_static_scale, float v_static_scale, const float* inv_freq,
                                           int pair_offset, void* stream) {
  return rope_kv_append_impl(qkv, positions, seq_index, block_table, max_blocks, k_pages, v_pages, k_scale, v_scale,
                             tokens, hq, hkv, hd, rotary_dim, page_size, kv_fp8, theta, k_static_scale, v_static_scale,
                             inv_freq, nullptr, 0, 0, stream, pair_offset);
}

// The same with 3-axis rotary positions rope_pos3 [3, tokens] (see RopeKvParams).
SLLM_EXPORT int sllm_rope_kv_append_mrope(void* qkv, const int* positions, const int* seq_index, const int* block_table,
                                          int max_blocks, void* k_pages, void* v_pages, float* k_scale, float* v_scale,
                                          int tokens, int hq, int hkv, int hd, int rotary_dim, int page_size, int kv_fp8,
                                          float theta, float k_static_scale, float v_static_scale, const float* inv_freq,
                                          const int* rope_pos3, int sec_t, int sec_h, void* stream) {
  if (!rope_pos3) return SLLM_ERR_INVALID_ARGUMENT;
  return rope_kv_append_impl(qkv, positions, seq_index, block_table, max_blocks, k_pages, v_pages, k_scale, v_scale,
                             tokens, hq, hkv, hd, rotary_dim, page_size, kv_fp8, theta, k_static_scale, v_static_scale,
                             inv_freq, rope_pos3, sec_t, sec_h, stream);
}

SLLM_EXPORT int sllm_elementwise(const void* a, const void* b, void* y, long long n, int d, int op, float s,
                                 void* stream) {
  if (!a || !y || n <= 0) return SLLM_ERR_INVALID_ARGUMENT;
  if ((op == 0 || op == 2 || op == 4) && !b) return SLLM_ERR_INVALID_ARGUMENT;
  const int blocks = static_cast<int>((n + 255) / 256);
  launch_kernel(elementwise_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream), 1u, 
      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), static_cast<__nv_bfloat16*>(y), n,
      d > 0 ? d : 1, op, s);
  return check_launch();
}

SLLM_EXPORT int sllm_argmax(const void* logits, int* out_idx, float* out_val, int rows, int n, int ld,
                            int index_offset, void* ws, long long ws_bytes, int* counters, int n_counters,
                            void* stream) {
  if (!logits || !out_idx || rows <= 0 || n <= 0) return SLLM_ERR_INVALID_ARGUMENT;
  // Enough CTAs to cover the machine, slices a multiple of 8 elements and at least 2048 long.
  int chunks = (2 * 148 + rows - 1) / rows;
  const int max_chunks = (n + 2047) / 2048;
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks < 1) chunks = 1;
  if (chunks > 1 && (!ws || !counters || ws_bytes < static_cast<long long>(rows) * chunks * 16 || n_counters < rows))
    chunks = 1;
  int chunk = (n + chunks - 1) / chunks;
  chunk = (chunk + 7) & ~7;
  chunks = (n + chunk - 1) / chunk;
  dim3 grid(rows, chunks);
  launch_kernel(argmax_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), 1u, 
      static_cast<const __nv_bfloat16*>(logits), out_idx, out_val, n, ld, index_offset, chunk,
      static_cast<ArgmaxPartial*>(ws), counters);
  return check_launch();
}

// ------------------------------------------------------------------------------------------------
// Row argmax for callers that must not allocate (declared in noalloc.h).
//
// Same kernel and same results as sllm_argmax, but the partial records and the per-row arrival
// counters live in a fixed array that is part of the loaded library image instead of a caller
// workspace.  Capacity: kNoAllocMaxRows rows; the array occupies kNoAllocScratchBytes on every GPU
// that loads the library, until the process exits.
namespace sllm {
constexpr int kNoAllocMaxRows = 256;
constexpr int kNoAllocMaxChunks = 64;
constexpr size_t kNoAllocPartialBytes = static_cast<size_t>(kNoAllocMaxRows) * kNoAllocMaxChunks * sizeof(ArgmaxPartial);
constexpr size_t kNoAllocScratchBytes = kNoAllocPartialBytes + kNoAllocMaxRows * sizeof(int);
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
}  // namespace sllm

SLLM_EXPORT int sllm_argmax_noalloc_max_rows(void) { return kNoAllocMaxRows; }

SLLM_EXPORT int sllm_argmax_noalloc(const void* logits, int* out_idx, float* out_val, int rows, int n, int ld,
                                    int index_offset, void* stream) {
  if (!logits || !out_idx || rows <= 0 || n <= 0 || ld < n) return SLLM_ERR_INVALID_ARGUMENT;   // rows may not overlap
  if (rows > kNoAllocMaxRows) return SLLM_ERR_LIMIT;   // larger batches must use sllm_argmax with a workspace
  // The array's name is only a host-side handle; the kernel needs its device address, which is looked
  // up once per device (with that device current) and remembered.
  constexpr int kMaxDevices = 64;
  static void* scratch_ptr[kMaxDevices] = {nullptr};
  static std::mutex setup_mutex;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SLLM_ERR_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  void* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(setup_mutex);
    if (!scratch_ptr[dev]) {
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) {
        cudaGetLastError();
        return SLLM_ERR_CUDA;
      }
      // the counters need no clearing here: a __device__ array is zero when the library image is loaded, and
      // the kernel returns every counter to zero before it ends
      scratch_ptr[dev] = p;
    }
    base = scratch_ptr[dev];
  }
  int chunks = (2 * 148 + rows - 1) / rows;
  const int max_chunks = (n + 2047) / 2048;
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks > kNoAllocMaxChunks) chunks = kNoAllocMaxChunks;
  if (chunks < 1) chunks = 1;
  int chunk = (n + chunks - 1) / chunks;
  chunk = (chunk + 7) & ~7;
  chunks = (n + chunk - 1) / chunk;
  dim3 grid(rows, chunks);
  cudaError_t e = launch_kernel(argmax_kernel, grid, dim3(256), 0, st, 1u, static_cast<const __nv_bfloat16*>(logits),
                                out_idx, out_val, n, ld, index_offset, chunk, static_cast<ArgmaxPartial*>(base),
                                reinterpret_cast<int*>(static_cast<unsigned char*>(base) + kNoAllocPartialBytes));
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}
