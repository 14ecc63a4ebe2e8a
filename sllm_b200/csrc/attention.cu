// Paged attention over the quantised KV cache (CUDA-core path): one kernel serves batched decode,
// speculative verification (k+1 query rows per sequence, each with its own causal limit) and short or
// cache-continuing prefill chunks.  Long fresh prefills use the tensor-core kernel in
// prefill_attention.cu.
//
// Work decomposition: grid = (query rows, kv heads, KV splits); a CTA of 4 warps owns the whole GQA
// group of one kv head for one query row and one slice of the visible keys, so each K/V byte is read
// once per group.  Inside a warp, keys are handled 32 at a time: lane <-> key for Q.K (no shuffles in
// the inner product), then lane <-> channel for P.V.  Per-(token, head) FP8 scales are folded into
// the score (K) and into the probability (V), so pages are consumed in their stored encoding.
// Partial (max, sum, acc) triples of the splits are merged by the last CTA to arrive (counter per
// (row, kv head)); nobody waits.
//
// KV page layout (per layer, K and V alike): values [num_pages, kv_heads, page, head_dim] in bf16 or
// E4M3FN, scales [num_pages, kv_heads, page] fp32 (head-major pages).
//
// Counterparts in the reference: causal_attention_kernel.hip.cpp:125-495 (online softmax, split-KV
// decode, GQA sharing, direct low-bit KV reads) and gemma_attention_kernel.hip.cpp:40 (sliding window).
#include "common.cuh"
#include "api.h"
#include "attention_common.cuh"

namespace sllm {

// kFmt: 0 bf16 pages, 1 E4M3 pages (scale per token and head, or static), 2 NVFP4 rows (E2M1 codes, E4M3 scale per 16
// channels inside the row, fp32 outer scale per token and head in the scale plane; see nvfp4_row_bytes).
template <int HD, int G, int kFmt>
__global__ void __launch_bounds__(128) paged_attention_kernel(const PagedAttnParams p) {
  pdl_wait();
  pdl_trigger();
  constexpr bool kFp8 = kFmt == 1;
  constexpr bool kNv4 = kFmt == 2;
  constexpr int EPL = HD / 32;  // channels per lane in the P.V phase
  extern __shared__ float smem[];
  float* q_s = smem;                       // [G][HD]
  float* p_s = q_s + G * HD;               // [4 warps][32][G]
  float* m_s = p_s + 4 * 32 * G;           // [4][G]
  float* l_s = m_s + 4 * G;                // [4][G]
  float* o_s = l_s + 4 * G;                // [4][G][HD]
  __shared__ int s_is_last;
  __shared__ float s_red[4];

  const int r = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z, splits = gridDim.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hq = p.hkv * G;
  const int seq = p.seq_index[r];
  const int kv_len = p.kv_lens[r];
  int first = 0;
  if (p.window > 0 && kv_len > p.window) first = kv_len - p.window;
  const int n = kv_len - first;
  int chunk = (n + splits - 1) / splits;
  chunk = (chunk + 31) & ~31;
  const int begin = first + split * chunk;
  int end = begin + chunk;
  if (end > kv_len) end = kv_len;

  for (int e = threadIdx.x; e < G * HD; e += blockDim.x) {
    const int g = e / HD, d = e % HD;
    // FP8 pages decode to value * 2^-120; half of the compensation (2^60) rides on q, half on the scale.
    q_s[e] = __bfloat162float(p.q[static_cast<size_t>(r) * p.q_ld + (kvh * G + g) * HD + d]) * p.sm_scale *
             (kFp8 ? kPow60 : 1.f);
  }
  __syncthreads();

  float m[G], l[G], o[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) o[g][e] = 0.f;
  }
  const int* bt = p.block_table + static_cast<size_t>(seq) * p.max_blocks;
  float* my_p = p_s + warp * 32 * G;

  for (int base = begin + warp * 32; base < end; base += 4 * 32) {
    const int tok = base + lane;
    const bool valid = tok < end;
    size_t slot = 0;
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = 0.f;
    float vsc = 0.f;
    if (valid) {
      const int blk = bt[tok / p.page_size];
      slot = (static_cast<size_t>(blk) * p.hkv + kvh) * p.page_size + tok % p.page_size;   // head-major pages
    }
    if (kNv4 && valid) {
      // the whole row (code words, then the block-scale words) is requested before any of it is used
      constexpr int kCodeWords = HD / 8, kScaleWords = (HD / 16 + 3) / 4;
      const uint8_t* rowp = static_cast<const uint8_t*>(p.k_pages) + slot * nvfp4_row_bytes(HD);
      uint32_t cw[kCodeWords], sw[kScaleWords];
#pragma unroll
      for (int i = 0; i < kCodeWords; ++i) cw[i] = reinterpret_cast<const uint32_t*>(rowp)[i];
#pragma unroll
      for (int i = 0; i < kScaleWords; ++i) {
        sw[i] = 0u;
#pragma unroll
        for (int b = 0; b < 4; ++b)
          if (4 * i + b < HD / 16) sw[i] |= static_cast<uint32_t>(rowp[HD / 2 + 4 * i + b]) << (8 * b);
      }
#pragma unroll
      for (int b = 0; b < HD / 16; ++b) {
        const float bs = e4m3_to_f32(static_cast<uint8_t>((sw[b >> 2] >> (8 * (b & 3))) & 0xffu));
        float kf[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) kf[j] = e2m1_to_f32((cw[2 * b + (j >> 3)] >> (4 * (j & 7))) & 0xfu);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float a = 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) a = fmaf(q_s[g * HD + 16 * b + j], kf[j], a);
          s[g] = fmaf(a, bs, s[g]);
        }
      }
      const float ksc = p.k_scale[slot];
      vsc = p.v_scale[slot];
#pragma unroll
      for (int g = 0; g < G; ++g) s[g] *= ksc;
    }
    if (!kNv4 && valid) {
      // All 16-byte pieces of (up to) 128 bytes of the key row are requested before any is used, so one
      // memory round trip covers the whole row.
      constexpr int kVecs = HD * (kFp8 ? 1 : 2) / 16;
      constexpr int kBatch = kVecs < 8 ? kVecs : 8;
      constexpr int kElemsPerVec = kFp8 ? 16 : 8;
      const uint4* krow = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.k_pages) +
                                                         slot * HD * (kFp8 ? 1 : 2));
#pragma unroll
      for (int b0 = 0; b0 < kVecs; b0 += kBatch) {
        uint4 raw[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) raw[u] = krow[b0 + u];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          float kf[kElemsPerVec];
          if (kFp8) {
            const uint32_t* w32 = reinterpret_cast<const uint32_t*>(&raw[u]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float f4[4];
              e4m3x4_to_f32x4_exp120(w32[j], f4);
#pragma unroll
              for (int b = 0; b < 4; ++b) kf[(4 * j + b) % kElemsPerVec] = f4[b];
            }
          } else {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              kf[2 * j] = __bfloat162float(h[j].x);
              kf[2 * j + 1] = __bfloat162float(h[j].y);
            }
          }
          const int d = (b0 + u) * kElemsPerVec;
#pragma unroll
          for (int g = 0; g < G; ++g) {
            float a = 0.f;
#pragma unroll
            for (int j = 0; j < kElemsPerVec; ++j) a = fmaf(q_s[g * HD + d + j], kf[j], a);
            s[g] += a;
          }
        }
      }
      if (kFp8) {
        const float ksc = kPow60 * (p.k_scale ? p.k_scale[slot] : p.k_static_scale);
        vsc = kPow60 * (p.v_scale ? p.v_scale[slot] : p.v_static_scale);  // second 2^60 applied to o at the end
#pragma unroll
        for (int g = 0; g < G; ++g) s[g] *= ksc;
      } else {
        vsc = 1.f;
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float sv = valid ? s[g] : -INFINITY;
      const float mx = warp_max(sv);
      const float m_new = fmaxf(m[g], mx);
      const float pr = valid ? __expf(sv - m_new) : 0.f;
      const float sum = warp_sum(pr);
      const float alpha = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - m_new);
      l[g] = l[g] * alpha + sum;
      m[g] = m_new;
#pragma unroll
      for (int e = 0; e < EPL; ++e) o[g][e] *= alpha;
      my_p[lane * G + g] = pr * vsc;
    }
    __syncwarp();
    const int cnt = min(32, end - base);
    // Values of 8 keys are requested together (8 independent loads in flight per lane).
    for (int j0 = 0; j0 < cnt; j0 += 8) {
      float vf[8][EPL];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const size_t vslot = __shfl_sync(0xffffffffu, slot, (j0 + u) & 31);
        const bool live = j0 + u < cnt;
        if (kNv4) {
          // this lane's EPL channels: EPL / 2 code bytes and the scale of the 16-channel block they lie in
          const uint8_t* rowp = static_cast<const uint8_t*>(p.v_pages) + vslot * nvfp4_row_bytes(HD);
          uint32_t codes = 0u;
          float bs = 0.f;
          if (live) {
#pragma unroll
            for (int b = 0; b < EPL / 2; ++b) codes |= static_cast<uint32_t>(rowp[lane * (EPL / 2) + b]) << (8 * b);
            bs = e4m3_to_f32(rowp[HD / 2 + (lane * EPL) / 16]);
          }
#pragma unroll
          for (int e = 0; e < EPL; ++e) vf[u][e] = e2m1_to_f32((codes >> (4 * e)) & 0xfu) * bs;
        } else if (kFp8) {
          const uint8_t* vp = static_cast<const uint8_t*>(p.v_pages) + vslot * HD + lane * EPL;
          float f4[4];
          if (EPL == 4) {
            const uint32_t raw = live ? *reinterpret_cast<const uint32_t*>(vp) : 0u;
            e4m3x4_to_f32x4_exp120(raw, f4);
#pragma unroll
            for (int e = 0; e < 4; ++e) vf[u][e % EPL] = f4[e];
          } else if (EPL == 2) {
            const uint32_t raw = live ? static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(vp)) : 0u;
            e4m3x4_to_f32x4_exp120(raw, f4);
            vf[u][0] = f4[0]; vf[u][1 % EPL] = f4[1];
          } else {
            const uint2 raw = live ? *reinterpret_cast<const uint2*>(vp) : make_uint2(0u, 0u);
            e4m3x4_to_f32x4_exp120(raw.x, f4);
#pragma unroll
            for (int e = 0; e < 4; ++e) vf[u][e % EPL] = f4[e];
            e4m3x4_to_f32x4_exp120(raw.y, f4);
#pragma unroll
            for (int e = 0; e < 4; ++e) vf[u][(4 + e) % EPL] = f4[e];
          }
        } else {
          const __nv_bfloat16* vp = static_cast<const __nv_bfloat16*>(p.v_pages) + vslot * HD + lane * EPL;
#pragma unroll
          for (int e = 0; e < EPL; e += 2) {
            const __nv_bfloat162 h = live ? *reinterpret_cast<const __nv_bfloat162*>(vp + e) : __nv_bfloat162();
            vf[u][e] = live ? __bfloat162float(h.x) : 0.f;
            vf[u][(e + 1) % EPL] = live ? __bfloat162float(h.y) : 0.f;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (j0 + u < cnt) {
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float pj = my_p[(j0 + u) * G + g];
#pragma unroll
            for (int e = 0; e < EPL; ++e) o[g][e] = fmaf(pj, vf[u][e], o[g][e]);
          }
        }
      }
    }
    __syncwarp();
  }

  // ---- merge the 4 warps
  if (kFp8) {
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int e = 0; e < EPL; ++e) o[g][e] *= kPow60;
  }
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) {
      m_s[warp * G + g] = m[g];
      l_s[warp * G + g] = l[g];
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) o_s[(warp * G + g) * HD + lane * EPL + e] = o[g][e];
  }
  __syncthreads();

  attention_tail<HD, G, 4, SyncCta>(p, r, kvh, split, splits, threadIdx.x, m_s, l_s, o_s, &s_is_last, s_red);
}

template <int HD, int G, int kFp8>
static int launch_paged(const PagedAttnParams& p, int rows, int splits, cudaStream_t st) {
  const size_t smem = sizeof(float) * (G * HD + 4 * 32 * G + 8 * G + 4 * G * HD);
  static bool cfg = false;
  if (!cfg) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(paged_attention_kernel<HD, G, kFp8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(smem));
    cfg = true;
  }
  dim3 grid(rows, p.hkv, splits);
  launch_kernel(paged_attention_kernel<HD, G, kFp8>, dim3(grid), dim3(128), smem, st, 1u, p);
  return cudaGetLastError() == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

template <int HD, int kFp8>
static int dispatch_g(const PagedAttnParams& p, int rows, int g, int splits, cudaStream_t st) {
  switch (g) {
    case 1: return launch_paged<HD, 1, kFp8>(p, rows, splits, st);
    case 2: return launch_paged<HD, 2, kFp8>(p, rows, splits, st);
    case 4: return launch_paged<HD, 4, kFp8>(p, rows, splits, st);
    case 8: return launch_paged<HD, 8, kFp8>(p, rows, splits, st);
    default: return SLLM_ERR_UNSUPPORTED_SHAPE;
  }
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT long long sllm_paged_attention_workspace_floats(int rows, int hq, int hd, int hkv, int splits) {
  if (splits <= 1) return 0;
  const long long g = hq / hkv;
  return static_cast<long long>(rows) * hkv * splits * (g * hd + g * 2);
}

SLLM_EXPORT int sllm_paged_attention(const void* q, int q_ld, const void* k_pages, const void* v_pages,
                                     const float* k_scale, const float* v_scale, float k_static_scale,
                                     float v_static_scale, const int* block_table, int max_blocks,
                                     const int* seq_index, const int* kv_lens, int rows, int hq, int hkv, int hd,
                                     int page_size, int window, float sm_scale, int kv_fp8, void* out_bf16,
                                     void* out_fp8, float* out_scale, int ld_scale, const float* sinks, int splits,
                                     float* ws, long long ws_floats, int* counters, int n_counters, void* stream) {
  if (!q || !k_pages || !v_pages || !block_table || !seq_index || !kv_lens || rows <= 0 || hkv <= 0 || hq % hkv)
    return SLLM_ERR_INVALID_ARGUMENT;
  if (!out_bf16 && !out_fp8) return SLLM_ERR_INVALID_ARGUMENT;
  if (out_fp8 && (hd != 128 || !out_scale)) return SLLM_ERR_UNSUPPORTED_SHAPE;
  if (kv_fp8 && !k_scale && !(k_static_scale > 0.f && v_static_scale > 0.f)) return SLLM_ERR_INVALID_ARGUMENT;
  if (splits < 1 || splits > 65535 || hkv > 65535) return SLLM_ERR_INVALID_ARGUMENT;
  const int g = hq / hkv;
  PagedAttnParams p = {};
  p.q = static_cast<const __nv_bfloat16*>(q); p.q_ld = q_ld;
  p.k_pages = k_pages; p.v_pages = v_pages; p.k_scale = k_scale; p.v_scale = v_scale;
  p.k_static_scale = k_static_scale; p.v_static_scale = v_static_scale;
  p.block_table = block_table; p.max_blocks = max_blocks; p.seq_index = seq_index; p.kv_lens = kv_lens;
  p.hkv = hkv; p.page_size = page_size; p.window = window; p.sm_scale = sm_scale;
  p.out_bf16 = static_cast<__nv_bfloat16*>(out_bf16); p.out_fp8 = static_cast<uint8_t*>(out_fp8);
  p.out_scale = out_scale; p.ld_scale = ld_scale; p.sinks = sinks;
  p.ws_o = nullptr; p.ws_ml = nullptr; p.counters = counters; p.status_word = nullptr;
  p.early_trigger = 0;
  if (splits > 1) {
    const long long units = static_cast<long long>(rows) * hkv;
    const long long need = units * splits * (static_cast<long long>(g) * hd + g * 2);
    if (!ws || !counters || ws_floats < need || n_counters < units) return SLLM_ERR_WORKSPACE_TOO_SMALL;
    p.ws_o = ws;
    p.ws_ml = ws + units * splits * g * hd;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (kv_fp8 == 2) {
    if (!k_scale || !v_scale) return SLLM_ERR_INVALID_ARGUMENT;       // the outer scales of the NVFP4 rows
    switch (hd) {
      case 64: return dispatch_g<64, 2>(p, rows, g, splits, st);
      case 128: return dispatch_g<128, 2>(p, rows, g, splits, st);
      case 256: return dispatch_g<256, 2>(p, rows, g, splits, st);
      default: return SLLM_ERR_UNSUPPORTED_SHAPE;
    }
  }
  if (kv_fp8) {
    switch (hd) {
      case 64: return dispatch_g<64, 1>(p, rows, g, splits, st);
      case 128: return dispatch_g<128, 1>(p, rows, g, splits, st);
      case 256: return dispatch_g<256, 1>(p, rows, g, splits, st);
    }
  } else {
    switch (hd) {
      case 64: return dispatch_g<64, 0>(p, rows, g, splits, st);
      case 128: return dispatch_g<128, 0>(p, rows, g, splits, st);
      case 256: return dispatch_g<256, 0>(p, rows, g, splits, st);
    }
  }
  return SLLM_ERR_UNSUPPORTED_SHAPE;
}
