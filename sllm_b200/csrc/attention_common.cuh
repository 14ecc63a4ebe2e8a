// Shared pieces of the paged attention kernels (CUDA-core kernel in attention.cu, tensor-core decode
// kernel in decode_attention_tc.cu): the launch parameters and the tail that merges KV splits, applies
// attention sinks, normalises and writes bf16 or FP8-quantised output.
#pragma once
#include "common.cuh"

namespace sllm {

struct PagedAttnParams {
  const __nv_bfloat16* q;  // [rows, hq * hd] (row stride q_ld)
  int q_ld;
  const void* k_pages;
  const void* v_pages;
  const float* k_scale;
  const float* v_scale;
  float k_static_scale, v_static_scale;  // used when the scale planes are null (fp8-static)
  const int* block_table;  // [num_seqs, max_blocks]
  int max_blocks;
  const int* seq_index;    // [rows]
  const int* kv_lens;      // [rows] keys visible to the row (its own position + 1)
  int hkv, page_size, window;
  float sm_scale;
  __nv_bfloat16* out_bf16;  // [rows, hq * hd] or null
  uint8_t* out_fp8;         // E4M3 [rows, hq * hd] (hd == 128 only) or null
  float* out_scale;         // [hq, ld_scale] kb-major scales for out_fp8
  int ld_scale;
  float* ws_o;              // [rows * hkv * splits, G, HD]
  float* ws_ml;             // [rows * hkv * splits, G, 2]
  int* counters;            // [rows * hkv]
  const float* sinks;       // optional [hq] attention-sink logits (added to the softmax denominator)
  int* status_word;         // device status word for bounded waits (tensor-core kernel)
  int early_trigger;        // tensor-core kernel: let dependent launches start once the CTA holds its TMEM
  STEP_TRACE_FIELD
};


struct SyncCta {
  static __device__ __forceinline__ void sync() { __syncthreads(); }
};
struct SyncBar1x128 {  // the 128 softmax threads of a warp-specialised CTA
  static __device__ __forceinline__ void sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
};

// Tail run by 128 threads (tid 0..127).  m_s / l_s: [W][G], o_s: [W][G][HD] partial softmax states of W
// producers inside the CTA (maxima in natural-log units); s_is_last / s_red: shared scratch.
template <int HD, int G, int W, class Sync>
__device__ __forceinline__ void attention_tail(const PagedAttnParams& p, int r, int kvh, int split, int splits,
                                               int tid, const float* m_s, const float* l_s, const float* o_s,
                                               int* s_is_last_p, float* s_red) {
  const int warp = tid >> 5, lane = tid & 31;
  const int hq = p.hkv * G;
  int& s_is_last = *s_is_last_p;
  const size_t unit = static_cast<size_t>(r) * p.hkv + kvh;
  bool finalize = true;
  if (splits > 1) {
    float* wo = p.ws_o + (unit * splits + split) * (G * HD);
    float* wml = p.ws_ml + (unit * splits + split) * (G * 2);
    for (int e = tid; e < G * HD; e += 128) {
      const int g = e / HD, d = e % HD;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < W; ++w) M = fmaxf(M, m_s[w * G + g]);
      float L = 0.f, O = 0.f;
      if (M != -INFINITY) {
#pragma unroll
        for (int w = 0; w < W; ++w) {
          const float f = __expf(m_s[w * G + g] - M);
          L += l_s[w * G + g] * f;
          O += o_s[(w * G + g) * HD + d] * f;
        }
      }
      wo[e] = O;
      if (d == 0) {
        wml[g * 2] = M;
        wml[g * 2 + 1] = L;
      }
    }
    __threadfence();
    Sync::sync();
    if (tid == 0) {
      const int old = atomicAdd(&p.counters[unit], 1);
      const int last = old == splits - 1;
      if (last) p.counters[unit] = 0;
      s_is_last = last;
      __threadfence();
    }
    Sync::sync();
    finalize = s_is_last != 0;
  }
  if (!finalize) return;

  // ---- final normalisation (+ optional FP8 1x128 quantisation: one block per head when HD == 128)
  for (int e0 = 0; e0 < G * HD; e0 += 128) {
    const int e = e0 + tid;
    const bool in = e < G * HD;
    const int g = in ? e / HD : 0, d = in ? e % HD : 0;
    float M = -INFINITY, L = 0.f, O = 0.f;
    if (in) {
      if (splits > 1) {
        const float* wo = p.ws_o + unit * splits * (G * HD);
        const float* wml = p.ws_ml + unit * splits * (G * 2);
        for (int s2 = 0; s2 < splits; ++s2) M = fmaxf(M, __ldcg(wml + (s2 * G + g) * 2));
        if (M != -INFINITY) {
          for (int s2 = 0; s2 < splits; ++s2) {
            const float ms = __ldcg(wml + (s2 * G + g) * 2);
            const float f = ms == -INFINITY ? 0.f : __expf(ms - M);
            L += __ldcg(wml + (s2 * G + g) * 2 + 1) * f;
            O += __ldcg(wo + static_cast<size_t>(s2) * G * HD + e) * f;
          }
        }
      } else {
#pragma unroll
        for (int w = 0; w < W; ++w) M = fmaxf(M, m_s[w * G + g]);
        if (M != -INFINITY) {
#pragma unroll
          for (int w = 0; w < W; ++w) {
            const float f = __expf(m_s[w * G + g] - M);
            L += l_s[w * G + g] * f;
            O += o_s[(w * G + g) * HD + d] * f;
          }
        }
      }
      if (p.sinks && M != -INFINITY) {
        // A per-head sink logit joins the denominator only.
        const float sk = p.sinks[kvh * G + g];
        const float M2 = fmaxf(M, sk);
        const float f = __expf(M - M2);
        L = L * f + __expf(sk - M2);
        O *= f;
      }
    }
    float val = (L > 0.f) ? O / L : 0.f;
    val = __bfloat162float(__float2bfloat16_rn(val));
    const size_t oidx = static_cast<size_t>(r) * hq * HD + (kvh * G + g) * HD + d;
    if (p.out_fp8) {
      // HD == 128 == blockDim: this iteration is exactly head g.
      float a = fabsf(val);
      if (!(a == a) || a > 3.0e38f) a = 0.f;
      a = warp_max(a);
      if (lane == 0) s_red[warp] = a;
      Sync::sync();
      const float amax = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
      const float scale = amax > 0.f ? amax / 448.f : 1.f;
      if (in) {
        p.out_fp8[oidx] = f32_to_e4m3(__fdiv_rn(val, scale));
        if (d == 0) p.out_scale[static_cast<size_t>(kvh * G + g) * p.ld_scale + r] = scale;
      }
      Sync::sync();
    } else if (in) {
      p.out_bf16[oidx] = __float2bfloat16_rn(val);
    }
  }
}

}  // namespace sllm
