// Gated delta net (linear attention) layers of the Qwen3.5 hybrid: depthwise causal convolution + SiLU with a
// rolling convolution state, and the gated delta-rule recurrence fused with the output RMSNorm and the SiLU(z)
// gate.  Both kernels work on a flat token batch in which the rows of one sequence are contiguous
// (row_off[s] .. row_off[s + 1]) and every sequence owns a state slot (slots[s]), so a decode step of many
// requests and a prefill of several prompts are the same launch.
//
// Recurrence per value head (state S[dv][dk], fp32), token by token:
//   q, k    L2-normalised over the head (eps 1e-6), rounded to bf16; q additionally scaled by 1/sqrt(dk)
//   beta    sigmoid(b) rounded to bf16;  decay = exp(-exp(A_log) * softplus(a + dt_bias))
//   S      <- decay * S;  r = v - S k;  S <- S + beta * r k^T;  o = S q
//   out     bf16(rmsnorm(bf16(o)) over dv, eps 1e-6) * norm_weight * silu(z)
// One CTA per (sequence, value head), thread d owns row d of the state in registers for the whole sequence
// (the reference re-reads the state from memory for every token: linear_attention_kernel.hip.cpp:128; same
// operation order here so that results agree with its fp32 oracle).
#include "common.cuh"
#include "api.h"

namespace sllm {

constexpr int kGdnHeadDim = 128;

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// x: [T, width] bf16 (the q|k|v projection), w: [width, taps] bf16, state: [slots, taps - 1, width] bf16.
// grid (ceil(width / 128), sequences).
__global__ void gdn_conv_silu_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                     __nv_bfloat16* __restrict__ state, __nv_bfloat16* __restrict__ y,
                                     const int* __restrict__ row_off, const int* __restrict__ slots, int width, int taps,
                                     int ldx) {
  pdl_wait();
  pdl_trigger();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y;
  if (c >= width) return;
  const int r0 = row_off[s], r1 = row_off[s + 1];
  const int hist = taps - 1;
  __nv_bfloat16* st = state + static_cast<size_t>(slots[s]) * hist * width;
  float win[8];       // sliding window of the last `taps` inputs (taps <= 8)
  float wt[8];
  for (int t = 0; t < taps; ++t) wt[t] = __bfloat162float(w[static_cast<size_t>(c) * taps + t]);
  for (int t = 0; t < hist; ++t) win[t] = __bfloat162float(st[static_cast<size_t>(t) * width + c]);
  for (int r = r0; r < r1; ++r) {
    win[hist] = __bfloat162float(x[static_cast<size_t>(r) * ldx + c]);
    float sum = 0.f;
    for (int t = 0; t < taps; ++t) sum += win[t] * wt[t];
    y[static_cast<size_t>(r) * width + c] = __float2bfloat16_rn(sum / (1.f + expf(-sum)));
    for (int t = 0; t < hist; ++t) win[t] = win[t + 1];
  }
  for (int t = 0; t < hist; ++t) st[static_cast<size_t>(t) * width + c] = __float2bfloat16_rn(win[t]);
}

// qkv: [T, 2 * qk_heads * 128 + v_heads * 128] bf16 after the convolution; z: [T, v_heads * 128];
// b, a: [T, v_heads]; a_log fp32 [v_heads]; dt_bias bf16 [v_heads]; norm_w fp32 [128];
// state: [slots, v_heads, 128 (dv), 128 (dk)] fp32; out: [T, v_heads * 128] bf16.
// grid (v_heads, sequences), 128 threads.
__global__ void __launch_bounds__(kGdnHeadDim)
gdn_recurrent_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ z,
                     const __nv_bfloat16* __restrict__ b_in, const __nv_bfloat16* __restrict__ a_in,
                     const float* __restrict__ a_log, const __nv_bfloat16* __restrict__ dt_bias,
                     const float* __restrict__ norm_w, float* __restrict__ state, __nv_bfloat16* __restrict__ out,
                     const int* __restrict__ row_off, const int* __restrict__ slots, int qk_heads, int v_heads, int ldz,
                     int ldg) {
  pdl_wait();
  pdl_trigger();
  constexpr int HD = kGdnHeadDim;
  const int vh = blockIdx.x, s = blockIdx.y, d = threadIdx.x;
  const int qh = vh / (v_heads / qk_heads);
  const int width = (2 * qk_heads + v_heads) * HD, ow = v_heads * HD;
  const int r0 = row_off[s], r1 = row_off[s + 1];
  if (r1 <= r0) return;
  __shared__ float q_s[HD], k_s[HD];
  __shared__ float red[3][4];
  __shared__ float sc[2];
  float* srow = state + ((static_cast<size_t>(slots[s]) * v_heads + vh) * HD + d) * HD;
  float S[HD];
#pragma unroll
  for (int i = 0; i < HD; i += 4) {
    const float4 v4 = *reinterpret_cast<const float4*>(srow + i);
    S[i] = v4.x; S[i + 1] = v4.y; S[i + 2] = v4.z; S[i + 3] = v4.w;
  }
  const int lane = d & 31, warp = d >> 5;
  const float a_neg = -expf(a_log[vh]);
  const float dtb = __bfloat162float(dt_bias[vh]);
  const float nw = norm_w[d];
  for (int r = r0; r < r1; ++r) {
    const size_t row = static_cast<size_t>(r) * width;
    const float qv = __bfloat162float(qkv[row + qh * HD + d]);
    const float kv = __bfloat162float(qkv[row + (qk_heads + qh) * HD + d]);
    const float vv = __bfloat162float(qkv[row + (2 * qk_heads + vh) * HD + d]);
    float qq = warp_sum(qv * qv), kk = warp_sum(kv * kv);
    if (lane == 0) { red[0][warp] = qq; red[1][warp] = kk; }
    __syncthreads();
    if (d == 0) {
      const float bq = __bfloat162float(b_in[static_cast<size_t>(r) * ldg + vh]);
      sc[0] = bf16_round(1.f / (1.f + expf(-bq)));
      const float av = __bfloat162float(a_in[static_cast<size_t>(r) * ldg + vh]) + dtb;
      sc[1] = expf(a_neg * softplus_f(av));
    }
    qq = red[0][0] + red[0][1] + red[0][2] + red[0][3];
    kk = red[1][0] + red[1][1] + red[1][2] + red[1][3];
    q_s[d] = bf16_round(qv * (1.f / sqrtf(qq + 1e-6f))) * (1.f / sqrtf(static_cast<float>(HD)));
    k_s[d] = bf16_round(kv * (1.f / sqrtf(kk + 1e-6f)));
    __syncthreads();
    const float beta = sc[0], decay = sc[1];
    float prev = 0.f;
#pragma unroll
    for (int i = 0; i < HD; ++i) {
      S[i] *= decay;
      prev += S[i] * k_s[i];
    }
    const float resid = beta * (vv - prev);
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < HD; ++i) {
      S[i] += resid * k_s[i];
      o += S[i] * q_s[i];
    }
    o = bf16_round(o);
    float oo = warp_sum(o * o);
    if (lane == 0) red[2][warp] = oo;
    __syncthreads();
    oo = red[2][0] + red[2][1] + red[2][2] + red[2][3];
    const float inv = 1.f / sqrtf(oo / static_cast<float>(HD) + 1e-6f);
    const float zv = __bfloat162float(z[static_cast<size_t>(r) * ldz + vh * HD + d]);
    out[static_cast<size_t>(r) * ow + vh * HD + d] = __float2bfloat16_rn(bf16_round(o * inv) * nw * (zv / (1.f + expf(-zv))));
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < HD; i += 4) *reinterpret_cast<float4*>(srow + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
}

// ---------------------------------------------------------------- prompt form of the recurrence: three stages
// The fused kernel above pays two block reductions and three barriers per token; on a prompt that is most of the
// ~1.7 us a token costs.  Everything that does not depend on the state is the same for all tokens and runs in
// parallel over them:
//   gdn_pre_kernel    per (token, head): normalised q and k (fp32, already rounded and scaled), beta, decay
//   gdn_scan_kernel   per (value head, sequence): the state update alone - thread d keeps row d of S in registers and
//                     reads a chunk of tokens' q / k from shared memory; no reduction, one barrier per 16 tokens
//   gdn_post_kernel   per (token, value head): RMSNorm over dv and the SiLU(z) gate
// (the reference's column pipeline: native/hip/src/linear_attention_kernel.hip.cpp, pre / recurrent / post process).
// Same arithmetic as the fused kernel except that the two dot products over dk are summed in four interleaved partial
// sums instead of one chain.
constexpr int kGdnChunk = 16;

// grid (T, qk_heads + ceil(v_heads / 128)), 128 threads.  qn / kn: [T, qk_heads, 128] fp32; gates: [T, v_heads, 2].
__global__ void __launch_bounds__(kGdnHeadDim)
gdn_pre_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ b_in,
               const __nv_bfloat16* __restrict__ a_in, const float* __restrict__ a_log,
               const __nv_bfloat16* __restrict__ dt_bias, float* __restrict__ qn, float* __restrict__ kn,
               float* __restrict__ gates, int qk_heads, int v_heads, int ldg) {
  pdl_wait();
  pdl_trigger();
  constexpr int HD = kGdnHeadDim;
  const int r = blockIdx.x, d = threadIdx.x;
  if (static_cast<int>(blockIdx.y) >= qk_heads) {
    const int vh = (blockIdx.y - qk_heads) * HD + d;
    if (vh < v_heads) {
      const float bq = __bfloat162float(b_in[static_cast<size_t>(r) * ldg + vh]);
      const float av = __bfloat162float(a_in[static_cast<size_t>(r) * ldg + vh]) + __bfloat162float(dt_bias[vh]);
      gates[(static_cast<size_t>(r) * v_heads + vh) * 2] = bf16_round(1.f / (1.f + expf(-bq)));
      gates[(static_cast<size_t>(r) * v_heads + vh) * 2 + 1] = expf(-expf(a_log[vh]) * softplus_f(av));
    }
    return;
  }
  const int qh = blockIdx.y;
  const int width = (2 * qk_heads + v_heads) * HD;
  __shared__ float red[2][4];
  const size_t row = static_cast<size_t>(r) * width;
  const float qv = __bfloat162float(qkv[row + qh * HD + d]);
  const float kv = __bfloat162float(qkv[row + (qk_heads + qh) * HD + d]);
  float qq = warp_sum(qv * qv), kk = warp_sum(kv * kv);
  if ((d & 31) == 0) { red[0][d >> 5] = qq; red[1][d >> 5] = kk; }
  __syncthreads();
  qq = red[0][0] + red[0][1] + red[0][2] + red[0][3];
  kk = red[1][0] + red[1][1] + red[1][2] + red[1][3];
  const size_t o = (static_cast<size_t>(r) * qk_heads + qh) * HD + d;
  qn[o] = bf16_round(qv * (1.f / sqrtf(qq + 1e-6f))) * (1.f / sqrtf(static_cast<float>(HD)));
  kn[o] = bf16_round(kv * (1.f / sqrtf(kk + 1e-6f)));
}

// grid (v_heads, sequences), 128 threads.  o_raw: [T, v_heads * 128] fp32 = bf16-rounded S q.
__global__ void __launch_bounds__(kGdnHeadDim)
gdn_scan_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ qn, const float* __restrict__ kn,
                const float* __restrict__ gates, float* __restrict__ state, float* __restrict__ o_raw,
                const int* __restrict__ row_off, const int* __restrict__ slots, int qk_heads, int v_heads) {
  pdl_wait();
  pdl_trigger();
  constexpr int HD = kGdnHeadDim;
  const int vh = blockIdx.x, s = blockIdx.y, d = threadIdx.x;
  const int qh = vh / (v_heads / qk_heads);
  const int width = (2 * qk_heads + v_heads) * HD, ow = v_heads * HD;
  const int r0 = row_off[s], r1 = row_off[s + 1];
  if (r1 <= r0) return;
  __shared__ __align__(16) float q_s[kGdnChunk][HD];
  __shared__ __align__(16) float k_s[kGdnChunk][HD];
  __shared__ float g_s[kGdnChunk][2];
  float* srow = state + ((static_cast<size_t>(slots[s]) * v_heads + vh) * HD + d) * HD;
  float S[HD];
#pragma unroll
  for (int i = 0; i < HD; i += 4) {
    const float4 v4 = *reinterpret_cast<const float4*>(srow + i);
    S[i] = v4.x; S[i + 1] = v4.y; S[i + 2] = v4.z; S[i + 3] = v4.w;
  }
  for (int c0 = r0; c0 < r1; c0 += kGdnChunk) {
    const int cn = min(kGdnChunk, r1 - c0);
    __syncthreads();                                       // the previous chunk has been consumed
    for (int t = 0; t < cn; ++t) {
      const size_t o = (static_cast<size_t>(c0 + t) * qk_heads + qh) * HD + d;
      q_s[t][d] = qn[o];
      k_s[t][d] = kn[o];
    }
    if (d < 2 * cn) g_s[d >> 1][d & 1] = gates[(static_cast<size_t>(c0 + (d >> 1)) * v_heads + vh) * 2 + (d & 1)];
    __syncthreads();
    for (int t = 0; t < cn; ++t) {
      const int r = c0 + t;
      const float vv = __bfloat162float(qkv[static_cast<size_t>(r) * width + (2 * qk_heads + vh) * HD + d]);
      const float beta = g_s[t][0], decay = g_s[t][1];
      float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
      for (int i = 0; i < HD; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(&k_s[t][i]);
        S[i] *= decay; S[i + 1] *= decay; S[i + 2] *= decay; S[i + 3] *= decay;
        p0 += S[i] * k4.x; p1 += S[i + 1] * k4.y; p2 += S[i + 2] * k4.z; p3 += S[i + 3] * k4.w;
      }
      const float resid = beta * (vv - ((p0 + p1) + (p2 + p3)));
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int i = 0; i < HD; i += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(&k_s[t][i]);
        const float4 q4 = *reinterpret_cast<const float4*>(&q_s[t][i]);
        S[i] += resid * k4.x; S[i + 1] += resid * k4.y; S[i + 2] += resid * k4.z; S[i + 3] += resid * k4.w;
        o0 += S[i] * q4.x; o1 += S[i + 1] * q4.y; o2 += S[i + 2] * q4.z; o3 += S[i + 3] * q4.w;
      }
      o_raw[static_cast<size_t>(r) * ow + vh * HD + d] = bf16_round((o0 + o1) + (o2 + o3));
    }
  }
#pragma unroll
  for (int i = 0; i < HD; i += 4) *reinterpret_cast<float4*>(srow + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
}

// grid (T, v_heads), 128 threads.
__global__ void __launch_bounds__(kGdnHeadDim)
gdn_post_kernel(const float* __restrict__ o_raw, const __nv_bfloat16* __restrict__ z, const float* __restrict__ norm_w,
                __nv_bfloat16* __restrict__ out, int v_heads, int ldz) {
  pdl_wait();
  pdl_trigger();
  constexpr int HD = kGdnHeadDim;
  const int r = blockIdx.x, vh = blockIdx.y, d = threadIdx.x;
  __shared__ float red[4];
  const size_t idx = static_cast<size_t>(r) * v_heads * HD + vh * HD + d;
  const float o = o_raw[idx];
  float oo = warp_sum(o * o);
  if ((d & 31) == 0) red[d >> 5] = oo;
  __syncthreads();
  oo = red[0] + red[1] + red[2] + red[3];
  const float inv = 1.f / sqrtf(oo / static_cast<float>(HD) + 1e-6f);
  const float zv = __bfloat162float(z[static_cast<size_t>(r) * ldz + vh * HD + d]);
  out[idx] = __float2bfloat16_rn(bf16_round(o * inv) * norm_w[d] * (zv / (1.f + expf(-zv))));
}

// In place per-head RMSNorm of the q and k heads inside a fused qkv activation (query/key normalisation of
// the Qwen3 / Gemma families): x [T, ld], heads 0 .. hq + hkv - 1 of width hd each; weight_q / weight_k fp32-exact
// bf16 [hd] (null: ones); offset_one: scale = 1 + w.  grid (T, heads), 128 threads; head0 = first head to touch;
// heads from hq + hkv on are value heads and take no weight.
__global__ void qk_headnorm_kernel(__nv_bfloat16* __restrict__ x, int ld, int hq, int hkv, int hd,
                                   const __nv_bfloat16* __restrict__ wq, const __nv_bfloat16* __restrict__ wk, float eps,
                                   int offset_one, int head0) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, h = head0 + blockIdx.y;
  __nv_bfloat16* p = x + static_cast<size_t>(t) * ld + static_cast<size_t>(h) * hd;
  const __nv_bfloat16* w = h < hq ? wq : (h < hq + hkv ? wk : nullptr);
  __shared__ float red[4];
  float ss = 0.f;
  for (int i = threadIdx.x; i < hd; i += blockDim.x) {
    const float v = __bfloat162float(p[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  ss = red[0] + red[1] + red[2] + red[3];
  const float inv = rsqrtf(ss / static_cast<float>(hd) + eps);
  for (int i = threadIdx.x; i < hd; i += blockDim.x) {
    const float g = w ? __bfloat162float(w[i]) + (offset_one ? 1.f : 0.f) : 1.f;
    p[i] = __float2bfloat16_rn(__bfloat162float(p[i]) * inv * g);
  }
}

}  // namespace sllm

using namespace sllm;

// ldx: row stride of x in elements (0: width) - x may be a column slice of a wider projection output.
SLLM_EXPORT int sllm_gdn_conv_silu(const void* x, const void* w, void* state, void* y, const int* row_off, const int* slots,
                                   int sequences, int width, int taps, int ldx, void* stream) {
  if (!x || !w || !state || !y || !row_off || !slots || sequences <= 0 || width <= 0 || taps < 2 || taps > 8)
    return SLLM_ERR_INVALID_ARGUMENT;
  cudaError_t e = launch_kernel(gdn_conv_silu_kernel, dim3((width + 127) / 128, sequences), dim3(128), 0,
                                static_cast<cudaStream_t>(stream), 1u, static_cast<const __nv_bfloat16*>(x),
                                static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(state),
                                static_cast<__nv_bfloat16*>(y), row_off, slots, width, taps, ldx > 0 ? ldx : width);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

// ldz / ldg: row strides in elements of z and of b / a (0: v_heads * 128 and v_heads) - they may be column slices of a
// wider projection output.
SLLM_EXPORT int sllm_gdn_recurrent(const void* qkv, const void* z, const void* b, const void* a, const float* a_log,
                                   const void* dt_bias, const float* norm_w, float* state, void* out, const int* row_off,
                                   const int* slots, int sequences, int qk_heads, int v_heads, int head_dim, int ldz, int ldg,
                                   void* stream) {
  if (!qkv || !z || !b || !a || !a_log || !dt_bias || !norm_w || !state || !out || !row_off || !slots || sequences <= 0 ||
      qk_heads <= 0 || v_heads <= 0 || (v_heads % qk_heads))
    return SLLM_ERR_INVALID_ARGUMENT;
  if (head_dim != kGdnHeadDim) return SLLM_ERR_UNSUPPORTED_SHAPE;
  cudaError_t e = launch_kernel(gdn_recurrent_kernel, dim3(v_heads, sequences), dim3(kGdnHeadDim), 0,
                                static_cast<cudaStream_t>(stream), 1u, static_cast<const __nv_bfloat16*>(qkv),
                                static_cast<const __nv_bfloat16*>(z), static_cast<const __nv_bfloat16*>(b),
                                static_cast<const __nv_bfloat16*>(a), a_log, static_cast<const __nv_bfloat16*>(dt_bias), norm_w,
                                state, static_cast<__nv_bfloat16*>(out), row_off, slots, qk_heads, v_heads,
                                ldz > 0 ? ldz : v_heads * kGdnHeadDim, ldg > 0 ? ldg : v_heads);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

// The prompt form (three launches).  tokens = rows of qkv; scratch: fp32, at least
// tokens * (2 * qk_heads * 128 + 2 * v_heads + v_heads * 128) elements.
SLLM_EXPORT int sllm_gdn_recurrent_prompt(const void* qkv, const void* z, const void* b, const void* a, const float* a_log,
                                          const void* dt_bias, const float* norm_w, float* state, void* out,
                                          const int* row_off, const int* slots, int sequences, int tokens, int qk_heads,
                                          int v_heads, int head_dim, int ldz, int ldg, float* scratch,
                                          long long scratch_floats, void* stream) {
  if (!qkv || !z || !b || !a || !a_log || !dt_bias || !norm_w || !state || !out || !row_off || !slots || !scratch ||
      sequences <= 0 || tokens <= 0 || qk_heads <= 0 || v_heads <= 0 || (v_heads % qk_heads))
    return SLLM_ERR_INVALID_ARGUMENT;
  if (head_dim != kGdnHeadDim) return SLLM_ERR_UNSUPPORTED_SHAPE;
  const long long nq = static_cast<long long>(tokens) * qk_heads * kGdnHeadDim;
  const long long ng = static_cast<long long>(tokens) * v_heads * 2;
  const long long no = static_cast<long long>(tokens) * v_heads * kGdnHeadDim;
  if (scratch_floats < 2 * nq + ng + no) return SLLM_ERR_WORKSPACE_TOO_SMALL;
  float* qn = scratch;
  float* kn = qn + nq;
  float* gates = kn + nq;
  float* o_raw = gates + ng;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int gate_blocks = (v_heads + kGdnHeadDim - 1) / kGdnHeadDim;
  cudaError_t e = launch_kernel(gdn_pre_kernel, dim3(tokens, qk_heads + gate_blocks), dim3(kGdnHeadDim), 0, st, 1u,
                                static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(b),
                                static_cast<const __nv_bfloat16*>(a), a_log, static_cast<const __nv_bfloat16*>(dt_bias), qn, kn,
                                gates, qk_heads, v_heads, ldg > 0 ? ldg : v_heads);
  if (e != cudaSuccess) return SLLM_ERR_CUDA;
  e = launch_kernel(gdn_scan_kernel, dim3(v_heads, sequences), dim3(kGdnHeadDim), 0, st, 1u,
                    static_cast<const __nv_bfloat16*>(qkv), static_cast<const float*>(qn), static_cast<const float*>(kn),
                    static_cast<const float*>(gates), state, o_raw, row_off, slots, qk_heads, v_heads);
  if (e != cudaSuccess) return SLLM_ERR_CUDA;
  e = launch_kernel(gdn_post_kernel, dim3(tokens, v_heads), dim3(kGdnHeadDim), 0, st, 1u, static_cast<const float*>(o_raw),
                    static_cast<const __nv_bfloat16*>(z), norm_w, static_cast<__nv_bfloat16*>(out), v_heads,
                    ldz > 0 ? ldz : v_heads * kGdnHeadDim);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

SLLM_EXPORT int sllm_qk_headnorm(void* x, int ld, int tokens, int hq, int hkv, int hd, const void* wq, const void* wk, float eps,
                                 int offset_one, void* stream) {
  if (!x || !wq || !wk || tokens <= 0 || hq <= 0 || hkv <= 0 || hd <= 0) return SLLM_ERR_INVALID_ARGUMENT;
  cudaError_t e = launch_kernel(qk_headnorm_kernel, dim3(tokens, hq + hkv), dim3(128), 0, static_cast<cudaStream_t>(stream), 1u,
                                static_cast<__nv_bfloat16*>(x), ld, hq, hkv, hd, static_cast<const __nv_bfloat16*>(wq),
                                static_cast<const __nv_bfloat16*>(wk), eps, offset_one, 0);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

// The same over a chosen span of heads: skip_qk leaves the q / k heads alone, norm_v adds the value heads (unweighted:
// reference crates/sllm-core/src/gemma4_graph.rs:740).  Null weights mean ones.
SLLM_EXPORT int sllm_qkv_headnorm(void* x, int ld, int tokens, int hq, int hkv, int hd, const void* wq, const void* wk,
                                  float eps, int offset_one, int skip_qk, int norm_v, void* stream) {
  if (!x || tokens <= 0 || hq <= 0 || hkv <= 0 || hd <= 0) return SLLM_ERR_INVALID_ARGUMENT;
  const int head0 = skip_qk ? hq + hkv : 0;
  const int heads = (skip_qk ? 0 : hq + hkv) + (norm_v ? hkv : 0);
  if (heads == 0) return SLLM_OK;
  // a q / k span followed by the value span is contiguous in head index; a lone value span starts at hq + hkv
  cudaError_t e = launch_kernel(qk_headnorm_kernel, dim3(tokens, heads), dim3(128), 0, static_cast<cudaStream_t>(stream), 1u,
                                static_cast<__nv_bfloat16*>(x), ld, hq, hkv, hd, static_cast<const __nv_bfloat16*>(wq),
                                static_cast<const __nv_bfloat16*>(wk), eps, offset_one, head0);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}
