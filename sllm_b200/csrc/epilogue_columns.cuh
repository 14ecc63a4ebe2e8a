// Row epilogues shared by the decode GEMM kernels (gemm_tcgen05.cu with its cluster split-K reduction, and the
// persistent decode_fused.cu): one warp finishes one token row of a 128-row output tile, lane l owning outputs
// 4 l .. 4 l + 3 of the tile.  What used to be separate kernels after the GEMM runs here on the fp32 sums:
//   PLAIN        (+ residual) (soft-cap) -> bf16
//   RESID_QUANT  + residual -> bf16 residual stream, its E4M3 form with one scale per 128 outputs, and the sum of
//                squares of the block (the statistics of the next RMSNorm)
//   SILU_QUANT   the already activated value -> E4M3 + scale
//   ROPE_KV      tile = attention head: rotary embedding of q / k heads, q written as bf16, k / v quantised (or
//                copied) into their KV page slot
// Counterparts in the reference are separate kernels: elementwise_kernel.hip.cpp:40-147 (residual add, silu-mul),
// matmul_kernel.hip.cpp:210-247 (activation quantisation), rotary_kernel.hip.cpp:40, kv_state_kernel.hip.cpp:161-335.
#pragma once
#include "common.cuh"
#include "decode_fused.h"

namespace sllm {

struct ColEpilogue {
  int mode;                          // SllmFdEpilogue
  int n, ldy, ld_s;
  float softcap;
  __nv_bfloat16* y;
  const __nv_bfloat16* residual;     // added here when non-null
  uint8_t* q_out;
  float* s_out;
  float* ssq_out;
  const SllmFdRope* rope;            // ROPE_KV
  const float* inv_freq;             // ROPE_KV: [rotary_dim / 2] frequencies (shared or global memory)
};

__device__ __forceinline__ float col_bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// E4M3 + scale (+ sum of squares) of the 128 values a warp holds (4 per lane), values rounded to bf16 first.
__device__ __forceinline__ void col_quant_store(float (&v)[4], uint8_t* q_dst, float* s_dst, float* ssq_dst, int lane) {
  float amax = 0.f, ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[j] = col_bf16r(v[j]);
    ss += v[j] * v[j];
    const float a = fabsf(v[j]);
    if (a == a && a <= 3.0e38f) amax = fmaxf(amax, a);
  }
  amax = warp_max(amax);
  const float scale = amax > 0.f ? amax / 448.f : 1.f;
  uint32_t q = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) q |= static_cast<uint32_t>(f32_to_e4m3(__fdiv_rn(v[j], scale))) << (8 * j);
  *reinterpret_cast<uint32_t*>(q_dst) = q;
  if (lane == 0) *s_dst = scale;
  if (ssq_dst) {
    ss = warp_sum(ss);
    if (lane == 0) *ssq_dst = ss;
  }
}

// v: the lane's four fp32 sums of token row c (norm factor and activation already applied).  pos / page: the token's
// position and KV page (ROPE_KV only).
__device__ __forceinline__ void col_epilogue(const ColEpilogue& e, int tile, int c, int lane, float (&v)[4], int pos,
                                             int page) {
  const int n0 = tile * 128 + lane * 4;
  if (e.mode == SLLM_FD_PLAIN) {
    __nv_bfloat16* y = e.y + static_cast<size_t>(c) * e.ldy + n0;
    const __nv_bfloat16* res = e.residual ? e.residual + static_cast<size_t>(c) * e.ldy + n0 : nullptr;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (n0 + j < e.n) {
        float o = v[j];
        if (res) o += __bfloat162float(res[j]);
        if (e.softcap > 0.f) o = e.softcap * tanhf(o / e.softcap);
        y[j] = __float2bfloat16_rn(o);
      }
    }
  } else if (e.mode == SLLM_FD_RESID_QUANT || e.mode == SLLM_FD_SILU_QUANT) {
    if (e.mode == SLLM_FD_RESID_QUANT) {
      if (e.residual) {
        const uint2 rr = *reinterpret_cast<const uint2*>(e.residual + static_cast<size_t>(c) * e.ldy + n0);
        const __nv_bfloat162 r0 = *reinterpret_cast<const __nv_bfloat162*>(&rr.x);
        const __nv_bfloat162 r1 = *reinterpret_cast<const __nv_bfloat162*>(&rr.y);
        v[0] += __bfloat162float(r0.x); v[1] += __bfloat162float(r0.y);
        v[2] += __bfloat162float(r1.x); v[3] += __bfloat162float(r1.y);
      }
      uint2 hw;
      *reinterpret_cast<__nv_bfloat162*>(&hw.x) = __floats2bfloat162_rn(v[0], v[1]);
      *reinterpret_cast<__nv_bfloat162*>(&hw.y) = __floats2bfloat162_rn(v[2], v[3]);
      *reinterpret_cast<uint2*>(e.y + static_cast<size_t>(c) * e.ldy + n0) = hw;
    }
    col_quant_store(v, e.q_out + static_cast<size_t>(c) * e.n + n0, e.s_out + static_cast<size_t>(tile) * e.ld_s + c,
                    e.ssq_out ? e.ssq_out + static_cast<size_t>(tile) * e.ld_s + c : nullptr, lane);
  } else {
    // ROPE_KV: tile = head index (q heads, then k heads, then v heads), lane holds dims 4 lane .. 4 lane + 3
    const SllmFdRope& rp = *e.rope;
    const int head = tile;
    const bool is_q = head < rp.hq;
    const bool is_v = head >= rp.hq + rp.hkv;
    if (!is_v) {
      const int half = rp.rotary_dim >> 1;
      const int lane_off = half >> 2;          // partner lane distance (half / 4), a power of two
      float pv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) pv[j] = __shfl_xor_sync(0xffffffffu, v[j], lane_off);
      const int i0 = lane * 4;
      if (i0 < rp.rotary_dim) {
        const bool lo = i0 < half;
        const int f0 = lo ? i0 : i0 - half;
#pragma unroll 1
        for (int j = 0; j < 4; ++j) {
          float sn, cs;
          sincosf(static_cast<float>(pos) * e.inv_freq[f0 + j], &sn, &cs);
          const float a = lo ? v[j] : pv[j], b = lo ? pv[j] : v[j];
          v[j] = lo ? a * cs - b * sn : b * cs + a * sn;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = col_bf16r(v[j]);
    uint2 hw;
    *reinterpret_cast<__nv_bfloat162*>(&hw.x) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(&hw.y) = __floats2bfloat162_rn(v[2], v[3]);
    if (is_q) {
      *reinterpret_cast<uint2*>(e.y + static_cast<size_t>(c) * e.ldy + n0) = hw;
    } else {
      const int kvh = is_v ? head - rp.hq - rp.hkv : head - rp.hq;
      const size_t slot = (static_cast<size_t>(page) * rp.hkv + kvh) * rp.page_size + pos % rp.page_size;
      if (!rp.kv_fp8) {
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(is_v ? rp.v_pages : rp.k_pages) + slot * 128 + lane * 4;
        *reinterpret_cast<uint2*>(dst) = hw;
      } else {
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = fabsf(v[j]);
          if (a == a && a <= 3.0e38f) amax = fmaxf(amax, a);
        }
        amax = warp_max(amax);
        const float st = is_v ? rp.v_static : rp.k_static;
        const float scale = st > 0.f ? st : (amax > 0.f ? amax / 448.f : 1.f);
        uint32_t q = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) q |= static_cast<uint32_t>(f32_to_e4m3(__fdiv_rn(v[j], scale))) << (8 * j);
        uint8_t* dst = static_cast<uint8_t*>(is_v ? rp.v_pages : rp.k_pages) + slot * 128 + lane * 4;
        *reinterpret_cast<uint32_t*>(dst) = q;
        if (lane == 0 && st <= 0.f) (is_v ? rp.v_scale : rp.k_scale)[slot] = scale;
      }
    }
  }
}

}  // namespace sllm
