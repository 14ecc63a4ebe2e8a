// Causal prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), head_dim 128.
//
// Fresh prompts only: every sequence's tokens are contiguous rows of the packed qkv activation
// [T, (hq + 2 hkv) * 128] (bf16, q and k already rotated) and start at position 0, so K and V are read
// from that tensor with TMA instead of from the paged cache.  Chunked or cache-continuing prefill goes
// through the paged kernel in attention.cu.
//
// One CTA = one (sequence, 128-row query tile, query head); 192 threads:
//   warp 0    TMA producer: Q once, then K/V tiles of 128 keys through a 2-stage ring
//   warp 1    TMEM owner + MMA issuer:  S = Q K^T  (M=128 queries, N=128 keys, K=128 channels)
//                                       PV = P V    (M=128 queries, N=128 channels, K=128 keys)
//   warps 2-5 softmax: thread r owns query row r (TMEM lane r): row max / sum are thread-local, P is
//             written to shared memory as the bf16 K-major A operand of the second MMA, the running
//             output lives in 128 fp32 registers and is rescaled when the row maximum moves.
// S_{j+1} is issued right after PV_j, so the tensor core computes the next scores while the softmax
// warps fold PV_j into the output.  V is consumed as an MN-major B operand straight from its
// [key, channel] layout.
//
// Replaces the reference's scalar prefill kernels (causal_attention_kernel.hip.cpp:388-495).
#include "common.cuh"
#include "api.h"
#include "tmap.h"

namespace sllm {

constexpr int kPfThreads = 192;
constexpr int kPfTile = 128;            // query rows per CTA and keys per KV tile
constexpr int kPfHd = 128;
constexpr int kChunkBytes = kPfTile * 128;  // one [128 rows x 64 bf16] swizzled chunk = 16 KB

struct PrefillParams {
  const int* tiles;        // [num_tiles][4]: first token row of the sequence, sequence length, q0, unused
  int hq, hkv;
  float scale_log2;        // softmax scale * log2(e)
  __nv_bfloat16* out_bf16; // [T, hq * 128] or null
  uint8_t* out_fp8;        // E4M3 [T, hq * 128] or null
  float* out_scale;        // [hq, ld_scale]
  int ld_scale;
  int* status;
};

struct __align__(8) PrefillBarriers {
  uint64_t q_full;
  uint64_t kv_full[2];
  uint64_t kv_empty[2];
  uint64_t s_full;
  uint64_t p_ready;
  uint64_t o_full;
  uint32_t tmem_base;
  int abort_flag;
};

// MN-major operand (rows = K index, 128-byte rows of 64 contiguous MN elements, two MN blocks of
// 64 elements `mn_block_stride` bytes apart), 128-byte swizzle: LBO = MN-block stride, SBO = 1024.
__device__ __forceinline__ uint64_t make_smem_desc_sw128_mn(uint32_t smem_addr, uint32_t mn_block_stride) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((mn_block_stride >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__global__ void __launch_bounds__(kPfThreads, 1)
prefill_attention_kernel(const __grid_constant__ CUtensorMap tm_qkv, const PrefillParams p) {
  pdl_wait();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // layout: Q (2 chunks) | P (2 chunks) | 2 stages x { K (2 chunks) | V (2 chunks) } | barriers
  uint8_t* q_s = smem;
  uint8_t* p_s = smem + 2 * kChunkBytes;
  uint8_t* kv_s = smem + 4 * kChunkBytes;
  PrefillBarriers* bars = reinterpret_cast<PrefillBarriers*>(smem + 12 * kChunkBytes);
  constexpr int kStageBytes = 4 * kChunkBytes;
  constexpr uint32_t kTmemCols = 256;  // S: columns [0,128), PV: columns [128,256)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int kvh = head / (p.hq / p.hkv);
  const int* tile = p.tiles + 4 * blockIdx.x;
  const int tok0 = tile[0], seq_len = tile[1], q0 = tile[2];
  const int nt = q0 / kPfTile + 1;  // causal: KV tiles 0 .. diagonal
  volatile int* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 1);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->p_ready, 128);
    mbar_init(&bars->o_full, 1);
    bars->abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_qkv);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  // No early trigger of dependent launches here: with one, the dependent GEMM's CTAs become resident
  // beside this kernel's for its whole run, and runs of a few hundred decode steps then showed an
  // occasional bounded wait of that GEMM running out (status 101, a 2 s stall); without it 1200 steps
  // ran clean.  Dependents therefore start when this grid completes.

  if (warp == 0) {
    if (lane == 0) {
      const int xq = head * kPfHd, xk = (p.hq + kvh) * kPfHd, xv = (p.hq + p.hkv + kvh) * kPfHd;
      mbar_expect_tx(&bars->q_full, 2 * kChunkBytes);
      tma_load_2d(q_s, &tm_qkv, &bars->q_full, xq, tok0 + q0);
      tma_load_2d(q_s + kChunkBytes, &tm_qkv, &bars->q_full, xq + 64, tok0 + q0);
      int issued = 0;
      for (int j = 0; j < nt; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&bars->kv_empty[st], ((j >> 1) & 1) ^ 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_SMEM_EMPTY)) break;
        uint8_t* dst = kv_s + st * kStageBytes;
        mbar_expect_tx(&bars->kv_full[st], kStageBytes);
        const int y = tok0 + j * kPfTile;
        tma_load_2d(dst, &tm_qkv, &bars->kv_full[st], xk, y);
        tma_load_2d(dst + kChunkBytes, &tm_qkv, &bars->kv_full[st], xk + 64, y);
        tma_load_2d(dst + 2 * kChunkBytes, &tm_qkv, &bars->kv_full[st], xv, y);
        tma_load_2d(dst + 3 * kChunkBytes, &tm_qkv, &bars->kv_full[st], xv + 64, y);
        issued = j + 1;
      }
      int dummy = 0;
      mbar_wait(&bars->q_full, 0, &dummy, p.status, SLLM_DEV_TIMEOUT_DRAIN, 200000000LL);
      for (int st = 0; st < 2; ++st) {
        const int fills = (issued > st) ? (issued - st + 1) / 2 : 0;
        if (fills > 0) mbar_wait(&bars->kv_full[st], (fills - 1) & 1, &dummy, p.status, SLLM_DEV_TIMEOUT_DRAIN, 200000000LL);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // S: A = Q (K-major), B = K tile (K-major).  PV: A = P (K-major), B = V tile (MN-major).
      constexpr uint32_t idesc_s = make_idesc(kFmtBf16, 128, 128, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc(kFmtBf16, 128, 128, 0, 1);
      const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s);
      auto issue_s = [&](int j) {
        const uint32_t k_addr = smem_u32(kv_s + (j & 1) * kStageBytes);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            umma_f16(tmem_base, make_smem_desc_sw128(q_addr + c * kChunkBytes) + 2 * k,
                     make_smem_desc_sw128(k_addr + c * kChunkBytes) + 2 * k, idesc_s, (c | k) != 0);
          }
        }
        tc_commit(&bars->s_full);
      };
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMA_FULL);
      if (ok) ok = mbar_wait(&bars->kv_full[0], 0, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMA_FULL);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; ok && j < nt; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&bars->p_ready, j & 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(kv_s + st * kStageBytes + 2 * kChunkBytes);
#pragma unroll
        for (int c = 0; c < 2; ++c) {      // P chunk c holds keys [64c, 64c + 64)
#pragma unroll
          for (int k = 0; k < 4; ++k) {    // 16 keys per MMA
            const int key0 = c * 64 + k * 16;
            umma_f16(tmem_base + 128, make_smem_desc_sw128(p_addr + c * kChunkBytes) + 2 * k,
                     make_smem_desc_sw128_mn(v_addr + key0 * 128, kChunkBytes), idesc_pv, (c | k) != 0);
          }
        }
        tc_commit(&bars->o_full);
        tc_commit(&bars->kv_empty[st]);
        if (j + 1 < nt) {
          if (!mbar_wait(&bars->kv_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMA_FULL))
            break;
          tc_fence_after();
          issue_s(j + 1);
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int qpos = q0 + r;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    float o[kPfHd];
#pragma unroll
    for (int i = 0; i < kPfHd; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nt; ++j) {
      if (ok) ok = mbar_wait(&bars->s_full, j & 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const bool diag = (j == nt - 1);
      const int key_base = j * kPfTile;
      // pass 1: row maximum
      float tmax = -INFINITY;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t v[16];
        tmem_ld16(lane_addr + c * 16, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float s = __uint_as_float(v[i]);
          if (diag && key_base + c * 16 + i > qpos) s = -INFINITY;
          tmax = fmaxf(tmax, s);
        }
      }
      const float m_new = fmaxf(m, tmax * p.scale_log2);
      const float alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      // pass 2: probabilities -> bf16 -> swizzled K-major shared memory
      float psum = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t v[16];
        tmem_ld16(lane_addr + c * 16, v);
        tmem_wait_ld();
        uint32_t packed[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float s0 = __uint_as_float(v[2 * i]), s1 = __uint_as_float(v[2 * i + 1]);
          float p0 = exp2f(s0 * p.scale_log2 - m_use), p1 = exp2f(s1 * p.scale_log2 - m_use);
          if (diag) {
            if (key_base + c * 16 + 2 * i > qpos) p0 = 0.f;
            if (key_base + c * 16 + 2 * i + 1 > qpos) p1 = 0.f;
          }
          const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          // the sum uses the rounded values, so the normaliser matches what the MMA multiplies
          psum += __bfloat162float(h.x) + __bfloat162float(h.y);
          packed[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        // 16 keys = two 16-byte units of this row; chunk = c / 4, unit index within the row = (c % 4) * 2 + {0, 1}
        uint8_t* rowp = p_s + (c >> 2) * kChunkBytes + r * 128;
        const int u0 = (c & 3) * 2;
        *reinterpret_cast<uint4*>(rowp + (((u0) ^ (r & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        *reinterpret_cast<uint4*>(rowp + (((u0 + 1) ^ (r & 7)) << 4)) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
      }
      l = l * alpha + psum;
      m = m_new;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bars->p_ready);
      // fold PV_j into the running output
      ok = mbar_wait(&bars->o_full, j & 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t v[16];
        tmem_ld16(lane_addr + 128 + c * 16, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) o[c * 16 + i] = fmaf(o[c * 16 + i], alpha, __uint_as_float(v[i]));
      }
      tc_fence_before();
    }
    if (ok && qpos < seq_len) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const size_t row = static_cast<size_t>(tok0 + qpos);
      const size_t base = row * p.hq * kPfHd + head * kPfHd;
      if (p.out_fp8) {
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < kPfHd; ++i) {
          o[i] = __bfloat162float(__float2bfloat16_rn(o[i] * inv));
          const float a = fabsf(o[i]);
          if (a == a && a <= 3.0e38f) amax = fmaxf(amax, a);
        }
        const float scale = amax > 0.f ? amax / 448.f : 1.f;
#pragma unroll
        for (int i = 0; i < kPfHd; i += 16) {
          uint32_t w[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            w[k] = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) w[k] |= static_cast<uint32_t>(f32_to_e4m3(__fdiv_rn(o[i + 4 * k + b], scale))) << (8 * b);
          }
          *reinterpret_cast<uint4*>(p.out_fp8 + base + i) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        p.out_scale[static_cast<size_t>(head) * p.ld_scale + row] = scale;
      } else {
#pragma unroll
        for (int i = 0; i < kPfHd; i += 8) {
          uint4 w;
          __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
          for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(o[i + 2 * k] * inv, o[i + 2 * k + 1] * inv);
          *reinterpret_cast<uint4*>(p.out_bf16 + base + i) = w;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace sllm

using namespace sllm;

// tiles: device int32 [num_tiles][4] = {first token row of the sequence, sequence length, q0, 0},
// ordered by the caller (longest first).  qkv row stride is qkv_ld elements.
SLLM_EXPORT int sllm_prefill_attention(const void* qkv, int total_tokens, int qkv_ld, const int* tiles, int num_tiles,
                                       int hq, int hkv, int hd, float sm_scale, void* out_bf16, void* out_fp8,
                                       float* out_scale, int ld_scale, int* status, void* stream) {
  if (!qkv || !tiles || num_tiles <= 0 || hq <= 0 || hkv <= 0 || hq % hkv) return SLLM_ERR_INVALID_ARGUMENT;
  if (hd != kPfHd) return SLLM_ERR_UNSUPPORTED_SHAPE;
  if (!out_bf16 && !(out_fp8 && out_scale)) return SLLM_ERR_INVALID_ARGUMENT;
  if (hq > 65535) return SLLM_ERR_LIMIT;
  CUtensorMap tm;
  int rc = cached_kmajor_tmap(&tm, qkv, 2, total_tokens, qkv_ld, static_cast<long long>(qkv_ld) * 2, kPfTile);
  if (rc != SLLM_OK) return rc;
  PrefillParams p;
  p.tiles = tiles; p.hq = hq; p.hkv = hkv; p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.out_bf16 = static_cast<__nv_bfloat16*>(out_bf16); p.out_fp8 = static_cast<uint8_t*>(out_fp8);
  p.out_scale = out_scale; p.ld_scale = ld_scale; p.status = status;
  const size_t smem = 12 * kChunkBytes + sizeof(PrefillBarriers) + 1024;
  static bool cfg = false;
  if (!cfg) {
    if (cudaFuncSetAttribute(prefill_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return SLLM_ERR_CUDA;
    cfg = true;
  }
  dim3 grid(num_tiles, hq);
  launch_kernel(prefill_attention_kernel, dim3(grid), dim3(kPfThreads), smem, static_cast<cudaStream_t>(stream), 1u, tm, p);
  return cudaGetLastError() == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}
