// Paged decode / verify attention over FP8 KV pages on the tensor cores (tcgen05 + TMEM + TMA),
// head_dim 128, GQA group <= 16.
//
// A CTA owns (query row, kv head, KV split) and walks its keys 128 at a time:
//   * the page table is walked by the producer warp: lane i issues the TMA box of page i of each tile
//     ({128 B of channels, 16 tokens} = 2 KB contiguous out of the head-major [pages, kv_heads, 16, 128]
//     E4M3 plane), eight boxes assembling a 128-key swizzled tile each for K and V, and stages the
//     tile's per-token scales with cp.async under the same barrier; 3-stage ring;
//   * S^T = K Q^T     : M = 128 keys, N = 16 (the group's heads, zero padded), K = 128 channels, E4M3
//     inputs (Q is quantised to E4M3 per head once per CTA), result in TMEM [key lane, head column];
//   * softmax        : thread t owns key t of the tile; per-head maxima cross the 128 threads by
//     shuffle + shared memory; probabilities are folded with the per-token V scale, scaled into the
//     E4M3 range and written as the K-major B operand P^T [head, key];
//   * O^T = V^T P    : M = 128 channels (V consumed MN-major, exactly as stored), N = 16 heads,
//     K = 128 keys; the running output is 16 fp32 registers per thread (thread = channel).
// Per-token K scales multiply the scores; KV splits are merged by attention_tail (shared with the
// CUDA-core kernel), which also applies sinks and the optional FP8 output quantisation.
//
// The CUDA-core kernel in attention.cu stays the path for bf16 pages and other head sizes.  Counterpart
// in the reference: causal_attention_decode_wave_split_kernel (causal_attention_kernel.hip.cpp:264).
#include <cstdio>
#include "common.cuh"
#include "api.h"
#include "attention_common.cuh"
#include <cudaTypedefs.h>
#include <cstddef>
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

namespace sllm {

constexpr int kDaThreads = 224;   // producer warp, S issuer, four softmax warps, PV issuer
constexpr int kDaTile = 128;
constexpr int kDaStages = 3;
constexpr int kDaTileBytes = kDaTile * 128;  // 16 KB per K or V tile
constexpr int kDaHeadsPad = 16;
// Status codes of this kernel's bounded waits are the shared ones plus 100, so that a recorded timeout
// names the kernel as well as the wait (201 KV tile, 203 S / PV accumulator, 204 probabilities).
constexpr int kDaStatusBase = 100;

struct __align__(16) DecodeTcBarriers {
  uint64_t kv_full[kDaStages];
  uint64_t kv_empty[kDaStages];
  uint64_t s_full[2];
  uint64_t p_ready[2];   // by tile parity: a waiter can then never fall a whole parity cycle behind
  uint64_t o_full[2];
  uint32_t tmem_base;
  int abort_flag;
  int is_last;
  float red[2][4][kDaHeadsPad + 1];   // per-warp maxima (heads + V scale), double buffered by tile parity
  alignas(16) float sc[kDaStages][2][kDaTile];  // per-token K and V scales of each staged tile (16-byte cp.async)
  float s_red[4];
};

// MN-major 8-bit operand: rows = K index (tokens), each row = 128 contiguous bytes of M (channels).
__device__ __forceinline__ uint64_t make_smem_desc_sw128_mn8(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Decode an E4M3 byte exactly (integer path, see e4m3x4_to_f32x4_exp120).
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
// Makes the barrier track this thread's earlier cp.async copies: the (pre-counted) arrival fires when they land.
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ float e4m3_to_f32_int(uint32_t b) {
  const uint32_t bits = ((b & 0x80u) << 24) | ((b & 0x7fu) << 20);
  return __uint_as_float(bits) * kPow60 * kPow60;
}

#ifdef SLLM_TRACE
// Development-only per-tile cycle stamps of CTA (0,0,0); never compiled into the product.
__device__ long long g_da_trace[256];
__device__ __forceinline__ void da_mark(int j, int slot) {
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && j < 24) g_da_trace[j * 10 + slot] = clock64();
}
#define DA_TRACE(j, slot) da_mark(j, slot)
#else
#define DA_TRACE(j, slot)
#endif

static_assert(offsetof(DecodeTcBarriers, sc) % 16 == 0, "cp.async 16-byte destinations");

template <int G>
__global__ void __launch_bounds__(kDaThreads, 2)
decode_attention_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                           const PagedAttnParams p) {
  STEP_TRACE_START(p);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // layout: stages x {K tile, V tile} | Q (16 x 128 B) | 2 x P^T (16 x 128 B) | barriers | tail scratch
  uint8_t* kv_s = smem;
  uint8_t* q_s = smem + kDaStages * 2 * kDaTileBytes;
  uint8_t* p_s = q_s + 2048;
  DecodeTcBarriers* bars = reinterpret_cast<DecodeTcBarriers*>(p_s + 2 * 2048);
  float* m_s = reinterpret_cast<float*>(bars + 1);  // [G]
  float* l_s = m_s + kDaHeadsPad;                   // [G]
  // [G][128] output staging of the tail, aliased onto the first K tile: it is written only after the last
  // PV MMA of this CTA has completed, when no tile is in flight any more.
  float* o_s = reinterpret_cast<float*>(kv_s);
  constexpr uint32_t kTmemCols = 64;  // S buffers at columns 0 and 16, PV buffers at columns 32 and 48

  const int r = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z, splits = gridDim.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = p.seq_index[r];
  const int kv_len = p.kv_lens[r];
  int first = 0;
  if (p.window > 0 && kv_len > p.window) first = kv_len - p.window;
  // Splits cover 128-aligned key ranges starting at the page-aligned beginning of the visible window.
  const int base0 = first & ~(p.page_size - 1);
  const int n = kv_len - base0;
  int chunk = (n + splits - 1) / splits;
  chunk = (chunk + kDaTile - 1) & ~(kDaTile - 1);
  const int begin = base0 + split * chunk;
  int end = begin + chunk;
  if (end > kv_len) end = kv_len;
  const int nt = end > begin ? (end - begin + kDaTile - 1) / kDaTile : 0;
  volatile int* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kDaStages; ++s) {
      mbar_init(&bars->kv_full[s], p.k_scale ? 33 : 1);   // TMA issuer + 32 lanes' scale copies
      mbar_init(&bars->kv_empty[s], 1);
    }
    mbar_init(&bars->s_full[0], 1);
    mbar_init(&bars->s_full[1], 1);
    mbar_init(&bars->p_ready[0], 128);
    mbar_init(&bars->p_ready[1], 128);
    mbar_init(&bars->o_full[0], 1);
    mbar_init(&bars->o_full[1], 1);
    bars->abort_flag = 0;
    bars->is_last = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  // Zero Q and P^T (rows >= G stay zero for the whole kernel).
  for (int i = threadIdx.x; i < 3 * 2048 / 16; i += blockDim.x) reinterpret_cast<uint4*>(q_s)[i] = make_uint4(0, 0, 0, 0);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  // Everything above reads only launch inputs no kernel writes (row -> sequence map, lengths); q and the newest
  // K / V slots come from the kernel before this one.
  pdl_wait();
  if (threadIdx.x == 64) STEP_TRACE_WAITED(p);
  // Dependents may start once this CTA holds its tensor memory: the next GEMM then requests its first weight
  // tiles while this grid drains.
  if (p.early_trigger) pdl_trigger();

  if (warp == 0) {
    // ------------------------------------------------------------ page-walking TMA producer
    // The warp reads 32 block-table entries at a time (one coalesced load, issued a whole batch of
    // tiles ahead of its first use, so a table row that misses the L2 costs no stall); lane i then
    // issues the TMA boxes of page i of the tile with its entry taken from the holder by shuffle.
    const int* bt = p.block_table + static_cast<size_t>(seq) * p.max_blocks;
    const int pages_per_tile = kDaTile / p.page_size;
    const int tiles_per_batch = 32 / pages_per_tile;
    const int box_bytes = p.page_size * 128;
    auto load_batch = [&](int b) -> int {
      int pi = begin / p.page_size + b * 32 + lane;
      if (pi >= p.max_blocks) pi = p.max_blocks - 1;   // beyond the table: any valid page, keys are masked
      return __ldg(bt + pi) * p.hkv + kvh;             // (page, head) row of the head-major plane
    };
    int rows_cur = nt > 0 ? load_batch(0) : 0;
    int rows_next = nt > tiles_per_batch ? load_batch(1) : 0;
    int issued = 0;
    for (int j = 0; j < nt; ++j) {
      const int within = j % tiles_per_batch;
      if (within == 0 && j > 0) {
        rows_cur = rows_next;
        if (j + tiles_per_batch < nt) rows_next = load_batch(j / tiles_per_batch + 1);
      }
      const int tok_row = __shfl_sync(0xffffffffu, rows_cur, within * pages_per_tile + (lane < pages_per_tile ? lane : 0));
      const int st = j % kDaStages;
      int ok = 1;
      if (lane == 0) {
        ok = mbar_wait(&bars->kv_empty[st], ((j / kDaStages) & 1) ^ 1, abort_flag, p.status_word,
                       kDaStatusBase + SLLM_DEV_TIMEOUT_SMEM_EMPTY) ? 1 : 0;
        if (!ok && p.status_word && p.status_word[0] == kDaStatusBase + SLLM_DEV_TIMEOUT_SMEM_EMPTY) {
          p.status_word[1] = j; p.status_word[2] = nt; p.status_word[3] = blockIdx.x; p.status_word[4] = blockIdx.y;
          p.status_word[5] = kv_len; p.status_word[6] = begin;
        }
        if (ok) mbar_expect_tx(&bars->kv_full[st], 2 * kDaTileBytes);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < pages_per_tile) {
        uint8_t* kd = kv_s + st * 2 * kDaTileBytes + lane * box_bytes;
        tma_load_3d(kd, &tm_k, &bars->kv_full[st], 0, 0, tok_row);
        tma_load_3d(kd + kDaTileBytes, &tm_v, &bars->kv_full[st], 0, 0, tok_row);
      }
      if (p.k_scale) {
        // lane l stages the scales of keys 4l .. 4l+3 (one page: page sizes are multiples of 8)
        const int key0 = lane * 4;
        const size_t slot = static_cast<size_t>(__shfl_sync(0xffffffffu, rows_cur,
                                                            within * pages_per_tile + key0 / p.page_size)) * p.page_size +
                            key0 % p.page_size;
        cp_async_16(&bars->sc[st][0][key0], p.k_scale + slot);
        cp_async_16(&bars->sc[st][1][key0], p.v_scale + slot);
      }
      if (p.k_scale) cp_async_mbar_arrive_noinc(&bars->kv_full[st]);
      issued = j + 1;
    }
    if (lane == 0) {
      int dummy = 0;
      for (int st = 0; st < kDaStages; ++st) {
        const int fills = (issued > st) ? (issued - st + kDaStages - 1) / kDaStages : 0;
        if (fills > 0) mbar_wait(&bars->kv_full[st], (fills - 1) & 1, &dummy, nullptr, 0, 200000000LL);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ S = K.Q^T issuer
    // One thread spends about 160 cycles per tcgen05.mma, so the S and the P.V MMAs of a tile come from two
    // threads in different warps, whose issue overlaps.  Each of them consumes every phase of the barriers
    // it waits on, in order.
    // The softmax warps quantise Q into shared memory first; barrier 2 joins them with this warp.
    if (nt > 0) asm volatile("bar.sync 2, 160;" ::: "memory");
    if (lane == 0 && nt > 0) {
      constexpr uint32_t idesc_s = make_idesc(kFmtE4M3, 128, kDaHeadsPad, 0, 0);
      const uint32_t q_addr = smem_u32(q_s);
      for (int j = 0; j < nt; ++j) {
        const int st = j % kDaStages;
        if (!mbar_wait(&bars->kv_full[st], (j / kDaStages) & 1, abort_flag, p.status_word, kDaStatusBase + SLLM_DEV_TIMEOUT_TMA_FULL))
          break;
        // S buffer j & 1 is free once the softmax warps have read S(j - 2), which they do before p_ready(j - 2)
        if (j >= 2 && !mbar_wait(&bars->p_ready[j & 1], ((j - 2) >> 1) & 1, abort_flag, p.status_word, kDaStatusBase + SLLM_DEV_TIMEOUT_TMEM_EMPTY))
          break;
        tc_fence_after();
        DA_TRACE(j, 6);
        const uint32_t k_addr = smem_u32(kv_s + st * 2 * kDaTileBytes);
#pragma unroll
        for (int k = 0; k < 4; ++k)  // 32 channels per MMA
          umma_f8(tmem_base + (j & 1) * 16, make_smem_desc_sw128(k_addr) + 2 * k, make_smem_desc_sw128(q_addr) + 2 * k,
                  idesc_s, k != 0);
        tc_commit(&bars->s_full[j & 1]);
        DA_TRACE(j, 8);
      }
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------ O = P.V issuer
    if (lane == 0 && nt > 0) {
      constexpr uint32_t idesc_pv = make_idesc(kFmtE4M3, 128, kDaHeadsPad, 1, 0);
      const uint32_t p_addr = smem_u32(p_s);
      for (int j = 0; j < nt; ++j) {
        const int st = j % kDaStages;
        // this thread's own view of the tile's TMA writes; the phase completed before S(j) was issued
        if (!mbar_wait(&bars->kv_full[st], (j / kDaStages) & 1, abort_flag, p.status_word, kDaStatusBase + SLLM_DEV_TIMEOUT_TMA_FULL))
          break;
        if (!mbar_wait(&bars->p_ready[j & 1], (j >> 1) & 1, abort_flag, p.status_word, kDaStatusBase + SLLM_DEV_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        DA_TRACE(j, 7);
        const uint32_t v_addr = smem_u32(kv_s + st * 2 * kDaTileBytes + kDaTileBytes);
#pragma unroll
        for (int k = 0; k < 4; ++k)  // 32 keys per MMA
          umma_f8(tmem_base + 32 + (j & 1) * 16, make_smem_desc_sw128_mn8(v_addr + k * 4096),
                  make_smem_desc_sw128(p_addr + (j & 1) * 2048) + 2 * k, idesc_pv, k != 0);
        tc_commit(&bars->o_full[j & 1]);
        // the K half of the stage was last read by S(j), which completed before p_ready(j) could be reached
        tc_commit(&bars->kv_empty[st]);
        DA_TRACE(j, 9);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / output (128 threads)
    const int qd = warp & 3;
    const int t = qd * 32 + lane;   // key index inside a tile, and channel index for the output phase
    const int tid = t;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
    const float log2e = 1.4426950408889634f;

    // ---- quantise Q: thread t holds channel t of every head of the group
    float qv[G], qsc[G];
#pragma unroll
    for (int g = 0; g < G; ++g)
      qv[g] = __bfloat162float(p.q[static_cast<size_t>(r) * p.q_ld + (kvh * G + g) * 128 + t]);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float a = fabsf(qv[g]);
      if (!(a == a) || a > 3.0e38f) a = 0.f;
      a = warp_max_redux(a);
      if (lane == 0) bars->red[1][qd][g] = a;
    }
    SyncBar1x128::sync();
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float amax = fmaxf(fmaxf(bars->red[1][0][g], bars->red[1][1][g]), fmaxf(bars->red[1][2][g], bars->red[1][3][g]));
      const float qs = amax > 0.f ? amax / 448.f : 1.f;
      // row g of the K-major tile: 16-byte unit (t / 16) lands at unit index ((t / 16) ^ (g % 8))
      q_s[g * 128 + ((((t >> 4) ^ (g & 7))) << 4) + (t & 15)] = f32_to_e4m3(__fdiv_rn(qv[g], qs));
      qsc[g] = qs * p.sm_scale * log2e;   // scores leave the MMA in log2 units after this factor
    }
    fence_proxy_async_smem();
    if (nt > 0) asm volatile("bar.sync 2, 160;" ::: "memory");

    float m[G], l[G], o[G], alpha_prev[G];
    float of_prev = 0.f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      m[g] = -INFINITY;
      l[g] = 0.f;
      o[g] = 0.f;
      alpha_prev[g] = 0.f;
    }
    bool ok = true;
    for (int j = 0; j < nt && ok; ++j) {
      const int tok = begin + j * kDaTile + t;
      const bool valid = tok < end && tok >= first;
      if (t == 0) DA_TRACE(j, 0);
      ok = mbar_wait(&bars->s_full[j & 1], (j >> 1) & 1, abort_flag, p.status_word, kDaStatusBase + SLLM_DEV_TIMEOUT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      // The tile's scales were staged by the producer warp under kv_full, which completed before the
      // S MMA was issued; observing it here (it returns at once) orders the reads below after the copies.
      float ksc = p.k_static_scale, vsc = p.v_static_scale;
      if (p.k_scale) {
        const int st = j % kDaStages;
        ok = mbar_wait(&bars->kv_full[st], (j / kDaStages) & 1, abort_flag, p.status_word, kDaStatusBase + SLLM_DEV_TIMEOUT_TMA_FULL);
        if (!ok) break;
        ksc = bars->sc[st][0][t];
        vsc = bars->sc[st][1][t];
      }
      uint32_t raw[16];
      if (t == 0) DA_TRACE(j, 1);
      tmem_ld16(lane_addr + (j & 1) * 16, raw);
      tmem_wait_ld();
      if (t == 0) DA_TRACE(j, 2);
      float s[G];
      float red_v[G + 1];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        s[g] = valid ? __uint_as_float(raw[g]) * ksc * qsc[g] : -INFINITY;
        red_v[g] = s[g];
      }
      red_v[G] = valid ? vsc : 0.f;
#pragma unroll
      for (int g = 0; g <= G; ++g) {
        red_v[g] = warp_max_redux(red_v[g]);
        if (lane == 0) bars->red[j & 1][qd][g] = red_v[g];
      }
      SyncBar1x128::sync();
      if (t == 0) DA_TRACE(j, 3);
      float tmax[G + 1];
#pragma unroll
      for (int g = 0; g <= G; ++g)
        tmax[g] = fmaxf(fmaxf(bars->red[j & 1][0][g], bars->red[j & 1][1][g]),
                        fmaxf(bars->red[j & 1][2][g], bars->red[j & 1][3][g]));
      const float vmax = tmax[G] > 0.f ? tmax[G] : 1.f;
      const float vfold = valid ? vsc / vmax * 256.f : 0.f;   // probabilities enter the MMA as p * vsc/vmax * 256
      const float inv_vfold = vfold > 0.f ? __fdividef(1.f, vfold) : 0.f;
      float alpha[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float m_new = fmaxf(m[g], tmax[g]);
        alpha[g] = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - m_new);
        const float pr = (valid && m_new != -INFINITY) ? exp2f(s[g] - m_new) : 0.f;
        const uint8_t p8 = f32_to_e4m3(pr * vfold);
        p_s[(j & 1) * 2048 + g * 128 + ((((t >> 4) ^ (g & 7))) << 4) + (t & 15)] = p8;
        // the normaliser uses the value the tensor core will actually multiply
        const float p_eff = e4m3_to_f32_int(p8) * inv_vfold;
        l[g] = l[g] * alpha[g] + p_eff;
        m[g] = m_new;
      }
      // m[], alpha[] and vmax are identical in all 128 threads (they come from the shared reduction),
      // so the output phase below needs no further exchange.
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bars->p_ready[j & 1]);
      if (t == 0) DA_TRACE(j, 4);
      // ---- fold P.V of the PREVIOUS tile into the output (thread = channel) while the tensor core
      // works on this tile: O <- O * alpha_{j-1} + PV_{j-1} * factor_{j-1}
      if (j > 0) {
        ok = mbar_wait(&bars->o_full[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, p.status_word, kDaStatusBase + SLLM_DEV_TIMEOUT_TMEM_FULL);
        if (!ok) break;
        tc_fence_after();
        tmem_ld16(lane_addr + 32 + ((j - 1) & 1) * 16, raw);
        tmem_wait_ld();
#pragma unroll
        for (int g = 0; g < G; ++g) o[g] = fmaf(o[g], alpha_prev[g], __uint_as_float(raw[g]) * of_prev);
        tc_fence_before();
      }
      if (t == 0) DA_TRACE(j, 5);
#pragma unroll
      for (int g = 0; g < G; ++g) alpha_prev[g] = alpha[g];
      of_prev = vmax / 256.f;
      // red[] and P^T are double buffered by tile parity: a fast thread may already be writing tile j+1's
      // maxima and probabilities while a slow one still reads tile j's maxima and the tensor core still
      // reads P^T(j); buffer j&1 is rewritten for tile j+2 only after this thread's wait on o_full(j)
      // (PV(j) finished) and after the block-wide barrier of tile j+1.
    }
    if (ok && nt > 0) {
      const int j = nt - 1;
      ok = mbar_wait(&bars->o_full[j & 1], (j >> 1) & 1, abort_flag, p.status_word, kDaStatusBase + SLLM_DEV_TIMEOUT_TMEM_FULL);
      if (ok) {
        uint32_t raw[16];
        tc_fence_after();
        tmem_ld16(lane_addr + 32 + (j & 1) * 16, raw);
        tmem_wait_ld();
#pragma unroll
        for (int g = 0; g < G; ++g) o[g] = fmaf(o[g], alpha_prev[g], __uint_as_float(raw[g]) * of_prev);
        tc_fence_before();
      }
    }

    // ---- hand the split's state to the common tail: l is a per-thread partial over keys -> reduce
    SyncBar1x128::sync();   // every thread has read the last tile's maxima before red[0] is reused
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float lg = warp_sum(l[g]);
      if (lane == 0) bars->red[0][qd][g] = lg;
    }
    SyncBar1x128::sync();
    if (t == 0) {
#pragma unroll
      for (int g = 0; g < G; ++g) {
        m_s[g] = (m[g] == -INFINITY) ? -INFINITY : m[g] * 0.6931471805599453f;  // back to natural-log units
        l_s[g] = bars->red[0][0][g] + bars->red[0][1][g] + bars->red[0][2][g] + bars->red[0][3][g];
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) o_s[g * 128 + t] = ok ? o[g] : 0.f;
    SyncBar1x128::sync();
    attention_tail<128, G, 1, SyncBar1x128>(p, r, kvh, split, splits, tid, m_s, l_s, o_s, &bars->is_last, bars->s_red);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  STEP_TRACE_END(p);
}

// [pages*kv_heads, page_size tokens, 128] E4M3 plane (head-major pages); box = {128 channels, page_size tokens, 1}.
static int make_page_tmap(CUtensorMap* out, const void* pages, long long total_tokens, int hkv, int page_size) {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  });
  if (!fn) return SLLM_ERR_DRIVER_ENTRY;
  if (reinterpret_cast<uintptr_t>(pages) & 15) return SLLM_ERR_ALIGNMENT;
  cuuint64_t gdim[3] = {128, static_cast<cuuint64_t>(page_size),
                        static_cast<cuuint64_t>(total_tokens / page_size) * static_cast<cuuint64_t>(hkv)};
  cuuint64_t gstride[2] = {128, static_cast<cuuint64_t>(page_size) * 128};
  cuuint32_t box[3] = {128, static_cast<cuuint32_t>(page_size), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(pages), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? SLLM_OK : SLLM_ERR_CUDA;
}

static std::map<std::tuple<const void*, long long, int, int>, CUtensorMap> g_page_tmaps;
static std::mutex g_page_mu;

static int cached_page_tmap(CUtensorMap* out, const void* pages, long long total_tokens, int hkv, int page_size) {
  auto key = std::make_tuple(pages, total_tokens, hkv, page_size);
  std::lock_guard<std::mutex> g(g_page_mu);
  auto it = g_page_tmaps.find(key);
  if (it != g_page_tmaps.end()) {
    *out = it->second;
    return SLLM_OK;
  }
  int rc = make_page_tmap(out, pages, total_tokens, hkv, page_size);
  if (rc == SLLM_OK) {
    if (g_page_tmaps.size() > 4096) g_page_tmaps.clear();
    g_page_tmaps[key] = *out;
  }
  return rc;
}

template <int G>
static int launch_da(const CUtensorMap& tk, const CUtensorMap& tv, const PagedAttnParams& p, int rows, int splits,
                     cudaStream_t st) {
  const size_t smem = kDaStages * 2 * kDaTileBytes + 3 * 2048 + sizeof(DecodeTcBarriers) +
                      sizeof(float) * (2 * kDaHeadsPad) + 1024;
  static bool cfg = false;
  if (!cfg) {
    if (cudaFuncSetAttribute(decode_attention_tc_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return SLLM_ERR_CUDA;
    cfg = true;
#ifdef SLLM_TRACE
    int per_sm = -1;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_attention_tc_kernel<G>, kDaThreads, smem);
    cudaFuncAttributes fa;
    cudaFuncGetAttributes(&fa, decode_attention_tc_kernel<G>);
    fprintf(stderr, "[trace] decode attention G=%d smem=%zu regs %d: %d CTAs/SM\n", G, smem, fa.numRegs, per_sm);
#endif
  }
  dim3 grid(rows, p.hkv, splits);
  launch_kernel(decode_attention_tc_kernel<G>, dim3(grid), dim3(kDaThreads), smem, st, 1u, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

}  // namespace sllm

using namespace sllm;

// Whether dependent kernels may start while the attention grid drains.  On one GPU that hides the start-up of the
// following GEMM (+1.4 % decode throughput); with tensor parallelism the follower is the GEMM fused with the
// all-reduce, whose early-resident CTAs cost 10 % at two GPUs, so the tensor-parallel context turns it off.
// SLLM_ATTN_EARLY_TRIGGER=0/1 overrides both.
static int g_attn_early = -1;
static int attn_early_trigger() {
  static const int env = [] {
    const char* e = getenv("SLLM_ATTN_EARLY_TRIGGER");
    return e ? (e[0] == '0' ? 0 : 1) : -1;
  }();
  if (env >= 0) return env;
  return g_attn_early < 0 ? 1 : g_attn_early;
}
SLLM_EXPORT void sllm_attention_set_early_trigger(int enabled) { g_attn_early = enabled ? 1 : 0; }

#ifdef SLLM_TRACE
SLLM_EXPORT int sllm_decode_attention_read_trace(long long* out256) {
  return cudaMemcpyFromSymbol(out256, g_da_trace, sizeof(long long) * 256) == cudaSuccess ? 0 : 5;
}
#endif

// Same contract as sllm_paged_attention, restricted to E4M3 pages with per-token scale planes or static
// scales, head_dim 128, page sizes dividing 128 and a GQA group of 1, 2, 4, 8 or 16.
SLLM_EXPORT int sllm_decode_attention_tc(const void* q, int q_ld, const void* k_pages, const void* v_pages,
                                         const float* k_scale, const float* v_scale, float k_static_scale,
                                         float v_static_scale, const int* block_table, int max_blocks,
                                         const int* seq_index, const int* kv_lens, int rows, int hq, int hkv,
                                         int num_pages, int page_size, int window, float sm_scale, void* out_bf16,
                                         void* out_fp8, float* out_scale, int ld_scale, const float* sinks,
                                         int splits, float* ws, long long ws_floats, int* counters, int n_counters,
                                         int* status, void* stream) {
  if (!q || !k_pages || !v_pages || !block_table || !seq_index || !kv_lens || rows <= 0 || hkv <= 0 || hq % hkv)
    return SLLM_ERR_INVALID_ARGUMENT;
  if (!out_bf16 && !(out_fp8 && out_scale)) return SLLM_ERR_INVALID_ARGUMENT;
  if (!k_scale && !(k_static_scale > 0.f && v_static_scale > 0.f)) return SLLM_ERR_INVALID_ARGUMENT;
  if (page_size <= 0 || (kDaTile % page_size) || (page_size & (page_size - 1)) || page_size < 8)
    return SLLM_ERR_UNSUPPORTED_SHAPE;
  if (splits < 1 || splits > 65535 || hkv > 65535 || max_blocks <= 0) return SLLM_ERR_INVALID_ARGUMENT;
  // the scale planes are staged with 16-byte copies
  if (k_scale && ((reinterpret_cast<uintptr_t>(k_scale) | reinterpret_cast<uintptr_t>(v_scale)) & 15)) return SLLM_ERR_ALIGNMENT;
  if (k_scale && !v_scale) return SLLM_ERR_INVALID_ARGUMENT;
  const int g = hq / hkv;
  PagedAttnParams p = {};
  p.q = static_cast<const __nv_bfloat16*>(q); p.q_ld = q_ld;
  p.k_pages = k_pages; p.v_pages = v_pages; p.k_scale = k_scale; p.v_scale = v_scale;
  p.k_static_scale = k_static_scale; p.v_static_scale = v_static_scale;
  p.block_table = block_table; p.max_blocks = max_blocks; p.seq_index = seq_index; p.kv_lens = kv_lens;
  p.hkv = hkv; p.page_size = page_size; p.window = window; p.sm_scale = sm_scale;
  p.out_bf16 = static_cast<__nv_bfloat16*>(out_bf16); p.out_fp8 = static_cast<uint8_t*>(out_fp8);
  p.out_scale = out_scale; p.ld_scale = ld_scale; p.sinks = sinks;
  p.ws_o = nullptr; p.ws_ml = nullptr; p.counters = counters; p.status_word = status;
  p.early_trigger = attn_early_trigger();
  STEP_TRACE_ASSIGN(p, 2);
  if (splits > 1) {
    const long long units = static_cast<long long>(rows) * hkv;
    const long long need = units * splits * (static_cast<long long>(g) * 128 + g * 2);
    if (!ws || !counters || ws_floats < need || n_counters < units) return SLLM_ERR_WORKSPACE_TOO_SMALL;
    p.ws_o = ws;
    p.ws_ml = ws + units * splits * g * 128;
  }
  CUtensorMap tk, tv;
  const long long total_tokens = static_cast<long long>(num_pages) * page_size;
  int rc = cached_page_tmap(&tk, k_pages, total_tokens, hkv, page_size);
  if (rc != SLLM_OK) return rc;
  rc = cached_page_tmap(&tv, v_pages, total_tokens, hkv, page_size);
  if (rc != SLLM_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (g) {
    case 1: return launch_da<1>(tk, tv, p, rows, splits, st);
    case 2: return launch_da<2>(tk, tv, p, rows, splits, st);
    case 4: return launch_da<4>(tk, tv, p, rows, splits, st);
    case 8: return launch_da<8>(tk, tv, p, rows, splits, st);
    case 16: return launch_da<16>(tk, tv, p, rows, splits, st);
    default: return SLLM_ERR_UNSUPPORTED_SHAPE;
  }
}
