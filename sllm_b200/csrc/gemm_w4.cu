// W4A16 GEMM on tcgen05: 4-bit block-scaled weights (MXFP4: E2M1 with an E8M0 scale per 32 elements;
// NVFP4: E2M1 with an E4M3 scale per 16 elements and an FP32 scale per tensor), bf16 activations, fp32
// accumulation in TMEM.  Dense (one weight matrix) or grouped (one matrix per expert, tokens permuted so that
// each expert's rows are contiguous).
//
// The weights stay 4-bit in HBM and in the TMA ring; they become bf16 only inside the SM:
//   warps 0, 21 producers (even / odd K chunks): per 128-element K chunk ONE bulk copy of the weight tile (128 rows x 64 B of codes
//               followed by the 128 x 4 or 8 B of their scales, contiguous in HBM) and two TMA boxes of
//               activations (BN tokens x 64 elements, 128-byte swizzle);
//   warps 2..17 converters, two groups of 256 threads taking alternate K chunks (thread = weight row x half
//               chunk; the conversion is instruction bound, so it is spread over as many warps as fit): unpack
//               eight E2M1 codes per 32-bit word with mask/shift into bf16 pairs whose exponent field holds
//               the code, multiply by (block scale * 2^110) in bf16x2 - exact, the product has at most six
//               significant bits - and store the chunk's two 128-byte-swizzled K-major A tiles (128 rows x 64
//               elements each) into the group's own tile buffers (two per half chunk at decode tile sizes); one generic->async proxy fence per
//               chunk, and while one group sits in its fence the other converts;
//   warps 1, 18..20  MMA issuers, one per (converter group, half chunk): D[128 weight rows, BN tokens] += A * B^T,
//               kind::f16, four K=16 steps per slot, each issuer into its own TMEM accumulator.  One thread
//               spends about 160 cycles per tcgen05.mma whatever its shape, but issuers in different warps
//               overlap, so four of them quadruple the rate at which small-N MMAs enter the tensor core;
//   epilogue    (the first converter group again) sum of the accumulators TMEM -> registers, times the tensor scale and 2^16 (the other half of
//               the exponent offset), optional per-token routing weight, optional residual, bf16 store
//               Y[token, row]; with split-K the partials go through an fp32 workspace and the last CTA of a tile
//               sums them.
// Storage is the "resident" layout the loader writes once: codes of eight consecutive elements e0..e7 sit in
// one 32-bit word as nibbles (e0,e2,e4,e6,e1,e3,e5,e7) from the low end, so that masking the word and the word
// shifted by 4, 8, 12 yields (e0,e1), (e2,e3), ... as ready bf16 pairs; codes and scales are tiled
// [group][row tile][K chunk]{128 rows x 64 B codes, 128 rows x 4|8 B scales}, so that a CTA streams one
// contiguous region of HBM (row-major codes gave 64-byte pieces at a K/2-byte stride, which held the kernel at
// a fifth of the DRAM bandwidth).
//
// Counterparts in the reference: sllm_matmul_nvfp4_block16_packed_dequant_v1 / _prefill_row8_tiled256_v2 (W4A16,
// native/hip/src/matmul_kernel.hip.cpp:830,881), the MXFP4 expert kernels (moe_expert_kernel.hip.cpp).
#include "common.cuh"
#include "api.h"
#include "tmap.h"
#include <cudaTypedefs.h>
#include <cuda_bf16.h>
#include <cstring>
#include <mutex>

namespace sllm {

constexpr int kW4Issuers = 4;          // MMA-issuing threads: (converter group, half chunk)
// warp 0 TMA producer of the even chunks, warp 1 MMA issuer, 16 converter warps, 3 more MMA issuers, warp 21
// TMA producer of the odd chunks
constexpr int kW4Threads = 576 + 32 * (kW4Issuers - 1) + 32;
constexpr int kW4Producer1 = 21;
constexpr int kW4Rows = 128;          // weight rows per CTA (MMA M)
constexpr int kW4Chunk = 128;         // K elements per TMA stage
constexpr int kW4PackedBytes = kW4Rows * (kW4Chunk / 2);   // 8 KB
// converted bf16 A tiles (128 rows x 64 elements = 16 KB each): one per (converter group, half chunk), doubled for
// the decode tile sizes so that a group converts its next chunk while the MMAs of its previous one still read
__host__ __device__ constexpr int w4_abufs(int bn) { return bn <= 32 ? 2 : 1; }
constexpr int kW4ASlotBytes = kW4Rows * 128;
constexpr int kW4MaxStages = 8;

struct W4Params {
  int n_rows;          // rows per group in the packed / scale arrays (multiple of 128)
  int n_valid;         // output features per group
  int k_chunks;        // K_pad / 128
  int groups;
  int scale_bytes;     // per row per chunk: 4 (MXFP4) or 8 (NVFP4)
  int stages;
  int splits;
  int total_tokens;
  int ldy;
  const uint8_t* wtiles;        // tiled codes + scales, see above
  const float* tensor_scale;    // [groups] or null (= 1)
  const int* tok_off;           // [groups + 1] first permuted token of each group, or null (dense)
  const float* tok_scale;       // [total_tokens] routing weight per permuted token, or null
  const __nv_bfloat16* residual;  // [total_tokens, ldy] or null
  __nv_bfloat16* y;             // [total_tokens, ldy]
  // scatter epilogue: when non-null, permuted token row t is stored at address row_ptr[t] (+ feature) instead of
  // y + t * ldy; the addresses may lie in another GPU's memory (expert-parallel combine: the row goes to its owner)
  const long long* row_ptr;
  float* ws;                    // split-K partials [splits][total_tokens][n_valid]
  int* counters;                // one per (group, row tile, token tile)
  int* status;
};

struct __align__(16) W4Barriers {
  uint64_t full[kW4MaxStages];
  uint64_t empty[kW4MaxStages];
  uint64_t conv_done[2][2][2];   // per (converter group, half chunk, buffer): the A tile is written
  uint64_t a_empty[2][2][2];     // per (converter group, half chunk, buffer): the MMAs that read it have completed
  uint64_t acc_full;          // every issuer has committed its last MMA
  uint32_t tmem_base;
  int abort_flag;
  int is_last;
};

__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Factor for one scale block as a bf16 pair: block scale * 2^110 (the remaining 2^16 of the 2^126 that turns an
// exponent field holding the E2M1 code into its value is applied in fp32 in the epilogue).
template <int kFmt>
__device__ __forceinline__ uint32_t block_factor(uint32_t code) {
  uint32_t bits;
  if (kFmt == 0) {
    // E8M0: 2^(code - 127) * 2^110 = 2^(code - 17), i.e. bf16 exponent field code + 110 (1..254 for the codes
    // 0..144 the loader admits; larger scales, above 2^17, are rejected when the weights are repacked).
    int e = static_cast<int>(code) + 110;
    bits = e > 0 ? static_cast<uint32_t>(e) << 7 : 0u;
  } else {
    // E4M3FN scale (never negative in this format's use): value * 2^110, exact in bf16 (3 mantissa bits).
    const uint32_t f = ((code & 0x7fu) << 20);                       // value * 2^-120 as fp32 bits
    const float val = __uint_as_float(f) * 0x1p+115f * 0x1p+115f;   // * 2^230 -> value * 2^110
    bits = __float_as_uint(val) >> 16;                               // three mantissa bits: the cut is exact
  }
  return bits | (bits << 16);
}

#ifdef SLLM_TRACE
__device__ long long g_w4_trace[1024];
__device__ __forceinline__ void w4_mark(int i, int slot) {
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && i < 64) g_w4_trace[i * 10 + slot] = clock64();
}
#define W4_TRACE(i, slot) w4_mark(i, slot)
#else
#define W4_TRACE(i, slot)
#endif

template <int BN, int kFmt>
__global__ void __launch_bounds__(kW4Threads, 1)
gemm_w4_kernel(const __grid_constant__ CUtensorMap tm_x, const W4Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kBBytes = 2 * BN * 128;                    // two 64-element sub-blocks of BN tokens
  constexpr int kScaleTile = kW4Rows * 8;                  // room for the larger (NVFP4) scale tile
  constexpr int kStageBytes = kW4PackedBytes + kScaleTile + kBBytes;
  static_assert(kStageBytes % 1024 == 0, "stage alignment");
  constexpr int kABufs = w4_abufs(BN);
  uint8_t* a_ring = smem;                                   // [group][half][buffer] x 16 KB
  uint8_t* stages = smem + 4 * kABufs * kW4ASlotBytes;
  W4Barriers* bars = reinterpret_cast<W4Barriers*>(stages + p.stages * kStageBytes);
  // one accumulator per issuer; the epilogue adds them up
  constexpr uint32_t kTmemCols = kW4Issuers * BN < 32 ? 32 : kW4Issuers * BN;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_tile = blockIdx.x, g = blockIdx.y;
  if (p.tok_off) pdl_wait();      // the group offsets come from the routing kernels just before this one
  const int tt = blockIdx.z / p.splits, split = blockIdx.z % p.splits;
  const int t_begin = (p.tok_off ? p.tok_off[g] : 0) + tt * BN;
  const int t_end_g = p.tok_off ? p.tok_off[g + 1] : p.total_tokens;
  const int count = min(BN, t_end_g - t_begin);
  if (count <= 0) return;                                   // uniform: an expert without tokens reads nothing
  const int per = (p.k_chunks + p.splits - 1) / p.splits;
  const int c0 = split * per;
  const int nk = max(0, min(per, p.k_chunks - c0));
  volatile int* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 258);                      // 256 converter threads + the two issuers' commits
    }
    for (int a = 0; a < 2; ++a)
      for (int b = 0; b < 2; ++b)
        for (int c = 0; c < 2; ++c) {
          mbar_init(&bars->conv_done[a][b][c], 128);
          mbar_init(&bars->a_empty[a][b][c], 1);
        }
    mbar_init(&bars->acc_full, kW4Issuers);
    bars->abort_flag = 0;
    bars->is_last = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  const size_t tile0 = (static_cast<size_t>(g) * (p.n_rows / kW4Rows) + row_tile) * p.k_chunks;
  const uint32_t tile_bytes = kW4PackedBytes + kW4Rows * p.scale_bytes;

  if (warp == 0 || warp == kW4Producer1) {
    // ------------------------------------------------------------ TMA producers
    // The converters keep the instruction issue slots busy, and one producer thread competing with them needed
    // about as long per chunk as the chunk takes to convert, so it never got ahead of the consumers; each
    // converter group therefore has its own producer (the ring has an even number of stages, so a stage always
    // carries chunks of one group).
    if (lane == 0) {
      const int pg = warp == 0 ? 0 : 1;
      int issued_end = 0;
      // the weights are constant: the first ring of weight tiles is requested before waiting for the
      // previous kernel, the activations after it
      const int pre = nk < p.stages ? nk : p.stages;
      auto load_w = [&](int i, int s) {
        bulk_load_1d(stages + s * kStageBytes, p.wtiles + (tile0 + c0 + i) * tile_bytes, tile_bytes, &bars->full[s]);
      };
      auto load_x = [&](int i, int s) {
        uint8_t* st = stages + s * kStageBytes + kW4PackedBytes + kScaleTile;
        tma_load_2d(st, &tm_x, &bars->full[s], (c0 + i) * kW4Chunk, t_begin);
        tma_load_2d(st + BN * 128, &tm_x, &bars->full[s], (c0 + i) * kW4Chunk + 64, t_begin);
      };
      const uint32_t tx = tile_bytes + kBBytes;
      for (int i = pg; i < pre; i += 2) {
        mbar_expect_tx(&bars->full[i], tx);
        load_w(i, i);
      }
      pdl_wait();
      for (int i = pg; i < pre; i += 2) {
        load_x(i, i);
        issued_end = i + 1;
      }
      for (int i = pre + ((pre & 1) != pg ? 1 : 0); i < nk; i += 2) {
        const int s = i % p.stages;
        if (!mbar_wait(&bars->empty[s], ((i / p.stages) & 1) ^ 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_SMEM_EMPTY)) break;
        W4_TRACE(i, 0);
        mbar_expect_tx(&bars->full[s], tx);
        load_w(i, s);
        load_x(i, s);
        W4_TRACE(i, 1);
        issued_end = i + 1;
      }
      if (pg == 0) pdl_trigger();
      // every copy this thread started must have landed before the CTA may exit
      for (int s = pg; s < p.stages; s += 2) {
        const int fills = (issued_end > s) ? (issued_end - s + p.stages - 1) / p.stages : 0;
        if (fills > 0) {
          int dummy = 0;
          mbar_wait(&bars->full[s], (fills - 1) & 1, &dummy, p.status, SLLM_DEV_TIMEOUT_DRAIN, 200000000LL);
        }
      }
    }
  } else if (warp == 1 || warp >= 18) {   // (warp 21 took the producer branch above)
    // ------------------------------------------------------------ MMA issuers
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(kFmtBf16, kW4Rows, BN < 16 ? 16 : BN);
      const int iw = warp == 1 ? 0 : warp - 17;   // 0..3
      const int grp = iw >> 1, sub = iw & 1;
      const uint32_t d = tmem_base + iw * BN;
      bool ok = true;
      for (int i = grp; ok && i < nk; i += 2) {
        const int s = i % p.stages;
        ok = mbar_wait(&bars->full[s], (i / p.stages) & 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMA_FULL);
        if (!ok) break;
        const uint32_t b_addr = smem_u32(stages + s * kStageBytes + kW4PackedBytes + kScaleTile);
        const int t = i >> 1;                       // the group's chunk counter
        const int ab = t % kABufs;
        ok = mbar_wait(&bars->conv_done[grp][sub][ab], (t / kABufs) & 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        if (sub == 0) W4_TRACE(i, 2);
        const uint64_t adesc = make_smem_desc_sw128(smem_u32(a_ring + ((grp * 2 + sub) * kABufs + ab) * kW4ASlotBytes));
        const uint64_t bdesc = make_smem_desc_sw128(b_addr + sub * BN * 128);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f16(d, adesc + 2 * k, bdesc + 2 * k, idesc, (i > grp) || (k > 0));
        tc_commit(&bars->a_empty[grp][sub][ab]);
        if (sub == 0) W4_TRACE(i, 3);
        tc_commit(&bars->empty[s]);
      }
      // an issuer without chunks (nk == 1) has nothing in flight: the commit arrives at once
      if (ok) tc_commit(&bars->acc_full);
    }
  } else {
    // ------------------------------------------------------------ converters, then epilogue (128 threads)
    const int q = warp & 3;
    const int r = q * 32 + lane;                 // weight row of the tile, TMEM lane
    const int grp = (warp - 2) >> 3;             // converter group: chunks i with (i & 1) == grp (warps 2..17 only)
    const int sub = ((warp - 2) >> 2) & 1;       // which 64-element half of the chunk this thread converts
    bool ok = true;
    // running stage index and phase (a division per chunk in 512 threads is worth avoiding: the converters are
    // bound by instruction issue); grp < stages and the ring is even, so s keeps the group's parity
    int s = grp;
    uint32_t full_ph = 0;
    for (int i = grp; ok && i < nk; i += 2, s += 2) {
      if (s >= p.stages) {
        s -= p.stages;
        full_ph ^= 1;
      }
      ok = mbar_wait(&bars->full[s], full_ph, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMA_FULL);
      if (!ok) break;
      if (r == 0 && sub == 0) W4_TRACE(i, 4);
      const uint8_t* st = stages + s * kStageBytes;
      // this row's scales of the chunk: 4 bytes (one per 32 elements) or 8 bytes (one per 16)
      uint32_t sc_lo = 0, sc_hi = 0;
      if (kFmt == 0) {
        sc_lo = *reinterpret_cast<const uint32_t*>(st + kW4PackedBytes + r * 4);
      } else {
        const uint2 v = *reinterpret_cast<const uint2*>(st + kW4PackedBytes + r * 8);
        sc_lo = v.x;
        sc_hi = v.y;
      }
      uint4 pk[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) pk[j] = *reinterpret_cast<const uint4*>(st + r * 64 + sub * 32 + j * 16);
      // the buffer is free once the MMAs of the chunk that used it last have completed
      const int t = i >> 1, ab = t % kABufs;
      ok = mbar_wait(&bars->a_empty[grp][sub][ab], ((t / kABufs) & 1) ^ 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_SMEM_EMPTY);
      if (!ok) break;
      if (r == 0 && sub == 0) W4_TRACE(i, 5);
      {
        const uint32_t words[8] = {pk[0].x, pk[0].y, pk[0].z, pk[0].w, pk[1].x, pk[1].y, pk[1].z, pk[1].w};
        uint8_t* dst_row = a_ring + ((grp * 2 + sub) * kABufs + ab) * kW4ASlotBytes + r * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {            // word c = elements 8c .. 8c+7 of the 64-element sub-block
          uint32_t code;
          if (kFmt == 0) {
            code = (sc_lo >> (8 * (sub * 2 + c / 4))) & 0xffu;              // block of 32 = 4 words
          } else {
            code = ((sub ? sc_hi : sc_lo) >> (8 * (c / 2))) & 0xffu;        // block of 16 = 2 words
          }
          const uint32_t f = block_factor<kFmt>(code);
          const uint32_t w = words[c];
          uint4 out;
          uint32_t* o = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
          for (int pr = 0; pr < 4; ++pr) {
            const uint32_t x = w >> (4 * pr);
            const uint32_t bits = ((x & 0x00070007u) << 6) | ((x & 0x00080008u) << 12);
            o[pr] = bf16x2_mul(bits, f);
          }
          *reinterpret_cast<uint4*>(dst_row + ((c ^ (r & 7)) << 4)) = out;
        }
      }
      if (r == 0 && sub == 0) W4_TRACE(i, 6);
      fence_proxy_async_smem();
      mbar_arrive(&bars->conv_done[grp][sub][ab]);
      mbar_arrive(&bars->empty[s]);
      if (r == 0 && sub == 0) W4_TRACE(i, 7);
    }
    if (grp == 0 && sub == 0) {
    // ---- epilogue, 16 token columns at a time
    pdl_wait();
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    if (ok && nk > 0) {
      ok = mbar_wait(&bars->acc_full, 0, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMEM_FULL);
      if (ok) tc_fence_after();
    }
    const int out_row = row_tile * kW4Rows + r;            // feature index inside the group
    const bool row_ok = out_row < p.n_valid;
    const float ts = (p.tensor_scale ? p.tensor_scale[g] : 1.f) * 65536.f;
    auto finalize = [&](int c, float a) {
      const int tok = t_begin + c;
      float v = a * ts;
      if (p.tok_scale) v *= p.tok_scale[tok];
      if (p.residual) v += __bfloat162float(p.residual[static_cast<size_t>(tok) * p.ldy + out_row]);
      __nv_bfloat16* dst = p.row_ptr ? reinterpret_cast<__nv_bfloat16*>(p.row_ptr[tok]) + out_row
                                     : p.y + static_cast<size_t>(tok) * p.ldy + out_row;
      *dst = __float2bfloat16_rn(v);
    };
#pragma unroll 1
    for (int cb = 0; cb < BN / 16; ++cb) {
      if (cb * 16 >= count) break;
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = 0.f;
      if (ok && nk > 0) {
#pragma unroll
        for (int a = 0; a < kW4Issuers; ++a) {
          if ((a >> 1) >= nk) continue;          // that issuer had no chunk: its accumulator was never written
          uint32_t t[16];
          tmem_ld16(lane_addr + a * BN + cb * 16, t);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] += __uint_as_float(t[j]);
        }
      }
      if (row_ok) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int c = cb * 16 + j;
          if (c < count) {
            // split-K partials are [split][token][feature]; the last CTA of the tile sums them in split order
            if (p.splits > 1)
              p.ws[(static_cast<size_t>(split) * p.total_tokens + t_begin + c) * p.n_valid + out_row] = v[j];
            else
              finalize(c, v[j]);
          }
        }
      }
    }
    tc_fence_before();
    if (p.splits > 1) {
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const int tile_id = (g * gridDim.x + row_tile) * (gridDim.z / p.splits) + tt;
      if (threadIdx.x == 64) {
        const int prev = atomicAdd(&p.counters[tile_id], 1);
        bars->is_last = (prev == p.splits - 1);
        if (prev == p.splits - 1) p.counters[tile_id] = 0;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (bars->is_last != 0) {
        __threadfence();
        if (row_ok)
          for (int c = 0; c < count; ++c) {
            float sum = 0.f;
            for (int sp = 0; sp < p.splits; ++sp)
              sum += __ldcg(&p.ws[(static_cast<size_t>(sp) * p.total_tokens + t_begin + c) * p.n_valid + out_row]);
            finalize(c, sum);
          }
      }
    }
    }   // first 128 converter threads = epilogue
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int BN, int kFmt>
static int launch_w4(const CUtensorMap& tx, W4Params& p, dim3 grid, cudaStream_t st) {
  constexpr int kStageBytes = kW4PackedBytes + kW4Rows * 8 + 2 * BN * 128;
  const int fixed = 4 * w4_abufs(BN) * kW4ASlotBytes + static_cast<int>(sizeof(W4Barriers)) + 1024;
  int stages = (227 * 1024 - fixed) / kStageBytes;
  if (stages > kW4MaxStages) stages = kW4MaxStages;
  if (stages > p.stages && p.stages >= 2) stages = p.stages;
  // an even ring keeps every stage with the same converter group and issuers: a parity wait is only sound
  // when the waiter has itself seen the barrier's previous phase complete (loads may land out of order)
  stages &= ~1;
  if (stages < 2) return SLLM_ERR_UNSUPPORTED_SHAPE;
  p.stages = stages;
  const size_t smem = static_cast<size_t>(fixed) + static_cast<size_t>(stages) * kStageBytes;
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(gemm_w4_kernel<BN, kFmt>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return SLLM_ERR_CUDA;
    configured = smem;
  }
  cudaError_t e = launch_kernel(gemm_w4_kernel<BN, kFmt>, grid, dim3(kW4Threads), smem, st, 1u, tx, p);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

}  // namespace sllm

using namespace sllm;

#ifdef SLLM_TRACE
SLLM_EXPORT int sllm_gemm_w4_read_trace(long long* out1024) {
  return cudaMemcpyFromSymbol(out1024, g_w4_trace, sizeof(long long) * 1024) == cudaSuccess ? 0 : 5;
}
#endif

// wtiles: the tiled resident weights (codes + scales, see the top of the file);
// x: bf16 [total_tokens, k] with row stride ldx elements (columns k .. k_pad read as zero); y: bf16 [total_tokens, ldy].
// fmt 0 = MXFP4, 1 = NVFP4.  bn in {16, 32, 64, 128}.  max_group_tokens bounds the tokens of any group
// (dense: total_tokens).  Workspace: splits * total_tokens * n_valid floats and one counter per tile when splits > 1.
static int gemm_w4_impl(const void* wtiles, const float* tensor_scale, const void* x, void* y,
                        const void* residual, const int* tok_off, const float* tok_scale, int fmt, int groups,
                        int n_rows, int n_valid, int k_pad, int k, int ldx, int total_tokens, int max_group_tokens,
                        int ldy, int bn,
                        int splits, int stages, float* ws, long long ws_floats, int* counters, int n_counters,
                        int* status, void* stream, const long long* row_ptr) {
  if (!wtiles || !x || (!y && !row_ptr) || groups <= 0 || n_rows <= 0 || (n_rows % kW4Rows) || n_valid <= 0 ||
      n_valid > n_rows || k_pad <= 0 || (k_pad % kW4Chunk) || k <= 0 || k > k_pad || ldx < k || (ldx % 8) ||
      total_tokens <= 0 || max_group_tokens <= 0)
    return SLLM_ERR_INVALID_ARGUMENT;
  if (fmt != 0 && fmt != 1) return SLLM_ERR_INVALID_ARGUMENT;
  if (groups > 1 && !tok_off) return SLLM_ERR_INVALID_ARGUMENT;
  if (bn != 16 && bn != 32 && bn != 64 && bn != 128) return SLLM_ERR_UNSUPPORTED_SHAPE;
  if (reinterpret_cast<uintptr_t>(wtiles) & 15) return SLLM_ERR_ALIGNMENT;
  const int k_chunks = k_pad / kW4Chunk;
  if (splits < 1) splits = 1;
  if (splits > k_chunks) splits = k_chunks;
  const int row_tiles = n_rows / kW4Rows;
  const int tok_tiles = (max_group_tokens + bn - 1) / bn;
  if (static_cast<long long>(tok_tiles) * splits > 65535 || groups > 65535) return SLLM_ERR_UNSUPPORTED_SHAPE;
  if (splits > 1) {
    if (!ws || !counters) return SLLM_ERR_INVALID_ARGUMENT;
    if (ws_floats < static_cast<long long>(splits) * total_tokens * n_valid ||
        n_counters < groups * row_tiles * tok_tiles)
      return SLLM_ERR_WORKSPACE_TOO_SMALL;
  }
  CUtensorMap tx;
  int rc = cached_kmajor_tmap(&tx, x, 2, total_tokens, k, static_cast<long long>(ldx) * 2, bn);
  if (rc != SLLM_OK) return rc;
  W4Params p;
  memset(&p, 0, sizeof(p));
  p.n_rows = n_rows; p.n_valid = n_valid; p.k_chunks = k_chunks; p.groups = groups;
  p.scale_bytes = fmt == 0 ? 4 : 8; p.stages = stages; p.splits = splits; p.total_tokens = total_tokens; p.ldy = ldy;
  p.wtiles = static_cast<const uint8_t*>(wtiles); p.tensor_scale = tensor_scale; p.tok_off = tok_off;
  p.tok_scale = tok_scale; p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.y = static_cast<__nv_bfloat16*>(y); p.ws = ws; p.counters = counters; p.status = status;
  p.row_ptr = row_ptr;
  dim3 grid(row_tiles, groups, tok_tiles * splits);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define SLLM_W4_CASE(BNV)                                                                      \
  case BNV:                                                                                    \
    return fmt == 0 ? launch_w4<BNV, 0>(tx, p, grid, st) : launch_w4<BNV, 1>(tx, p, grid, st);
  switch (bn) {
    SLLM_W4_CASE(16)
    SLLM_W4_CASE(32)
    SLLM_W4_CASE(64)
    SLLM_W4_CASE(128)
  }
#undef SLLM_W4_CASE
  return SLLM_ERR_UNSUPPORTED_SHAPE;
}

SLLM_EXPORT int sllm_gemm_w4(const void* wtiles, const float* tensor_scale, const void* x, void* y,
                             const void* residual, const int* tok_off, const float* tok_scale, int fmt, int groups,
                             int n_rows, int n_valid, int k_pad, int k, int ldx, int total_tokens, int max_group_tokens,
                             int ldy, int bn,
                             int splits, int stages, float* ws, long long ws_floats, int* counters, int n_counters,
                             int* status, void* stream) {
  return gemm_w4_impl(wtiles, tensor_scale, x, y, residual, tok_off, tok_scale, fmt, groups, n_rows, n_valid, k_pad, k, ldx,
                      total_tokens, max_group_tokens, ldy, bn, splits, stages, ws, ws_floats, counters, n_counters, status,
                      stream, nullptr);
}

// The same with a scatter epilogue: row t of the result is stored at row_ptr[t] (a device array of bf16 row addresses,
// 2-byte aligned, possibly in peer memory) instead of y + t * ldy; no residual.
SLLM_EXPORT int sllm_gemm_w4_scatter(const void* wtiles, const float* tensor_scale, const void* x, const long long* row_ptr,
                                     const int* tok_off, const float* tok_scale, int fmt, int groups, int n_rows,
                                     int n_valid, int k_pad, int k, int ldx, int total_tokens, int max_group_tokens, int bn,
                                     int splits, int stages, float* ws, long long ws_floats, int* counters, int n_counters,
                                     int* status, void* stream) {
  if (!row_ptr) return SLLM_ERR_INVALID_ARGUMENT;
  return gemm_w4_impl(wtiles, tensor_scale, x, nullptr, nullptr, tok_off, tok_scale, fmt, groups, n_rows, n_valid, k_pad, k,
                      ldx, total_tokens, max_group_tokens, n_valid, bn, splits, stages, ws, ws_floats, counters, n_counters,
                      status, stream, row_ptr);
}
