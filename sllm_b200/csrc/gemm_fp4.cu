// W4A4 GEMM on the block-scaled tensor-core path: 4-bit weights AND 4-bit activations go to tcgen05.mma as E2M1
// codes, their block scales ride in TMEM and are applied by the tensor core itself
//   NVFP4: kind::mxf4nvf4.block_scale.block16, one UE4M3 scale per 16 elements (+ an FP32 scale per weight tensor and
//          per activation row, applied in the epilogue)
//   MXFP4: kind::mxf4.block_scale.block32, one UE8M0 scale per 32 elements
// so no CUDA core touches a weight: the W4A16 kernel (gemm_w4.cu) spends its time unpacking E2M1 into bf16 with integer
// instructions and tops out at about a third of the copy bandwidth; here a weight tile goes HBM -> shared memory ->
// tensor core as the bulk copy delivered it.
//
// Swap-AB like the other decode GEMMs: D[128 weight rows, BN tokens] += A[128, 64] * B[BN, 64]^T per instruction
// (K = 64 four-bit elements = 32 bytes), fp32 accumulators in TMEM.
//   warp 0      producer: per 256-element K block ONE bulk copy of the weight tile - the 128-byte-swizzled image of
//               128 rows x 128 B of codes followed by its scale "atoms" - and one TMA box of the activations' codes
//               (BN tokens x 128 B, 128-byte swizzle);
//   warps 1-3, 8  MMA issuers (K blocks round robin, each into its own accumulator and its own scale columns):
//               tcgen05.cp of the block's scale atoms into TMEM, then four MMAs.  One thread needs about 150 ns per
//               tcgen05 instruction and a block-16 K block takes eleven of them, so the issue work is spread over four
//               threads.  tcgen05.cp and tcgen05.mma of one thread execute in issue order, so an issuer reuses its scale
//               columns for its next K block without a barrier;
//   warps 4..7  (tiles of more than 32 tokens only: first stage the activations' scales of the CTA's K range into
//               shared memory in atom order), then the epilogue: TMEM -> registers, times weight-tensor scale x activation-row scale (x routing weight),
//               (+ residual), bf16 store Y[token, row]; split-K partials go through an fp32 workspace.
// A scale atom is 512 bytes = 32 rows x 16 B, the 16 B of row r holding 4 scale bytes each of matrix rows r, r + 32,
// r + 64, r + 96: the form tcgen05.cp.32x128b.warpx4 copies into four TMEM columns, after which row m's four scales
// sit in lane m % 32 (replicated to all four lane quarters), column m / 32.  An MMA that needs fewer than four scales
// per row (block 32: two) names the byte it starts at through the scale-factor id of the instruction descriptor.
// Activation scales are stored per token in 8-byte units, [4 scale bytes | 4 unused], so that a K block of a token is
// 32 bytes (block 16) or 16 bytes (block 32).  With at most 32 tokens per tile only column 0 of an activation atom
// would be read, so the decode tiles use the token-major rows themselves as atoms: a TMA box of {16 B, 32 tokens} of the
// scale matrix lands in the stage as an atom whose columns 0 and 2 hold the scales of two consecutive MMAs (the unused
// bytes fall into columns 1 and 3).  A scale address handed to tcgen05.mma must name an even column: an odd one raises
// "misaligned address".
//
// Counterparts in the reference: activation quantisers sllm_matmul_bf16_to_nvfp4_block16_v1 / bf16_to_mxfp4_block32_even
// (native/hip/src/matmul_kernel.hip.cpp:343,457) and the W4A4 dot kernels (:396, :562, :574), scalar there.
#include "common.cuh"
#include "api.h"
#include "tmap.h"
#include <cudaTypedefs.h>
#include <cuda_bf16.h>
#include <cstring>

namespace sllm {

constexpr int kF4Rows = 128;                    // weight rows per CTA (MMA M)
constexpr int kF4KBlock = 256;                  // K elements per stage = one 128-byte row
constexpr int kF4ABytes = kF4Rows * 128;        // 16 KB of codes per weight tile
constexpr int kF4AtomBytes = 512;
constexpr int kF4MaxAtoms = 4;                  // scale atoms per K block: 4 (block 16) or 2 (block 32)
constexpr int kF4MaxKb = 8;                     // K blocks per CTA; split-K keeps a CTA's share within it
constexpr int kF4Threads = 288;                 // warp 0 producer, warps 1-3 and 8 issuers, warps 4-7 epilogue
constexpr int kF4MaxStages = 8;
__host__ __device__ constexpr int f4_issuers(int bn) { return bn <= 64 ? 4 : 2; }   // bounded by the 512 TMEM columns

struct F4Params {
  int n_rows, n_valid, k_blocks, groups;
  int atoms;                 // scale atoms per K block (4: NVFP4, 2: MXFP4)
  int stages, splits, total_tokens, ldy;
  int sf_ld;                 // bytes per token row of xsf (8 per four scales: see the top)
  const uint8_t* wtiles;     // [group][row tile][K block]{16 KB code image | atoms x 512 B}
  const float* tensor_scale; // [groups] or null
  const int* tok_off;        // [groups + 1] or null (dense)
  const float* tok_scale;    // [total_tokens] or null
  const float* x_outer;      // [total_tokens] activation row scales or null (= 1)
  const uint8_t* xsf;        // [total_tokens, sf_ld] activation block scales, token-major
  const __nv_bfloat16* residual;
  __nv_bfloat16* y;
  const long long* row_ptr;  // scatter epilogue (see gemm_w4.cu)
  float* ws;
  int* counters;
  int* status;
};

struct __align__(16) F4Barriers {
  uint64_t full[kF4MaxStages];
  uint64_t empty[kF4MaxStages];
  uint64_t sfb_ready;
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
  int is_last;
  float tok_mult[128];        // per token of the tile: weight-tensor scale x activation-row scale x routing weight
  long long tok_ptr[128];     // per token: destination row address of the scatter epilogue
};

__device__ __forceinline__ void f4_bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// K-major descriptor without swizzle for one scale atom: rows of 16 bytes, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc_atom(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(16 >> 4) << 16;      // LBO (one 16-byte column only: unused)
  d |= static_cast<uint64_t>(128 >> 4) << 32;     // SBO
  d |= static_cast<uint64_t>(1) << 46;            // version
  return d;                                       // layout type 0: no swizzle
}

__device__ __forceinline__ void tmem_cp_atom(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// Block-scaled instruction descriptor: E2M1 x E2M1, K-major, fp32 accumulate.
//   [4,6) B scale id   [7,10) A format (1 = E2M1)   [10,13) B format   [17,23) N >> 3   [23] scale format (0 UE4M3,
//   1 UE8M0)   [24,29) M >> 4   [29,31) A scale id
__host__ __device__ constexpr uint32_t make_idesc_f4(uint32_t n, uint32_t ue8m0) {
  return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | (ue8m0 << 23) | ((128u >> 4) << 24);
}

template <int kBlock>
__device__ __forceinline__ void umma_f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa,
                                        uint32_t sfb, uint32_t accumulate) {
  if (kBlock == 16) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  }
}

// kBlock: elements per scale (16: NVFP4, 32: MXFP4).
template <int BN, int kBlock>
__global__ void __launch_bounds__(kF4Threads, 1)
gemm_fp4_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_sf, const F4Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kAtoms = kBlock == 16 ? 4 : 2;
  constexpr int kBBytes = BN * 128;
  constexpr bool kTmaSfb = BN <= 32;           // activation scales by TMA straight into the stage (see the top)
  constexpr int kSfbBoxes = kBlock == 16 ? 2 : 1;   // 16-byte boxes per token and K block
  constexpr int kSfbStage = kTmaSfb ? 1024 : 0;
  constexpr int kOffB = kF4ABytes + kF4MaxAtoms * kF4AtomBytes;
  constexpr int kOffSfb = kOffB + kBBytes;
  constexpr int kStageBytes = kOffSfb + kSfbStage;
  static_assert(kStageBytes % 1024 == 0, "stage alignment");
  constexpr int kSfbBytes = kTmaSfb ? 0 : kF4MaxKb * kAtoms * kF4AtomBytes;
  // TMEM: one accumulator per issuer, then per issuer (weight scales | activation scales), four columns per atom
  constexpr int kIss = f4_issuers(BN);
  constexpr uint32_t kSfCols = 4 * kAtoms;
  constexpr uint32_t kNeed = kIss * (BN + 2 * kSfCols);
  constexpr uint32_t kTmemCols = kNeed <= 32 ? 32 : kNeed <= 64 ? 64 : kNeed <= 128 ? 128 : kNeed <= 256 ? 256 : 512;
  uint8_t* sfb_region = smem;
  uint8_t* stages = smem + ((kSfbBytes + 1023) & ~1023);
  F4Barriers* bars = reinterpret_cast<F4Barriers*>(stages + p.stages * kStageBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_tile = blockIdx.x, g = blockIdx.y;
  if (p.tok_off) pdl_wait();
  const int tt = blockIdx.z / p.splits, split = blockIdx.z % p.splits;
  const int t_begin = (p.tok_off ? p.tok_off[g] : 0) + tt * BN;
  const int t_end_g = p.tok_off ? p.tok_off[g + 1] : p.total_tokens;
  const int count = min(BN, t_end_g - t_begin);
  if (count <= 0) return;
  const int per = (p.k_blocks + p.splits - 1) / p.splits;      // <= kF4MaxKb, checked on the host
  const int c0 = split * per;
  const int nk = max(0, min(per, p.k_blocks - c0));
  volatile int* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->sfb_ready, 128);
    mbar_init(&bars->acc_full, kIss);
    bars->abort_flag = 0;
    bars->is_last = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_x);
    if (kTmaSfb) tma_prefetch_desc(&tm_sf);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t tile_bytes = kF4ABytes + kAtoms * kF4AtomBytes;
  const size_t tile0 = (static_cast<size_t>(g) * (p.n_rows / kF4Rows) + row_tile) * p.k_blocks + c0;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int issued = 0;
      const int pre = nk < p.stages ? nk : p.stages;
      const uint32_t tx = tile_bytes + kBBytes + (kTmaSfb ? 512u * kSfbBoxes : 0u);
      auto load_x = [&](int i, int s) {
        uint8_t* st = stages + s * kStageBytes;
        tma_load_2d(st + kOffB, &tm_x, &bars->full[s], (c0 + i) * 128, t_begin);
        // the tokens' scale bytes of this K block: 16 per box
        if (kTmaSfb) {
#pragma unroll
          for (int b = 0; b < kSfbBoxes; ++b)
            tma_load_2d(st + kOffSfb + b * kF4AtomBytes, &tm_sf, &bars->full[s], ((c0 + i) * kSfbBoxes + b) * 16, t_begin);
        }
      };
      // weights are constant: their first ring is requested before the dependency wait
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&bars->full[i], tx);
        f4_bulk_load(stages + i * kStageBytes, p.wtiles + (tile0 + i) * tile_bytes, tile_bytes, &bars->full[i]);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i) {
        load_x(i, i);
        issued = i + 1;
      }
      for (int i = pre; i < nk; ++i) {
        const int s = i % p.stages;
        if (!mbar_wait(&bars->empty[s], ((i / p.stages) & 1) ^ 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_SMEM_EMPTY)) break;
        mbar_expect_tx(&bars->full[s], tx);
        f4_bulk_load(stages + s * kStageBytes, p.wtiles + (tile0 + i) * tile_bytes, tile_bytes, &bars->full[s]);
        load_x(i, s);
        issued = i + 1;
      }
      pdl_trigger();
      // every copy this thread started must have landed before the CTA may exit
      for (int s = 0; s < p.stages; ++s) {
        const int fills = (issued > s) ? (issued - s + p.stages - 1) / p.stages : 0;
        if (fills > 0) {
          int dummy = 0;
          mbar_wait(&bars->full[s], (fills - 1) & 1, &dummy, p.status, SLLM_DEV_TIMEOUT_DRAIN, 200000000LL);
        }
      }
    }
  } else if (warp < 4 || warp == 8) {
    // ------------------------------------------------------------ MMA issuers
    // (the number of stages is a multiple of the number of issuers, so a stage always carries K blocks of one issuer:
    // a parity wait is only sound for a waiter that has itself seen the barrier's previous phase complete)
    const int iw = warp < 4 ? warp - 1 : 3;
    if (lane == 0 && iw < kIss) {
      constexpr uint32_t idesc = make_idesc_f4(BN, kBlock == 32 ? 1u : 0u);
      const uint32_t d_tmem = tmem_base + iw * BN;
      const uint32_t sfa_t = tmem_base + kIss * BN + iw * 2 * kSfCols;
      const uint32_t sfb_t = sfa_t + kSfCols;
      bool ok = kTmaSfb || nk <= iw || mbar_wait(&bars->sfb_ready, 0, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMA_FULL);
      for (int i = iw; ok && i < nk; i += kIss) {
        const int s = i % p.stages;
        ok = mbar_wait(&bars->full[s], (i / p.stages) & 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMA_FULL);
        if (!ok) break;
        tc_fence_after();
        const uint32_t st = smem_u32(stages + s * kStageBytes);
#pragma unroll
        for (int a = 0; a < kAtoms; ++a) {
          tmem_cp_atom(sfa_t + 4 * a, make_smem_desc_atom(st + kF4ABytes + a * kF4AtomBytes));
          if (!kTmaSfb)
            tmem_cp_atom(sfb_t + 4 * a, make_smem_desc_atom(smem_u32(sfb_region) + (i * kAtoms + a) * kF4AtomBytes));
        }
        if (kTmaSfb) {
#pragma unroll
          for (int b = 0; b < kSfbBoxes; ++b)
            tmem_cp_atom(sfb_t + 4 * b, make_smem_desc_atom(st + kOffSfb + b * kF4AtomBytes));
        }
        const uint64_t adesc = make_smem_desc_sw128(st);
        const uint64_t bdesc = make_smem_desc_sw128(st + kOffB);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // block 16: MMA j takes atom j whole; block 32: atom j / 2, bytes 2 (j % 2) .. + 1 of each row's four
          const uint32_t col = kBlock == 16 ? 4u * j : 4u * (j >> 1);
          const uint32_t id = kBlock == 16 ? 0u : 2u * (j & 1);
          // decode tiles: the four scale bytes MMA j starts in are the j-th (block 32: (j / 2)-th) 8-byte unit of the
          // token's K block, i.e. column 2 j (2 (j / 2)) of its boxes - always an even column
          const uint32_t colb = kTmaSfb ? (kBlock == 16 ? 2u * j : 2u * (j >> 1)) : col;
          umma_f4<kBlock>(d_tmem, adesc + 2 * j, bdesc + 2 * j, idesc | (id << 29) | (id << 4),
                          (sfa_t + col) | (id << 30), (sfb_t + colb) | (id << 30), (i > iw) || (j > 0));
        }
        tc_commit(&bars->empty[s]);
      }
      // an issuer without K blocks has nothing in flight: its commit arrives at once
      if (ok) tc_commit(&bars->acc_full);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ activation scales, then the epilogue
    const int q = warp & 3;
    const int r = q * 32 + lane;                 // weight row of the tile = TMEM lane
    const int e = threadIdx.x - 128;
    pdl_wait();
    if (!kTmaSfb) {
      // token n's scales of K block i, atom a: the four bytes that open 8-byte unit (c0 + i) kAtoms + a of its row
      for (int w = e; w < nk * kAtoms * BN; w += 128) {
        const int n = w % BN, ia = w / BN;
        uint32_t v = 0;
        if (n < count)
          v = *reinterpret_cast<const uint32_t*>(p.xsf + static_cast<size_t>(t_begin + n) * p.sf_ld +
                                                 (static_cast<size_t>(c0) * kAtoms + ia) * 8);
        *reinterpret_cast<uint32_t*>(sfb_region + ia * kF4AtomBytes + (n & 31) * 16 + (n >> 5) * 4) = v;
      }
      fence_proxy_async_smem();
      mbar_arrive(&bars->sfb_ready);
    }

    bool ok = true;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const int out_row = row_tile * kF4Rows + r;
    const bool row_ok = out_row < p.n_valid;
    // Everything the epilogue reads from memory is fetched while the main loop runs: a load per token inside the
    // store loop costs a memory latency per token (32 dependent residual loads were a third of the o-projection).
    if (e < BN) {
      float m = 0.f;
      long long ptr = 0;
      if (e < count) {
        const int tok = t_begin + e;
        m = p.tensor_scale ? p.tensor_scale[g] : 1.f;
        if (p.x_outer) m *= p.x_outer[tok];
        if (p.tok_scale) m *= p.tok_scale[tok];
        if (p.row_ptr) ptr = p.row_ptr[tok];
      }
      bars->tok_mult[e] = m;
      bars->tok_ptr[e] = ptr;
    }
    constexpr int kResRegs = BN <= 32 ? BN : 1;
    float res[kResRegs];
    const bool res_ready = BN <= 32 && p.residual != nullptr && p.splits == 1;
    if (res_ready) {
#pragma unroll
      for (int c = 0; c < kResRegs; ++c)
        res[c] = (row_ok && c < count) ? __bfloat162float(p.residual[static_cast<size_t>(t_begin + c) * p.ldy + out_row]) : 0.f;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (nk > 0) {
      ok = mbar_wait(&bars->acc_full, 0, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMEM_FULL);
      if (ok) tc_fence_after();
    }
    auto finalize = [&](int c, float a, float resid) {
      const int tok = t_begin + c;
      const float v = a * bars->tok_mult[c] + resid;
      __nv_bfloat16* dst = p.row_ptr ? reinterpret_cast<__nv_bfloat16*>(bars->tok_ptr[c]) + out_row
                                     : p.y + static_cast<size_t>(tok) * p.ldy + out_row;
      *dst = __float2bfloat16_rn(v);
    };
    auto resid_at = [&](int c) {
      return p.residual ? __bfloat162float(p.residual[static_cast<size_t>(t_begin + c) * p.ldy + out_row]) : 0.f;
    };
#pragma unroll
    for (int cb = 0; cb < BN / 16; ++cb) {
      if (cb * 16 >= count) break;
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = 0.f;
      if (ok && nk > 0) {
#pragma unroll
        for (int a = 0; a < kIss; ++a) {
          if (a >= nk) continue;                 // that issuer had no K block: its accumulator was never written
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
            if (p.splits > 1)
              p.ws[(static_cast<size_t>(split) * p.total_tokens + t_begin + c) * p.n_valid + out_row] = v[j];
            else
              finalize(c, v[j], res_ready ? res[c < kResRegs ? c : 0] : resid_at(c));
          }
        }
      }
    }
    tc_fence_before();
    if (p.splits > 1) {
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const int tile_id = (g * gridDim.x + row_tile) * (gridDim.z / p.splits) + tt;
      if (e == 0) {
        const int prev = atomicAdd(&p.counters[tile_id], 1);
        bars->is_last = (prev == p.splits - 1);
        if (prev == p.splits - 1) p.counters[tile_id] = 0;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (bars->is_last != 0) {
        __threadfence();
        if (row_ok) {
          // four tokens at a time so that their loads are in flight together
          for (int cq = 0; cq < count; cq += 4) {
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
            for (int sp = 0; sp < p.splits; ++sp) {
              const float* src = p.ws + (static_cast<size_t>(sp) * p.total_tokens + t_begin + cq) * p.n_valid + out_row;
#pragma unroll
              for (int u = 0; u < 4; ++u)
                if (cq + u < count) sum[u] += __ldcg(src + static_cast<size_t>(u) * p.n_valid);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
              if (cq + u < count) finalize(cq + u, sum[u], resid_at(cq + u));
          }
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

template <int BN, int kBlock>
static int launch_f4(const CUtensorMap& tx, const CUtensorMap& tsf, F4Params& p, dim3 grid, cudaStream_t st) {
  constexpr int kAtoms = kBlock == 16 ? 4 : 2;
  constexpr int kStageBytes = kF4ABytes + kF4MaxAtoms * kF4AtomBytes + BN * 128 + (BN <= 32 ? 1024 : 0);
  constexpr int kSfb = BN <= 32 ? 0 : ((kF4MaxKb * kAtoms * kF4AtomBytes + 1023) & ~1023);
  const int fixed = kSfb + static_cast<int>(sizeof(F4Barriers)) + 1024;
  // An SM's share of the HBM bandwidth (~44 GB/s) needs ~190 KB of copies in flight at the loaded memory latency:
  // two CTAs per SM with four stages each at the decode tile sizes, or, when the launch has no more CTAs than the
  // device has SMs, one CTA with eight stages (a four-stage CTA alone on its SM streamed 22 GB/s, an eight-stage
  // one 40 GB/s).
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      sms = 148;
  }
  const long long ctas = static_cast<long long>(grid.x) * grid.y * grid.z;
  const int budget = (BN <= 32 && ctas > sms) ? 113 * 1024 : 227 * 1024;
  int stages = (budget - fixed) / kStageBytes;
  if (stages > kF4MaxStages) stages = kF4MaxStages;
  stages -= stages % f4_issuers(BN);             // a stage stays with one issuer
  if (stages < 2) return SLLM_ERR_UNSUPPORTED_SHAPE;
  p.stages = stages;
  const size_t smem = static_cast<size_t>(fixed) + static_cast<size_t>(stages) * kStageBytes;
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(gemm_fp4_kernel<BN, kBlock>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return SLLM_ERR_CUDA;
    configured = smem;
  }
  cudaError_t e = launch_kernel(gemm_fp4_kernel<BN, kBlock>, grid, dim3(kF4Threads), smem, st, 1u, tx, tsf, p);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

// ---------------------------------------------------------------- activation quantiser
// One CTA per token row: bf16 [k] -> E2M1 codes (element 2 i in the low nibble of byte i) and one scale byte per
// block (four scale bytes, then four unused ones: scale b sits at byte (b / 4) * 8 + b % 4), zero-filled up to k_pad.  fmt 1 (NVFP4): row scale = amax / (448 * 6) in fp32, block scale UE4M3 of
// (block amax / 6) / row scale; fmt 0 (MXFP4): block scale UE8M0 with the same exponent rule as the weight
// quantiser, row scale 1.  (Reference: native/hip/src/matmul_kernel.hip.cpp:343,457 - a calibrated global scale
// there, the row's own maximum here.)
__device__ __forceinline__ float f4_silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float f4_gelu_tanh(float x) {
  const float c = 0.7978845608028654f;
  return 0.5f * x * (1.f + tanhf(c * (x + 0.044715f * x * x * x)));
}

// Eight consecutive values of the row to quantise.  gated (1 SiLU, 2 GELU-tanh): the row is [gate (k) | up (k)] and the
// value is act(gate) * up with the bf16 roundings of the stand-alone gated-activation kernel (elementwise.cu).
// norm_w: the value is the RMS-normalised element x * inv * weight (weight + 1 with offset_one), rounded to bf16 as the
// stand-alone norm kernel writes it.
__device__ __forceinline__ void f4_load8(const __nv_bfloat16* row, int i, int k, int gated, const __nv_bfloat16* norm_w,
                                         float inv, int offset_one, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(row + i);
  const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
  if (norm_w) {
    const uint4 raww = *reinterpret_cast<const uint4*>(norm_w + i);
    const __nv_bfloat16* wv = reinterpret_cast<const __nv_bfloat16*>(&raww);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float g = offset_one ? 1.f + __bfloat162float(wv[j]) : __bfloat162float(wv[j]);
      v[j] = __bfloat162float(__float2bfloat16_rn(__bfloat162float(h[j]) * inv * g));
    }
  } else if (!gated) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(h[j]);
  } else {
    const uint4 rawu = *reinterpret_cast<const uint4*>(row + k + i);
    const __nv_bfloat16* u = reinterpret_cast<const __nv_bfloat16*>(&rawu);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float g = __bfloat162float(h[j]);
      const float a = gated == 1 ? f4_silu(g) : f4_gelu_tanh(g);
      v[j] = __bfloat162float(__float2bfloat16_rn(__bfloat162float(__float2bfloat16_rn(a)) * __bfloat162float(u[j])));
    }
  }
}

__device__ __forceinline__ void f4_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void f4_st_peer(float* local_ptr, uint32_t cta_rank, float v) {
  uint32_t ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(local_ptr)), "r"(cta_rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(ra), "f"(v) : "memory");
}

// Block reduction (sum or max) of `v`, then the same over the CTAs of the row's cluster: every CTA stores its partial
// into slot `rank` of every peer's exchange array and reads all slots after the cluster barrier (in rank order, so
// the result is the same in every CTA and from run to run).
template <bool kMax>
__device__ __forceinline__ float f4_row_reduce(float v, float* red, float* xch, int rank, int nctas) {
  v = kMax ? warp_max(v) : warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) t = kMax ? fmaxf(t, red[w]) : t + red[w];
  __syncthreads();                                     // red is reused by the next reduction
  if (nctas == 1) return t;
  if (threadIdx.x < nctas) f4_st_peer(&xch[rank], threadIdx.x, t);
  f4_cluster_sync();
  float r = xch[0];
  for (int c = 1; c < nctas; ++c) r = kMax ? fmaxf(r, xch[c]) : r + xch[c];
  return r;
}

// grid (tokens, 1, chunks) with the chunks of a row forming one thread-block cluster: every CTA quantises its share of
// the row's blocks, and the row's statistics (sum of squares for the norm, maximum for the NVFP4 row scale) are reduced
// over the cluster instead of being recomputed by every CTA.
template <int kBlock>
__global__ void __launch_bounds__(256) act_quant_fp4_kernel(const __nv_bfloat16* __restrict__ x, int ldx, int k, int k_pad,
                                                            const int* __restrict__ src_row, const int* __restrict__ n_rows_ptr,
                                                            int gated, const __nv_bfloat16* __restrict__ norm_w, float eps,
                                                            int offset_one, uint8_t* __restrict__ xq,
                                                            uint8_t* __restrict__ xsf, int sf_ld, float* __restrict__ outer) {
  __shared__ float red[8];
  __shared__ float xch[2][8];
  pdl_wait();
  const int t = blockIdx.x;
  const int rank = blockIdx.z, nctas = gridDim.z;
  // rows past the routed ones: their source index is not defined.  (Uniform over the row's cluster: no CTA is left
  // waiting at a cluster barrier.)
  if (n_rows_ptr && t >= *n_rows_ptr) return;
  const __nv_bfloat16* row = x + static_cast<size_t>(src_row ? src_row[t] : t) * ldx;
  const int blocks = k_pad / kBlock;
  const int per_cta = (blocks + nctas - 1) / nctas;
  const int b_begin = rank * per_cta, b_end = min(blocks, (rank + 1) * per_cta);
  const int e_begin = b_begin * kBlock, e_end = min(k, b_end * kBlock);     // this CTA's share of the row's elements
  float inv = 1.f;
  if (norm_w) {
    float ss = 0.f;
    for (int i = e_begin + threadIdx.x * 8; i < e_end; i += 256 * 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(row + i);
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = __bfloat162float(h[j]);
        ss += f * f;
      }
    }
    inv = rsqrtf(f4_row_reduce<false>(ss, red, xch[0], rank, nctas) / k + eps);
  }
  float outer_s = 1.f;
  if (kBlock == 16) {
    float amax = 0.f;
    for (int i = e_begin + threadIdx.x * 8; i < e_end; i += 256 * 8) {
      float v[8];
      f4_load8(row, i, k, gated, norm_w, inv, offset_one, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float a = fabsf(v[j]);
        if (a == a && a <= 3.0e38f) amax = fmaxf(amax, a);
      }
    }
    amax = f4_row_reduce<true>(amax, red, xch[1], rank, nctas);
    outer_s = amax > 0.f ? __fdiv_rn(amax, 2688.f) : 1.f;
    if (threadIdx.x == 0 && rank == 0) outer[t] = outer_s;
  } else if (threadIdx.x == 0 && rank == 0) {
    outer[t] = 1.f;
  }
  pdl_trigger();
  for (int b = b_begin + threadIdx.x; b < b_end; b += 256) {
    float v[kBlock];
    float bamax = 0.f;
#pragma unroll
    for (int c = 0; c < kBlock / 8; ++c) {
      const int i = b * kBlock + c * 8;
      float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (i < k) f4_load8(row, i, k, gated, norm_w, inv, offset_one, f);   // k is a multiple of 8
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[c * 8 + j] = f[j];
        const float a = fabsf(f[j]);
        if (a == a && a <= 3.0e38f) bamax = fmaxf(bamax, a);
      }
    }
    float scale;
    uint32_t code;
    if (kBlock == 16) {
      const float want = fminf(__fdiv_rn(__fdiv_rn(bamax, 6.f), outer_s), 448.f);
      code = f32_to_e4m3(want);
      scale = e4m3_to_f32(static_cast<uint8_t>(code)) * outer_s;
    } else {
      const uint32_t bits = __float_as_uint(bamax) + 0x00200000u;
      int ec = static_cast<int>((bits >> 23) & 0xffu) - 2;
      ec = bamax > 0.f ? max(0, min(254, ec)) : 0;
      code = static_cast<uint32_t>(ec);
      scale = bamax > 0.f ? __uint_as_float(ec > 0 ? static_cast<uint32_t>(ec) << 23 : 0x00400000u) : 0.f;
    }
    xsf[static_cast<size_t>(t) * sf_ld + (b >> 2) * 8 + (b & 3)] = static_cast<uint8_t>(code);
    uint32_t words[kBlock / 8];
#pragma unroll
    for (int c = 0; c < kBlock / 8; ++c) {
      uint32_t w = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t qv = scale > 0.f ? f32_to_e2m1(__fdiv_rn(v[c * 8 + j], scale)) : 0u;
        w |= qv << (4 * j);
      }
      words[c] = w;
    }
    uint32_t* dst = reinterpret_cast<uint32_t*>(xq + static_cast<size_t>(t) * (k_pad / 2) + b * (kBlock / 2));
#pragma unroll
    for (int c = 0; c < kBlock / 8; ++c) dst[c] = words[c];
  }
}

}  // namespace sllm

using namespace sllm;

// x: bf16 [rows of the source, k] (row stride ldx elements, k a multiple of 8); token t reads source row src_row[t]
// (or t when src_row is null: gathering the rows of a routed batch costs nothing extra); with n_rows_ptr (device int)
// tokens >= *n_rows_ptr are skipped.  gated (0 none, 1 SiLU, 2 GELU-tanh): x rows are [gate (k) | up (k)] and the
// quantised value is act(gate) * up.  norm_w (bf16 [k], optional, not with gated): the row is RMS-normalised first
// (eps; weight + 1 with offset_one).  xq: [tokens, k_pad / 2]; xsf: [tokens, sf_ld] with sf_ld >= 2 k_pad / block
// (8 bytes per four scales), a multiple of 16; outer: [tokens] fp32.  fmt 0 = MXFP4 (block 32), 1 = NVFP4 (16).
SLLM_EXPORT int sllm_act_quant_fp4(const void* x, int ldx, int tokens, int k, int k_pad, const int* src_row,
                                   const int* n_rows_ptr, int gated, const void* norm_w, float eps, int offset_one, int fmt,
                                   void* xq, void* xsf, int sf_ld, float* outer, void* stream) {
  if (!x || !xq || !xsf || !outer || tokens <= 0 || k <= 0 || (k % 8) || k_pad < k || (k_pad % kF4KBlock) || (ldx % 8) ||
      (fmt != 0 && fmt != 1) || gated < 0 || gated > 2 || ldx < (gated ? 2 * k : k) || (norm_w && gated) ||
      (reinterpret_cast<uintptr_t>(norm_w) & 15))
    return SLLM_ERR_INVALID_ARGUMENT;
  const __nv_bfloat16* nw = static_cast<const __nv_bfloat16*>(norm_w);
  if (sf_ld < 2 * k_pad / (fmt ? 16 : 32) || (sf_ld % 16)) return SLLM_ERR_INVALID_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  // a row's blocks are shared out over a cluster of 1, 2, 4 or 8 CTAs: enough CTAs for two per SM, at least 256
  // blocks (one per thread) each (a launch of a few token rows would otherwise keep a few SMs busy for tens of
  // microseconds)
  const int blocks = k_pad / (fmt ? 16 : 32);
  int chunks = 1;
  while (chunks < 8 && tokens * chunks < 296 && blocks >= 256 * chunks * 2) chunks *= 2;
  const dim3 qgrid(tokens, 1, chunks);
  const unsigned cz = static_cast<unsigned>(chunks);
  if (fmt)
    e = launch_kernel(act_quant_fp4_kernel<16>, qgrid, dim3(256), 0, st, cz, static_cast<const __nv_bfloat16*>(x), ldx,
                      k, k_pad, src_row, n_rows_ptr, gated, nw, eps, offset_one, static_cast<uint8_t*>(xq),
                      static_cast<uint8_t*>(xsf), sf_ld, outer);
  else
    e = launch_kernel(act_quant_fp4_kernel<32>, qgrid, dim3(256), 0, st, cz, static_cast<const __nv_bfloat16*>(x), ldx,
                      k, k_pad, src_row, n_rows_ptr, gated, nw, eps, offset_one, static_cast<uint8_t*>(xq),
                      static_cast<uint8_t*>(xsf), sf_ld, outer);
  return e == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

// wtiles: native tiles [group][row tile][K block]{16 KB swizzled code image | scale atoms}; xq / xsf / x_outer: what
// sllm_act_quant_fp4 wrote.  bn in {16, 32, 64, 128}; with bn > 32 splits must keep ceil(k_blocks / splits) <= 8; with
// bn <= 32 the scale rows are read by TMA.  sf_ld and the address of xsf are multiples of 16.
// Workspace as sllm_gemm_w4.  row_ptr (optional): scatter epilogue, no residual then.
SLLM_EXPORT int sllm_gemm_fp4(const void* wtiles, const float* tensor_scale, const void* xq, const void* xsf, int sf_ld,
                              const float* x_outer, void* y, const void* residual, const int* tok_off, const float* tok_scale,
                              const long long* row_ptr, int fmt, int groups, int n_rows, int n_valid, int k_pad,
                              int total_tokens, int max_group_tokens, int ldy, int bn, int splits, float* ws,
                              long long ws_floats, int* counters, int n_counters, int* status, void* stream) {
  if (!wtiles || !xq || !xsf || (!y && !row_ptr) || groups <= 0 || n_rows <= 0 || (n_rows % kF4Rows) || n_valid <= 0 ||
      n_valid > n_rows || k_pad <= 0 || (k_pad % kF4KBlock) || total_tokens <= 0 || max_group_tokens <= 0 ||
      (fmt != 0 && fmt != 1) || (row_ptr && residual))
    return SLLM_ERR_INVALID_ARGUMENT;
  if (groups > 1 && !tok_off) return SLLM_ERR_INVALID_ARGUMENT;
  if (bn != 16 && bn != 32 && bn != 64 && bn != 128) return SLLM_ERR_UNSUPPORTED_SHAPE;
  if ((reinterpret_cast<uintptr_t>(wtiles) & 15) || (reinterpret_cast<uintptr_t>(xsf) & 15) || (sf_ld % 16))
    return SLLM_ERR_ALIGNMENT;
  const int k_blocks = k_pad / kF4KBlock;
  if (splits < 1) splits = 1;
  if (splits > k_blocks) splits = k_blocks;
  if (bn > 32 && (k_blocks + splits - 1) / splits > kF4MaxKb) return SLLM_ERR_UNSUPPORTED_SHAPE;
  if (sf_ld < 2 * k_pad / (fmt ? 16 : 32)) return SLLM_ERR_INVALID_ARGUMENT;
  const int row_tiles = n_rows / kF4Rows;
  const int tok_tiles = (max_group_tokens + bn - 1) / bn;
  if (static_cast<long long>(tok_tiles) * splits > 65535 || groups > 65535) return SLLM_ERR_UNSUPPORTED_SHAPE;
  if (splits > 1) {
    if (!ws || !counters) return SLLM_ERR_INVALID_ARGUMENT;
    if (ws_floats < static_cast<long long>(splits) * total_tokens * n_valid || n_counters < groups * row_tiles * tok_tiles)
      return SLLM_ERR_WORKSPACE_TOO_SMALL;
  }
  CUtensorMap tx, tsf;
  int rc = cached_kmajor_tmap(&tx, xq, 1, total_tokens, k_pad / 2, k_pad / 2, bn);
  if (rc != SLLM_OK) return rc;
  memset(&tsf, 0, sizeof(tsf));
  if (bn <= 32) {
    // a box always spans 32 token rows: rows past the tile (or the matrix) are never read by an MMA of N = bn
    rc = cached_plain_tmap(&tsf, xsf, total_tokens, sf_ld, sf_ld, 16, 32);
    if (rc != SLLM_OK) return rc;
  }
  F4Params p;
  memset(&p, 0, sizeof(p));
  p.n_rows = n_rows; p.n_valid = n_valid; p.k_blocks = k_blocks; p.groups = groups; p.atoms = fmt ? 4 : 2;
  p.splits = splits; p.total_tokens = total_tokens; p.ldy = row_ptr ? n_valid : ldy; p.sf_ld = sf_ld;
  p.wtiles = static_cast<const uint8_t*>(wtiles); p.tensor_scale = tensor_scale; p.tok_off = tok_off;
  p.tok_scale = tok_scale; p.x_outer = x_outer; p.xsf = static_cast<const uint8_t*>(xsf);
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.y = static_cast<__nv_bfloat16*>(y); p.row_ptr = row_ptr;
  p.ws = ws; p.counters = counters; p.status = status;
  dim3 grid(row_tiles, groups, tok_tiles * splits);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define SLLM_F4_CASE(BNV)                                                                      \
  case BNV:                                                                                    \
    return fmt ? launch_f4<BNV, 16>(tx, tsf, p, grid, st) : launch_f4<BNV, 32>(tx, tsf, p, grid, st);
  switch (bn) {
    SLLM_F4_CASE(16)
    SLLM_F4_CASE(32)
    SLLM_F4_CASE(64)
    SLLM_F4_CASE(128)
  }
#undef SLLM_F4_CASE
  return SLLM_ERR_UNSUPPORTED_SHAPE;
}
