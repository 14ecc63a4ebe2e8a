// Fused decode kernel: the weight-streaming GEMMs of a decoder layer as phases of ONE persistent kernel.
//
// Decode at small batch is bound by streaming the weights once per step.  A chain of separate GEMM kernels
// stalls HBM at every kernel boundary (prologue, first TMA round trip, epilogue, grid drain), which costs more
// than the transfer itself for the smaller projections.  Here one CTA per SM stays resident across up to four
// dependent GEMMs; because weights do not depend on activations, the TMA producer of every CTA keeps
// streaming the NEXT phase's weight tiles into its shared-memory ring while the current phase finishes and the
// grid barrier between phases resolves, so the HBM pipe never drains inside a launch.
//
// Work decomposition ("stream-K"): a phase is tiles x K-blocks units of 128 weight rows x 128 K bytes; CTA c
// owns the contiguous unit range [c U / G, (c + 1) U / G), i.e. every SM streams the same number of bytes
// whatever the shape.  A tile whose K range is split over several CTAs is finished by the CTA that arrives
// last (partials in a workspace, summed in a fixed order, so results do not depend on arrival order).
//
// Roles (256 threads): warp 0 weight producer (TMA, never waits for a grid barrier), warp 1 activation producer
// (TMA, waits for the barrier that publishes the phase's input), warps 2-3 MMA issuers (tcgen05.mma
// kind::f8f6f4, one K block per TMEM accumulator; each issuer has its own rings and accumulators), warps 4-7
// epilogue (promotion of every K block with scaleA * scaleB into fp32 registers, then the fused tile epilogue).
//
// Epilogues fold what used to be separate kernels into the GEMM that produces their input: residual add,
// RMSNorm statistics, FP8 1x128 quantisation of the next operand, SiLU*up, RoPE and the quantising KV-page
// append.  RMSNorm itself never runs: its weight vector is folded into the next weight matrix at load and
// its per-row factor rsqrt(mean(h^2) + eps) is applied to the accumulators of the next phase.
//
// Waits (mbarrier, grid barrier, peer flag) are bounded; a wait that gives up records a status code, and the
// CTA runs to its normal teardown.
//
// Replaces, for decode, the reference's per-op layer sequence (crates/sllm-core/src/qwen_graph.rs:2524-3501:
// rmsnorm, matmul, rotary + KV append, silu-mul, residual add as separate kernels).
#include "common.cuh"
#include "api.h"
#include "decode_fused.h"
#include "epilogue_columns.cuh"
#include <cstddef>
#include <cstring>

namespace sllm {

int cached_kmajor_tmap(CUtensorMap* out, const void* ptr, int elem_bytes, long long rows, long long k_elems,
                       long long row_stride_bytes, int box_rows);

constexpr int kFdThreads = 384;                    // 2 producer + 2 MMA warps, two epilogue groups of 4 warps
constexpr int kFdASlots = 4;                       // weight-ring slots (16 KB) per issuer, released by the MMA commit
constexpr int kFdBSlots = 6;                       // activation-ring slots per issuer, released by the epilogue
constexpr int kFdATile = 128 * 128;                // 128 weight rows x 128 K bytes
constexpr int kFdASlotBytes = kFdATile;
constexpr int kFdMaxWorld = 8;
constexpr int kFdLookaheadDefault = 12;            // weight tiles (16 KB each) prefetched into L2 ahead of the ring, per CTA
constexpr float kFdE4M3Max = 448.f;
constexpr unsigned long long kFdSyncQuantum = 4096;   // grid-barrier arrivals per launch (>= phases x CTAs)

template <int BN> constexpr int fd_b_tile() { return BN * 128; }
template <int BN> constexpr int fd_b_slot() { return BN * 128; }

struct FdComm {
  int world, rank;
  long long cap_elems;
  __nv_bfloat16* recv[kFdMaxWorld];
  uint32_t* flags[kFdMaxWorld];
  uint32_t* epoch;
};

struct FdMaps {
  CUtensorMap a[SLLM_FD_MAX_PHASES];
  CUtensorMap b[SLLM_FD_MAX_PHASES];
};

struct FdParams {
  int n_phases, rows;
  SllmFdPhase ph[SLLM_FD_MAX_PHASES];
  SllmFdRope rope;
  float* ws;
  int* counters;
  unsigned long long* sync;
  int* status;
  long long wait_limit;
  int lookahead;               // L2 prefetch distance of the weight producer in tiles
  int debug;                   // experiment switches (timing studies only; results are wrong when set)
  unsigned long long* trace;   // optional [CTAs][MAX_PHASES][8] globaltimer stamps (profiling aid), null = off
  FdComm comm;
};

struct __align__(16) FdShared {
  uint64_t afull[2][kFdASlots], aempty[2][kFdASlots];
  uint64_t bfull[2][kFdBSlots], bempty[2][kFdBSlots];
  uint64_t tfull[4], tempty[4];
  uint32_t tmem_base;
  int abort_flag;
  int is_last;
  uint32_t epoch;
  float rnorm[32];
  float norm_scratch[128];
  float inv_freq[64];
  int rope_pos[32];            // position and KV page of every token row (ROPE_KV launches)
  int rope_page[32];
  // the launch descriptors, copied from kernel-parameter space once: a run-time phase index (and the out-of-line
  // tile epilogue) would otherwise read them through generic loads of the parameter window on every use
  SllmFdPhase ph[SLLM_FD_MAX_PHASES];
  SllmFdRope rope;
  FdComm comm;
};

__device__ __forceinline__ float fd_silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float fd_gelu_tanh(float x) {
  const float c = 0.7978845608028654f;
  return 0.5f * x * (1.f + tanhf(c * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float fd_bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ unsigned long long fd_ld_acquire_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fd_red_release_add_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void fd_st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t fd_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// 1-D bulk copy global -> shared completing on an mbarrier; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void fd_bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void fd_fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
// TMA prefetch of a 2-D tile into L2 only (no shared-memory destination, nothing to wait for).
__device__ __forceinline__ void fd_tma_prefetch_l2(const CUtensorMap* m, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y)
               : "memory");
}
// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread, no wait.
__device__ __forceinline__ void fd_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
template <int BN>
__device__ __forceinline__ void fd_tmem_ld(uint32_t taddr, uint32_t (&r)[BN]) {
  if constexpr (BN == 32) fd_tmem_ld32(taddr, r);
  else tmem_ld16(taddr, r);
}

// Bounded wait until the grid-barrier counter reaches `target`.
__device__ __forceinline__ bool fd_grid_wait(const unsigned long long* ctr, unsigned long long target,
                                             volatile int* abort_flag, int* status, long long limit) {
  uint32_t spins = 0;
  long long t0 = 0;
  while (fd_ld_acquire_u64(ctr) < target) {
    ++spins;
    if (spins == 64) t0 = clock64();
    if (spins > 64 && (spins & 15) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, SLLM_DEV_TIMEOUT_GRID_BARRIER);
        return false;
      }
    }
  }
  return true;
}

// Barrier 1 over the 128 epilogue threads that also ORs a predicate, so that every thread takes the same branch
// on a flag another role may set at any moment.
__device__ __forceinline__ bool fd_epi_any(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.or.pred q, 1, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(pred))
      : "memory");
  return r != 0;
}

__device__ __forceinline__ void fd_stamp(unsigned long long* trace, int cta, int pi, int slot) {
  if (trace) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    trace[(static_cast<size_t>(cta) * SLLM_FD_MAX_PHASES + pi) * 8 + slot] = t;
  }
}

#ifdef SLLM_FD_PROFILE
// Cycle accounting of the pipeline roles (timing studies; never compiled into the product library).
#define FD_PROF_DECL(n) long long prof_##n = 0
#define FD_PROF_T0() const long long prof_t0 = clock64()
#define FD_PROF_ADD(n) prof_##n += clock64() - prof_t0
#define FD_PROF_OUT(slot, n) if (p.trace) p.trace[static_cast<size_t>(gridDim.x) * 32 + static_cast<size_t>(blockIdx.x) * 32 + (slot)] = prof_##n
#else
#define FD_PROF_DECL(n)
#define FD_PROF_T0()
#define FD_PROF_ADD(n)
#define FD_PROF_OUT(slot, n)
#endif

// CTA that owns unit u when U units are dealt to G CTAs as [c U / G, (c + 1) U / G).
// (all unit arithmetic is 32-bit: the launcher checks that units x (CTAs + 1) stays below 2^31)
__device__ __forceinline__ int fd_cta_of_unit(uint32_t u, uint32_t U, int G) {
  return static_cast<int>(((u + 1u) * static_cast<uint32_t>(G) - 1u) / U);
}

struct FdPhaseGeom {
  int tiles, nkb, dual;
  uint32_t U, u0, u1;
};
__device__ __forceinline__ FdPhaseGeom fd_geom(const SllmFdPhase& ph, int cta, int G) {
  FdPhaseGeom g;
  g.tiles = (ph.n + 127) >> 7;
  g.nkb = ph.k >> 7;
  g.dual = ph.dual_off > 0 ? 1 : 0;
  g.U = static_cast<uint32_t>(g.tiles) * static_cast<uint32_t>(g.nkb);
  g.u0 = static_cast<uint32_t>(cta) * g.U / static_cast<uint32_t>(G);
  g.u1 = static_cast<uint32_t>(cta + 1) * g.U / static_cast<uint32_t>(G);
  return g;
}

// Barrier 2 over the 256 threads of both epilogue groups, ORing a predicate (see fd_epi_any).
__device__ __forceinline__ bool fd_all_any(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.or.pred q, 2, 256, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(pred))
      : "memory");
  return r != 0;
}
__device__ __forceinline__ void mbar_arrive_cnt(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// Cross-rank sum of a staged tile (tensor parallelism), run by the 128 threads of epilogue group 0: push the partial
// (bf16) to every rank, flag, wait (bounded), sum in rank order back into the staging buffer.
template <int BN>
__device__ __noinline__ bool fd_comm_sum_tile(int* status, FdShared* sh, float* stage, int tile, int ew, int lane, int et,
                                              int T, volatile int* abort_flag, long long limit) {
  {
    // ---- cross-rank sum of the tile: push the partial (bf16) to every rank, flag, wait, sum in rank order
    const FdComm& cm = sh->comm;
    if (et == 0) {
      const uint32_t e1 = cm.epoch[tile] + 1;
      cm.epoch[tile] = e1;
      sh->epoch = e1;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const uint32_t e = sh->epoch;
    const long long region = static_cast<long long>(e & 1) * cm.world;
    const long long toff = static_cast<long long>(tile) * (128 * BN);
#pragma unroll 1
    for (int c = ew; c < T; c += 4) {
      const float4 x = *reinterpret_cast<const float4*>(stage + c * 128 + lane * 4);
      uint2 w;
      *reinterpret_cast<__nv_bfloat162*>(&w.x) = __floats2bfloat162_rn(x.x, x.y);
      *reinterpret_cast<__nv_bfloat162*>(&w.y) = __floats2bfloat162_rn(x.z, x.w);
      const long long off = (region + cm.rank) * cm.cap_elems + toff + c * 128 + lane * 4;
      for (int peer = 0; peer < cm.world; ++peer) *reinterpret_cast<uint2*>(cm.recv[peer] + off) = w;
    }
    __threadfence_system();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (et < cm.world && et != cm.rank) {
      fd_st_release_sys(cm.flags[et] + static_cast<size_t>(tile) * cm.world + cm.rank, e);
      const uint32_t* f = cm.flags[cm.rank] + static_cast<size_t>(tile) * cm.world + et;
      uint32_t spins = 0;
      long long t0 = 0;
      while (static_cast<int32_t>(fd_ld_acquire_sys(f) - e) < 0) {
        ++spins;
        if (spins == 1024) t0 = clock64();
        if (spins > 1024 && (spins & 63) == 0) {
          if (*abort_flag) break;
          if (clock64() - t0 > limit) {
            *abort_flag = 1;
            if (status) atomicCAS(status, 0, SLLM_DEV_TIMEOUT_PEER_FLAG);
            break;
          }
        }
      }
    }
    if (fd_epi_any(*abort_flag != 0)) return false;
#pragma unroll 1
    for (int c = ew; c < T; c += 4) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int src = 0; src < cm.world; ++src) {
        const uint2 w = __ldcg(reinterpret_cast<const uint2*>(cm.recv[cm.rank] + (region + src) * cm.cap_elems + toff +
                                                              c * 128 + lane * 4));
        const __nv_bfloat162 h0 = *reinterpret_cast<const __nv_bfloat162*>(&w.x);
        const __nv_bfloat162 h1 = *reinterpret_cast<const __nv_bfloat162*>(&w.y);
        s.x += __bfloat162float(h0.x); s.y += __bfloat162float(h0.y);
        s.z += __bfloat162float(h1.x); s.w += __bfloat162float(h1.y);
      }
      *reinterpret_cast<float4*>(stage + c * 128 + lane * 4) = s;
    }
  }

  return true;
}

// Tile epilogue, run by all 256 epilogue threads.  On entry the raw sums of the tile are in stage[token][row]
// (group 1's share of a plain tile, or the up sums of a gate/up tile, in xchg).  Step 1: every thread rewrites half of
// the token columns of its row in place (residual, norm factor, activation).  Step 2 (tensor-parallel launches): the
// tile is summed across ranks.  Step 3: warp w of 8 takes token rows w, w + 8, ...; lane l owns outputs 4 l .. 4 l + 3
// and writes / quantises them.  Kept out of line and rolled: it runs once per tile.
// Returns false when the cross-rank exchange gave up.
template <int BN>
__device__ __noinline__ bool fd_finish_tile(int* status, const SllmFdPhase& ph, FdShared* sh, float* stage,
                                            const float* xchg, int tile, int grp, int ew, int lane, int et, int T,
                                            int dual, int add_xchg, float norm_part, bool& norm_ready,
                                            volatile int* abort_flag, long long limit) {
  const int row = ew * 32 + lane;
  const bool has_norm = ph.norm_tiles > 0;
  if (!norm_ready) {
    // the norm factors of the phase are reduced the first time a tile needs them
    constexpr int kParts = 128 / BN;
    if (grp == 0) sh->norm_scratch[et] = norm_part;      // [part][token]
    asm volatile("bar.sync 2, 256;" ::: "memory");
    if (grp == 0 && et < BN) {
      float ss = 0.f;
#pragma unroll
      for (int q = 0; q < kParts; ++q) ss += sh->norm_scratch[q * BN + et];
      sh->rnorm[et] = rsqrtf(ss / static_cast<float>(ph.norm_dim) + ph.eps);
    }
    norm_ready = true;
  }
  asm volatile("bar.sync 2, 256;" ::: "memory");          // sums and norm factors visible
  {
    // tensor-parallel launches sum the tile across ranks afterwards: the residual then joins on rank 0 only
    const bool resid = ph.epilogue == SLLM_FD_RESID_QUANT && (sh->comm.world <= 1 || sh->comm.rank == 0);
    const int act = ph.act;
    // residual stream: this thread owns feature tile * 128 + row; the loads of its token columns are in flight together
    const __nv_bfloat16* res = static_cast<const __nv_bfloat16*>(ph.residual) + static_cast<size_t>(tile) * 128 + row;
    float rv[BN / 2];
#pragma unroll
    for (int i = 0; i < BN / 2; ++i) {
      const int c = grp + 2 * i;
      rv[i] = (resid && c < T) ? __bfloat162float(res[static_cast<size_t>(c) * ph.ldy]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < BN / 2; ++i) {
      const int c = grp + 2 * i;
      const float rn = has_norm ? sh->rnorm[c] : 1.f;
      float v = stage[c * 128 + row];
      if (add_xchg) v += xchg[c * 128 + row];
      v = (v + rv[i]) * rn;
      if (dual) {
        const float a = act == 0 ? fd_silu(v) : fd_gelu_tanh(v);
        v = fd_bf16r(a) * (xchg[c * 128 + row] * rn);
      }
      stage[c * 128 + row] = v;
    }
  }
  asm volatile("bar.sync 2, 256;" ::: "memory");
  bool comm_ok = true;
  if (ph.epilogue == SLLM_FD_RESID_QUANT && sh->comm.world > 1) {
    if (grp == 0) comm_ok = fd_comm_sum_tile<BN>(status, sh, stage, tile, ew, lane, et, T, abort_flag, limit);
    if (fd_all_any(!comm_ok)) return false;
  }
  ColEpilogue e;
  e.mode = ph.epilogue; e.n = ph.n; e.ldy = ph.ldy; e.ld_s = ph.ld_s_out; e.softcap = ph.softcap;
  e.y = static_cast<__nv_bfloat16*>(ph.y);
  // the residual of a RESID_QUANT tile is already part of the staged values
  e.residual = ph.epilogue == SLLM_FD_PLAIN ? static_cast<const __nv_bfloat16*>(ph.residual) : nullptr;
  e.q_out = static_cast<uint8_t*>(ph.q_out); e.s_out = ph.s_out; e.ssq_out = ph.ssq_out;
  e.rope = &sh->rope; e.inv_freq = sh->inv_freq;
#pragma unroll 1
  for (int c = grp * 4 + ew; c < T; c += 8) {
    const float4 x = *reinterpret_cast<const float4*>(stage + c * 128 + lane * 4);
    float v[4] = {x.x, x.y, x.z, x.w};
    col_epilogue(e, tile, c, lane, v, sh->rope_pos[c], sh->rope_page[c]);
  }
  asm volatile("bar.sync 2, 256;" ::: "memory");          // the staging buffers are free again
  return true;
}

constexpr int kFdFastParts = 6;   // parts of a split tile whose loads are kept in flight together
// dst[(col0 + c) * 128] = sum over parts jj < np (in order) of base[offs[jj] + (col0 + c) * 128], c < CH: all loads are
// issued before the first one is used, and the sums go to shared memory so that no accumulator array is live here.
template <int NP, int CH>
__device__ __forceinline__ void fd_sum_parts(const float* base, const uint32_t (&offs)[kFdFastParts], int np, int col0,
                                             float* dst) {
  float t[NP][CH];
#pragma unroll
  for (int jj = 0; jj < NP; ++jj) {
    if (jj < np) {
#pragma unroll
      for (int c = 0; c < CH; ++c) t[jj][c] = __ldcg(base + offs[jj] + static_cast<size_t>(col0 + c) * 128);
    }
  }
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    float sum = 0.f;
#pragma unroll
    for (int jj = 0; jj < NP; ++jj)
      if (jj < np) sum += t[jj][c];
    dst[(col0 + c) * 128] = sum;
  }
}

template <int BN>
__global__ void __launch_bounds__(kFdThreads, 1)
fused_decode_kernel(const __grid_constant__ FdMaps maps, const __grid_constant__ FdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kBSlot = fd_b_slot<BN>();
  constexpr int kBTile = fd_b_tile<BN>();
  constexpr uint32_t kTmemCols = 8 * BN;            // 4 accumulators x (gate, up) x BN columns
  uint8_t* a_ring = smem;                                         // [2][kFdASlots][kFdASlotBytes]
  uint8_t* b_ring = a_ring + 2 * kFdASlots * kFdASlotBytes;       // [2][kFdBSlots][kBSlot]
  float* b_scale = reinterpret_cast<float*>(b_ring + 2 * kFdBSlots * kBSlot);   // [2][kFdBSlots][BN] activation scales
  float* stage = b_scale + 2 * kFdBSlots * BN;                                  // [BN][128] tile staged for the row epilogue
  float* xchg = stage + BN * 128;                                             // [BN][128] group 1 -> group 0 hand-over
  FdShared* sh = reinterpret_cast<FdShared*>(xchg + BN * 128);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const int G = gridDim.x;
  volatile int* abort_flag = &sh->abort_flag;
  const long long limit = p.wait_limit;

  {
    constexpr int kPhWords = sizeof(SllmFdPhase) * SLLM_FD_MAX_PHASES / 4, kRopeWords = sizeof(SllmFdRope) / 4,
                  kCommWords = sizeof(FdComm) / 4;
    const uint32_t* src_ph = reinterpret_cast<const uint32_t*>(&p.ph[0]);
    const uint32_t* src_rope = reinterpret_cast<const uint32_t*>(&p.rope);
    const uint32_t* src_comm = reinterpret_cast<const uint32_t*>(&p.comm);
    for (int i = threadIdx.x; i < kPhWords; i += kFdThreads) reinterpret_cast<uint32_t*>(&sh->ph[0])[i] = src_ph[i];
    for (int i = threadIdx.x; i < kRopeWords; i += kFdThreads) reinterpret_cast<uint32_t*>(&sh->rope)[i] = src_rope[i];
    for (int i = threadIdx.x; i < kCommWords; i += kFdThreads) reinterpret_cast<uint32_t*>(&sh->comm)[i] = src_comm[i];
  }
  if (threadIdx.x == 0) {
    for (int r = 0; r < 2; ++r) {
      for (int s = 0; s < kFdASlots; ++s) { mbar_init(&sh->afull[r][s], 1); mbar_init(&sh->aempty[r][s], 1); }
      for (int s = 0; s < kFdBSlots; ++s) { mbar_init(&sh->bfull[r][s], 1); mbar_init(&sh->bempty[r][s], 8); }
    }
    for (int a = 0; a < 4; ++a) { mbar_init(&sh->tfull[a], 1); mbar_init(&sh->tempty[a], 8); }
    sh->abort_flag = 0;
    sh->is_last = 0;
    mbar_fence_init();
    for (int i = 0; i < p.n_phases; ++i) { tma_prefetch_desc(&maps.a[i]); tma_prefetch_desc(&maps.b[i]); }
  }
  if (warp == 2) {
    tmem_alloc(&sh->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  if (threadIdx.x >= 128 && threadIdx.x < 192) {
    const int fi = threadIdx.x - 128;
    const int rd = p.rope.rotary_dim > 0 ? p.rope.rotary_dim : 128;
    sh->inv_freq[fi] = (p.rope.inv_freq && fi < rd / 2) ? p.rope.inv_freq[fi] : 0.f;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  if (threadIdx.x == 0) fd_stamp(p.trace, cta, 0, 0);       // CTA set up

  if (warp == 0) {
    // ------------------------------------------------------------------ weight producer
    if (lane == 0) {
      uint32_t apos[2] = {0u, 0u};
      uint32_t n = 0;
      bool ok = true;
      FD_PROF_DECL(pa);
      // L2 prefetch cursor: runs kFdLookahead tile loads ahead of the shared-memory ring, across phase
      // boundaries, so HBM keeps streaming while a phase's reduction / epilogue / grid barrier resolves.
      int f_pi = 0, f_half = 0;
      FdPhaseGeom fg = fd_geom(sh->ph[0], cta, G);
      uint32_t f_u = fg.u0;
      auto prefetch_next = [&]() {
        while (f_pi < p.n_phases && f_u >= fg.u1) {
          if (++f_pi < p.n_phases) { fg = fd_geom(sh->ph[f_pi], cta, G); f_u = fg.u0; f_half = 0; }
        }
        if (f_pi >= p.n_phases) return;
        const int ft = static_cast<int>(f_u / fg.nkb), fk = static_cast<int>(f_u % fg.nkb);
        const SllmFdPhase& fp = sh->ph[f_pi];
        const int frow = ft * 128 + f_half * fp.dual_off;
        fd_tma_prefetch_l2(&maps.a[f_pi], fk * 128, frow);
        int fs = fp.dual_off + fp.n - frow;      // the row scales the epilogue will read from L2
        if (fs > 128) fs = 128;
        prefetch_l2_bulk(fp.w_scale + static_cast<size_t>(fk) * fp.ld_sa + frow, fs * 4);
        if (f_half < fg.dual) ++f_half; else { f_half = 0; ++f_u; }
      };
      for (int i = 0; i < p.lookahead; ++i) prefetch_next();
      for (int pi = 0; pi < p.n_phases && ok; ++pi) {
        const SllmFdPhase& ph = sh->ph[pi];
        const FdPhaseGeom g = fd_geom(ph, cta, G);
        int tile = static_cast<int>(g.u0 / g.nkb), kb = static_cast<int>(g.u0 % g.nkb);
        for (uint32_t u = g.u0; u < g.u1 && ok; ++u, ++n) {
          const int r = n & 1;
          for (int half = 0; half <= g.dual; ++half) {
            const uint32_t slot = apos[r] % kFdASlots, fill = apos[r] / kFdASlots;
            { FD_PROF_T0();
            if (!mbar_wait(&sh->aempty[r][slot], (fill & 1) ^ 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_SMEM_EMPTY, limit)) {
              ok = false;
              break;
            }
            FD_PROF_ADD(pa); }
            uint8_t* dst = a_ring + (r * kFdASlots + slot) * kFdASlotBytes;
            const int row0 = tile * 128 + half * ph.dual_off;
            if (p.debug & 1) {
              mbar_arrive(&sh->afull[r][slot]);                       // no weight traffic at all
            } else if (p.debug & 4) {
              mbar_expect_tx(&sh->afull[r][slot], kFdATile);          // one contiguous 16 KB copy instead of a tiled box
              fd_bulk_load(dst, static_cast<const uint8_t*>(ph.w) + (static_cast<size_t>(tile) * g.nkb + kb) * kFdATile,
                           kFdATile, &sh->afull[r][slot]);
            } else {
              mbar_expect_tx(&sh->afull[r][slot], kFdATile);
              tma_load_2d(dst, &maps.a[pi], &sh->afull[r][slot], kb * 128, row0);
            }
            ++apos[r];
            if (p.lookahead > 0) prefetch_next();
          }
          if (++kb == g.nkb) { kb = 0; ++tile; }
        }
      }
      pdl_trigger();
      FD_PROF_OUT(16, pa);
      // Drain: every copy this thread started must have landed before the CTA may exit (on the normal path
      // all of them have been consumed already and the waits return at once).
      for (int r = 0; r < 2; ++r)
        for (int s = 0; s < kFdASlots; ++s) {
          const uint32_t fills = apos[r] > static_cast<uint32_t>(s) ? (apos[r] - s + kFdASlots - 1) / kFdASlots : 0u;
          if (fills > 0) {
            int dummy = 0;
            mbar_wait(&sh->afull[r][s], (fills - 1) & 1, &dummy, p.status, SLLM_DEV_TIMEOUT_DRAIN, 200000000LL);
          }
        }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ activation producer
    if (lane == 0) {
      uint32_t bpos[2] = {0u, 0u};
      uint32_t n = 0;
      bool ok = true;
      unsigned long long base = 0;
      FD_PROF_DECL(pb); FD_PROF_DECL(pg);
      for (int pi = 0; pi < p.n_phases && ok; ++pi) {
        const SllmFdPhase& ph = sh->ph[pi];
        const FdPhaseGeom g = fd_geom(ph, cta, G);
        FD_PROF_T0();
        if (pi == 0) {
          pdl_wait();
          base = fd_ld_acquire_u64(p.sync) / kFdSyncQuantum * kFdSyncQuantum;
        } else if (!fd_grid_wait(p.sync, base + static_cast<unsigned long long>(pi) * G, abort_flag, p.status, limit)) {
          ok = false;
          break;
        }
        fd_fence_proxy_async();
        FD_PROF_ADD(pg);
        int kb = static_cast<int>(g.u0 % g.nkb);
        for (uint32_t u = g.u0; u < g.u1 && ok; ++u, ++n) {
          const int r = n & 1;
          const uint32_t slot = bpos[r] % kFdBSlots, fill = bpos[r] / kFdBSlots;
          { FD_PROF_T0();
          if (!mbar_wait(&sh->bempty[r][slot], (fill & 1) ^ 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_SMEM_EMPTY, limit)) {
            ok = false;
            break;
          }
          FD_PROF_ADD(pb); }
          uint8_t* dst = b_ring + (r * kFdBSlots + slot) * kBSlot;
          mbar_expect_tx(&sh->bfull[r][slot], kBTile + BN * 4);
          tma_load_2d(dst, &maps.b[pi], &sh->bfull[r][slot], kb * 128, 0);
          fd_bulk_load(b_scale + (r * kFdBSlots + slot) * BN, ph.x_scale + static_cast<size_t>(kb) * ph.ld_sb, BN * 4,
                       &sh->bfull[r][slot]);
          ++bpos[r];
          if (++kb == g.nkb) kb = 0;
        }
      }
      FD_PROF_OUT(17, pb); FD_PROF_OUT(18, pg);
      for (int r = 0; r < 2; ++r)
        for (int s = 0; s < kFdBSlots; ++s) {
          const uint32_t fills = bpos[r] > static_cast<uint32_t>(s) ? (bpos[r] - s + kFdBSlots - 1) / kFdBSlots : 0u;
          if (fills > 0) {
            int dummy = 0;
            mbar_wait(&sh->bfull[r][s], (fills - 1) & 1, &dummy, p.status, SLLM_DEV_TIMEOUT_DRAIN, 200000000LL);
          }
        }
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ MMA issuers
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(kFmtE4M3, 128, BN);
      const int iw = warp - 2;
      uint32_t apos = 0, bpos = 0, mine = 0, n = 0;
      bool ok = true;
      FD_PROF_DECL(wa); FD_PROF_DECL(wb); FD_PROF_DECL(wt); FD_PROF_DECL(is);
      for (int pi = 0; pi < p.n_phases && ok; ++pi) {
        const FdPhaseGeom g = fd_geom(sh->ph[pi], cta, G);
        for (uint32_t u = g.u0; u < g.u1 && ok; ++u, ++n) {
          if (static_cast<int>(n & 1) != iw) continue;
          const int acc = iw * 2 + (mine & 1);
          const uint32_t use = mine >> 1;
          const uint32_t bslot = bpos % kFdBSlots, bfill = bpos / kFdBSlots;
          uint32_t aslot[2];
          { FD_PROF_T0();
          for (int half = 0; half <= g.dual && ok; ++half) {
            aslot[half] = (apos + half) % kFdASlots;
            const uint32_t afill = (apos + half) / kFdASlots;
            ok = mbar_wait(&sh->afull[iw][aslot[half]], afill & 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMA_FULL, limit);
          }
          FD_PROF_ADD(wa); }
          { FD_PROF_T0();
          if (ok) ok = mbar_wait(&sh->bfull[iw][bslot], bfill & 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMA_FULL, limit);
          FD_PROF_ADD(wb); }
          { FD_PROF_T0();
          if (ok) ok = mbar_wait(&sh->tempty[acc], (use & 1) ^ 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMEM_EMPTY, limit);
          FD_PROF_ADD(wt); }
          if (!ok) break;
          FD_PROF_T0();
          tc_fence_after();
          const uint64_t bdesc = make_smem_desc_sw128(smem_u32(b_ring + (iw * kFdBSlots + bslot) * kBSlot));
          for (int half = 0; half <= g.dual; ++half) {
            const uint64_t adesc = make_smem_desc_sw128(smem_u32(a_ring + (iw * kFdASlots + aslot[half]) * kFdASlotBytes));
            const uint32_t d = tmem_base + acc * (2 * BN) + half * BN;
#pragma unroll
            for (int k = 0; k < 4; ++k)
              if (k == 0 || !(p.debug & 2)) umma_f8(d, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0);
          }
          for (int half = 0; half <= g.dual; ++half) tc_commit(&sh->aempty[iw][aslot[half]]);   // slot reusable once read
          tc_commit(&sh->tfull[acc]);
          FD_PROF_ADD(is);
          apos += 1 + g.dual;
          ++bpos;
          ++mine;
        }
      }
      FD_PROF_OUT(iw * 4 + 0, wa); FD_PROF_OUT(iw * 4 + 1, wb); FD_PROF_OUT(iw * 4 + 2, wt); FD_PROF_OUT(iw * 4 + 3, is);
    }
  } else {
    // ------------------------------------------------------------------ epilogue: two groups of 128 threads
    // Promotion is a chain of long-latency steps per K block (barrier wait, TMEM load, release), so two groups
    // work on different accumulators at the same time: in a plain phase group g promotes the K blocks of issuer
    // g; in a gate/up phase group 0 promotes every gate accumulator and group 1 every up accumulator.  At the
    // end of a tile segment group 1 hands its registers to group 0 through shared memory; group 0 finishes tiles.
    const int grp = (warp - 4) >> 2;
    const int ew = (warp - 4) & 3;           // TMEM lane quarter (= warp % 4)
    const int row = ew * 32 + lane;          // row of the weight tile
    const int et = threadIdx.x - 128 - grp * 128;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16);
    const int T = p.rows;
    uint32_t bpos[2] = {0u, 0u};
    uint32_t n = 0;
    bool ok = true;
    unsigned long long base = 0;
    float acc[BN];
    FD_PROF_DECL(wf); FD_PROF_DECL(ld); FD_PROF_DECL(fm); FD_PROF_DECL(xc); FD_PROF_DECL(pr); FD_PROF_DECL(fn);

    for (int pi = 0; pi < p.n_phases; ++pi) {
      const SllmFdPhase& ph = sh->ph[pi];
      const FdPhaseGeom g = fd_geom(ph, cta, G);
      float norm_part = 0.f;
      bool norm_ready = ph.norm_tiles == 0;
      if (grp == 0) {
        if (pi == 0) {
          pdl_wait();
          base = fd_ld_acquire_u64(p.sync) / kFdSyncQuantum * kFdSyncQuantum;
          if (sh->rope.positions && et < T) {
            // page lookups of the KV append, long before the q/k/v phase needs them
            const int pos = sh->rope.positions[et];
            sh->rope_pos[et] = pos;
            sh->rope_page[et] = sh->rope.block_table[static_cast<size_t>(sh->rope.seq_index[et]) * sh->rope.max_blocks +
                                                     pos / sh->rope.page_size];
          }
        } else if (ok) {
          if (et == 0) fd_grid_wait(p.sync, base + static_cast<unsigned long long>(pi) * G, abort_flag, p.status, limit);
          fd_epi_any(false);                 // the group resumes together; a failed wait shows at the next segment end
        }
        if (et == 0) fd_stamp(p.trace, cta, pi, 1);         // phase input visible
        // RMSNorm factor of every token row from the per-block sums of squares of the phase's input: the loads
        // are issued here (token = et % BN, every (128 / BN)-th block) and first used when a tile is finished,
        // so their latency hides under the promotion loop.
        if (ph.norm_tiles > 0) {
          constexpr int kParts = 128 / BN;
          const int tok = et % BN, part = et / BN;
          if (tok < T)
            for (int i = part; i < ph.norm_tiles; i += kParts)
              norm_part += __ldcg(ph.ssq_in + static_cast<size_t>(i) * ph.ld_s_out + tok);
        }
      }
      bool first_unit = true;
      const size_t part_floats = static_cast<size_t>(1 + g.dual) * BN * 128;
      int pend[2];          // split tiles this CTA arrived last for (a CTA's range touches at most two)
      int npend = 0;
      // Weight scales (one fp32 per weight row and K block) come straight from L2, where the producer's prefetch
      // cursor has put them: each thread keeps the scales of its next two K blocks in registers.
      const uint32_t nkb_u = static_cast<uint32_t>(g.nkb);
      const uint32_t u_end = static_cast<uint32_t>(g.u1);
      const uint32_t s_stride = g.dual ? 1u : 2u;
      const int s_rows = ph.dual_off + ph.n;
      const int s_row_off = row + ((g.dual && grp == 1) ? ph.dual_off : 0);
      auto load_sa = [&](uint32_t uu) -> float {
        if (uu >= u_end) return 0.f;
        const uint32_t t = uu / nkb_u, k = uu - t * nkb_u;
        const int rg = static_cast<int>(t) * 128 + s_row_off;
        return rg < s_rows ? __ldg(ph.w_scale + static_cast<size_t>(k) * ph.ld_sa + rg) : 0.f;
      };
      uint32_t s_next = static_cast<uint32_t>(g.u0) + (g.dual ? 0u : ((static_cast<uint32_t>(grp) - n) & 1u));
      float sa_q0 = load_sa(s_next), sa_q1 = load_sa(s_next + s_stride);
      s_next += 2 * s_stride;

      uint32_t u = g.u0;
      while (u < g.u1 && ok) {
        const int tile = static_cast<int>(u / g.nkb);
        const int kb0 = static_cast<int>(u - static_cast<uint32_t>(tile) * static_cast<uint32_t>(g.nkb));
        int kbe = g.nkb;
        if (g.u1 - u < g.nkb - kb0) kbe = kb0 + static_cast<int>(g.u1 - u);
        const bool split = !(kb0 == 0 && kbe == g.nkb);
        const bool seg_first = u == g.u0;
#pragma unroll
        for (int c = 0; c < BN; ++c) acc[c] = 0.f;
        // ---- promotion: one K block per TMEM accumulator
        for (int kb = kb0; kb < kbe; ++kb, ++n) {
          const int iw = n & 1;
          const uint32_t bs = bpos[iw] % kFdBSlots;
          ++bpos[iw];
          if (!g.dual && iw != grp) continue;
          const uint32_t m = n >> 1;
          const int a = iw * 2 + (m & 1);
          // a wait that gives up leaves the loop warp-uniformly; the CTA-wide decision follows the segment
          { FD_PROF_T0();
          if (!__all_sync(0xffffffffu, mbar_wait(&sh->tfull[a], (m >> 1) & 1, abort_flag, p.status,
                                                  SLLM_DEV_TIMEOUT_TMEM_FULL, limit))) {
            *abort_flag = 1;
            break;
          }
          FD_PROF_ADD(wf); }
          tc_fence_after();
          if (first_unit) {
            first_unit = false;
            if (et == 0 && grp == 0) fd_stamp(p.trace, cta, pi, 2);       // first accumulator ready
          }
          const float sa = sa_q0;
          sa_q0 = sa_q1;
          sa_q1 = load_sa(s_next);
          s_next += s_stride;
          const float* sb_p = b_scale + (iw * kFdBSlots + bs) * BN;
          uint32_t r[BN];
          { FD_PROF_T0();
          fd_tmem_ld<BN>(lane_addr + a * (2 * BN) + ((g.dual && grp == 1) ? BN : 0), r);
          tmem_wait_ld();
          FD_PROF_ADD(ld); }
          { FD_PROF_T0();
#pragma unroll
          for (int c = 0; c < BN; ++c) acc[c] = fmaf(__uint_as_float(r[c]), sa * sb_p[c], acc[c]);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            // either release barrier expects 8 arrivals: both groups' warps once each, or one group's warps twice
            const uint32_t cnt = g.dual ? 1u : 2u;
            mbar_arrive_cnt(&sh->tempty[a], cnt);
            mbar_arrive_cnt(&sh->bempty[iw][bs], cnt);
          }
          FD_PROF_ADD(fm); }
        }
        u += kbe - kb0;

        // ---- hand-over: group 1's accumulators travel through shared memory, or, for a split gate/up tile,
        // both halves go to the workspace
        const bool both_to_ws = split && g.dual;
        float* my_part = p.ws + (static_cast<size_t>(2 * cta) + (seg_first ? 0 : 1)) * part_floats;
        { FD_PROF_T0();
        if (both_to_ws) {
          float* dst = my_part + grp * (BN * 128);
#pragma unroll
          for (int c = 0; c < BN; ++c) dst[c * 128 + row] = acc[c];
          __threadfence();
        } else if (grp == 1) {
#pragma unroll
          for (int c = 0; c < BN; ++c) xchg[c * 128 + row] = acc[c];
        }
        if (fd_all_any(*abort_flag != 0)) {      // barrier 2 (256 threads)
          ok = false;
          break;
        }
        if (grp == 0 && et == 0) fd_stamp(p.trace, cta, pi, 3);         // segment promoted
        if (!split) {
          // ---- a whole tile: group 0's sums go to the staging buffer (group 1's are in xchg), then both groups
          // run the tile epilogue
          if (grp == 0) {
#pragma unroll
            for (int c = 0; c < BN; ++c) stage[c * 128 + row] = acc[c];
          }
          FD_PROF_ADD(xc);
          {
            FD_PROF_T0();
            if (grp == 0 && et == 0) fd_stamp(p.trace, cta, pi, 4);
            if (!fd_finish_tile<BN>(p.status, ph, sh, stage, xchg, tile, grp, ew, lane, et, T, g.dual, g.dual ? 0 : 1,
                                    norm_part, norm_ready, abort_flag, limit))
              *abort_flag = 1;
            FD_PROF_ADD(fn);
          }
        } else {
          // ---- a tile shared with other CTAs: publish the partial now; whoever arrives last finishes the tile
          // after its own segments, so that no CTA delays the parts it still owes to other tiles
          if (grp == 0) {
            if (!g.dual) {
#pragma unroll
              for (int c = 0; c < BN; ++c) my_part[c * 128 + row] = acc[c] + xchg[c * 128 + row];
              __threadfence();
              asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            if (et == 0) {
              const uint32_t tu0 = static_cast<uint32_t>(tile) * static_cast<uint32_t>(g.nkb);
              const int first_c = fd_cta_of_unit(tu0, g.U, G);
              const int last_c = fd_cta_of_unit(tu0 + g.nkb - 1, g.U, G);
              // CTAs with an empty unit range (fewer units than CTAs) contribute no part
              int nparts = 0;
              for (int j = first_c; j <= last_c; ++j)
                nparts += (static_cast<uint32_t>(j + 1) * g.U / G > static_cast<uint32_t>(j) * g.U / G) ? 1 : 0;
              const int old = atomicAdd(&p.counters[tile], 1);
              const int last = old == nparts - 1;
              if (last) p.counters[tile] = 0;
              sh->is_last = last;
              __threadfence();
            }
          }
          asm volatile("bar.sync 3, 256;" ::: "memory");     // xchg consumed, is_last visible
          if (sh->is_last != 0) pend[npend++] = tile;
          FD_PROF_ADD(xc);
        }
        }
      }

      // ---- tiles this CTA arrived last for: sum the parts in CTA order, then the tile epilogue.  With up to
      // kFdFastParts parts the loads of all parts of 8 token columns are in flight together; in a plain phase the
      // two groups share the columns, in a gate/up phase each sums its own half of the accumulators.
      if (npend > 0 && ok) asm volatile("bar.sync 3, 256;" ::: "memory");   // group 0 is done with the staging buffer
      for (int pd = 0; pd < npend && ok; ++pd) {
        const int tile = pend[pd];
        FD_PROF_T0();
        const uint32_t tu0 = static_cast<uint32_t>(tile) * static_cast<uint32_t>(g.nkb);
        const int first_c = fd_cta_of_unit(tu0, g.U, G);
        const int last_c = fd_cta_of_unit(tu0 + g.nkb - 1, g.U, G);
        const int np = last_c - first_c + 1;
        const bool fast = np <= kFdFastParts && g.U >= G;   // every CTA of the range holds a part
        const float* base0 = p.ws + (g.dual ? grp * (BN * 128) : 0) + row;
        float* dst = ((g.dual && grp == 1) ? xchg : stage) + row;
        if (fast) {
          uint32_t offs[kFdFastParts];
#pragma unroll
          for (int jj = 0; jj < kFdFastParts; ++jj) {
            const uint32_t j = static_cast<uint32_t>(first_c + jj);
            const uint32_t sj = j * g.U / static_cast<uint32_t>(G);
            offs[jj] = static_cast<uint32_t>((static_cast<size_t>(2 * j) + (sj >= tu0 ? 0 : 1)) * part_floats);
          }
          const int col0 = g.dual ? 0 : grp * (BN / 2);
          const int ncol = g.dual ? BN : BN / 2;
          if (np <= 3 && ncol >= 16) {
#pragma unroll 1
            for (int cc = 0; cc < ncol; cc += 16) fd_sum_parts<3, 16>(base0, offs, np, col0 + cc, dst);
          } else {
#pragma unroll 1
            for (int cc = 0; cc < ncol; cc += 8) fd_sum_parts<kFdFastParts, 8>(base0, offs, np, col0 + cc, dst);
          }
        } else if (grp == 0 || g.dual) {
#pragma unroll
          for (int c = 0; c < BN; ++c) acc[c] = 0.f;
          for (int j = first_c; j <= last_c; ++j) {
            const uint32_t sj = static_cast<uint32_t>(j) * g.U / static_cast<uint32_t>(G);
            if (static_cast<uint32_t>(j + 1) * g.U / static_cast<uint32_t>(G) == sj) continue;
            const float* src = base0 + (static_cast<size_t>(2 * j) + (sj >= tu0 ? 0 : 1)) * part_floats;
#pragma unroll
            for (int c = 0; c < BN; ++c) acc[c] += __ldcg(src + c * 128);
          }
#pragma unroll
          for (int c = 0; c < BN; ++c) dst[c * 128] = acc[c];
        }
        FD_PROF_ADD(pr);
        {
          FD_PROF_T0();
          if (grp == 0 && et == 0) fd_stamp(p.trace, cta, pi, 4);
          if (!fd_finish_tile<BN>(p.status, ph, sh, stage, xchg, tile, grp, ew, lane, et, T, g.dual, 0, norm_part,
                                  norm_ready, abort_flag, limit))
            *abort_flag = 1;
          FD_PROF_ADD(fn);
        }
        if (fd_all_any(*abort_flag != 0)) ok = false;
      }

      if (grp == 0) {
        // ---- publish the phase: every output of this CTA is written; arrive at the grid barrier
        if (et == 0) fd_stamp(p.trace, cta, pi, 5);           // all tiles of this CTA written
        __threadfence();
        fd_fence_proxy_async();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et == 0) {
          // Barrier k of a launch completes at base + k G.  The arrivals of a whole launch add up to kFdSyncQuantum
          // whatever the grid and the phase count (CTA 0 tops up its last arrival), so the counter is a multiple of
          // the quantum between launches and a CTA that starts late still derives the same base from it.
          unsigned long long add = 1ull;
          if (pi == p.n_phases - 1 && cta == 0) add += kFdSyncQuantum - static_cast<unsigned long long>(p.n_phases) * G;
          fd_red_release_add_u64(p.sync, add);
          fd_stamp(p.trace, cta, pi, 6);
        }
      }
    }
    if (et == 0) {
      FD_PROF_OUT(8 + grp * 4 + 0, wf); FD_PROF_OUT(8 + grp * 4 + 1, ld); FD_PROF_OUT(8 + grp * 4 + 2, fm);
      FD_PROF_OUT(20 + grp * 3 + 0, xc); FD_PROF_OUT(20 + grp * 3 + 1, pr); FD_PROF_OUT(20 + grp * 3 + 2, fn);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------- embedding + quantisation
// One CTA per token: h = table[id] * scale (bf16), E4M3 + scale per 128 columns, sum of squares per 128 columns.
__global__ void __launch_bounds__(256)
embed_quant_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ ids, __nv_bfloat16* __restrict__ h,
                   uint8_t* __restrict__ q_out, float* __restrict__ s_out, float* __restrict__ ssq_out, int ld_s, int d,
                   int vocab, float scale) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const __nv_bfloat16* src = table + static_cast<size_t>(id) * d;
  for (int blk = warp; blk < d / 128; blk += 8) {
    const int i0 = blk * 128 + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(src + i0);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    float v[4] = {__bfloat162float(a.x), __bfloat162float(a.y), __bfloat162float(b.x), __bfloat162float(b.y)};
    float amax = 0.f, ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (scale != 1.f) v[j] = fd_bf16r(v[j] * scale);
      ss += v[j] * v[j];
      const float x = fabsf(v[j]);
      if (x == x && x <= 3.0e38f) amax = fmaxf(amax, x);
    }
    uint2 hw;
    *reinterpret_cast<__nv_bfloat162*>(&hw.x) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(&hw.y) = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(h + static_cast<size_t>(t) * d + i0) = hw;
    amax = warp_max(amax);
    ss = warp_sum(ss);
    const float sc = amax > 0.f ? amax / kFdE4M3Max : 1.f;
    uint32_t q = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) q |= static_cast<uint32_t>(f32_to_e4m3(__fdiv_rn(v[j], sc))) << (8 * j);
    *reinterpret_cast<uint32_t*>(q_out + static_cast<size_t>(t) * d + i0) = q;
    if (lane == 0) {
      s_out[static_cast<size_t>(blk) * ld_s + t] = sc;
      ssq_out[static_cast<size_t>(blk) * ld_s + t] = ss;
    }
  }
}

static int fd_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
      n = v;
    else
      n = 148;
  }
  return n;
}

template <int BN>
constexpr size_t fd_smem_bytes() {
  return 1024 + 2 * kFdASlots * kFdASlotBytes + 2 * kFdBSlots * (fd_b_slot<BN>() + BN * 4) + 2 * BN * 128 * 4 +
         sizeof(FdShared);
}

template <int BN>
static int fd_launch(const FdMaps& maps, const FdParams& p, int grid, cudaStream_t stream) {
  constexpr size_t smem = fd_smem_bytes<BN>();
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(fused_decode_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return SLLM_ERR_CUDA;
    configured = true;
  }
  if (launch_kernel(fused_decode_kernel<BN>, dim3(grid), dim3(kFdThreads), smem, stream, 1u, maps, p) != cudaSuccess) {
    cudaGetLastError();
    return SLLM_ERR_CUDA;
  }
  return SLLM_OK;
}

}  // namespace sllm

using namespace sllm;

struct SllmCommDescFd {   // same layout as the descriptor of sllm_gemm_allreduce
  int world, rank;
  long long cap_elems;
  int max_tiles;
  int reserved;
  void* recv[kFdMaxWorld];
  void* flags[kFdMaxWorld];
  void* epoch;
};

static unsigned long long* g_fd_trace = nullptr;
static int g_fd_lookahead = kFdLookaheadDefault;
static int g_fd_debug = 0;
SLLM_EXPORT void sllm_fused_decode_set_debug(int bits) { g_fd_debug = bits; }
// Tuning knob: L2 prefetch distance of the weight producer in 16 KB tiles per CTA (0 = no prefetch).
SLLM_EXPORT void sllm_fused_decode_set_lookahead(int tiles) { g_fd_lookahead = tiles < 0 ? 0 : (tiles > 256 ? 256 : tiles); }
// Profiling aid: device buffer of [CTAs][4][8] u64 that subsequent launches fill with globaltimer stamps
// (0 set-up done, 1 phase input visible, 2 first accumulator ready, 3 last segment promoted, 4 last tile complete,
// 5 outputs written, 6 arrived at the barrier); null switches it off.
SLLM_EXPORT void sllm_fused_decode_set_trace(void* dev_buf) { g_fd_trace = static_cast<unsigned long long*>(dev_buf); }

SLLM_EXPORT long long sllm_fused_decode_ws_floats(int grid) {
  if (grid <= 0) grid = fd_sm_count();
  return static_cast<long long>(2) * grid * 2 * 32 * 128;
}

SLLM_EXPORT int sllm_fused_decode(const SllmFdDesc* d, void* stream) {
  if (!d || d->n_phases < 1 || d->n_phases > SLLM_FD_MAX_PHASES || d->rows < 1 || d->rows > 32 || !d->ws ||
      !d->counters || !d->sync)
    return SLLM_ERR_INVALID_ARGUMENT;
  const int bn = d->rows <= 16 ? 16 : 32;
  const int grid = d->grid > 0 ? d->grid : fd_sm_count();
  if (static_cast<unsigned long long>(grid) * SLLM_FD_MAX_PHASES > kFdSyncQuantum) return SLLM_ERR_UNSUPPORTED_SHAPE;
  if (d->ws_floats < sllm_fused_decode_ws_floats(grid)) return SLLM_ERR_WORKSPACE_TOO_SMALL;
  FdMaps maps;
  FdParams p;
  memset(&p, 0, sizeof(p));
  p.n_phases = d->n_phases;
  p.rows = d->rows;
  p.rope = d->rope;
  p.ws = d->ws; p.counters = d->counters; p.sync = d->sync; p.status = d->status;
  p.wait_limit = d->wait_limit_cycles > 0 ? d->wait_limit_cycles : kWaitLimitCycles;
  p.trace = g_fd_trace;
  p.lookahead = g_fd_lookahead;
  p.debug = g_fd_debug;
  for (int i = 0; i < d->n_phases; ++i) {
    const SllmFdPhase& ph = d->phase[i];
    if (!ph.w || !ph.w_scale || !ph.x || !ph.x_scale || ph.n <= 0 || ph.k <= 0 || (ph.k & 127) || (ph.n & 3))
      return SLLM_ERR_INVALID_ARGUMENT;
    const int tiles = (ph.n + 127) / 128;
    if (tiles > d->n_counters) return SLLM_ERR_WORKSPACE_TOO_SMALL;
    if (static_cast<long long>(tiles) * (ph.k / 128) * (grid + 1) >= (1LL << 31)) return SLLM_ERR_UNSUPPORTED_SHAPE;
    if (ph.ld_sb < bn || (ph.ld_sb & 3) || (ph.ld_sa & 3) || ph.ld_sa < ph.dual_off + ph.n) return SLLM_ERR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(ph.w_scale) & 15) || (reinterpret_cast<uintptr_t>(ph.x_scale) & 15))
      return SLLM_ERR_ALIGNMENT;
    if (ph.norm_tiles > 0 && (!ph.ssq_in || ph.norm_dim <= 0)) return SLLM_ERR_INVALID_ARGUMENT;
    switch (ph.epilogue) {
      case SLLM_FD_PLAIN:
        if (!ph.y || ph.dual_off || (ph.ldy & 3)) return SLLM_ERR_INVALID_ARGUMENT;
        break;
      case SLLM_FD_RESID_QUANT:
        if (!ph.y || !ph.residual || !ph.q_out || !ph.s_out || ph.dual_off || (ph.n & 127) || (ph.ldy & 3) ||
            ph.ld_s_out < d->rows)
          return SLLM_ERR_INVALID_ARGUMENT;
        break;
      case SLLM_FD_SILU_QUANT:
        if (!ph.q_out || !ph.s_out || ph.dual_off < ph.n || (ph.dual_off & 3) || (ph.n & 127) || ph.ld_s_out < d->rows)
          return SLLM_ERR_INVALID_ARGUMENT;
        break;
      case SLLM_FD_ROPE_KV: {
        const SllmFdRope& r = d->rope;
        if (!ph.y || ph.dual_off || (ph.ldy & 3) || !r.positions || !r.seq_index || !r.block_table || !r.k_pages ||
            !r.v_pages || r.hq <= 0 || r.hkv <= 0 || ph.n != (r.hq + 2 * r.hkv) * 128 || r.page_size <= 0)
          return SLLM_ERR_INVALID_ARGUMENT;
        if (r.rotary_dim != 32 && r.rotary_dim != 64 && r.rotary_dim != 128) return SLLM_ERR_UNSUPPORTED_SHAPE;
        if (!r.inv_freq) return SLLM_ERR_INVALID_ARGUMENT;     // [rotary_dim / 2] frequencies, computed by the caller
        if (r.kv_fp8 && (r.k_static <= 0.f || r.v_static <= 0.f) && (!r.k_scale || !r.v_scale))
          return SLLM_ERR_INVALID_ARGUMENT;
        break;
      }
      default:
        return SLLM_ERR_INVALID_ARGUMENT;
    }
    p.ph[i] = ph;
    int rc = cached_kmajor_tmap(&maps.a[i], ph.w, 1, ph.dual_off + ph.n, ph.k, ph.k, 128);
    if (rc != SLLM_OK) return rc;
    rc = cached_kmajor_tmap(&maps.b[i], ph.x, 1, d->rows, ph.k, ph.k, bn);
    if (rc != SLLM_OK) return rc;
  }
  for (int i = d->n_phases; i < SLLM_FD_MAX_PHASES; ++i) { maps.a[i] = maps.a[0]; maps.b[i] = maps.b[0]; }
  if (d->comm) {
    const SllmCommDescFd* c = static_cast<const SllmCommDescFd*>(d->comm);
    if (c->world < 2 || c->world > kFdMaxWorld || c->rank < 0 || c->rank >= c->world || !c->epoch)
      return SLLM_ERR_INVALID_ARGUMENT;
    for (int i = 0; i < d->n_phases; ++i) {
      if (d->phase[i].epilogue != SLLM_FD_RESID_QUANT) continue;
      const long long tiles = (d->phase[i].n + 127) / 128;
      if (tiles > c->max_tiles || tiles * 128 * bn > c->cap_elems) return SLLM_ERR_WORKSPACE_TOO_SMALL;
    }
    p.comm.world = c->world; p.comm.rank = c->rank; p.comm.cap_elems = c->cap_elems;
    for (int i = 0; i < c->world; ++i) {
      if (!c->recv[i] || !c->flags[i]) return SLLM_ERR_INVALID_ARGUMENT;
      p.comm.recv[i] = static_cast<__nv_bfloat16*>(c->recv[i]);
      p.comm.flags[i] = static_cast<uint32_t*>(c->flags[i]);
    }
    p.comm.epoch = static_cast<uint32_t*>(c->epoch);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return bn == 16 ? fd_launch<16>(maps, p, grid, st) : fd_launch<32>(maps, p, grid, st);
}

SLLM_EXPORT int sllm_embed_quant(const void* table, const int* ids, void* h, void* q_out, float* s_out, float* ssq_out,
                                 int ld_s, int rows, int d, int vocab, float scale, void* stream) {
  if (!table || !ids || !h || !q_out || !s_out || !ssq_out || rows <= 0 || d <= 0 || (d & 127) || ld_s < rows || vocab <= 0)
    return SLLM_ERR_INVALID_ARGUMENT;
  launch_kernel(embed_quant_kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream), 1u,
                static_cast<const __nv_bfloat16*>(table), ids, static_cast<__nv_bfloat16*>(h),
                static_cast<uint8_t*>(q_out), s_out, ssq_out, ld_s, d, vocab, scale);
  return cudaGetLastError() == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

SLLM_EXPORT int sllm_fused_decode_abi(int* out, int n) {
  const int rec[] = {
      static_cast<int>(sizeof(SllmFdPhase)), static_cast<int>(offsetof(SllmFdPhase, eps)),
      static_cast<int>(offsetof(SllmFdPhase, w)), static_cast<int>(offsetof(SllmFdPhase, ssq_out)),
      static_cast<int>(sizeof(SllmFdRope)), static_cast<int>(offsetof(SllmFdRope, theta)),
      static_cast<int>(offsetof(SllmFdRope, k_pages)), static_cast<int>(offsetof(SllmFdRope, inv_freq)),
      static_cast<int>(sizeof(SllmFdDesc)), static_cast<int>(offsetof(SllmFdDesc, phase)),
      static_cast<int>(offsetof(SllmFdDesc, rope)), static_cast<int>(offsetof(SllmFdDesc, ws)),
      static_cast<int>(offsetof(SllmFdDesc, sync)), static_cast<int>(offsetof(SllmFdDesc, comm)),
      static_cast<int>(offsetof(SllmFdDesc, wait_limit_cycles)),
      static_cast<int>(sizeof(SllmCommDescFd)), static_cast<int>(offsetof(SllmCommDescFd, recv)),
      static_cast<int>(offsetof(SllmCommDescFd, epoch)),
  };
  const int have = static_cast<int>(sizeof(rec) / sizeof(rec[0]));
  for (int i = 0; i < n && i < have; ++i) out[i] = rec[i];
  return have;
}
