// tcgen05 / TMEM / TMA GEMM for sm_100a:  D[a, b] = sum_k A[a, k] * B[b, k]
//
// Both operands are K-major (row-major with K contiguous), which is how activations [M, K] and
// weights [N, K] are stored, so no transpose is ever materialised.  The 128-row operand A fills the
// tensor-core M dimension; B supplies BN in {16, 32, 64, 128} columns.  Callers pick which tensor
// plays which role:
//   * prefill (many tokens): A = activations, B = weights, Y[a, b]            (transpose_out = 0)
//   * decode  (few tokens) : A = weights, B = activations, Y[b, a] ("swap-AB", transpose_out = 1)
//     so a batch of 1..128 tokens still drives full 128-row MMAs and the kernel streams the weight
//     matrix once at HBM rate.
// Two numeric modes:
//   * bf16 x bf16 -> fp32 accumulate in TMEM over the whole K range (kind::f16)
//   * E4M3 x E4M3 with fp32 scales per 128-element K block on both operands (the 1x128 block-scaled
//     FP8 format).  Each K block is accumulated in its own TMEM buffer (double buffered) and promoted
//     into fp32 registers with scaleA[kb, a] * scaleB[kb, b] by the epilogue warps while the tensor
//     core works on the next block.
// Split-K: gridDim.z CTAs share one output tile; each writes its fp32 partial to a workspace, bumps
// a per-tile counter, and the CTA that arrives last sums the partials in split order (deterministic)
// and writes the tile.  No CTA ever waits for another one.
//
// Fused all-reduce (tensor-parallel row-parallel projections): with a communicator attached, the CTA
// that holds a finished tile of this rank's partial product pushes it (bf16) straight into every
// peer's receive buffer with plain NVLink stores, raises a per-(tile, source) flag on the peer,
// waits (bounded) for the peers' flags for the same tile, and sums the world's partials in rank order
// before the usual residual/store epilogue - one kernel, tile-granular overlap of transfer and MMA,
// bit-identical results on every rank.  Receive buffers are double-buffered by call parity; epochs
// are per-tile device counters so CUDA-graph replays need no host-side argument changes.
//
// Warp roles: warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..5 = epilogue (TMEM lane
// quarter = warp index % 4), warps 6.. = further MMA issuers.  One thread spends about 160 cycles per
// tcgen05.mma whatever its shape, which is more than the tensor core needs for a 128x128 tile and far more
// than for a decode tile; issuers in different warps overlap, so K blocks are dealt round-robin to
// gemm_issuers(BN) issuing threads, each K block (scaled) or each issuer (unscaled) with its own TMEM
// accumulator out of four.
//
// Replaces the reference's scalar-FMA matmul family and its library GEMM calls
// (native/hip/src/matmul_kernel.hip.cpp:586-830, native/hip/src/matmul_runtime.inc:690).
#include <cstdio>
#include "common.cuh"
#include "api.h"
#include "epilogue_columns.cuh"
#include <cudaTypedefs.h>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

namespace sllm {

constexpr int kTileA = 128;        // rows of the A operand per CTA (tensor-core M)
constexpr int kBoxBytes = 128;     // K bytes per pipeline stage row (one 128-byte swizzle row)
constexpr int kMaxStages = 8;
constexpr int kAccBufs = 4;        // TMEM accumulators of BN columns each
// MMA-issuing threads per CTA.  BN = 64 keeps one: its epilogue needs the registers that two CTAs per SM of
// 192 threads leave.  The stage count and kAccBufs are multiples of the issuer count, so a pipeline stage and
// a TMEM accumulator always belong to the same issuer: a parity wait is only sound when the waiter has
// itself seen the barrier's previous phase complete, and TMA loads in flight together may land out of order.
__host__ __device__ constexpr int gemm_issuers(int bn) { return bn == 64 ? 1 : 2; }
__host__ __device__ constexpr int gemm_threads(int bn) { return 192 + 32 * (gemm_issuers(bn) - 1); }

constexpr int kMaxWorld = 8;
constexpr int kMaxSlices = 8;   // cluster split-K slices per tile (flag / epoch slots per tile)

struct CommParams {
  int world, rank;
  long long cap_elems;                 // bf16 elements per (buffer, source) region
  __nv_bfloat16* recv[kMaxWorld];      // recv[p]: base of rank p's receive buffer [2][world][cap_elems]
  uint32_t* flags[kMaxWorld];          // flags[p]: base of rank p's flag array [max_tiles * kMaxSlices][world]
  uint32_t* epoch;                     // local call counters [max_tiles * kMaxSlices]
};

// All-gather fused into a column-parallel GEMM: the K range of the B operand (activations) is spread over the
// ranks, K blocks [src * kb_per_rank, (src + 1) * kb_per_rank) live in rank src's symmetric buffer.  The producer
// reads them straight out of peer memory with plain (non-multicast) TMA loads, own shard first, after a bounded
// wait on the flag the owner raises when its shard is written; the MMAs of the shards that have arrived run while
// the later ones cross NVLink.
struct GatherParams {
  int world, rank;
  int kb_per_rank;
  const CUtensorMap* maps;   // device array [world]: maps[src] covers rank src's shard [b_rows, K / world]
  const uint32_t* flags;     // local [world]: flags[src] = last epoch rank src published
  const uint32_t* epoch;     // local: the epoch this call consumes
};

// Fused row epilogue of a decode GEMM (swap-AB, block-scaled FP8, cluster split-K or no split): the work of the
// kernels that used to follow the projection happens on the fp32 sums of each token row (epilogue_columns.cuh).
// SILU_QUANT expects the gate / up weight rows interleaved per tile (rows 0..63 gate, 64..127 up of the same 64
// features) and a cluster of two tiles along x: the two CTAs exchange the row maxima of their 64 features so that
// the 128 features they cover share one E4M3 scale.
struct FusedEpi {
  int mode;            // 0 = off, else SllmFdEpilogue + 1
  int n;               // logical outputs per row (SILU_QUANT: the gated width)
  int norm_tiles, norm_dim;
  float eps, softcap;
  int act, ld_s;
  const float* ssq_in;
  uint8_t* q_out;
  float* s_out;
  float* ssq_out;
  const float* inv_freq;
  SllmFdRope rope;
};

struct GemmParams {
  int a_rows, b_rows;
  int num_kb;          // K blocks (of kBoxBytes) over the whole K range
  int kb_per_split;    // K blocks handled by one blockIdx.z
  int stages;
  int transpose_out;   // 0: Y[a, b]; 1: Y[b, a]
  int ldy;
  int ld_sa, ld_sb;    // leading dimensions of the kb-major scale arrays
  int epilogue;        // 0 = store, 1 = add residual
  int cluster_split;   // 1: gridDim.z CTAs form one cluster and reduce split-K partials over DSMEM
  int const_operand;   // operand that no kernel writes (weights): 0 none, 1 A, 2 B; loaded before the PDL wait
  int early_trigger;   // 1: dependents may become resident as soon as this CTA holds its resources
  const float* scale_a;  // [num_kb, ld_sa]
  const float* scale_b;  // [num_kb, ld_sb]
  __nv_bfloat16* y;
  const __nv_bfloat16* residual;
  float* ws;           // split-K partials
  int* counters;       // one per output tile, zero between launches
  int* status;         // device status word (0 = ok)
  CommParams comm;     // used by the kComm instantiation only
  GatherParams gather; // world > 1: B operand gathered from the peers (unscaled GEMM only)
  FusedEpi fe;         // mode != 0: fused row epilogue (scaled, swap-AB launches)
  STEP_TRACE_FIELD
};

#ifdef SLLM_TRACE
// Development-only phase timestamps of CTA (0,0,0) (globaltimer ns); never compiled into the product.
__device__ unsigned long long g_trace[32];
__device__ __forceinline__ void trace_mark(int slot) {
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_trace[slot] = t;
  }
}
#define TRACE(slot) trace_mark(slot)
#else
#define TRACE(slot)
#endif

constexpr int kScaleChunk = 16;  // K blocks of scales staged in shared memory at a time

template <int BN>
struct __align__(16) GemmBarriers {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[kAccBufs];
  uint64_t tmem_empty[kAccBufs];
  uint32_t tmem_base;
  int abort_flag;
  int is_last;
  uint32_t epoch;
  float famax[128];       // fused SiLU epilogue: row maxima of this tile ...
  float famax_peer[128];  // ... and of the other tile of the scale block, written by that tile's CTA over DSMEM
  float inv_freq[64];     // fused rotary epilogue: the frequency table, staged while the main loop runs
};

template <int BN>
struct __align__(16) GemmScales {
  float sa[2][kScaleChunk][kTileA];
  float sb[2][kScaleChunk][BN];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// 4-byte async copy global -> shared; src_bytes == 0 writes zero instead of reading.
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Store into the shared memory of CTA `cta_rank` of the cluster, at the address `local_ptr` has in this CTA.
// Partials travel by stores (fire and forget, made visible by the cluster barrier that follows) rather than by
// loads, whose round trips over the cluster network would sit on the critical path one after another.
__device__ __forceinline__ void st_dsmem_f32(float* local_ptr, uint32_t cta_rank, float v) {
  uint32_t ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(local_ptr)), "r"(cta_rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(ra), "f"(v) : "memory");
}

template <int BN, bool kScaled, bool kComm>
// Two CTAs per SM for the decode tiles (BN <= 64): 128 registers a thread and at most ~110 KB of shared memory each.
// Measured: with the pipeline deepened to fill one CTA's 227 KB the same grids run a third slower (the second CTA of
// an SM hides the first one's start-up, reduction and exit), although the occupancy query reports one CTA per SM for
// every kernel that allocates tensor memory.
__global__ void __launch_bounds__((BN <= 64 ? 256 : gemm_threads(BN)), (BN <= 64 ? 2 : 1))
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // Tiles need 1024-byte alignment for the 128-byte swizzle atom.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kABytes = kTileA * kBoxBytes;
  constexpr int kBBytes = BN * kBoxBytes;
  constexpr int kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = (kAccBufs * BN < 32) ? 32 : kAccBufs * BN;
  constexpr int kIssuers = gemm_issuers(BN);
  constexpr int kElemsPerBox = kScaled ? 128 : 64;
  GemmBarriers<BN>* bars = reinterpret_cast<GemmBarriers<BN>*>(smem + p.stages * kStageBytes);
  GemmScales<BN>* sc = reinterpret_cast<GemmScales<BN>*>(bars + 1);
  // Output staging in the drained pipeline memory: red[(s * cw + cl) * 128 + row] = the partial of K slice s for
  // column c0 + cl of this CTA's column slice [c0, c0 + cw) (one slice s = 0 holding all BN columns without a
  // cluster split).
  float* red = reinterpret_cast<float*>(smem);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int a_tile = blockIdx.x, b_tile = blockIdx.y, split = blockIdx.z;
  const int kb0 = split * p.kb_per_split;
  int nkb = p.num_kb - kb0;
  if (nkb > p.kb_per_split) nkb = p.kb_per_split;
  if (nkb < 0) nkb = 0;
  volatile int* abort_flag = &bars->abort_flag;
  const bool cluster_split = p.cluster_split != 0;
  if (threadIdx.x == 0) TRACE(0);
  STEP_TRACE_START(p);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < kAccBufs; ++b) {
      mbar_init(&bars->tmem_full[b], 1);
      mbar_init(&bars->tmem_empty[b], 128);
    }
    bars->abort_flag = 0;
    bars->is_last = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  if (threadIdx.x == 0) TRACE(1);
  // With the early trigger the next kernel's CTAs become resident while this one runs (where shared memory and
  // TMEM allow): their set-up and the first ring of weight tiles then overlap this kernel instead of following it.
  if (p.early_trigger && threadIdx.x == 0) pdl_trigger();

  // Epilogue-thread coordinates (meaningful for warps 2..5 only).
  const int q = warp & 3;              // TMEM lane quarter this warp may read
  const int row = q * 32 + lane;       // row of the A tile
  const int et = threadIdx.x - 64;     // 0..127
  const int a_row = a_tile * kTileA + row;
  float acc[BN];
  bool ok = true;
  bool active = true;   // this CTA takes part in the output phase (false for non-final global split-K CTAs)
  float rn_lane = 1.f;  // fused row epilogue: RMSNorm factor of token row `lane`
  int my_pos = 0, my_page = 0;  // fused rotary epilogue: position and KV page of token row c0 + lane of this CTA's slice

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int issued = 0;
      // The constant operand (the weights) of the first ring of stages is requested before waiting for
      // the previous kernel, so its HBM latency overlaps that kernel's tail; the dependent operand
      // (activations) follows after the wait.
      const int pre = nkb < p.stages ? nkb : p.stages;
      const bool gather = p.gather.world > 1;
      // gathered K blocks are visited own shard first, then the peers in ring order
      auto kmap = [&](int j) {
        if (!gather) return j;
        int kb = j + p.gather.rank * p.gather.kb_per_rank;
        return kb >= p.num_kb ? kb - p.num_kb : kb;
      };
      int gather_ready = gather ? p.gather.rank : -1;      // the last source whose flag has been seen
      // the epoch is written by the publishing kernel just before this one: it is read on the first gathered
      // load, which comes after the wait for that kernel
      uint32_t gather_epoch = 0u;
      bool gather_have_epoch = false, gather_ok = true;
      auto load_a = [&](int i, int s) {
        tma_load_2d(smem + s * kStageBytes, &tm_a, &bars->full[s], kmap(kb0 + i) * kElemsPerBox, a_tile * kTileA);
      };
      auto load_b = [&](int i, int s) {
        if (gather) {
          const int kb = kmap(kb0 + i);
          const int src = kb / p.gather.kb_per_rank;
          if (!gather_have_epoch) {
            gather_epoch = *reinterpret_cast<const volatile uint32_t*>(p.gather.epoch);
            gather_have_epoch = true;
          }
          if (src != gather_ready) {
            // bounded wait for the owner's flag, then order the TMA (async proxy) reads after it
            uint32_t spins = 0;
            long long t0 = 0;
            while (gather_ok && static_cast<int32_t>(ld_acquire_sys(p.gather.flags + src) - gather_epoch) < 0) {
              ++spins;
              if (spins == 1024) t0 = clock64();
              if (spins > 1024 && (spins & 63) == 0 && clock64() - t0 > kWaitLimitCycles) {
                if (p.status) atomicCAS(p.status, 0, SLLM_DEV_TIMEOUT_PEER_FLAG);
                gather_ok = false;
              }
            }
            asm volatile("fence.proxy.async;" ::: "memory");
            gather_ready = src;
          }
          // a shard that never arrived is replaced by this rank's own rows: the result is wrong, the status word
          // says so, and every barrier still completes
          const int from = gather_ok ? src : p.gather.rank;
          // two buffers per rank, chosen by the parity of the epoch: maps[parity][source]
          tma_load_2d(smem + s * kStageBytes + kABytes, p.gather.maps + (gather_epoch & 1u) * p.gather.world + from,
                      &bars->full[s],
                      (kb - src * p.gather.kb_per_rank) * kElemsPerBox, b_tile * BN);
          return;
        }
        tma_load_2d(smem + s * kStageBytes + kABytes, &tm_b, &bars->full[s], (kb0 + i) * kElemsPerBox, b_tile * BN);
      };
      if (p.const_operand != 0) {
        for (int i = 0; i < pre; ++i) {
          mbar_expect_tx(&bars->full[i], kStageBytes);
          if (p.const_operand == 1) load_a(i, i); else load_b(i, i);
        }
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i) {
        if (p.const_operand == 0) {
          mbar_expect_tx(&bars->full[i], kStageBytes);
          load_a(i, i);
          load_b(i, i);
        } else if (p.const_operand == 1) {
          load_b(i, i);
        } else {
          load_a(i, i);
        }
        issued = i + 1;
      }
      for (int i = pre; i < nkb; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (i / p.stages) & 1;
        if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_SMEM_EMPTY)) break;
        mbar_expect_tx(&bars->full[s], kStageBytes);
        load_a(i, s);
        load_b(i, s);
        issued = i + 1;
      }
      pdl_trigger();
      // Drain: every copy this thread started must have landed before the CTA may exit.  On the
      // normal path these phases are already complete and the waits return at once.
      for (int s = 0; s < p.stages; ++s) {
        const int fills = (issued > s) ? (issued - s + p.stages - 1) / p.stages : 0;
        if (fills > 0) {
          int dummy_abort = 0;
          mbar_wait(&bars->full[s], (fills - 1) & 1, &dummy_abort, p.status, SLLM_DEV_TIMEOUT_DRAIN, 200000000LL);
        }
      }
    }
  } else if (warp == 1 || warp >= 6) {
    // ------------------------------------------------------------ MMA issuers
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(kScaled ? kFmtE4M3 : kFmtBf16, kTileA, BN);
      const int iw = warp == 1 ? 0 : warp - 5;
      bool issued_any = false;
      for (int i = iw; i < nkb; i += kIssuers) {
        const int s = i % p.stages;
        const uint32_t ph = (i / p.stages) & 1;
        if (!mbar_wait(&bars->full[s], ph, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMA_FULL)) break;
        if (i == 0) TRACE(2);
        if (i == nkb - 1) TRACE(3);
        // scaled: one accumulator per K block (the epilogue promotes it); unscaled: one per issuer
        const int buf = kScaled ? (i % kAccBufs) : iw;
        if (kScaled) {
          if (!mbar_wait(&bars->tmem_empty[buf], ((i / kAccBufs) & 1) ^ 1, abort_flag, p.status,
                         SLLM_DEV_TIMEOUT_TMEM_EMPTY))
            break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + s * kStageBytes);
        const uint64_t adesc = make_smem_desc_sw128(sa);
        const uint64_t bdesc = make_smem_desc_sw128(sa + kABytes);
        const uint32_t d = tmem_base + buf * BN;
#pragma unroll
        for (int k = 0; k < 4; ++k) {  // 4 x 32 bytes of K per stage row
          const uint32_t accum = kScaled ? (k > 0) : ((i > iw) || (k > 0));
          if (kScaled)
            umma_f8(d, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
          else
            umma_f16(d, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
        }
        tc_commit(&bars->empty[s]);  // stage reusable once these MMAs have read it
        if (kScaled) tc_commit(&bars->tmem_full[buf]);
        issued_any = true;
      }
      if (!kScaled && issued_any) tc_commit(&bars->tmem_full[iw]);
    }
  } else {
    // ------------------------------------------------------------ epilogue main loop (128 threads)
    pdl_wait();
    if (threadIdx.x == 64) STEP_TRACE_WAITED(p);
    if constexpr (kScaled && BN <= 32) {
      // norm factor of every token row from the sums of squares its producer wrote: requested now, used after the
      // last K block, so the L2 round trip hides under the main loop
      if (p.fe.mode != 0 && p.fe.norm_tiles > 0 && lane < p.b_rows) {
        float ss = 0.f;
        for (int i = 0; i < p.fe.norm_tiles; ++i) ss += __ldcg(p.fe.ssq_in + static_cast<size_t>(i) * p.fe.ld_s + lane);
        rn_lane = rsqrtf(ss / static_cast<float>(p.fe.norm_dim) + p.fe.eps);
      }
      if (p.fe.mode == SLLM_FD_ROPE_KV + 1) {
        // position -> page walk (three dependent loads) and the frequency table: also requested now
        const int cwp = cluster_split ? BN / static_cast<int>(gridDim.z) : BN;
        const int c0p = cluster_split ? split * cwp : 0;
        if (lane < cwp && c0p + lane < p.b_rows) {
          my_pos = p.fe.rope.positions[c0p + lane];
          my_page = p.fe.rope.block_table[static_cast<size_t>(p.fe.rope.seq_index[c0p + lane]) * p.fe.rope.max_blocks +
                                          my_pos / p.fe.rope.page_size];
        }
        if (et < 64) bars->inv_freq[et] = et < (p.fe.rope.rotary_dim >> 1) ? p.fe.inv_freq[et] : 0.f;
      }
    }
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
    for (int c = 0; c < BN; ++c) acc[c] = 0.f;

    if (kScaled) {
      // Scales of 16 K blocks at a time are staged in shared memory with cp.async (double buffered),
      // so no global-memory latency sits on the per-block critical path.
      const int b_row0 = b_tile * BN;
      auto stage_scales = [&](int chunk, int buf) {
        const int base_kb = kb0 + chunk * kScaleChunk;
        int cnt = kb0 + nkb - base_kb;
        if (cnt > kScaleChunk) cnt = kScaleChunk;
        for (int j = 0; j < cnt; ++j) {
          const bool in = a_row < p.a_rows;
          cp_async4(&sc->sa[buf][j][row], p.scale_a + static_cast<size_t>(base_kb + j) * p.ld_sa + (in ? a_row : 0),
                    in ? 4 : 0);
        }
        for (int idx = et; idx < cnt * BN; idx += 128) {
          const int j = idx / BN, c = idx % BN;
          const bool in = b_row0 + c < p.b_rows;
          cp_async4(&sc->sb[buf][j][c], p.scale_b + static_cast<size_t>(base_kb + j) * p.ld_sb + (in ? b_row0 + c : 0),
                    in ? 4 : 0);
        }
      };
      const int nchunks = (nkb + kScaleChunk - 1) / kScaleChunk;
      if (nchunks > 0) stage_scales(0, 0);
      cp_async_wait_all();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      for (int ci = 0; ci < nchunks; ++ci) {
        const int sbuf = ci & 1;
        if (ci + 1 < nchunks) stage_scales(ci + 1, sbuf ^ 1);
        int cnt = nkb - ci * kScaleChunk;
        if (cnt > kScaleChunk) cnt = kScaleChunk;
        for (int j = 0; j < cnt; ++j) {
          const int i = ci * kScaleChunk + j;
          const int buf = i % kAccBufs;
          const float sa = sc->sa[sbuf][j][row];
          if (ok) ok = mbar_wait(&bars->tmem_full[buf], (i / kAccBufs) & 1, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMEM_FULL);
          if (et == 0 && i == 0) TRACE(4);
          if (et == 0 && i == 1) TRACE(5);
          if (et == 0 && i == nkb - 1) TRACE(6);
          if (ok) {
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < BN / 16; ++c) {
              uint32_t r[16];
              tmem_ld16(lane_addr + buf * BN + c * 16, r);
              tmem_wait_ld();
#pragma unroll
              for (int jj = 0; jj < 16; ++jj)
                acc[c * 16 + jj] = fmaf(__uint_as_float(r[jj]), sa * sc->sb[sbuf][j][c * 16 + jj], acc[c * 16 + jj]);
            }
            tc_fence_before();
            mbar_arrive(&bars->tmem_empty[buf]);
          }
        }
        cp_async_wait_all();
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
    } else {
      // one partial accumulator per issuer that had at least one K block
#pragma unroll
      for (int a = 0; a < kIssuers; ++a) {
        if (a < nkb && ok) {
          ok = mbar_wait(&bars->tmem_full[a], 0, abort_flag, p.status, SLLM_DEV_TIMEOUT_TMEM_FULL);
          if (ok) {
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < BN / 16; ++c) {
              uint32_t r[16];
              tmem_ld16(lane_addr + a * BN + c * 16, r);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[c * 16 + j] += __uint_as_float(r[j]);
            }
            tc_fence_before();
          }
        }
      }
    }
    // ---- global split-K fix-up (more than 8 splits, or clusters unavailable): the CTA that arrives
    // last for this tile sums all partials in split order; nobody waits.
    if (!cluster_split && gridDim.z > 1) {
      const int tile_id = a_tile * gridDim.y + b_tile;
      float* my = p.ws + (static_cast<size_t>(tile_id) * gridDim.z + split) * (BN * kTileA);
#pragma unroll
      for (int c = 0; c < BN; ++c) my[c * kTileA + row] = acc[c];
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (et == 0) {
        const int old = atomicAdd(&p.counters[tile_id], 1);
        const int last = (old == static_cast<int>(gridDim.z) - 1);
        if (last) p.counters[tile_id] = 0;  // ready for the next launch
        bars->is_last = last;
        __threadfence();
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      active = bars->is_last != 0;
      if (active) {
        const float* base = p.ws + static_cast<size_t>(tile_id) * gridDim.z * (BN * kTileA);
#pragma unroll
        for (int c = 0; c < BN; ++c) acc[c] = 0.f;
        for (int s = 0; s < static_cast<int>(gridDim.z); ++s) {
          const float* src = base + static_cast<size_t>(s) * (BN * kTileA);
#pragma unroll
          for (int c = 0; c < BN; ++c) acc[c] += __ldcg(src + c * kTileA + row);
        }
      }
    }
    // Without a cluster split the fp32 tile is parked in this CTA's shared memory as red[column][row] (the
    // pipeline stages are drained by now); the output phase below works on 16-byte units out of this buffer.
    if (!cluster_split) {
      if (active) {
#pragma unroll
        for (int c = 0; c < BN; ++c) red[c * kTileA + row] = acc[c];
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
  }

  if (threadIdx.x == 64) TRACE(7);
  constexpr bool kFusable = kScaled && BN <= 32;      // instantiations that carry the fused row epilogue
  const bool pair_x = kFusable && p.fe.mode == SLLM_FD_SILU_QUANT + 1;     // cluster of two tiles along x (no K split)
  if (cluster_split) {
    // Cluster split-K: CTA j of the cluster finishes the columns [j cw, (j + 1) cw) of the tile.  Once every CTA's
    // pipeline memory is drained (first barrier), each CTA stores its partial of those columns straight into CTA j's
    // staging buffer, slot = its own K slice; after the second barrier every CTA sums its slots out of its OWN
    // shared memory and nothing reads another CTA's memory again, so CTAs leave without a closing barrier.
    cluster_sync_all();
    if (warp >= 2 && warp < 6) {
      const int cwp = BN / static_cast<int>(gridDim.z);       // a power of two
      const int sh = 31 - __clz(cwp);
#pragma unroll
      for (int c = 0; c < BN; ++c)
        st_dsmem_f32(red + (split * cwp + (c & (cwp - 1))) * kTileA + row, static_cast<uint32_t>(c >> sh), acc[c]);
    }
    cluster_sync_all();
  }
  if (threadIdx.x == 64) TRACE(8);

  if (kFusable && p.fe.mode != 0) {
    // ------------------------------------------------------------ fused row epilogue
    // Each CTA finishes the token rows [c0, c0 + cw) of its tile (all of them without a K split): a warp sums the
    // cluster's partials of one row over DSMEM (lane l: outputs 4 l .. 4 l + 3), applies the norm factor and runs
    // the row epilogue.
    const FusedEpi& fe = p.fe;
    const int nslice = cluster_split ? static_cast<int>(gridDim.z) : 1;
    const int cw = BN / nslice;
    const int c0 = (cluster_split ? split : 0) * cw;
    const int T = p.b_rows;
    const int ew = warp - 2;
    const bool epi_warp = warp >= 2 && warp < 6 && active && ok;
    if (epi_warp) {
      ColEpilogue e;
      e.mode = fe.mode - 1; e.n = fe.n; e.ldy = p.ldy; e.ld_s = fe.ld_s; e.softcap = fe.softcap;
      e.y = p.y; e.residual = p.residual;
      e.q_out = fe.q_out; e.s_out = fe.s_out; e.ssq_out = fe.ssq_out;
      e.rope = &fe.rope; e.inv_freq = bars->inv_freq;
      [[maybe_unused]] uint32_t comm_epoch = 0;
      [[maybe_unused]] long long comm_region = 0, comm_toff = 0;
      [[maybe_unused]] bool comm_ok = true;
      if constexpr (kComm) {
        // ---- tensor parallelism: this rank's partial of every row of the slice goes (bf16) to all ranks, then
        // flags, a bounded wait for the peers' flags, and below the rows are summed in rank order
        const CommParams& cm = p.comm;
        const int tile_id = a_tile * gridDim.y + b_tile;
        const int slot = tile_id * kMaxSlices + (cluster_split ? split : 0);
        if (et == 0) {
          const uint32_t e1 = cm.epoch[slot] + 1;
          cm.epoch[slot] = e1;
          bars->epoch = e1;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        comm_epoch = bars->epoch;
        comm_region = static_cast<long long>(comm_epoch & 1) * cm.world;
        comm_toff = static_cast<long long>(tile_id) * (kTileA * BN);
        for (int cl = ew; cl < cw; cl += 4) {
          const int col = c0 + cl;
          if (col >= T) break;
          const float* src = red + cl * kTileA + lane * 4;
          float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int s = 0; s < nslice; ++s) {
            const float4 x = *reinterpret_cast<const float4*>(src + s * cw * kTileA);
            sum.x += x.x; sum.y += x.y; sum.z += x.z; sum.w += x.w;
          }
          uint2 w;
          *reinterpret_cast<__nv_bfloat162*>(&w.x) = __floats2bfloat162_rn(sum.x, sum.y);
          *reinterpret_cast<__nv_bfloat162*>(&w.y) = __floats2bfloat162_rn(sum.z, sum.w);
          const long long off = (comm_region + cm.rank) * cm.cap_elems + comm_toff + col * kTileA + lane * 4;
          for (int peer = 0; peer < cm.world; ++peer) *reinterpret_cast<uint2*>(cm.recv[peer] + off) = w;
        }
        __threadfence_system();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et < cm.world && et != cm.rank) {
          st_release_sys(cm.flags[et] + static_cast<size_t>(slot) * cm.world + cm.rank, comm_epoch);
          const uint32_t* f = cm.flags[cm.rank] + static_cast<size_t>(slot) * cm.world + et;
          uint32_t spins = 0;
          long long t0 = 0;
          while (static_cast<int32_t>(ld_acquire_sys(f) - comm_epoch) < 0) {
            ++spins;
            if (spins == 1024) t0 = clock64();
            if (spins > 1024 && (spins & 63) == 0) {
              if (*abort_flag) break;
              if (clock64() - t0 > kWaitLimitCycles) {
                *abort_flag = 1;
                if (p.status) atomicCAS(p.status, 0, SLLM_DEV_TIMEOUT_PEER_FLAG);
                break;
              }
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*abort_flag) comm_ok = false;
      }
      if (pair_x) {
        // ---- SiLU(gate) * up of 64 features: a half warp per token row (lane l: features 4 l .. 4 l + 3, gate
        // rows 0..63 and up rows 64..127 of the tile), two rows per warp step; the result goes back over the gate
        // half of the staging buffer, the row maximum to both CTAs of the scale block
        const int l16 = lane & 15;
        for (int base = 2 * ew; base < T; base += 8) {
          const int col = base + (lane >> 4);
          const bool live = col < T;
          const int cc = live ? col : base;
          const float rn = __shfl_sync(0xffffffffu, rn_lane, cc);
          float* slot = red + cc * kTileA + l16 * 4;
          const float4 g = *reinterpret_cast<const float4*>(slot);
          const float4 u = *reinterpret_cast<const float4*>(slot + 64);
          float v[4] = {g.x * rn, g.y * rn, g.z * rn, g.w * rn};
          const float up[4] = {u.x * rn, u.y * rn, u.z * rn, u.w * rn};
          float amax = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float a = fe.act == 0 ? v[j] / (1.f + __expf(-v[j]))
                                        : 0.5f * v[j] * (1.f + tanhf(0.7978845608028654f * (v[j] + 0.044715f * v[j] * v[j] * v[j])));
            v[j] = col_bf16r(col_bf16r(a) * up[j]);
            const float x = fabsf(v[j]);
            if (x == x && x <= 3.0e38f) amax = fmaxf(amax, x);
          }
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));   // within the half warp
          if (live) {
            *reinterpret_cast<float4*>(slot) = make_float4(v[0], v[1], v[2], v[3]);
            if (l16 == 0) {
              bars->famax[col] = amax;
              st_dsmem_f32(&bars->famax_peer[col], (blockIdx.x & 1u) ^ 1u, amax);   // the other tile of the scale block
            }
          }
        }
      }
      for (int cl = ew; cl < cw && comm_ok && !pair_x; cl += 4) {
        const int col = c0 + cl;
        if (col >= T) break;
        const float rn = __shfl_sync(0xffffffffu, rn_lane, col);
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        if constexpr (kComm) {
          const CommParams& cm = p.comm;
          for (int src = 0; src < cm.world; ++src) {
            const uint2 w = __ldcg(reinterpret_cast<const uint2*>(cm.recv[cm.rank] + (comm_region + src) * cm.cap_elems +
                                                                  comm_toff + col * kTileA + lane * 4));
            const __nv_bfloat162 h0 = *reinterpret_cast<const __nv_bfloat162*>(&w.x);
            const __nv_bfloat162 h1 = *reinterpret_cast<const __nv_bfloat162*>(&w.y);
            sum.x += __bfloat162float(h0.x); sum.y += __bfloat162float(h0.y);
            sum.z += __bfloat162float(h1.x); sum.w += __bfloat162float(h1.y);
          }
        } else {
          const float* src = red + cl * kTileA + lane * 4;
          for (int s = 0; s < nslice; ++s) {
            const float4 x = *reinterpret_cast<const float4*>(src + s * cw * kTileA);
            sum.x += x.x; sum.y += x.y; sum.z += x.z; sum.w += x.w;
          }
        }
        float v[4] = {sum.x * rn, sum.y * rn, sum.z * rn, sum.w * rn};
        col_epilogue(e, a_tile, col, lane, v, __shfl_sync(0xffffffffu, my_pos, cl), __shfl_sync(0xffffffffu, my_page, cl));
      }
    }
    if (pair_x) {
      // both tiles' row maxima are written, each into both CTAs (all threads of both CTAs take part); nothing
      // reads the other CTA's memory afterwards
      cluster_sync_all();
      if (epi_warp) {
        const int l16 = lane & 15;
        for (int base = 2 * ew; base < T; base += 8) {
          const int col = base + (lane >> 4);
          if (col < T) {
            const float amax = fmaxf(bars->famax[col], bars->famax_peer[col]);
            const float scale = amax > 0.f ? amax / 448.f : 1.f;
            const float4 x = *reinterpret_cast<const float4*>(red + col * kTileA + l16 * 4);
            const float v[4] = {x.x, x.y, x.z, x.w};
            uint32_t q = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) q |= static_cast<uint32_t>(f32_to_e4m3(__fdiv_rn(v[j], scale))) << (8 * j);
            *reinterpret_cast<uint32_t*>(fe.q_out + static_cast<size_t>(col) * fe.n + a_tile * 64 + l16 * 4) = q;
            if (l16 == 0 && (blockIdx.x & 1u) == 0) fe.s_out[static_cast<size_t>(a_tile >> 1) * fe.ld_s + col] = scale;
          }
        }
      }
    }
  } else if (warp >= 2 && warp < 6 && active && ok) {
    const int nslice = cluster_split ? static_cast<int>(gridDim.z) : 1;
    const int cw = BN / nslice;            // columns of the tile this CTA finishes
    const int c0 = (cluster_split ? split : 0) * cw;
    const int tile_id = a_tile * gridDim.y + b_tile;
    const bool tr = p.transpose_out != 0;
    // unit u -> (column, first row) of 8 consecutive outputs along the contiguous axis of Y
    const int units = tr ? cw * (kTileA / 8) : kTileA * (cw / 8);
    auto unit_pos = [&](int u, int& col, int& r0) {
      if (tr) { col = c0 + u / (kTileA / 8); r0 = (u % (kTileA / 8)) * 8; }   // 8 rows of one column
      else    { r0 = u % kTileA; col = c0 + (u / kTileA) * 8; }                // 8 columns of one row
    };
    auto load_unit = [&](int col, int r0, float (&v)[8]) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
      for (int s = 0; s < nslice; ++s) {
        const float* slot = red + (s * cw + col - c0) * kTileA + r0;     // this CTA's own shared memory
        if (tr) {
          const float4 x0 = *reinterpret_cast<const float4*>(slot);
          const float4 x1 = *reinterpret_cast<const float4*>(slot + 4);
          v[0] += x0.x; v[1] += x0.y; v[2] += x0.z; v[3] += x0.w;
          v[4] += x1.x; v[5] += x1.y; v[6] += x1.z; v[7] += x1.w;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] += slot[j * kTileA];
        }
      }
    };
    // offset of a unit inside a tile-sized bf16 exchange region ([column][row] or [row][column])
    auto unit_off = [&](int col, int r0) -> long long {
      return static_cast<long long>(tile_id) * (kTileA * BN) + (tr ? col * kTileA + r0 : r0 * BN + col);
    };
    auto store_unit = [&](int col, int r0, float (&v)[8]) {
      if (tr) {
        const int b_row = b_tile * BN + col;
        const int a0 = a_tile * kTileA + r0;
        if (b_row >= p.b_rows || a0 >= p.a_rows) return;
        const size_t idx = static_cast<size_t>(b_row) * p.ldy + a0;
        if (a0 + 8 <= p.a_rows && (p.ldy & 7) == 0) {
          if (p.epilogue == 1) {
            const uint4 rr = *reinterpret_cast<const uint4*>(p.residual + idx);
            const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
            for (int j = 0; j < 4; ++j) { v[2 * j] += __bfloat162float(r2[j].x); v[2 * j + 1] += __bfloat162float(r2[j].y); }
          }
          uint4 out;
          __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
          for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
          *reinterpret_cast<uint4*>(p.y + idx) = out;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (a0 + j < p.a_rows) {
              float x = v[j];
              if (p.epilogue == 1) x += bf16_to_f32(p.residual[idx + j]);
              p.y[idx + j] = f32_to_bf16(x);
            }
          }
        }
      } else {
        const int a_row = a_tile * kTileA + r0;
        const int b0 = b_tile * BN + col;
        if (a_row >= p.a_rows || b0 >= p.b_rows) return;
        const size_t idx = static_cast<size_t>(a_row) * p.ldy + b0;
        if (b0 + 8 <= p.b_rows && (p.ldy & 7) == 0) {
          if (p.epilogue == 1) {
            const uint4 rr = *reinterpret_cast<const uint4*>(p.residual + idx);
            const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
            for (int j = 0; j < 4; ++j) { v[2 * j] += __bfloat162float(r2[j].x); v[2 * j + 1] += __bfloat162float(r2[j].y); }
          }
          uint4 out;
          __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
          for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
          *reinterpret_cast<uint4*>(p.y + idx) = out;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (b0 + j < p.b_rows) {
              float x = v[j];
              if (p.epilogue == 1) x += bf16_to_f32(p.residual[idx + j]);
              p.y[idx + j] = f32_to_bf16(x);
            }
          }
        }
      }
    };

    if (threadIdx.x == 64) TRACE(9);
    if (!kComm) {
      for (int u = et; u < units; u += 128) {
        int col, r0;
        unit_pos(u, col, r0);
        float v[8];
        load_unit(col, r0, v);
        store_unit(col, r0, v);
      }
    } else {
      // ---- fused all-reduce: push this CTA's slice (bf16) to every rank, flag, wait, sum in rank order
      const CommParams& cm = p.comm;
      const int slot = tile_id * kMaxSlices + (cluster_split ? split : 0);
      if (et == 0) {
        const uint32_t e1 = cm.epoch[slot] + 1;
        cm.epoch[slot] = e1;
        bars->epoch = e1;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const uint32_t e = bars->epoch;
      const long long region = static_cast<long long>(e & 1) * cm.world;
      for (int u = et; u < units; u += 128) {
        int col, r0;
        unit_pos(u, col, r0);
        float v[8];
        load_unit(col, r0, v);
        uint4 w;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        const long long off = (region + cm.rank) * cm.cap_elems + unit_off(col, r0);
        for (int peer = 0; peer < cm.world; ++peer) *reinterpret_cast<uint4*>(cm.recv[peer] + off) = w;
      }
      __threadfence_system();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      bool comm_ok = true;
      if (et < cm.world && et != cm.rank) {
        st_release_sys(cm.flags[et] + static_cast<size_t>(slot) * cm.world + cm.rank, e);
        const uint32_t* f = cm.flags[cm.rank] + static_cast<size_t>(slot) * cm.world + et;
        uint32_t spins = 0;
        long long t0 = 0;
        while (static_cast<int32_t>(ld_acquire_sys(f) - e) < 0) {
          ++spins;
          if (spins == 1024) t0 = clock64();
          if (spins > 1024 && (spins & 63) == 0) {
            if (*abort_flag) break;
            if (clock64() - t0 > kWaitLimitCycles) {
              *abort_flag = 1;
              if (p.status) atomicCAS(p.status, 0, SLLM_DEV_TIMEOUT_PEER_FLAG);
              break;
            }
          }
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*abort_flag) comm_ok = false;
      if (comm_ok) {
        for (int u = et; u < units; u += 128) {
          int col, r0;
          unit_pos(u, col, r0);
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = 0.f;
          const long long uo = unit_off(col, r0);
          for (int src = 0; src < cm.world; ++src) {
            const uint4 w = __ldcg(reinterpret_cast<const uint4*>(cm.recv[cm.rank] + (region + src) * cm.cap_elems + uo));
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
            for (int j = 0; j < 4; ++j) { v[2 * j] += __bfloat162float(h[j].x); v[2 * j + 1] += __bfloat162float(h[j].y); }
          }
          store_unit(col, r0, v);
        }
      }
    }
  }

  if (threadIdx.x == 64) TRACE(10);
  if (threadIdx.x == 64) TRACE(11);

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  STEP_TRACE_END(p);
}

// ---------------------------------------------------------------- host side
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  });
  return fn;
}

// K-major 2-D tensor map: global [rows, k_elems], box = {128 bytes of K, box_rows}, 128-byte swizzle.
int make_kmajor_tmap(CUtensorMap* out, const void* ptr, int elem_bytes, long long rows, long long k_elems,
                     long long row_stride_bytes, int box_rows) {
  auto fn = get_encode_fn();
  if (!fn) return SLLM_ERR_DRIVER_ENTRY;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (row_stride_bytes & 15)) return SLLM_ERR_ALIGNMENT;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(k_elems), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstride[1] = {static_cast<cuuint64_t>(row_stride_bytes)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBoxBytes / elem_bytes), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUresult r = fn(out, dt, 2, const_cast<void*>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SLLM_OK : SLLM_ERR_CUDA;
}

struct TmapKey {
  const void* ptr;
  long long rows, k, stride;
  int elem, box;
  bool operator<(const TmapKey& o) const {
    return std::tie(ptr, rows, k, stride, elem, box) < std::tie(o.ptr, o.rows, o.k, o.stride, o.elem, o.box);
  }
};
static std::map<TmapKey, CUtensorMap> g_tmap_cache;
static std::mutex g_tmap_mutex;

int cached_kmajor_tmap(CUtensorMap* out, const void* ptr, int elem_bytes, long long rows, long long k_elems,
                       long long row_stride_bytes, int box_rows) {
  TmapKey key{ptr, rows, k_elems, row_stride_bytes, elem_bytes, box_rows};
  std::lock_guard<std::mutex> g(g_tmap_mutex);
  auto it = g_tmap_cache.find(key);
  if (it != g_tmap_cache.end()) {
    *out = it->second;
    return SLLM_OK;
  }
  int rc = make_kmajor_tmap(out, ptr, elem_bytes, rows, k_elems, row_stride_bytes, box_rows);
  if (rc == SLLM_OK) {
    if (g_tmap_cache.size() > 65536) g_tmap_cache.clear();
    g_tmap_cache[key] = *out;
  }
  return rc;
}

int cached_plain_tmap(CUtensorMap* out, const void* ptr, long long rows, long long row_bytes, long long row_stride_bytes,
                      int box_bytes, int box_rows) {
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (row_stride_bytes & 15) || (box_bytes & 15) || box_bytes <= 0 ||
      box_rows <= 0 || box_rows > 256)
    return SLLM_ERR_ALIGNMENT;
  TmapKey key{ptr, rows, row_bytes, row_stride_bytes, -box_bytes, box_rows};   // negative element size: plain maps
  std::lock_guard<std::mutex> g(g_tmap_mutex);
  auto it = g_tmap_cache.find(key);
  if (it != g_tmap_cache.end()) {
    *out = it->second;
    return SLLM_OK;
  }
  auto fn = get_encode_fn();
  if (!fn) return SLLM_ERR_DRIVER_ENTRY;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstride[1] = {static_cast<cuuint64_t>(row_stride_bytes)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_bytes), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return SLLM_ERR_CUDA;
  if (g_tmap_cache.size() > 65536) g_tmap_cache.clear();
  g_tmap_cache[key] = *out;
  return SLLM_OK;
}

template <int BN, bool kScaled>
constexpr size_t gemm_fixed_smem() {
  return sizeof(GemmBarriers<BN>) + (kScaled ? sizeof(GemmScales<BN>) : 0) + 1024;
}

template <int BN, bool kScaled, bool kComm>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, dim3 grid,
                       cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(p.stages) * (kTileA + BN) * kBoxBytes + gemm_fixed_smem<BN, kScaled>();
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, kScaled, kComm>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return SLLM_ERR_CUDA;
    configured = smem;
  }
  GemmParams pp = p;
  if (pp.cluster_split) {
    // Validate this cluster shape once per (instantiation, size); fall back to the global fix-up
    // when the device cannot co-schedule it.
    static int cluster_ok[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};  // 0 unknown, 1 ok, -1 unusable
    static size_t cluster_smem[9] = {0};
    const int z = static_cast<int>(grid.z);
    if (cluster_ok[z] == 0 || cluster_smem[z] < smem) {
      cudaLaunchConfig_t probe = {};
      probe.gridDim = grid;
      probe.blockDim = dim3(gemm_threads(BN));
      probe.dynamicSmemBytes = smem;
      cudaLaunchAttribute pa[1];
      pa[0].id = cudaLaunchAttributeClusterDimension;
      pa[0].val.clusterDim.x = 1;
      pa[0].val.clusterDim.y = 1;
      pa[0].val.clusterDim.z = grid.z;
      probe.attrs = pa;
      probe.numAttrs = 1;
      int n_clusters = 0;
      const cudaError_t e = cudaOccupancyMaxActiveClusters(&n_clusters, gemm_tcgen05_kernel<BN, kScaled, kComm>, &probe);
      if (e != cudaSuccess) cudaGetLastError();
      cluster_ok[z] = (e == cudaSuccess && n_clusters > 0) ? 1 : -1;
      cluster_smem[z] = smem;
    }
    if (cluster_ok[z] < 0) {
      if (pp.fe.mode != 0) return SLLM_ERR_UNSUPPORTED_SHAPE;   // the fused row epilogue needs the DSMEM reduction
      pp.cluster_split = 0;
      if (!pp.ws || !pp.counters) return SLLM_ERR_WORKSPACE_TOO_SMALL;
    }
  }
  const unsigned cluster_x = pp.fe.mode == SLLM_FD_SILU_QUANT + 1 ? 2u : 1u;
#ifdef SLLM_TRACE
  {
    // development aid: how many clusters of this shape the device holds at once, printed once per shape
    static unsigned seen[64];
    static int n_seen = 0;
    const unsigned key = (BN << 16) | (cluster_x << 8) | (pp.cluster_split ? grid.z : 1u) | (kComm ? 1u << 30 : 0u);
    bool have = false;
    for (int i = 0; i < n_seen; ++i) have = have || seen[i] == key;
    if (!have && n_seen < 64) {
      seen[n_seen++] = key;
      cudaLaunchConfig_t probe = {};
      probe.gridDim = grid;
      probe.blockDim = dim3(gemm_threads(BN));
      probe.dynamicSmemBytes = smem;
      cudaLaunchAttribute pa[1];
      pa[0].id = cudaLaunchAttributeClusterDimension;
      pa[0].val.clusterDim.x = cluster_x;
      pa[0].val.clusterDim.y = 1;
      pa[0].val.clusterDim.z = pp.cluster_split ? grid.z : 1u;
      probe.attrs = pa;
      probe.numAttrs = 1;
      int n_clusters = -1, per_sm = -1;
      if (cudaOccupancyMaxActiveClusters(&n_clusters, gemm_tcgen05_kernel<BN, kScaled, kComm>, &probe) != cudaSuccess) cudaGetLastError();
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_tcgen05_kernel<BN, kScaled, kComm>, gemm_threads(BN), smem);
      fprintf(stderr, "[trace] gemm BN=%d cluster=(%u,1,%u) smem=%zu grid=(%u,%u,%u): max active clusters %d, CTAs per SM %d\n", BN,
              cluster_x, pp.cluster_split ? grid.z : 1u, smem, grid.x, grid.y, grid.z, n_clusters, per_sm);
      cudaFuncAttributes fa;
      cudaFuncGetAttributes(&fa, gemm_tcgen05_kernel<BN, kScaled, kComm>);
      cudaDeviceProp dp;
      cudaGetDeviceProperties(&dp, 0);
      fprintf(stderr, "[trace]   regs %d static smem %zu max dyn %d max threads %d | SM: regs %d smem %zu reserved/block %zu max blocks %d\n",
              fa.numRegs, fa.sharedSizeBytes, fa.maxDynamicSharedSizeBytes, fa.maxThreadsPerBlock, dp.regsPerMultiprocessor,
              dp.sharedMemPerMultiprocessor, dp.reservedSharedMemPerBlock, dp.maxBlocksPerMultiProcessor);
      for (int th : {192, 224, 256})
        for (size_t sm : {size_t(0), size_t(65536), size_t(104912), size_t(112000), size_t(115000)}) {
          int n = -1;
          cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, gemm_tcgen05_kernel<BN, kScaled, kComm>, th, sm);
          fprintf(stderr, "[trace]   threads %d smem %zu -> %d CTAs/SM\n", th, sm, n);
        }
    }
  }
#endif
  if (launch_kernel_cluster(gemm_tcgen05_kernel<BN, kScaled, kComm>, grid, dim3(gemm_threads(BN)), smem, stream, cluster_x,
                            pp.cluster_split ? grid.z : 1u, ta, tb, pp) != cudaSuccess) {
    cudaGetLastError();
    return SLLM_ERR_CUDA;
  }
  return SLLM_OK;
}

}  // namespace sllm

using namespace sllm;

SLLM_EXPORT long long sllm_gemm_workspace_floats(int a_rows, int b_rows, int bn, int splits) {
  if (splits <= 1) return 0;
  const long long tiles = static_cast<long long>((a_rows + kTileA - 1) / kTileA) * ((b_rows + bn - 1) / bn);
  return tiles * splits * bn * kTileA;
}

static int g_disable_cluster_split = 0;

// SLLM_GEMM_EARLY_TRIGGER=0/1 (default 0) or sllm_gemm_set_early_trigger: see GemmParams::early_trigger.
static int g_gemm_early = -1;
static int gemm_early_trigger() {
  if (g_gemm_early < 0) {
    const char* e = getenv("SLLM_GEMM_EARLY_TRIGGER");
    g_gemm_early = (e && e[0] == '1') ? 1 : 0;
  }
  return g_gemm_early;
}
SLLM_EXPORT void sllm_gemm_set_early_trigger(int enabled) { g_gemm_early = enabled ? 1 : 0; }

struct SllmCommDesc {   // host-side mirror passed by the Python layer (ctypes.Structure)
  int world, rank;
  long long cap_elems;
  int max_tiles;
  int reserved;
  void* recv[kMaxWorld];
  void* flags[kMaxWorld];
  void* epoch;
};

struct SllmGatherDesc {   // host-side mirror passed by the Python layer (ctypes.Structure)
  int world, rank;
  void* maps;      // device array [4 tile widths (16, 32, 64, 128)][2 parities][world] of CUtensorMap
  void* flags;     // local flags [world]
  void* epoch;     // local epoch counter
};

static int gemm_impl(const void* a, const void* b, void* y, const float* scale_a, const float* scale_b,
                     const void* residual, int a_rows, int b_rows, int k, int scaled, int transpose_out, int ldy,
                     int ld_sa, int ld_sb, int bn, int splits, int stages, float* ws, long long ws_floats,
                     int* counters, int n_counters, int* status, void* stream, const SllmCommDesc* comm,
                     const SllmGatherDesc* gather = nullptr, const FusedEpi* fused = nullptr) {
  if (gather) b = a;    // the B operand comes from the peers' buffers; keep the argument checks below simple
  if (!a || !b || !y || a_rows <= 0 || b_rows <= 0 || k <= 0 || splits < 1) return SLLM_ERR_INVALID_ARGUMENT;
  if (bn != 16 && bn != 32 && bn != 64 && bn != 128) return SLLM_ERR_UNSUPPORTED_SHAPE;
  const int elem = scaled ? 1 : 2;
  if ((static_cast<long long>(k) * elem) % 16) return SLLM_ERR_ALIGNMENT;
  if (scaled && (!scale_a || !scale_b)) return SLLM_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(y) & 15) return SLLM_ERR_ALIGNMENT;
  const int elems_per_box = kBoxBytes / elem;
  const int num_kb = (k + elems_per_box - 1) / elems_per_box;
  if (splits > num_kb) splits = num_kb;
  const int kb_per_split = (num_kb + splits - 1) / splits;
  splits = (num_kb + kb_per_split - 1) / kb_per_split;
  const int a_tiles = (a_rows + kTileA - 1) / kTileA, b_tiles = (b_rows + bn - 1) / bn;
  if (b_tiles > 65535 || splits > 65535) return SLLM_ERR_UNSUPPORTED_SHAPE;
  if (splits > 1) {
    if (!ws || !counters) return SLLM_ERR_INVALID_ARGUMENT;
    if (ws_floats < static_cast<long long>(a_tiles) * b_tiles * splits * bn * kTileA || n_counters < a_tiles * b_tiles)
      return SLLM_ERR_WORKSPACE_TOO_SMALL;
  }
  const int fixed_smem = 2048 + static_cast<int>(sizeof(GemmBarriers<128>)) +
                         (scaled ? static_cast<int>(sizeof(float)) * 2 * kScaleChunk * (kTileA + bn) : 0);
  const int max_stages_smem = (227 * 1024 - fixed_smem) / ((kTileA + bn) * kBoxBytes);
  if (stages < 2) stages = 2;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages > max_stages_smem) stages = max_stages_smem;
  stages -= stages % gemm_issuers(bn);   // each stage stays with one issuer
  if (stages < 2) return SLLM_ERR_UNSUPPORTED_SHAPE;

  GemmParams p;
  memset(&p, 0, sizeof(p));
  if (comm) {
    if (comm->world < 2 || comm->world > kMaxWorld || comm->rank < 0 || comm->rank >= comm->world || !comm->epoch)
      return SLLM_ERR_INVALID_ARGUMENT;
    const long long tiles = static_cast<long long>(a_tiles) * b_tiles;
    // flags and epochs hold kMaxSlices slots per tile
    if (tiles > comm->max_tiles || tiles * kTileA * bn > comm->cap_elems) return SLLM_ERR_WORKSPACE_TOO_SMALL;
    p.comm.world = comm->world; p.comm.rank = comm->rank; p.comm.cap_elems = comm->cap_elems;
    for (int i = 0; i < comm->world; ++i) {
      if (!comm->recv[i] || !comm->flags[i]) return SLLM_ERR_INVALID_ARGUMENT;
      p.comm.recv[i] = static_cast<__nv_bfloat16*>(comm->recv[i]);
      p.comm.flags[i] = static_cast<uint32_t*>(comm->flags[i]);
    }
    p.comm.epoch = static_cast<uint32_t*>(comm->epoch);
  }

  CUtensorMap ta, tb;
  int rc = cached_kmajor_tmap(&ta, a, elem, a_rows, k, static_cast<long long>(k) * elem, kTileA);
  if (rc != SLLM_OK) return rc;
  rc = cached_kmajor_tmap(&tb, b, elem, b_rows, k, static_cast<long long>(k) * elem, bn);
  if (rc != SLLM_OK) return rc;

  p.a_rows = a_rows; p.b_rows = b_rows; p.num_kb = num_kb; p.kb_per_split = kb_per_split; p.stages = stages;
  p.transpose_out = transpose_out; p.ldy = ldy; p.ld_sa = ld_sa; p.ld_sb = ld_sb;
  p.epilogue = residual ? 1 : 0;
  // 2..8 splits reduce inside one thread-block cluster over DSMEM; more use the global fix-up.
  // (the output phase needs whole 16-byte units per slice: any slice width when Y is written
  // transposed, at least 8 columns otherwise)
  const bool pow2 = splits == 2 || splits == 4 || splits == 8;
  p.cluster_split = (pow2 && bn % splits == 0 && (transpose_out || bn / splits >= 8) && !g_disable_cluster_split) ? 1 : 0;
  p.const_operand = transpose_out ? 1 : 2;   // swap-AB: A is the weight matrix, else B is
  p.early_trigger = gemm_early_trigger();
  STEP_TRACE_ASSIGN(p, 1);
  p.scale_a = scale_a; p.scale_b = scale_b;
  p.y = static_cast<__nv_bfloat16*>(y);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ws = ws; p.counters = counters; p.status = status;
  if (fused) {
    // the row epilogue works on whole token rows of a tile: no K split, or a cluster split reduced over DSMEM
    if (!scaled || !transpose_out || gather || (splits > 1 && !p.cluster_split) || bn > 32)
      return SLLM_ERR_UNSUPPORTED_SHAPE;
    if (comm && fused->mode != SLLM_FD_RESID_QUANT + 1) return SLLM_ERR_UNSUPPORTED_SHAPE;   // only row-parallel phases sum
    if (fused->mode == SLLM_FD_SILU_QUANT + 1 && (splits != 1 || (a_tiles & 1))) return SLLM_ERR_UNSUPPORTED_SHAPE;
    p.fe = *fused;
  }
  if (gather) {
    if (scaled || !transpose_out || comm || gather->world < 2 || gather->world > kMaxWorld || gather->rank < 0 ||
        gather->rank >= gather->world || !gather->maps || !gather->flags || !gather->epoch || num_kb % gather->world)
      return SLLM_ERR_INVALID_ARGUMENT;
    const int bi = bn == 16 ? 0 : bn == 32 ? 1 : bn == 64 ? 2 : 3;
    p.gather.world = gather->world; p.gather.rank = gather->rank; p.gather.kb_per_rank = num_kb / gather->world;
    p.gather.maps = static_cast<const CUtensorMap*>(gather->maps) + static_cast<size_t>(bi) * 2 * gather->world;
    p.gather.flags = static_cast<const uint32_t*>(gather->flags);
    p.gather.epoch = static_cast<const uint32_t*>(gather->epoch);
  }
  dim3 grid(a_tiles, b_tiles, splits);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define SLLM_GEMM_CASE(BN_)                                                                                 \
  case BN_:                                                                                                 \
    if (comm)                                                                                               \
      return scaled ? launch_gemm<BN_, true, true>(ta, tb, p, grid, st)                                     \
                    : launch_gemm<BN_, false, true>(ta, tb, p, grid, st);                                   \
    return scaled ? launch_gemm<BN_, true, false>(ta, tb, p, grid, st)                                      \
                  : launch_gemm<BN_, false, false>(ta, tb, p, grid, st);
  switch (bn) {
    SLLM_GEMM_CASE(16)
    SLLM_GEMM_CASE(32)
    SLLM_GEMM_CASE(64)
    SLLM_GEMM_CASE(128)
  }
#undef SLLM_GEMM_CASE
  return SLLM_ERR_UNSUPPORTED_SHAPE;
}

#ifdef SLLM_TRACE
static unsigned long long* g_step_buf = nullptr;
static int g_step_cap = 0, g_step_next = 0;
namespace sllm {
unsigned long long* step_trace_next(int kind) {
  if (!g_step_buf || g_step_next >= g_step_cap) return nullptr;
  unsigned long long* rec = g_step_buf + 4 * static_cast<size_t>(g_step_next++);
  const unsigned long long k = static_cast<unsigned long long>(kind);
  cudaMemcpy(rec + 3, &k, sizeof(k), cudaMemcpyHostToDevice);
  return rec;
}
}  // namespace sllm
// dev_buf: records * 4 64-bit words on the device (null switches the timeline off); numbering restarts at 0.
SLLM_EXPORT void sllm_step_trace_set(void* dev_buf, int records) {
  g_step_buf = static_cast<unsigned long long*>(dev_buf);
  g_step_cap = records;
  g_step_next = 0;
}
SLLM_EXPORT int sllm_step_trace_count() { return g_step_next; }
SLLM_EXPORT int sllm_gemm_read_trace(unsigned long long* out32) {
  return cudaMemcpyFromSymbol(out32, g_trace, sizeof(unsigned long long) * 32) == cudaSuccess ? 0 : 5;
}
#endif

// Test hook: force the global-memory split-K fix-up even when a cluster reduction is possible.
SLLM_EXPORT void sllm_gemm_set_cluster_split(int enabled) { g_disable_cluster_split = enabled ? 0 : 1; }

SLLM_EXPORT int sllm_gemm(const void* a, const void* b, void* y, const float* scale_a, const float* scale_b,
                          const void* residual, int a_rows, int b_rows, int k, int scaled, int transpose_out,
                          int ldy, int ld_sa, int ld_sb, int bn, int splits, int stages, float* ws,
                          long long ws_floats, int* counters, int n_counters, int* status, void* stream) {
  return gemm_impl(a, b, y, scale_a, scale_b, residual, a_rows, b_rows, k, scaled, transpose_out, ldy, ld_sa, ld_sb,
                   bn, splits, stages, ws, ws_floats, counters, n_counters, status, stream, nullptr);
}

// Same GEMM with the cross-rank sum of the partial products fused into the epilogue (see the file
// comment).  `comm` points to a host SllmCommDesc whose device pointers come from sllm_symm_open.
SLLM_EXPORT int sllm_gemm_allreduce(const void* a, const void* b, void* y, const float* scale_a,
                                    const float* scale_b, const void* residual, int a_rows, int b_rows, int k,
                                    int scaled, int transpose_out, int ldy, int ld_sa, int ld_sb, int bn, int splits,
                                    int stages, float* ws, long long ws_floats, int* counters, int n_counters,
                                    int* status, void* stream, const void* comm) {
  if (!comm) return SLLM_ERR_INVALID_ARGUMENT;
  return gemm_impl(a, b, y, scale_a, scale_b, residual, a_rows, b_rows, k, scaled, transpose_out, ldy, ld_sa, ld_sb,
                   bn, splits, stages, ws, ws_floats, counters, n_counters, status, stream,
                   static_cast<const SllmCommDesc*>(comm));
}

// ---------------------------------------------------------------- all-gather -> column-parallel GEMM
namespace sllm {
// Copies this rank's activation shard [rows, ks] into its symmetric buffer of the next epoch's parity and raises
// flag[rank] = epoch on every rank.  One CTA: the shard is small (decode / verify rows).
__global__ void __launch_bounds__(1024)
gather_publish_kernel(const __nv_bfloat16* __restrict__ x, int rows, int ks, int ldx, __nv_bfloat16* buf0,
                      __nv_bfloat16* buf1, int cap_rows, uint32_t* epoch, CommParams peers) {
  pdl_wait();
  __shared__ uint32_t s_e;
  if (threadIdx.x == 0) {
    s_e = *epoch + 1;
    *epoch = s_e;
  }
  __syncthreads();
  const uint32_t e = s_e;
  __nv_bfloat16* dst = (e & 1u) ? buf1 : buf0;
  const int units = ks / 8;                      // 16-byte units per row
  for (int i = threadIdx.x; i < rows * units; i += blockDim.x) {
    const int r = i / units, u = i % units;
    reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * ks)[u] =
        *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * ldx + u * 8);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < peers.world) st_release_sys(peers.flags[threadIdx.x] + peers.rank, e);
  pdl_trigger();
}
}  // namespace sllm

// Builds the tensor maps of every rank's two shard buffers for the four token-tile widths and copies them to
// `dev_maps` ([4][2][world] CUtensorMap).  bufs[p * 2 + parity]: rank p's buffer as mapped in this process.
SLLM_EXPORT int sllm_gather_build_maps(void* dev_maps, const void* const* bufs, int world, int cap_rows, int k_shard) {
  if (!dev_maps || !bufs || world < 2 || world > kMaxWorld || cap_rows <= 0 || k_shard <= 0 || (k_shard % 64))
    return SLLM_ERR_INVALID_ARGUMENT;
  static const int widths[4] = {16, 32, 64, 128};
  std::vector<CUtensorMap> host(static_cast<size_t>(4) * 2 * world);
  for (int bi = 0; bi < 4; ++bi)
    for (int par = 0; par < 2; ++par)
      for (int pr = 0; pr < world; ++pr) {
        const int rc = make_kmajor_tmap(&host[(static_cast<size_t>(bi) * 2 + par) * world + pr], bufs[pr * 2 + par], 2,
                                        cap_rows, k_shard, static_cast<long long>(k_shard) * 2, widths[bi]);
        if (rc != SLLM_OK) return rc;
      }
  return cudaMemcpy(dev_maps, host.data(), host.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice) == cudaSuccess
             ? SLLM_OK : SLLM_ERR_CUDA;
}

// flags_on_peers[p]: rank p's flag array as mapped in this process.
SLLM_EXPORT int sllm_gather_publish(const void* x, int rows, int k_shard, int ldx, void* buf0, void* buf1, int cap_rows,
                                    void* epoch, const void* const* flags_on_peers, int world, int rank, void* stream) {
  if (!x || !buf0 || !buf1 || !epoch || !flags_on_peers || rows <= 0 || rows > cap_rows || (k_shard % 8) || (ldx % 8) ||
      world < 2 || world > kMaxWorld || rank < 0 || rank >= world || (reinterpret_cast<uintptr_t>(x) & 15))
    return SLLM_ERR_INVALID_ARGUMENT;
  CommParams peers;
  memset(&peers, 0, sizeof(peers));
  peers.world = world; peers.rank = rank;
  for (int i = 0; i < world; ++i) peers.flags[i] = static_cast<uint32_t*>(const_cast<void*>(flags_on_peers[i]));
  launch_kernel(gather_publish_kernel, dim3(1), dim3(1024), 0, static_cast<cudaStream_t>(stream), 1u,
                static_cast<const __nv_bfloat16*>(x), rows, k_shard, ldx, static_cast<__nv_bfloat16*>(buf0),
                static_cast<__nv_bfloat16*>(buf1), cap_rows, static_cast<uint32_t*>(epoch), peers);
  return cudaGetLastError() == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

// Y[rows, n] = concat over ranks of X_r[rows, k / world] times W[n, k]^T, bf16, weights as the 128-row operand.
// The shards must have been published with sllm_gather_publish on every rank (same stream order everywhere).
SLLM_EXPORT int sllm_gemm_allgather(const void* w, void* y, const void* residual, int n, int rows, int k, int ldy, int bn,
                                    int splits, int stages, float* ws, long long ws_floats, int* counters, int n_counters,
                                    int* status, void* stream, const void* gather) {
  if (!gather) return SLLM_ERR_INVALID_ARGUMENT;
  return gemm_impl(w, nullptr, y, nullptr, nullptr, residual, n, rows, k, 0, 1, ldy, 0, 0, bn, splits, stages, ws,
                   ws_floats, counters, n_counters, status, stream, nullptr, static_cast<const SllmGatherDesc*>(gather));
}

// One decode GEMM with a fused row epilogue, described by a phase record of the fused decode path (decode_fused.h):
// Y[t, n] = X[t, :] . W[n, :] (block-scaled FP8, weights as the 128-row operand), K split over a thread-block cluster
// and reduced over DSMEM, then the PLAIN / RESID_QUANT / SILU_QUANT / ROPE_KV row epilogue.  For SILU_QUANT `ph->w`
// is the gate / up matrix with rows interleaved per 128-row tile (64 gate rows, then the 64 up rows of the same
// features) and `ph->w_scale` its scales in the same row order; dual_off is ignored.  `comm` (a host SllmCommDesc, or
// null) makes RESID_QUANT phases sum their rows across the tensor-parallel ranks before the residual joins.
SLLM_EXPORT int sllm_gemm_fused(const SllmFdPhase* ph, const SllmFdRope* rope, int rows, int bn, int splits, int stages,
                                float* ws, long long ws_floats, int* counters, int n_counters, int* status, void* stream,
                                const void* comm) {
  if (!ph || rows < 1 || rows > 32 || !ph->w || !ph->w_scale || !ph->x || !ph->x_scale || ph->n <= 0 || ph->k <= 0 ||
      (ph->k & 127))
    return SLLM_ERR_INVALID_ARGUMENT;
  FusedEpi fe;
  memset(&fe, 0, sizeof(fe));
  fe.mode = ph->epilogue + 1;
  fe.n = ph->n; fe.norm_tiles = ph->norm_tiles; fe.norm_dim = ph->norm_dim; fe.eps = ph->eps; fe.softcap = ph->softcap;
  fe.act = ph->act; fe.ld_s = ph->ld_s_out; fe.ssq_in = ph->ssq_in;
  fe.q_out = static_cast<uint8_t*>(ph->q_out); fe.s_out = ph->s_out; fe.ssq_out = ph->ssq_out;
  int w_rows = ph->n;
  void* y = ph->y;
  switch (ph->epilogue) {
    case SLLM_FD_PLAIN:
      if (!ph->y || (ph->ldy & 3)) return SLLM_ERR_INVALID_ARGUMENT;
      break;
    case SLLM_FD_RESID_QUANT:
      if (!ph->y || !ph->residual || !ph->q_out || !ph->s_out || (ph->n & 127) || (ph->ldy & 3)) return SLLM_ERR_INVALID_ARGUMENT;
      break;
    case SLLM_FD_SILU_QUANT:
      if (!ph->q_out || !ph->s_out || (ph->n & 127)) return SLLM_ERR_INVALID_ARGUMENT;
      w_rows = 2 * ph->n;
      y = ph->q_out;      // no bf16 output; the GEMM launcher only needs a non-null, aligned pointer
      break;
    case SLLM_FD_ROPE_KV:
      if (!rope || !ph->y || (ph->ldy & 3) || !rope->positions || !rope->seq_index || !rope->block_table || !rope->k_pages ||
          !rope->v_pages || !rope->inv_freq || ph->n != (rope->hq + 2 * rope->hkv) * 128 ||
          (rope->rotary_dim != 32 && rope->rotary_dim != 64 && rope->rotary_dim != 128))
        return SLLM_ERR_INVALID_ARGUMENT;
      fe.rope = *rope;
      fe.inv_freq = rope->inv_freq;
      break;
    default:
      return SLLM_ERR_INVALID_ARGUMENT;
  }
  if (ph->norm_tiles > 0 && (!ph->ssq_in || ph->norm_dim <= 0)) return SLLM_ERR_INVALID_ARGUMENT;
  return gemm_impl(ph->w, ph->x, y, ph->w_scale, ph->x_scale, ph->epilogue == SLLM_FD_SILU_QUANT ? nullptr : ph->residual,
                   w_rows, rows, ph->k, 1, 1, ph->ldy > 0 ? ph->ldy : ph->n, ph->ld_sa, ph->ld_sb, bn, splits, stages, ws,
                   ws_floats, counters, n_counters, status, stream,
                   ph->epilogue == SLLM_FD_RESID_QUANT ? static_cast<const SllmCommDesc*>(comm) : nullptr, nullptr, &fe);
}

// sizeof / offsetof records of the two descriptor structs that foreign-language bindings mirror by hand
// (SllmCommDesc: size, recv, flags, epoch; SllmGatherDesc: size, maps, flags, epoch): writes up to n ints and returns
// how many there are.  A binding compares them with its own layout before it passes a descriptor.
SLLM_EXPORT int sllm_comm_abi(int* out, int n) {
  const int rec[] = {
      static_cast<int>(sizeof(SllmCommDesc)), static_cast<int>(offsetof(SllmCommDesc, recv)),
      static_cast<int>(offsetof(SllmCommDesc, flags)), static_cast<int>(offsetof(SllmCommDesc, epoch)),
      static_cast<int>(sizeof(SllmGatherDesc)), static_cast<int>(offsetof(SllmGatherDesc, maps)),
      static_cast<int>(offsetof(SllmGatherDesc, flags)), static_cast<int>(offsetof(SllmGatherDesc, epoch)),
  };
  const int have = static_cast<int>(sizeof(rec) / sizeof(rec[0]));
  for (int i = 0; i < n && i < have; ++i) out[i] = rec[i];
  return have;
}
