// Shared device helpers for the sm_100a kernels: mbarrier, TMA, tcgen05/TMEM wrappers, numeric
// conversions and the bounded-wait policy.
//
// Bounded waits: every spin in this library (mbarrier, peer flag) gives up after kWaitLimitCycles,
// records a non-zero code in a caller-supplied status word and lets the kernel run to its normal
// teardown (TMEM freed, copies in flight drained).  A kernel never traps and never spins forever.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdlib.h>

#define SLLM_EXPORT extern "C" __attribute__((visibility("default")))

// Status codes returned by every launcher (0 = launched).
enum SllmStatus : int {
  SLLM_OK = 0,
  SLLM_ERR_INVALID_ARGUMENT = 1,
  SLLM_ERR_UNSUPPORTED_SHAPE = 2,
  SLLM_ERR_ALIGNMENT = 3,
  SLLM_ERR_WORKSPACE_TOO_SMALL = 4,
  SLLM_ERR_CUDA = 5,
  SLLM_ERR_DRIVER_ENTRY = 6,
  SLLM_ERR_LIMIT = 7,
};

// Device-side status codes written to the status word when a bounded wait gives up.
enum SllmDeviceStatus : int {
  SLLM_DEV_OK = 0,
  SLLM_DEV_TIMEOUT_TMA_FULL = 101,
  SLLM_DEV_TIMEOUT_SMEM_EMPTY = 102,
  SLLM_DEV_TIMEOUT_TMEM_FULL = 103,
  SLLM_DEV_TIMEOUT_TMEM_EMPTY = 104,
  SLLM_DEV_TIMEOUT_PEER_FLAG = 105,
  SLLM_DEV_TIMEOUT_DRAIN = 106,
  SLLM_DEV_TIMEOUT_GRID_BARRIER = 107,
};

namespace sllm {

// Host: launch with programmatic dependent launch enabled (and an optional cluster size along z).
// SLLM_PDL=0 in the environment turns the attribute off (plain stream order).
inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SLLM_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                         unsigned cluster_x, unsigned cluster_z, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_z > 1 || cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x > 1 ? cluster_x : 1;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = cluster_z > 1 ? cluster_z : 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 unsigned cluster_z, Args&&... args) {
  return launch_kernel_cluster(kernel, grid, block, smem, stream, 1u, cluster_z, static_cast<Args&&>(args)...);
}

// ~2 s at 2 GHz; a healthy wait finishes in microseconds.
constexpr long long kWaitLimitCycles = 4000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and records `code`) when the limit runs out or another role of the
// CTA has already given up (`*abort_flag` set).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code, long long limit = kWaitLimitCycles) {
  uint32_t spins = 0;
  long long t0 = 0;
  while (!mbar_try_wait(bar, parity)) {
    ++spins;
    if (spins == 2048) t0 = clock64();
    if (spins > 2048 && (spins & 255) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- TMA (no cluster multicast anywhere)
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load gmem -> smem.  x (innermost coordinate) times the element size must be a multiple
// of 16 bytes; callers only pass multiples of the 128-byte box.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], bf16/f16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same for 8-bit float inputs (E4M3 here).
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 16 consecutive fp32 columns -> 16 registers per thread (thread t reads lane base+t).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Instruction descriptor for kind::f16 / kind::f8f6f4, fp32 accumulate, both operands K-major.
//   bits [4,6)  accumulator format (1 = F32)       bits [7,10) / [10,13) A / B element format
//   bits [17,23) N >> 3                            bits [24,29) M >> 4
constexpr uint32_t kFmtBf16 = 1;  // kind::f16: 0 = F16, 1 = BF16
constexpr uint32_t kFmtE4M3 = 0;  // kind::f8f6f4: 0 = E4M3
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt, uint32_t m, uint32_t n, uint32_t a_mn_major = 0,
                                                  uint32_t b_mn_major = 0) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

// Shared-memory matrix descriptor for a K-major operand stored as rows of 128 bytes with the
// 128-byte swizzle (what a TMA box of {128 B, rows} with SWIZZLE_128B writes): 8-row groups are
// 1024 bytes apart (SBO), LBO is unused for swizzled K-major layouts, descriptor version 1.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(1) << 16;             // LBO (ignored)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;     // SBO
  d |= static_cast<uint64_t>(1) << 46;             // version
  d |= static_cast<uint64_t>(2) << 61;             // SWIZZLE_128B
  return d;
}

// ---------------------------------------------------------------- programmatic dependent launch
// Every kernel of the library is launched with the programmatic-stream-serialization attribute and
// calls pdl_wait() before it touches memory that an earlier kernel may have written (or may still be
// reading); what runs before the wait (barrier set-up, TMEM allocation, descriptor prefetch, loads of
// constant weights) overlaps the tail of the previous kernel.  pdl_trigger() lets the next kernel in
// the stream start its own preamble.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- step timeline (trace builds only)
// Under -DSLLM_TRACE every launch of the pipelined kernels gets the next 4-word record of a device buffer set with
// sllm_step_trace_set: [0] earliest CTA start, [1] CTA 0 past its dependency wait, [2] latest CTA end (globaltimer
// ns), [3] kernel kind.  Records are assigned on the host when the launch is enqueued (or captured), so a replayed
// graph fills the same records again; clear the buffer to ~0 / 0 between replays.  Never compiled into the product.
#ifdef SLLM_TRACE
unsigned long long* step_trace_next(int kind);      // host: record for the launch being enqueued, or null
__device__ __forceinline__ unsigned long long step_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void step_trace_start(unsigned long long* rec) {
  if (rec && threadIdx.x == 0) atomicMin(rec, step_now());
}
__device__ __forceinline__ void step_trace_waited(unsigned long long* rec) {
  if (rec && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) rec[1] = step_now();
}
__device__ __forceinline__ void step_trace_end(unsigned long long* rec) {
  if (rec && threadIdx.x == 0) atomicMax(rec + 2, step_now());
}
#define STEP_TRACE_FIELD unsigned long long* step_rec;
#define STEP_TRACE_START(p) step_trace_start((p).step_rec)
#define STEP_TRACE_WAITED(p) step_trace_waited((p).step_rec)
#define STEP_TRACE_END(p) step_trace_end((p).step_rec)
#define STEP_TRACE_ASSIGN(p, kind) (p).step_rec = step_trace_next(kind)
#else
#define STEP_TRACE_FIELD
#define STEP_TRACE_START(p)
#define STEP_TRACE_WAITED(p)
#define STEP_TRACE_END(p)
#define STEP_TRACE_ASSIGN(p, kind)
#endif

// ---------------------------------------------------------------- E2M1 (4-bit float: sign | 2-bit exponent | 1-bit mantissa)
// Values 0, 0.5, 1, 1.5, 2, 3, 4, 6.  Encoding rounds to the nearest value, ties to the even index, saturates at 6
// and maps NaN to +0, like the host codec.
__device__ __forceinline__ uint32_t f32_to_e2m1(float v) {
  if (v != v) return 0u;
  const float a = fabsf(v);
  const uint32_t idx = a <= 0.25f ? 0u : a < 0.75f ? 1u : a <= 1.25f ? 2u : a < 1.75f ? 3u : a <= 2.5f ? 4u : a < 3.5f ? 5u
                                                                                                 : a <= 5.0f ? 6u : 7u;
  return idx | ((v < 0.f && idx != 0u) ? 8u : 0u);
}
__device__ __forceinline__ float e2m1_to_f32(uint32_t code) {
  const uint32_t e = (code >> 1) & 3u, m = code & 1u;
  const float mag = e ? __uint_as_float(((126u + e) << 23) | (m << 22)) : 0.5f * static_cast<float>(m);
  return (code & 8u) ? -mag : mag;
}
// Bytes of one NVFP4 KV row of `hd` channels: hd / 2 code bytes (element 2 i in the low nibble of byte i) followed
// by hd / 16 E4M3 block scales; the fp32 outer scale of the row lives in the scale plane.
__host__ __device__ constexpr int nvfp4_row_bytes(int hd) { return hd / 2 + hd / 16; }

// ---------------------------------------------------------------- L2 prefetch
// Requests bytes into L2 with no destination in shared memory and nothing to wait for (16-byte aligned, multiple of 16).
__device__ __forceinline__ void prefetch_l2_bulk(const void* gsrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gsrc), "r"(bytes) : "memory");
}

// ---------------------------------------------------------------- numerics
__device__ __forceinline__ float bf16_to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ __nv_bfloat16 f32_to_bf16(float v) { return __float2bfloat16_rn(v); }

// E4M3FN encode with saturation to +-448 and NaN -> 0x7f (sign dropped), matching the host codec.
__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
  if (v != v) return 0x7f;
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}
// Two packed E4M3 bytes -> float2.
__device__ __forceinline__ float2 e4m3x2_to_f32x2(uint16_t b) {
  __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(b), __NV_E4M3);
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}

// Four packed E4M3 bytes -> four floats, each multiplied by 2^-120, with integer instructions only.
// The 7 exponent/mantissa bits of an E4M3 byte placed at bits [26:20] of an fp32 word (sign at 31) are
// the fp32 encoding of value * 2^-120 (exponent bias 127 vs 7), subnormals included; no conversion
// instruction is issued, which keeps the special-function pipe free.  Callers fold 2^120 into their
// scales in two factors of 2^60 (see kPow60).  0x7f (NaN) decodes as a finite number.
constexpr float kPow60 = 1152921504606846976.f;  // 2^60
__device__ __forceinline__ void e4m3x4_to_f32x4_exp120(uint32_t x, float (&o)[4]) {
  const uint32_t t0 = __byte_perm(x, 0u, 0x1404);  // bytes 0, 1 in the upper byte of each 16-bit lane
  const uint32_t t1 = __byte_perm(x, 0u, 0x3424);  // bytes 2, 3
  const uint32_t h0 = ((t0 & 0x7f007f00u) >> 4) | (t0 & 0x80008000u);  // two bf16 words
  const uint32_t h1 = ((t1 & 0x7f007f00u) >> 4) | (t1 & 0x80008000u);
  o[0] = __uint_as_float(h0 << 16);
  o[1] = __uint_as_float(h0 & 0xffff0000u);
  o[2] = __uint_as_float(h1 << 16);
  o[3] = __uint_as_float(h1 & 0xffff0000u);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Warp-wide maximum in one instruction (f32 redux is an sm_100a feature).
__device__ __forceinline__ float warp_max_redux(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace sllm
