// Symmetric peer memory for the fused compute+collective kernels, and small stand-alone collectives
// built on it (used where no GEMM precedes the exchange).
//
// Every rank allocates the same-sized device region, exports it as a CUDA IPC handle, and opens the
// peers' handles; the resulting pointer table lets a kernel on any rank store into, or load from,
// any other rank's region over NVLink / NVSwitch.  NCCL (through torch.distributed) is used only to
// exchange the 64-byte handles at start-up.  The reference has no multi-GPU path at all
// (docs/architecture/runtime.md:547-555); this file has no counterpart there.
//
// Rules kept here: plain ld/st/red to peer addresses only and no cluster multicast anywhere; the one place
// that reads peer memory with TMA is the all-gather GEMM (gemm_tcgen05.cu), through plain, non-multicast tiled
// loads whose tensor maps are built per peer buffer.  Every wait on a peer flag is bounded and reports through
// the status word.
#include "common.cuh"
#include "api.h"
#include <cstring>

using namespace sllm;

SLLM_EXPORT int sllm_symm_alloc(long long bytes, void** dev_ptr, unsigned char* handle64) {
  if (bytes <= 0 || !dev_ptr || !handle64) return SLLM_ERR_INVALID_ARGUMENT;
  void* p = nullptr;
  if (cudaMalloc(&p, static_cast<size_t>(bytes)) != cudaSuccess) return SLLM_ERR_CUDA;
  if (cudaMemset(p, 0, static_cast<size_t>(bytes)) != cudaSuccess) {
    cudaFree(p);
    return SLLM_ERR_CUDA;
  }
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaFree(p);
    return SLLM_ERR_CUDA;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  cudaDeviceSynchronize();
  *dev_ptr = p;
  return SLLM_OK;
}

SLLM_EXPORT int sllm_symm_open(const unsigned char* handle64, void** dev_ptr) {
  if (!handle64 || !dev_ptr) return SLLM_ERR_INVALID_ARGUMENT;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return SLLM_ERR_CUDA;
  }
  *dev_ptr = p;
  return SLLM_OK;
}

SLLM_EXPORT int sllm_symm_close(void* peer_ptr) {
  if (!peer_ptr) return SLLM_ERR_INVALID_ARGUMENT;
  return cudaIpcCloseMemHandle(peer_ptr) == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

SLLM_EXPORT int sllm_symm_free(void* dev_ptr) {
  if (!dev_ptr) return SLLM_ERR_INVALID_ARGUMENT;
  return cudaFree(dev_ptr) == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

namespace sllm {

struct PeerTable {
  int world, rank;
  void* base[8];  // base[p]: rank p's region as mapped in this process
};

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded wait until *flag >= target (wrap-safe).  Returns false when the limit ran out.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t target, int* status) {
  uint32_t spins = 0;
  long long t0 = 0;
  while (static_cast<int32_t>(ld_acquire_sys_u32(flag) - target) < 0) {
    ++spins;
    if (spins == 1024) t0 = clock64();
    if (spins > 1024 && (spins & 63) == 0 && clock64() - t0 > kWaitLimitCycles) {
      if (status) atomicCAS(status, 0, SLLM_DEV_TIMEOUT_PEER_FLAG);
      return false;
    }
  }
  return true;
}

// One-shot all-gather of a small per-rank record (e.g. the (value, index) pair of a vocabulary-shard
// argmax, or sampling statistics): every rank stores its `bytes` into slot [rank] of every peer's
// region and raises a flag; each rank then waits for all flags.  Region layout: data
// [2 parities][world][slot_bytes] at `offset`, [world] uint32 flags at the fixed `flag_offset`
// (independent of the record size of a call); `epoch` is a local counter.
__global__ void allgather_small_kernel(PeerTable pt, long long offset, long long flag_offset, int slot_bytes,
                                       const uint8_t* src, uint8_t* dst, uint32_t* epoch, int* status) {
  pdl_wait();
  pdl_trigger();
  __shared__ uint32_t s_e;
  if (threadIdx.x == 0) {
    s_e = *epoch + 1;
    *epoch = s_e;
  }
  __syncthreads();
  const uint32_t e = s_e;
  const long long par = static_cast<long long>(e & 1) * pt.world * slot_bytes;
  for (int p = 0; p < pt.world; ++p) {
    uint8_t* region = static_cast<uint8_t*>(pt.base[p]) + offset;
    for (int i = threadIdx.x; i < slot_bytes; i += blockDim.x) region[par + pt.rank * slot_bytes + i] = src[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < pt.world) {
    uint32_t* pf = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(pt.base[threadIdx.x]) + flag_offset);
    st_release_sys_u32(pf + pt.rank, e);
    const uint32_t* mf = reinterpret_cast<const uint32_t*>(static_cast<uint8_t*>(pt.base[pt.rank]) + flag_offset);
    wait_flag(mf + threadIdx.x, e, status);
  }
  __syncthreads();
  const uint8_t* mine = static_cast<const uint8_t*>(pt.base[pt.rank]) + offset + par;
  for (int i = threadIdx.x; i < pt.world * slot_bytes; i += blockDim.x) dst[i] = __ldcg(mine + i);
}

// Merge per-shard argmax records: rows x world (value fp32, index int32) -> best index per row
// (largest value, ties to the lowest index, any -1 (NaN shard) wins).
__global__ void argmax_merge_kernel(const float* vals, const int* idx, int* out, int rows, int world) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  bool nan = false;
  for (int w = 0; w < world; ++w) {
    const float v = vals[w * rows + r];
    const int i = idx[w * rows + r];
    if (i < 0) nan = true;
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
  out[r] = nan ? -1 : bi;
}

}  // namespace sllm

SLLM_EXPORT int sllm_allgather_small(const void* const* bases, int world, int rank, long long offset,
                                     long long flag_offset, int slot_bytes, const void* src, void* dst, void* epoch,
                                     int* status, void* stream) {
  if (!bases || world < 2 || world > 8 || rank < 0 || rank >= world || slot_bytes <= 0 || !src || !dst || !epoch)
    return SLLM_ERR_INVALID_ARGUMENT;
  PeerTable pt;
  pt.world = world;
  pt.rank = rank;
  for (int i = 0; i < world; ++i) pt.base[i] = const_cast<void*>(bases[i]);
  launch_kernel(allgather_small_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream), 1u, 
      pt, offset, flag_offset, slot_bytes, static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst),
      static_cast<uint32_t*>(epoch), status);
  return cudaGetLastError() == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}

SLLM_EXPORT int sllm_argmax_merge(const float* vals, const int* idx, int* out, int rows, int world, void* stream) {
  if (!vals || !idx || !out || rows <= 0 || world <= 0) return SLLM_ERR_INVALID_ARGUMENT;
  launch_kernel(argmax_merge_kernel, dim3((rows + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream), 1u, vals, idx, out, rows, world);
  return cudaGetLastError() == cudaSuccess ? SLLM_OK : SLLM_ERR_CUDA;
}
