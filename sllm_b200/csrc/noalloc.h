/* Entry point for callers that are not allowed to allocate device memory.
 *
 * This has no counterpart in the reference engine; it exists for embedders of this library.
 *
 * Who needs it: code that runs where cudaMalloc is off limits - a plug-in living inside another
 * process's memory budget, a real-time or safety-audited component whose allocations are frozen
 * after start-up, or a host that hands this library raw device pointers from its own arena and
 * forbids it to take more.  Every other compute entry point of the library already takes its
 * workspace from the caller; this one removes even that requirement for one operation, the row
 * argmax that turns logits into greedy tokens, by keeping the scratch it needs inside the library.
 *
 *   int sllm_argmax_noalloc(logits, out_idx, out_val, rows, n, ld, index_offset, stream)
 *
 * Arguments and results are those of sllm_argmax (bf16 logits [rows, n] with row stride ld; a NaN
 * anywhere in a row gives -1; ties give the lowest index; out_val may be null).  Differences:
 *   - rows may not exceed sllm_argmax_noalloc_max_rows() (256); a larger value is refused with
 *     status 7 (limit exceeded) and nothing is launched;
 *   - the scratch (about 257 KiB: partial records plus one counter per row) is a fixed array in the
 *     library image, so every GPU that loads the library carries it until the process ends;
 *   - the first call on each device looks up the array's device address (the array itself starts zeroed when
 *     the library is loaded).  Make that first call before any stream capture; later calls only launch the kernel;
 *   - ld (the row stride) must be at least n: overlapping rows are refused with status 1;
 *   - all calls share the one array.  It keeps whatever the previous call left there; the counters
 *     are returned to zero by every launch, the records are overwritten before they are read.  Two
 *     calls whose kernels may overlap on the GPU (different streams, no ordering) would race on it:
 *     order them.
 * No cudaMalloc, cudaFree or other allocating routine is called on any path.
 */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

int sllm_argmax_noalloc_max_rows(void);
int sllm_argmax_noalloc(const void* logits, int* out_idx, float* out_val, int rows, int n, int ld, int index_offset,
                        void* stream);

#ifdef __cplusplus
}
#endif
