// TMA tensor-map helpers shared by the kernels that stream K-major matrices (defined in gemm_tcgen05.cu).
#pragma once
#include <cuda.h>

namespace sllm {

// Tensor map over a row-major [rows, k_elems] matrix (row stride in bytes) with a box of
// {128 bytes of the row, box_rows rows} and the 128-byte swizzle.  Results are cached per
// (pointer, shape, box); returns an SllmStatus code.
int cached_kmajor_tmap(CUtensorMap* out, const void* ptr, int elem_bytes, long long rows, long long k_elems,
                       long long row_stride_bytes, int box_rows);

// Tensor map over a row-major byte matrix [rows, row_bytes] with a box of {box_bytes, box_rows} and no swizzle
// (box_bytes, the row stride and the base address are multiples of 16).  Cached like the one above.
int cached_plain_tmap(CUtensorMap* out, const void* ptr, long long rows, long long row_bytes, long long row_stride_bytes,
                      int box_bytes, int box_rows);

}  // namespace sllm
