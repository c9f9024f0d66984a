// C entry points of the tcgen05 GEMM family (loaded through ctypes).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Tile / split-K plan for a problem size: BN (token tile), number of K splits, scratch bytes
// and number of tile counters the split-K path needs.
int b200_gemm_plan(int T, int N, int K, int num_sms, int* bn_out, int* splits_out, size_t* ws_bytes,
                   int* counters_needed);

// Y[T,N] = X[T,K] * W[N,K]^T (+ bias[N]); bf16 in/out, fp32 accumulate.  ld* in elements.
// ws/counters are split-K scratch (counters zero before first use; re-armed by the kernel).
// status: optional device int that receives a b200 status code if a bounded wait expires.
int b200_gemm_bf16(const void* X, const void* W, void* Y, const void* bias, int T, int N, int K, int ldx,
                   int ldw, int ldy, void* ws, size_t ws_bytes, int* counters, int counters_len, int* status,
                   int num_sms, int force_splits, cudaStream_t stream);

int b200_make_tmap_2d(void* out_map, const void* ptr, int elem_bytes, uint64_t rows, uint64_t cols,
                      uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols);
int b200_make_tmap_2d_bytes_linear(void* out_map, const void* ptr, uint64_t rows, uint64_t cols,
                                   uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols);
int b200_make_tmap_3d_bf16(void* out_map, const void* ptr, uint64_t dx, uint64_t dy, uint64_t dz,
                           uint64_t stride_y_bytes, uint64_t stride_z_bytes, uint32_t bx, uint32_t by,
                           uint32_t bz);

#ifdef __cplusplus
}
#endif
