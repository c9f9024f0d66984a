// Paged-KV block mover: the data plane of disaggregated prefill/decode and of KV offload.
//
// One launch copies `n` blocks of EVERY layer from a source pool to a destination pool:
//   dst_layers[l] + dst_ids[i] * block_bytes  <-  src_layers[l] + src_ids[i] * block_bytes
// Either side may be another GPU's memory mapped through CUDA IPC (the consumer pulls from the
// producer's pool over NVLink, or the producer pushes), or pinned host memory (offload tier).
// The id lists and layer-pointer tables live in device memory, so a transfer is a single kernel
// regardless of how many blocks or layers it touches, and no batched-memcpy API is involved.
//
// Role of the reference's multi-layer block scatter and native DMA engine
// (reference: src/vllm_torchtpu/distributed/kv_transfer/kv_scatter.py:14-251, tpu_connector.py:1063).
#include "common.cuh"

namespace b200 {

__global__ void kv_copy_blocks_kernel(const uint8_t* const* __restrict__ src_layers,
                                      uint8_t* const* __restrict__ dst_layers, const int* __restrict__ src_ids,
                                      const int* __restrict__ dst_ids, int n, int num_layers,
                                      size_t block_bytes, long long src_blocks, long long dst_blocks,
                                      int* status) {
  // grid: x = block index i, y = layer
  const int l = blockIdx.y;
  for (int i = blockIdx.x; i < n; i += gridDim.x) {
    const long long s = src_ids[i], d = dst_ids[i];
    if (s < 0 || s >= src_blocks || d < 0 || d >= dst_blocks) {
      if (threadIdx.x == 0 && status) atomicCAS(status, ST_OK, ST_BAD_INDEX);
      continue;
    }
    const uint4* sp = reinterpret_cast<const uint4*>(src_layers[l] + (size_t)s * block_bytes);
    uint4* dp = reinterpret_cast<uint4*>(dst_layers[l] + (size_t)d * block_bytes);
    const size_t nvec = block_bytes >> 4;
    for (size_t v = threadIdx.x; v < nvec; v += blockDim.x) dp[v] = sp[v];
  }
}

// Part of a block: `chunks` pieces of `span_bytes`, piece c at src_off + c * src_stride of the source block and at
// dst_off + c * dst_stride of the destination block.  Source and destination blocks may differ in size: this is
// the move between engines whose tensor-parallel degrees differ (a [2, heads, block_size, head_dim] block of a
// rank holds that rank's KV heads only; a head range is one piece of the K half and one of the V half).
__global__ void kv_copy_block_spans_kernel(const uint8_t* const* __restrict__ src_layers,
                                           uint8_t* const* __restrict__ dst_layers,
                                           const int* __restrict__ src_ids, const int* __restrict__ dst_ids, int n,
                                           size_t src_block_bytes, size_t dst_block_bytes, size_t src_off,
                                           size_t dst_off, size_t span_bytes, int chunks, size_t src_stride,
                                           size_t dst_stride, long long src_blocks, long long dst_blocks,
                                           int* status) {
  const int l = blockIdx.y;
  const size_t nvec = span_bytes >> 4;
  for (int i = blockIdx.x; i < n; i += gridDim.x) {
    const long long s = src_ids[i], d = dst_ids[i];
    if (s < 0 || s >= src_blocks || d < 0 || d >= dst_blocks) {
      if (threadIdx.x == 0 && status) atomicCAS(status, ST_OK, ST_BAD_INDEX);
      continue;
    }
    const uint8_t* sb = src_layers[l] + (size_t)s * src_block_bytes + src_off;
    uint8_t* db = dst_layers[l] + (size_t)d * dst_block_bytes + dst_off;
    for (size_t v = threadIdx.x; v < nvec * (size_t)chunks; v += blockDim.x) {
      const size_t c = v / nvec, e = v - c * nvec;
      reinterpret_cast<uint4*>(db + c * dst_stride)[e] = reinterpret_cast<const uint4*>(sb + c * src_stride)[e];
    }
  }
}

// NaN/Inf screen of the rows about to be saved: flags[i] = 1 if block i of any layer holds a
// non-finite bf16 value (asynchronous KV stores are gated on it,
// reference: src/vllm_torchtpu/distributed/kv_transfer/kv_save_nan_check.py:14-163).
__global__ void kv_nan_check_kernel(const uint8_t* const* __restrict__ layers, const int* __restrict__ ids,
                                    int n, size_t block_bytes, int* __restrict__ flags) {
  const int l = blockIdx.y;
  for (int i = blockIdx.x; i < n; i += gridDim.x) {
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(layers[l] + (size_t)ids[i] * block_bytes);
    int bad = 0;
    for (size_t e = threadIdx.x; e < (block_bytes >> 1); e += blockDim.x) {
      const float f = __bfloat162float(p[e]);
      bad |= !(fabsf(f) <= 3.3e38f);
    }
    if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(&flags[i], 1);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_kv_copy_blocks(const void* const* src_layers_dev, void* const* dst_layers_dev,
                                   const int* src_ids_dev, const int* dst_ids_dev, int n, int num_layers,
                                   size_t block_bytes, long long src_blocks, long long dst_blocks, int* status,
                                   cudaStream_t stream) {
  if (n <= 0 || num_layers <= 0) return 0;
  if (block_bytes % 16) {
    b200_set_last_error("kv_copy_blocks: block size must be a multiple of 16 bytes", __FILE__, __LINE__);
    return -1;
  }
  dim3 grid(n < 1024 ? n : 1024, num_layers);
  kv_copy_blocks_kernel<<<grid, 256, 0, stream>>>((const uint8_t* const*)src_layers_dev,
                                                  (uint8_t* const*)dst_layers_dev, src_ids_dev, dst_ids_dev, n,
                                                  num_layers, block_bytes, src_blocks, dst_blocks, status);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_kv_copy_block_spans(const void* const* src_layers_dev, void* const* dst_layers_dev,
                                        const int* src_ids_dev, const int* dst_ids_dev, int n, int num_layers,
                                        size_t src_block_bytes, size_t dst_block_bytes, size_t src_off,
                                        size_t dst_off, size_t span_bytes, int chunks, size_t src_stride,
                                        size_t dst_stride, long long src_blocks, long long dst_blocks, int* status,
                                        cudaStream_t stream) {
  if (n <= 0 || num_layers <= 0 || chunks <= 0 || span_bytes == 0) return 0;
  if ((src_block_bytes | dst_block_bytes | src_off | dst_off | span_bytes | src_stride | dst_stride) % 16) {
    b200_set_last_error("kv_copy_block_spans: sizes and offsets must be multiples of 16 bytes", __FILE__, __LINE__);
    return -1;
  }
  if (src_off + (size_t)(chunks - 1) * src_stride + span_bytes > src_block_bytes ||
      dst_off + (size_t)(chunks - 1) * dst_stride + span_bytes > dst_block_bytes) {
    b200_set_last_error("kv_copy_block_spans: span leaves the block", __FILE__, __LINE__);
    return -1;
  }
  dim3 grid(n < 1024 ? n : 1024, num_layers);
  kv_copy_block_spans_kernel<<<grid, 256, 0, stream>>>(
      (const uint8_t* const*)src_layers_dev, (uint8_t* const*)dst_layers_dev, src_ids_dev, dst_ids_dev, n,
      src_block_bytes, dst_block_bytes, src_off, dst_off, span_bytes, chunks, src_stride, dst_stride, src_blocks,
      dst_blocks, status);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_kv_nan_check(const void* const* layers_dev, const int* ids_dev, int n, int num_layers,
                                 size_t block_bytes, int* flags_dev, cudaStream_t stream) {
  if (n <= 0) return 0;
  dim3 grid(n < 1024 ? n : 1024, num_layers);
  kv_nan_check_kernel<<<grid, 256, 0, stream>>>((const uint8_t* const*)layers_dev, ids_dev, n, block_bytes,
                                                flags_dev);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_host_register(void* p, size_t bytes) {
  B200_CUDA_CHECK(cudaHostRegister(p, bytes, cudaHostRegisterPortable | cudaHostRegisterMapped));
  return 0;
}
extern "C" int b200_host_alloc(size_t bytes, void** out) {
  B200_CUDA_CHECK(cudaHostAlloc(out, bytes, cudaHostAllocPortable | cudaHostAllocMapped));
  return 0;
}
extern "C" int b200_host_free(void* p) {
  B200_CUDA_CHECK(cudaFreeHost(p));
  return 0;
}
