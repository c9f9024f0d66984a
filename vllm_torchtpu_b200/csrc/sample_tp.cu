// Vocab-parallel greedy sampling: every tensor-parallel rank takes the arg-max of its own vocab
// shard (value + local index); after a tiny all-gather of those pairs this kernel picks, per row,
// the winning shard and converts the local index to a global token id.  Avoids gathering the
// full [rows, vocab] logits (reference: src/vllm_torchtpu/runner/greedy_top_tokens.py).
#include "common.cuh"

namespace b200 {

template <typename T>
__device__ __forceinline__ float ldl(const T* p, int i);
template <>
__device__ __forceinline__ float ldl<__nv_bfloat16>(const __nv_bfloat16* p, int i) { return __bfloat162float(p[i]); }
template <>
__device__ __forceinline__ float ldl<float>(const float* p, int i) { return p[i]; }

template <typename T>
__global__ void __launch_bounds__(1024)
argmax_pair_kernel(const T* __restrict__ logits, int ld, int V, float* __restrict__ val_out,
                   int* __restrict__ idx_out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const T* row = logits + (size_t)blockIdx.x * ld;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = ldl(row, i);
    if (v > bv) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = lane < (blockDim.x >> 5) ? sv[lane] : -INFINITY;
    bi = lane < (blockDim.x >> 5) ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) {
      val_out[blockIdx.x] = bv;
      idx_out[blockIdx.x] = bi < V ? bi : 0;
    }
  }
}

// vals/idx: [world, R] gathered pairs; token = shard * shard_size + local index of the best value
// (lowest shard wins ties, matching an arg-max over the concatenated vocab).
__global__ void select_best_kernel(const float* __restrict__ vals, const int* __restrict__ idx, int world,
                                   int R, int shard_size, int* __restrict__ out) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  float bv = -INFINITY;
  int best = 0;
  for (int w = 0; w < world; ++w) {
    const float v = vals[(size_t)w * R + r];
    if (v > bv) { bv = v; best = w * shard_size + idx[(size_t)w * R + r]; }
  }
  out[r] = best;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_argmax_pair(const void* logits, int dtype, int R, int V, int ld, float* val_out,
                                int* idx_out, cudaStream_t stream) {
  if (R == 0) return 0;
  if (dtype == 0)
    argmax_pair_kernel<__nv_bfloat16><<<R, 1024, 0, stream>>>((const __nv_bfloat16*)logits, ld, V, val_out,
                                                              idx_out);
  else
    argmax_pair_kernel<float><<<R, 1024, 0, stream>>>((const float*)logits, ld, V, val_out, idx_out);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_select_best(const float* vals, const int* idx, int world, int R, int shard_size, int* out,
                                cudaStream_t stream) {
  if (R == 0) return 0;
  select_best_kernel<<<(R + 127) / 128, 128, 0, stream>>>(vals, idx, world, R, shard_size, out);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}
