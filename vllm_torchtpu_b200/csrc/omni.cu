// Diffusion-transformer helpers: q/k RMSNorm over all channels fused with interleaved RoPE.
//
// A Wan-style self-attention block normalises q and k with an RMSNorm over all heads * head_dim
// channels and then rotates the (even, odd) channel pairs of every head by per-token angles that come
// from a table (the angles of a video token mix its frame, row and column, so they are not
// position * inv_freq).  One pass reads the q and k columns of the fused QKV projection and writes the
// normalised, rotated q and k:
//     y   = bf16(x * rsqrt(mean(x^2) + eps) * w)                          fp32 math, one rounding
//     out[2i]     = y[2i] * cos[i] - y[2i + 1] * sin[i]
//     out[2i + 1] = y[2i + 1] * cos[i] + y[2i] * sin[i]                   fp32 math, one rounding
// (reference: src/vllm_torchtpu/kernels/diffusion_attention/qk_norm_rope.py:1-60, omni/rope.py:1-80).
#include "common.cuh"

namespace b200 {

// grid (T, 2): blockIdx.y = 0 handles the q slice of row t, 1 the k slice.  Channel counts are
// multiples of 8, head_dim a multiple of 8; cos / sin are fp32 [T, head_dim / 2].
__global__ void qk_norm_rope_kernel(const __nv_bfloat16* __restrict__ qkv, long long row_stride,
                                    const __nv_bfloat16* __restrict__ wq, const __nv_bfloat16* __restrict__ wk,
                                    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                    __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out,
                                    int Cq, int Ck, int D, float eps) {
  __shared__ float red[32];
  extern __shared__ __align__(16) uint8_t dyn[];
  bf16x8* row_cache = reinterpret_cast<bf16x8*>(dyn);
  const size_t t = blockIdx.x;
  const bool is_k = blockIdx.y != 0;
  const int C = is_k ? Ck : Cq;
  const __nv_bfloat16* x = qkv + t * (size_t)row_stride + (is_k ? Cq : 0);
  const __nv_bfloat16* w = is_k ? wk : wq;
  __nv_bfloat16* y = is_k ? k_out + t * (size_t)Ck : q_out + t * (size_t)Cq;
  const int nvec = C >> 3;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const bf16x8 a = *reinterpret_cast<const bf16x8*>(x + i * 8);
    row_cache[i] = a;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(a.v[j]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  const float tot = block_sum(ss, red);
  const float inv = rsqrtf(tot / (float)C + eps);
  const int half = D >> 1;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const bf16x8 a = row_cache[i];
    const bf16x8 ww = *reinterpret_cast<const bf16x8*>(w + i * 8);
    const int pair0 = ((i * 8) % D) >> 1;                 // first of the four pairs this vector holds
    const float4 c4 = *reinterpret_cast<const float4*>(cos_t + t * half + pair0);
    const float4 s4 = *reinterpret_cast<const float4*>(sin_t + t * half + pair0);
    const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(a.v[j]), g = __bfloat1622float2(ww.v[j]);
      const float2 n = __bfloat1622float2(__floats2bfloat162_rn(f.x * inv * g.x, f.y * inv * g.y));
      o.v[j] = __floats2bfloat162_rn(n.x * cs[j] - n.y * sn[j], n.y * cs[j] + n.x * sn[j]);
    }
    *reinterpret_cast<bf16x8*>(y + i * 8) = o;
  }
}

}  // namespace b200

using namespace b200;

// qkv [T, row_stride] bf16 with q in columns [0, Cq) and k in [Cq, Cq + Ck); wq [Cq], wk [Ck] bf16;
// cos / sin fp32 [T, head_dim / 2]; q_out [T, Cq], k_out [T, Ck] bf16.
extern "C" int b200_qk_norm_rope(const void* qkv, long long row_stride, const void* wq, const void* wk,
                                 const void* cos_t, const void* sin_t, void* q_out, void* k_out, int T, int Cq,
                                 int Ck, int head_dim, float eps, cudaStream_t stream) {
  if (T == 0) return 0;
  if (Cq % 8 || Ck % 8 || head_dim % 8 || row_stride % 8 || Cq % head_dim || Ck % head_dim || Cq <= 0 || Ck <= 0) {
    b200_set_last_error("qk_norm_rope: channel counts, head_dim and the row stride must be multiples of 8 and the "
                        "channel counts multiples of head_dim", __FILE__, __LINE__);
    return -1;
  }
  const int cmax = Cq > Ck ? Cq : Ck;
  int threads = cmax / 8 >= 1024 ? 1024 : ((cmax / 8 + 31) / 32) * 32;
  if (threads < 32) threads = 32;
  const size_t smem = (size_t)cmax * 2;
  if (smem > 200 * 1024) {
    b200_set_last_error("qk_norm_rope: more than 102400 channels per row", __FILE__, __LINE__);
    return -1;
  }
  if (smem > 48 * 1024)
    B200_CUDA_CHECK(cudaFuncSetAttribute(qk_norm_rope_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  qk_norm_rope_kernel<<<dim3(T, 2), threads, smem, stream>>>(
      (const __nv_bfloat16*)qkv, row_stride, (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk,
      (const float*)cos_t, (const float*)sin_t, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out, Cq, Ck, head_dim, eps);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}
