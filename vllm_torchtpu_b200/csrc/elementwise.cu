// Memory-bound bf16 kernels: RMSNorm (+residual), SiLU*mul, embedding gather with
// on-device token substitution, row gather for the sampling rows, RoPE + per-head
// q/k norm + paged KV-cache write.
//
// Numerics follow the reference's CUDA-style norm providers: normalise and scale in
// fp32, cast once; the fused-add variant first rounds x+residual to bf16 and
// normalises the rounded value (reference: src/vllm_torchtpu/layers/adapter/ir_ops.py:50-88).
// RoPE rotates in fp32 with angles position * inv_freq computed in the kernel
// (reference: src/vllm_torchtpu/layers/adapter/rotary_embedding.py:14-44, rope_patch.py).
#include "common.cuh"

namespace b200 {

// One CTA per row; H % 8 == 0.  ADD: residual += x (rounded to bf16) first.
template <bool ADD>
__global__ void rms_norm_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ residual,
                                const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, int H,
                                float eps) {
  pdl_launch_dependents();      // the GEMM that follows may start and prefetch its weights now
  pdl_wait();                   // this grid may itself have started early
  __shared__ float red[32];
  extern __shared__ __align__(16) uint8_t dyn[];
  bf16x8* row_cache = reinterpret_cast<bf16x8*>(dyn);     // the (summed) row, kept for the second pass
  const size_t base = (size_t)blockIdx.x * H;
  const int nvec = H >> 3;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    bf16x8 a = *reinterpret_cast<const bf16x8*>(x + base + i * 8);
    if (ADD) {
      bf16x8 r = *reinterpret_cast<const bf16x8*>(residual + base + i * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 fa = __bfloat1622float2(a.v[j]), fr = __bfloat1622float2(r.v[j]);
        a.v[j] = __floats2bfloat162_rn(fa.x + fr.x, fa.y + fr.y);
      }
      *reinterpret_cast<bf16x8*>(residual + base + i * 8) = a;
    }
    row_cache[i] = a;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(a.v[j]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  const float tot = block_sum(ss, red);
  const float inv = rsqrtf(tot / (float)H + eps);
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    bf16x8 a = row_cache[i];
    bf16x8 ww = *reinterpret_cast<const bf16x8*>(w + i * 8);
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(a.v[j]), g = __bfloat1622float2(ww.v[j]);
      o.v[j] = __floats2bfloat162_rn(f.x * inv * g.x, f.y * inv * g.y);
    }
    *reinterpret_cast<bf16x8*>(y + base + i * 8) = o;
  }
}

// y[t, i] = silu(x[t, i]) * x[t, I + i]
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int T,
                                int I) {
  const int nvec = I >> 3;
  const size_t total = (size_t)T * nvec;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / nvec;
    const int i = (int)(idx - t * nvec);
    const bf16x8 g = *reinterpret_cast<const bf16x8*>(x + t * 2 * I + i * 8);
    const bf16x8 u = *reinterpret_cast<const bf16x8*>(x + t * 2 * I + I + i * 8);
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 fg = __bfloat1622float2(g.v[j]), fu = __bfloat1622float2(u.v[j]);
      // round silu(g) the way a bf16 elementwise op would not: keep fp32 until the product
      float a = fg.x / (1.f + __expf(-fg.x)), b = fg.y / (1.f + __expf(-fg.y));
      o.v[j] = __floats2bfloat162_rn(a * fu.x, b * fu.y);
    }
    *reinterpret_cast<bf16x8*>(y + t * I + i * 8) = o;
  }
}

// Gated activations of MoE / MLP blocks, y[t, i] = act(gate, up) with gate = x[t, i], up = x[t, I + i]:
//   0 silu(g) * u            1 gelu(g) * u (erf)          2 gelu_tanh(g) * u
//   3 swigluoai: g' = min(g, limit), u' = clamp(u, +-limit), (u' + 1) * g' * sigmoid(alpha * g')   (a = alpha, b = limit)
//   4 silu with clamp: silu(min(g, limit)) * clamp(u, +-limit)                                         (b = limit)
//   5 situ: beta * tanh(g / beta) * sigmoid(g) * (linear_beta > 0 ? linear_beta * tanh(u / linear_beta) : u)
//      (a = beta, b = linear_beta or 0)
// (reference: src/vllm_torchtpu/kernels/megablox/gmm_v2.py:30-58, 100-121)
template <int ACT>
__device__ __forceinline__ float gated_act(float g, float u, float a, float b) {
  if (ACT == 0) return g / (1.f + __expf(-g)) * u;
  if (ACT == 1) return 0.5f * g * (1.f + erff(g * 0.70710678118654752f)) * u;
  if (ACT == 2) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
  if (ACT == 3) {
    const float gc = fminf(g, b), uc = fminf(fmaxf(u, -b), b);
    return (uc + 1.f) * gc / (1.f + __expf(-a * gc));
  }
  if (ACT == 4) {
    const float gc = fminf(g, b), uc = fminf(fmaxf(u, -b), b);
    return gc / (1.f + __expf(-gc)) * uc;
  }
  const float gg = a * tanhf(g / a) / (1.f + __expf(-g));
  return gg * (b > 0.f ? b * tanhf(u / b) : u);
}

template <int ACT>
__global__ void gated_act_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int T, int I,
                                 float a, float b) {
  const int nvec = I >> 3;
  const size_t total = (size_t)T * nvec;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / nvec;
    const int i = (int)(idx - t * nvec);
    const bf16x8 g = *reinterpret_cast<const bf16x8*>(x + t * 2 * I + i * 8);
    const bf16x8 u = *reinterpret_cast<const bf16x8*>(x + t * 2 * I + I + i * 8);
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 fg = __bfloat1622float2(g.v[j]), fu = __bfloat1622float2(u.v[j]);
      o.v[j] = __floats2bfloat162_rn(gated_act<ACT>(fg.x, fu.x, a, b), gated_act<ACT>(fg.y, fu.y, a, b));
    }
    *reinterpret_cast<bf16x8*>(y + t * I + i * 8) = o;
  }
}

// out[t] = table[ token_src[t] >= 0 ? last_tokens[token_src[t]] : ids[t] ]
__global__ void embedding_kernel(const int* __restrict__ ids, const int* __restrict__ token_src,
                                 const int* __restrict__ last_tokens, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, int H, int vocab) {
  const int t = blockIdx.x;
  int id = ids[t];
  if (token_src != nullptr) {
    const int src = token_src[t];
    if (src >= 0) id = last_tokens[src];
  }
  id = min(max(id, 0), vocab - 1);
  const bf16x8* srcp = reinterpret_cast<const bf16x8*>(table + (size_t)id * H);
  bf16x8* dst = reinterpret_cast<bf16x8*>(out + (size_t)t * H);
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) dst[i] = srcp[i];
}

// out_h[r] = hidden[idx[r]], out_r[r] = residual[idx[r]]
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ hidden,
                                   const __nv_bfloat16* __restrict__ residual, const int* __restrict__ idx,
                                   __nv_bfloat16* __restrict__ out_h, __nv_bfloat16* __restrict__ out_r, int H,
                                   int T) {
  const int r = blockIdx.x;
  const int t = min(max(idx[r], 0), T - 1);
  const bf16x8* h = reinterpret_cast<const bf16x8*>(hidden + (size_t)t * H);
  bf16x8* oh = reinterpret_cast<bf16x8*>(out_h + (size_t)r * H);
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) oh[i] = h[i];
  if (residual != nullptr) {
    const bf16x8* rr = reinterpret_cast<const bf16x8*>(residual + (size_t)t * H);
    bf16x8* orr = reinterpret_cast<bf16x8*>(out_r + (size_t)r * H);
    for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) orr[i] = rr[i];
  }
}

__global__ void scatter_tokens_kernel(const int* __restrict__ tokens, const int* __restrict__ slots,
                                      int* __restrict__ last_tokens, int R, int cap) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < R) {
    const int s = slots[r];
    if (s >= 0 && s < cap) last_tokens[s] = tokens[r];
  }
}

// ------------------------------------------------------------------ RoPE + KV write
// One CTA per token, one warp per head (q heads, then k heads, then v heads).
// qkv: [T, (Hq + 2 Hkv) * D] packed.  q_out: [T, Hq, D].  Cache: [blocks, 2, Hkv, bs, D].
template <int D, typename CacheT>
__global__ void rope_cache_kernel(const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int rot_pairs,
                                  const int* __restrict__ slot_mapping, __nv_bfloat16* __restrict__ q_out,
                                  CacheT* __restrict__ kv_cache, const __nv_bfloat16* __restrict__ q_norm_w,
                                  const __nv_bfloat16* __restrict__ k_norm_w, float eps, int Hq, int Hkv,
                                  int block_size, int interleaved, float k_inv_scale, float v_inv_scale,
                                  long long num_slots) {
  constexpr int EPL = D / 32;               // elements per lane
  __shared__ float cs[D];                   // cos[0..rot_pairs) | sin[0..rot_pairs)
  pdl_launch_dependents();
  pdl_wait();                               // qkv comes from the GEMM before this grid
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < rot_pairs; i += blockDim.x) {
    float s, c;
    sincosf(pos * inv_freq[i], &s, &c);
    cs[i] = c;
    cs[D / 2 + i] = s;
  }
  __syncthreads();
  const long long slot = slot_mapping[t];
  const int heads = Hq + 2 * Hkv;
  const __nv_bfloat16* row = qkv + (size_t)t * heads * D;
  for (int h = warp; h < heads; h += nw) {
    const int kind = h < Hq ? 0 : (h < Hq + Hkv ? 1 : 2);       // q, k, v
    const __nv_bfloat16* src = row + (size_t)h * D;
    // lane owns elements e(u): neox -> pairs (i, i + D/2) with i = lane*EPL/2 + u; interleaved -> (2i, 2i+1)
    float x[EPL];
    int idx[EPL];
#pragma unroll
    for (int u = 0; u < EPL / 2; ++u) {
      const int i = lane * (EPL / 2) + u;
      if (interleaved) {
        idx[2 * u] = 2 * i;
        idx[2 * u + 1] = 2 * i + 1;
      } else {
        idx[2 * u] = i;
        idx[2 * u + 1] = i + D / 2;
      }
    }
#pragma unroll
    for (int u = 0; u < EPL; ++u) x[u] = __bfloat162float(src[idx[u]]);
    if (kind < 2) {
      const __nv_bfloat16* nw_ptr = kind == 0 ? q_norm_w : k_norm_w;
      if (nw_ptr != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int u = 0; u < EPL; ++u) ss += x[u] * x[u];
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
        for (int u = 0; u < EPL; ++u)
          x[u] = __bfloat162float(__float2bfloat16(x[u] * inv * __bfloat162float(nw_ptr[idx[u]])));
      }
#pragma unroll
      for (int u = 0; u < EPL / 2; ++u) {
        const int i = lane * (EPL / 2) + u;
        if (i < rot_pairs) {
          const float c = cs[i], s = cs[D / 2 + i];
          const float a = x[2 * u], b = x[2 * u + 1];
          x[2 * u] = a * c - b * s;
          x[2 * u + 1] = b * c + a * s;
        }
      }
    }
    if (kind == 0) {
      __nv_bfloat16* dst = q_out + ((size_t)t * Hq + h) * D;
#pragma unroll
      for (int u = 0; u < EPL; ++u) dst[idx[u]] = __float2bfloat16(x[u]);
    } else if (kv_cache != nullptr && slot >= 0 && slot < num_slots) {
      const int hk = kind == 1 ? h - Hq : h - Hq - Hkv;
      const long long blk = slot / block_size;
      const int off = (int)(slot - blk * block_size);
      CacheT* dst = kv_cache + ((((size_t)blk * 2 + (kind - 1)) * Hkv + hk) * block_size + off) * D;
      const float sc = kind == 1 ? k_inv_scale : v_inv_scale;
#pragma unroll
      for (int u = 0; u < EPL; ++u) {
        if constexpr (sizeof(CacheT) == 2) {
          dst[idx[u]] = __float2bfloat16(x[u]);
        } else {
          dst[idx[u]] = CacheT(x[u] * sc);
        }
      }
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_rms_norm(const void* x, void* residual, const void* w, void* y, int T, int H, float eps,
                             cudaStream_t stream) {
  if (T == 0) return 0;
  if (H % 8) {
    b200_set_last_error("rms_norm: hidden size must be a multiple of 8", __FILE__, __LINE__);
    return -1;
  }
  int threads = H / 8 >= 1024 ? 1024 : ((H / 8 + 31) / 32) * 32;
  if (threads < 32) threads = 32;
  size_t smem = (size_t)H * 2;
  if (residual)
    B200_CUDA_CHECK(launch_pdl(rms_norm_kernel<true>, dim3(T), dim3(threads), smem, stream,
                               (const __nv_bfloat16*)x, (__nv_bfloat16*)residual, (const __nv_bfloat16*)w,
                               (__nv_bfloat16*)y, H, eps));
  else
    B200_CUDA_CHECK(launch_pdl(rms_norm_kernel<false>, dim3(T), dim3(threads), smem, stream,
                               (const __nv_bfloat16*)x, (__nv_bfloat16*)nullptr, (const __nv_bfloat16*)w,
                               (__nv_bfloat16*)y, H, eps));
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_silu_and_mul(const void* x, void* y, int T, int I, cudaStream_t stream) {
  if (T == 0) return 0;
  if (I % 8) {
    b200_set_last_error("silu_and_mul: width must be a multiple of 8", __FILE__, __LINE__);
    return -1;
  }
  size_t total = (size_t)T * (I / 8);
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  silu_mul_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, T, I);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// x [T, 2I] (gate columns first) -> y [T, I]; act and its parameters a, b as listed at gated_act.
extern "C" int b200_gated_act(const void* x, void* y, int T, int I, int act, float a, float b,
                              cudaStream_t stream) {
  if (T == 0) return 0;
  if (I % 8 || act < 0 || act > 5) {
    b200_set_last_error("gated_act: width must be a multiple of 8, activation 0..5", __FILE__, __LINE__);
    return -1;
  }
  size_t total = (size_t)T * (I / 8);
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
  __nv_bfloat16* yp = (__nv_bfloat16*)y;
  switch (act) {
    case 0: gated_act_kernel<0><<<blocks, 256, 0, stream>>>(xp, yp, T, I, a, b); break;
    case 1: gated_act_kernel<1><<<blocks, 256, 0, stream>>>(xp, yp, T, I, a, b); break;
    case 2: gated_act_kernel<2><<<blocks, 256, 0, stream>>>(xp, yp, T, I, a, b); break;
    case 3: gated_act_kernel<3><<<blocks, 256, 0, stream>>>(xp, yp, T, I, a, b); break;
    case 4: gated_act_kernel<4><<<blocks, 256, 0, stream>>>(xp, yp, T, I, a, b); break;
    default: gated_act_kernel<5><<<blocks, 256, 0, stream>>>(xp, yp, T, I, a, b); break;
  }
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_embedding(const int* ids, const int* token_src, const int* last_tokens, const void* table,
                              void* out, int T, int H, int vocab, cudaStream_t stream) {
  if (T == 0) return 0;
  embedding_kernel<<<T, 128, 0, stream>>>(ids, token_src, last_tokens, (const __nv_bfloat16*)table,
                                          (__nv_bfloat16*)out, H, vocab);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_gather_rows(const void* hidden, const void* residual, const int* idx, void* out_h,
                                void* out_r, int R, int H, int T, cudaStream_t stream) {
  if (R == 0) return 0;
  gather_rows_kernel<<<R, 128, 0, stream>>>((const __nv_bfloat16*)hidden, (const __nv_bfloat16*)residual, idx,
                                            (__nv_bfloat16*)out_h, (__nv_bfloat16*)out_r, H, T);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_scatter_tokens(const int* tokens, const int* slots, int* last_tokens, int R, int cap,
                                   cudaStream_t stream) {
  if (R == 0) return 0;
  scatter_tokens_kernel<<<(R + 127) / 128, 128, 0, stream>>>(tokens, slots, last_tokens, R, cap);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// cache_elem_bytes: 2 = bf16 cache, 1 = fp8 e4m3 cache (values divided by k_scale / v_scale)
extern "C" int b200_rope_and_cache(const void* qkv, const int* positions, const float* inv_freq, int rot_pairs,
                                   const int* slot_mapping, void* q_out, void* kv_cache, const void* q_norm_w,
                                   const void* k_norm_w, float eps, int T, int Hq, int Hkv, int D,
                                   int block_size, long long num_blocks, int interleaved, int cache_elem_bytes,
                                   float k_scale, float v_scale, cudaStream_t stream) {
  if (T == 0) return 0;
  const long long num_slots = num_blocks * block_size;
  int heads = Hq + 2 * Hkv;
  int threads = heads >= 8 ? 256 : heads * 32;
#define LAUNCH(DD, CT)                                                                                       \
  B200_CUDA_CHECK(launch_pdl(rope_cache_kernel<DD, CT>, dim3(T), dim3(threads), 0, stream,                   \
      (const __nv_bfloat16*)qkv, positions, inv_freq, rot_pairs, slot_mapping, (__nv_bfloat16*)q_out,        \
      (CT*)kv_cache, (const __nv_bfloat16*)q_norm_w, (const __nv_bfloat16*)k_norm_w, eps, Hq, Hkv,           \
      block_size, interleaved, 1.f / k_scale, 1.f / v_scale, num_slots))
  if (cache_elem_bytes == 2) {
    if (D == 128) LAUNCH(128, __nv_bfloat16);
    else if (D == 64) LAUNCH(64, __nv_bfloat16);
    else if (D == 256) LAUNCH(256, __nv_bfloat16);
    else {
      b200_set_last_error("rope_and_cache: head_dim must be 64, 128 or 256", __FILE__, __LINE__);
      return -1;
    }
  } else {
    if (D == 128) LAUNCH(128, __nv_fp8_e4m3);
    else if (D == 64) LAUNCH(64, __nv_fp8_e4m3);
    else {
      b200_set_last_error("rope_and_cache: fp8 cache needs head_dim 64 or 128", __FILE__, __LINE__);
      return -1;
    }
  }
#undef LAUNCH
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}
