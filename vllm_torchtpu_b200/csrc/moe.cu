// MoE routing and token permutation kernels.
//
//  * route: scoring (softmax | sigmoid) -> optional score-correction bias and grouped
//    top-k -> top-k -> renormalise -> scale, one warp per token
//    (semantics: reference src/vllm_torchtpu/layers/adapter/moe_routing.py:161-343).
//  * permute plan: counting sort of the (token, k) entries by local expert, giving
//    per-expert row offsets, the source token of every sorted row and the inverse map
//    (the reference's counting-sort permute, src/vllm_torchtpu/layers/core/fused_moe_gmm.py:242-337).
//  * gather: copy token rows into expert order for the grouped GEMM.
//  * unpermute: out[t] = sum_j w[t,j] * y[pos(t,j)] in fp32.
// Everything is sized by T*k on the host and reads the actual counts from device memory, so
// the sequence is CUDA-graph safe.
#include "common.cuh"

namespace b200 {

constexpr int ROUTE_MAX_E = 512;
constexpr int ROUTE_WARPS = 4;

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ logits, int ld, int Tn, int E, int top_k, int sigmoid,
                                 int renorm, float scaling, const float* __restrict__ bias, int n_group,
                                 int topk_group, int* __restrict__ ids_out, float* __restrict__ w_out) {
  __shared__ float s_score[ROUTE_WARPS][ROUTE_MAX_E];
  __shared__ float s_choice[ROUTE_WARPS][ROUTE_MAX_E];
  __shared__ float s_group[ROUTE_WARPS][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= Tn) return;
  float* score = s_score[warp];
  float* choice = s_choice[warp];
  const T* row = logits + (size_t)t * ld;
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) {
    const float v = to_f(row[e]);
    score[e] = v;
    mx = fmaxf(mx, v);
  }
  mx = warp_max(mx);
  if (sigmoid) {
    for (int e = lane; e < E; e += 32) score[e] = 1.f / (1.f + __expf(-score[e]));
  } else {
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float p = __expf(score[e] - mx);
      score[e] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int e = lane; e < E; e += 32) score[e] *= inv;
  }
  for (int e = lane; e < E; e += 32) choice[e] = score[e] + (bias != nullptr ? bias[e] : 0.f);
  __syncwarp();
  if (n_group > 1) {
    const int per = E / n_group;
    // group score: max, or sum of the two best when a bias is in play
    if (lane < n_group) {
      float a = -INFINITY, b = -INFINITY;
      for (int i = 0; i < per; ++i) {
        const float v = choice[lane * per + i];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      s_group[warp][lane] = bias != nullptr ? a + b : a;
    }
    __syncwarp();
    // keep the topk_group best groups (lowest index wins ties)
    unsigned keep = 0;
    for (int j = 0; j < topk_group; ++j) {
      float best = -INFINITY;
      int bi = 0;
      for (int g = 0; g < n_group; ++g) {
        if (!((keep >> g) & 1u) && s_group[warp][g] > best) { best = s_group[warp][g]; bi = g; }
      }
      keep |= 1u << bi;
    }
    for (int e = lane; e < E; e += 32)
      if (!((keep >> (e / per)) & 1u)) choice[e] = -INFINITY;
    __syncwarp();
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int j = 0; j < top_k; ++j) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = choice[e];
      if (v > bv) { bv = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (bi >= E) bi = 0;
    const float w = score[bi];
    wsum += w;
    if (lane == j) { my_w = w; my_id = bi; }
    __syncwarp();
    if (lane == 0) choice[bi] = -INFINITY;
    __syncwarp();
  }
  if (lane < top_k) {
    float w = my_w;
    if (renorm) w = w / fmaxf(wsum, 1e-20f);
    ids_out[(size_t)t * top_k + lane] = my_id;
    w_out[(size_t)t * top_k + lane] = w * scaling;
  }
}

// One CTA.  entries = T * k.  Experts outside [e_lo, e_lo + E_local) are not local (inv_pos = -1).
__global__ void __launch_bounds__(1024)
moe_permute_plan_kernel(const int* __restrict__ ids, int entries, int top_k, int e_lo, int E_local,
                        int* __restrict__ group_off, int* __restrict__ row_src, int* __restrict__ inv_pos) {
  extern __shared__ int s_cnt[];                 // [E_local + 1] counts, then cursors
  for (int e = threadIdx.x; e <= E_local; e += blockDim.x) s_cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int e = ids[i] - e_lo;
    if (e >= 0 && e < E_local) atomicAdd(&s_cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E_local; ++e) {
      const int c = s_cnt[e];
      group_off[e] = run;
      s_cnt[e] = run;                            // becomes the cursor
      run += c;
    }
    group_off[E_local] = run;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int e = ids[i] - e_lo;
    int pos = -1;
    if (e >= 0 && e < E_local) {
      pos = atomicAdd(&s_cnt[e], 1);
      row_src[pos] = i / top_k;
    }
    inv_pos[i] = pos;
  }
}

// x_perm[pos] = x[row_src[pos]] for pos < group_off[E_local]
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_src,
                                  const int* __restrict__ group_off, int E_local,
                                  __nv_bfloat16* __restrict__ x_perm, int H, int T) {
  const int total = group_off[E_local];
  for (int pos = blockIdx.x; pos < total; pos += gridDim.x) {
    const int t = min(max(row_src[pos], 0), T - 1);
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * H);
    uint4* dst = reinterpret_cast<uint4*>(x_perm + (size_t)pos * H);
    for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) dst[i] = src[i];
  }
}

// out[t] = sum_j w[t,j] * y[inv_pos[t,j]]   (rows with inv_pos < 0 belong to other ranks)
__global__ void moe_unpermute_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ inv_pos,
                                     const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int H,
                                     int top_k, int rows_cap) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      const int pos = inv_pos[(size_t)t * top_k + j];
      if (pos < 0 || pos >= rows_cap) continue;
      const float wt = w[(size_t)t * top_k + j];
      const uint4 raw = *(reinterpret_cast<const uint4*>(y + (size_t)pos * H) + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h[q]);
        acc[2 * q] += wt * f.x;
        acc[2 * q + 1] += wt * f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) oh[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    *(reinterpret_cast<uint4*>(out + (size_t)t * H) + i) = o;
  }
}

}  // namespace b200

namespace b200 {
// After routing: rows at or beyond *num_valid (padding of a captured bucket or of a lockstep step) lose their
// experts (id -1 is ignored by permute, dispatch and combine), and a routing simulation may replace the
// router's choice: 1 = round-robin over (token, k), perfectly balanced; 2 = hashed start expert per token with
// the k experts E / k apart.  Simulated weights are 1 / k.
// (reference: src/vllm_torchtpu/layers/adapter/token_padding.py, moe_routing.py routing simulation)
__global__ void moe_route_post_kernel(int* __restrict__ ids, float* __restrict__ w, int T, int k, int E,
                                      const int* __restrict__ num_valid, int sim) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * k) return;
  const int t = i / k, j = i - t * k;
  if (num_valid != nullptr && t >= *num_valid) {
    ids[i] = -1;
    w[i] = 0.f;
    return;
  }
  if (sim == 1) {
    ids[i] = i % E;
    w[i] = 1.f / (float)k;
  } else if (sim == 2) {
    uint32_t h = (uint32_t)t * 2654435761u;
    h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
    const int stride = E / k > 0 ? E / k : 1;
    ids[i] = (int)((h % (uint32_t)E + (uint32_t)(j * stride)) % (uint32_t)E);
    w[i] = 1.f / (float)k;
  }
}
// y[r, :] += bias[e, :] for the rows r of expert e (rows grouped by expert: group_off[e] <= r < group_off[e + 1]);
// expert biases of MoE blocks whose experts carry them (in front of the activation and behind the down projection).
__global__ void group_bias_add_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ bias,
                                      const int* __restrict__ group_off, int R, int N, int ldy, int E) {
  for (int r = blockIdx.x; r < R; r += gridDim.x) {
    if (r >= group_off[E]) break;                   // rows behind the last group are padding
    int lo = 0, hi = E;                             // largest e with group_off[e] <= r
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (group_off[mid] <= r) lo = mid; else hi = mid;
    }
    const bf16x8* b = reinterpret_cast<const bf16x8*>(bias + (size_t)lo * N);
    bf16x8* row = reinterpret_cast<bf16x8*>(y + (size_t)r * ldy);
    for (int i = threadIdx.x; i < (N >> 3); i += blockDim.x) {
      bf16x8 v = row[i];
      const bf16x8 w = b[i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 a = __bfloat1622float2(v.v[j]), c = __bfloat1622float2(w.v[j]);
        v.v[j] = __floats2bfloat162_rn(a.x + c.x, a.y + c.y);
      }
      row[i] = v;
    }
  }
}
}  // namespace b200

using namespace b200;

extern "C" int b200_group_bias_add(void* y, const void* bias, const int* group_off, int R, int N, int ldy, int E,
                                   cudaStream_t stream) {
  if (R <= 0 || N <= 0 || E <= 0) return 0;
  if (N % 8 || ldy % 8) {
    b200_set_last_error("group_bias_add: width and row stride must be multiples of 8", __FILE__, __LINE__);
    return -1;
  }
  const int blocks = R < 148 * 8 ? R : 148 * 8;
  group_bias_add_kernel<<<blocks, 128, 0, stream>>>((__nv_bfloat16*)y, (const __nv_bfloat16*)bias, group_off, R, N,
                                                    ldy, E);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_moe_route_post(int* ids, float* w, int T, int k, int E, const int* num_valid, int sim,
                                   cudaStream_t stream) {
  if (T * k == 0 || (num_valid == nullptr && sim == 0)) return 0;
  moe_route_post_kernel<<<(T * k + 255) / 256, 256, 0, stream>>>(ids, w, T, k, E, num_valid, sim);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// dtype: 0 = bf16 logits, 1 = fp32 logits
extern "C" int b200_moe_route(const void* logits, int dtype, int ld, int T, int E, int top_k, int sigmoid,
                              int renorm, float scaling, const float* bias, int n_group, int topk_group,
                              int* ids_out, float* w_out, cudaStream_t stream) {
  if (T == 0) return 0;
  if (E > ROUTE_MAX_E || top_k > 32 || n_group > 32 || (n_group > 1 && E % n_group)) {
    b200_set_last_error("moe_route: E <= 512, top_k <= 32, n_group <= 32 required", __FILE__, __LINE__);
    return -1;
  }
  const int blocks = (T + ROUTE_WARPS - 1) / ROUTE_WARPS;
  if (dtype == 0)
    moe_route_kernel<__nv_bfloat16><<<blocks, ROUTE_WARPS * 32, 0, stream>>>(
        (const __nv_bfloat16*)logits, ld, T, E, top_k, sigmoid, renorm, scaling, bias, n_group, topk_group,
        ids_out, w_out);
  else
    moe_route_kernel<float><<<blocks, ROUTE_WARPS * 32, 0, stream>>>(
        (const float*)logits, ld, T, E, top_k, sigmoid, renorm, scaling, bias, n_group, topk_group, ids_out,
        w_out);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_moe_permute(const void* x, const int* ids, int T, int top_k, int H, int e_lo, int E_local,
                                int* group_off, int* row_src, int* inv_pos, void* x_perm,
                                cudaStream_t stream) {
  if (T == 0) return 0;
  if (H % 8 || E_local > 8191) {
    b200_set_last_error("moe_permute: H % 8 == 0 required", __FILE__, __LINE__);
    return -1;
  }
  moe_permute_plan_kernel<<<1, 1024, (E_local + 1) * sizeof(int), stream>>>(ids, T * top_k, top_k, e_lo,
                                                                           E_local, group_off, row_src, inv_pos);
  int blocks = T * top_k;
  if (blocks > 148 * 16) blocks = 148 * 16;
  moe_gather_kernel<<<blocks, 128, 0, stream>>>((const __nv_bfloat16*)x, row_src, group_off, E_local,
                                                (__nv_bfloat16*)x_perm, H, T);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_moe_unpermute(const void* y, const int* inv_pos, const float* w, void* out, int T, int H,
                                  int top_k, int rows_cap, cudaStream_t stream) {
  if (T == 0) return 0;
  moe_unpermute_kernel<<<T, 128, 0, stream>>>((const __nv_bfloat16*)y, inv_pos, w, (__nv_bfloat16*)out, H,
                                              top_k, rows_cap);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}
