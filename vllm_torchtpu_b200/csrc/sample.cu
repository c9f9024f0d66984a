// Sampling kernels: greedy argmax, and temperature / top-k / top-p / Gumbel-max
// sampling without a sort.
//
// Top-k and top-p thresholds are found by 32-step bisection over the
// order-preserving integer image of the fp32 logits, the same sort-free idea as
// the reference's sampler (reference: src/vllm_torchtpu/layers/adapter/sample/top_k_top_p.py:33-366);
// the draw itself is argmax(logit/T + Gumbel(u)) over the kept set
// (reference: src/vllm_torchtpu/runner/tpu_runner.py:9240-9274).  Uniform noise is
// either supplied (tests) or generated in the kernel with Philox keyed by
// (seed, step, row, column), so every tensor-parallel rank draws the same token.
// One CTA per row; each pass re-reads the row (bf16, L2 resident).
#include <cstdlib>

#include "common.cuh"

namespace b200 {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ uint32_t f2key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key2f(uint32_t k) {
  uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

// Philox-4x32-10
__device__ __forceinline__ uint4 philox(uint4 ctr, uint2 key) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}
__device__ __forceinline__ float uniform_at(unsigned long long seed, unsigned long long step, int row,
                                            int col) {
  const uint4 r = philox(make_uint4((uint32_t)col, (uint32_t)row, (uint32_t)step, (uint32_t)(step >> 32)),
                         make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
  return (float)(r.x >> 8) * (1.0f / 16777216.0f) + (0.5f / 16777216.0f);     // (0, 1)
}

template <typename T>
__device__ __forceinline__ float load_logit(const T* p, int i);
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* p, int i) {
  return __bfloat162float(p[i]);
}
template <>
__device__ __forceinline__ float load_logit<float>(const float* p, int i) {
  return p[i];
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ ArgMax block_argmax(ArgMax a, ArgMax* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b{__shfl_xor_sync(0xffffffffu, a.v, o), __shfl_xor_sync(0xffffffffu, a.i, o)};
    a = better(a, b);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = a;
  __syncthreads();
  ArgMax t = lane < nw ? red[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
    t = better(t, b);
  }
  return t;
}
__device__ __forceinline__ float block_sum_f(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ int block_sum_i(int v, int* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  int t = lane < nw ? red[lane] : 0;
  return warp_sum(t);
}

template <typename T>
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const T* __restrict__ logits, int ld, int V, int* __restrict__ out) {
  __shared__ ArgMax red[32];
  const T* row = logits + (size_t)blockIdx.x * ld;
  ArgMax a{-INFINITY, 0x7fffffff};
  int head = 0;                                  // elements before the 16-byte aligned body
  if (sizeof(T) == 2) {
    // bf16 rows: 16-byte loads over the aligned body (a thread's indices still grow, so `>` keeps the
    // smallest index among equal values), scalar loads for the ragged ends
    const uintptr_t addr = reinterpret_cast<uintptr_t>(row);
    head = min(V, (int)(((16 - (addr & 15)) & 15) >> 1));
    const int nvec = (V - head) >> 3;
    const uint4* body = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(row) + head);
    for (int q = threadIdx.x; q < nvec; q += blockDim.x) {
      const uint4 w = body[q];
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h2[j]);
        const int i = head + q * 8 + 2 * j;
        if (f.x > a.v) a = ArgMax{f.x, i};
        if (f.y > a.v) a = ArgMax{f.y, i + 1};
      }
    }
    for (int i = threadIdx.x; i < head; i += blockDim.x) {
      const float v = load_logit(row, i);
      if (v > a.v || (v == a.v && i < a.i)) a = ArgMax{v, i};
    }
    for (int i = head + nvec * 8 + threadIdx.x; i < V; i += blockDim.x) {
      const float v = load_logit(row, i);
      if (v > a.v) a = ArgMax{v, i};
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = load_logit(row, i);
      if (v > a.v) a = ArgMax{v, i};
    }
  }
  a = block_argmax(a, red);
  if (threadIdx.x == 0) out[blockIdx.x] = a.i < V ? a.i : 0;
}

// Full sampler.  temperature <= 1e-5 -> greedy.  top_k <= 0 and top_p >= 1 disable the filters.
template <typename T>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const T* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ uniform, unsigned long long seed, unsigned long long step,
              const long long* __restrict__ step_ptr, int* __restrict__ out) {
  if (step_ptr != nullptr) step += (unsigned long long)(*step_ptr);   // graph replays read a fresh offset
  __shared__ ArgMax red[32];
  __shared__ float redf[32];
  __shared__ int redi[32];
  const int r = blockIdx.x;
  const T* row = logits + (size_t)r * ld;
  const float temp = temperature[r];
  if (temp <= 1e-5f) {
    ArgMax a{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = load_logit(row, i);
      if (v > a.v) a = ArgMax{v, i};
    }
    a = block_argmax(a, red);
    if (threadIdx.x == 0) out[r] = a.i < V ? a.i : 0;
    return;
  }
  const float inv_t = 1.f / temp;
  int k = top_k[r];
  if (k <= 0 || k > V) k = V;
  const float pp = top_p[r];

  // ---- top-k threshold: largest key with count(x >= key) >= k
  uint32_t kth = 0;                                     // keep everything
  if (k < V) {
    uint32_t lo = 0, hi = 0xffffffffu;                  // invariant: count(>= lo) >= k
    for (int it = 0; it < 32 && lo < hi; ++it) {
      const uint32_t mid = lo + ((hi - lo) >> 1) + 1;   // upper mid so the loop terminates
      int c = 0;
      for (int i = threadIdx.x; i < V; i += blockDim.x) c += f2key(load_logit(row, i) * inv_t) >= mid;
      c = block_sum_i(c, redi);
      if (c >= k) lo = mid; else hi = mid - 1;
    }
    kth = lo;
  }
  // ---- softmax statistics over the kept set
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float x = load_logit(row, i) * inv_t;
    if (f2key(x) >= kth) mx = fmaxf(mx, x);
  }
  {
    ArgMax a = block_argmax(ArgMax{mx, 0}, red);
    mx = a.v;
  }
  uint32_t thr = kth;
  if (pp < 1.f) {
    float z = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float x = load_logit(row, i) * inv_t;
      if (f2key(x) >= kth) z += __expf(x - mx);
    }
    z = block_sum_f(z, redf);
    // largest key such that mass(x >= key) >= top_p * Z  (ties at the threshold are all kept)
    uint32_t lo = kth, hi = f2key(mx);
    const float want = pp * z;
    for (int it = 0; it < 32 && lo < hi; ++it) {
      const uint32_t mid = lo + ((hi - lo) >> 1) + 1;
      float ms = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float x = load_logit(row, i) * inv_t;
        if (f2key(x) >= mid) ms += __expf(x - mx);
      }
      ms = block_sum_f(ms, redf);
      if (ms >= want) lo = mid; else hi = mid - 1;
    }
    thr = lo;
  }
  // ---- Gumbel-max over the kept set
  ArgMax a{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float x = load_logit(row, i) * inv_t;
    if (f2key(x) >= thr) {
      float u = uniform != nullptr ? uniform[(size_t)r * V + i] : uniform_at(seed, step, r, i);
      u = fminf(fmaxf(u, 1e-20f), 1.f - 1e-7f);
      const float g = -__logf(-__logf(u));
      const float v = x + g;
      if (v > a.v) a = ArgMax{v, i};
    }
  }
  a = block_argmax(a, red);
  if (threadIdx.x == 0) out[r] = a.i < V ? a.i : 0;
}

// ---- the same sampler with the row held in registers by a cluster of four CTAs ------------------------
// The single-CTA kernel above re-reads its row from L2 in every bisection pass (about 70 passes over 128 K
// logits: 1.2 ms for 64 rows).  Here a cluster of SAMPLE_CL CTAs owns a row: CTA c keeps elements
// [c * seg, (c + 1) * seg) as packed bf16 logits in registers (64 per thread), so a pass is 64 compares per
// thread, a block reduction and one exchange of a few words over distributed shared memory.  The threshold
// searches are 4-ary (three thresholds per pass), which halves the number of cluster barriers.  Same
// thresholds, same Philox noise and same Gumbel-max draw as the single-CTA kernel.
constexpr int SAMPLE_CL = 4;
constexpr int SAMPLE_CT = 512;                    // threads per CTA of the cluster kernel
constexpr int SAMPLE_NPT = 64;                    // elements per thread: V <= 4 * 512 * 64 = 131072

struct ClusterXchg {
  float f[2][4];                                  // [parity][word]
  int i[2][4];
};

__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ int ld_dsmem_s32(uint32_t addr) {
  int v;
  asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}

// Every thread of every CTA of the cluster passes up to three per-thread values; all threads get the three
// cluster-wide sums.  `par` alternates between calls, so a slot is rewritten only after a later barrier.
// three block sums with one pair of barriers; red holds 3 x 32 words; every thread of warp 0 gets the sums
__device__ __forceinline__ void block_sum3_f(float& a, float& b, float& c, float* red) {
  a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) { red[warp] = a; red[32 + warp] = b; red[64 + warp] = c; }
  __syncthreads();
  if (warp == 0) {
    a = warp_sum(lane < nw ? red[lane] : 0.f);
    b = warp_sum(lane < nw ? red[32 + lane] : 0.f);
    c = warp_sum(lane < nw ? red[64 + lane] : 0.f);
  }
}
__device__ __forceinline__ void block_sum3_i(int& a, int& b, int& c, int* red) {
  a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) { red[warp] = a; red[32 + warp] = b; red[64 + warp] = c; }
  __syncthreads();
  if (warp == 0) {
    a = warp_sum(lane < nw ? red[lane] : 0);
    b = warp_sum(lane < nw ? red[32 + lane] : 0);
    c = warp_sum(lane < nw ? red[64 + lane] : 0);
  }
}

__device__ __forceinline__ void cluster_sum3_f(float& a, float& b, float& c, ClusterXchg* x, float* red, int& par) {
  block_sum3_f(a, b, c, red);
  if (threadIdx.x == 0) { x->f[par][0] = a; x->f[par][1] = b; x->f[par][2] = c; }
  cluster_arrive_release();
  cluster_wait_acquire();
  const uint32_t base = smem_u32(&x->f[par][0]);
  float sa = 0.f, sb = 0.f, sc = 0.f;
#pragma unroll
  for (int r = 0; r < SAMPLE_CL; ++r) {
    const uint32_t ra = mapa_shared(base, r);
    sa += ld_dsmem_f32(ra);
    sb += ld_dsmem_f32(ra + 4);
    sc += ld_dsmem_f32(ra + 8);
  }
  a = sa; b = sb; c = sc;
  par ^= 1;
}
__device__ __forceinline__ void cluster_sum3_i(int& a, int& b, int& c, ClusterXchg* x, int* red, int& par) {
  block_sum3_i(a, b, c, red);
  if (threadIdx.x == 0) { x->i[par][0] = a; x->i[par][1] = b; x->i[par][2] = c; }
  cluster_arrive_release();
  cluster_wait_acquire();
  const uint32_t base = smem_u32(&x->i[par][0]);
  int sa = 0, sb = 0, sc = 0;
#pragma unroll
  for (int r = 0; r < SAMPLE_CL; ++r) {
    const uint32_t ra = mapa_shared(base, r);
    sa += ld_dsmem_s32(ra);
    sb += ld_dsmem_s32(ra + 4);
    sc += ld_dsmem_s32(ra + 8);
  }
  a = sa; b = sb; c = sc;
  par ^= 1;
}
// cluster-wide arg-max of (value, index): smaller index wins ties
__device__ __forceinline__ ArgMax cluster_argmax(ArgMax a, ClusterXchg* x, ArgMax* red, int& par) {
  a = block_argmax(a, red);
  if (threadIdx.x == 0) { x->f[par][3] = a.v; x->i[par][3] = a.i; }
  cluster_arrive_release();
  cluster_wait_acquire();
  const uint32_t bf = smem_u32(&x->f[par][3]), bi = smem_u32(&x->i[par][3]);
  ArgMax best{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int r = 0; r < SAMPLE_CL; ++r) {
    const ArgMax o{ld_dsmem_f32(mapa_shared(bf, r)), ld_dsmem_s32(mapa_shared(bi, r))};
    best = better(best, o);
  }
  par ^= 1;
  return best;
}

// bf16 logits only (fp32 rows would not fit the register budget): a thread keeps 32 packed pairs, element j of
// thread t is row index cr * seg + ((j >> 1) * 512 + t) * 2 + (j & 1).
__global__ void __launch_bounds__(SAMPLE_CT, 1)
sample_cluster_kernel(const __nv_bfloat16* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
                      const int* __restrict__ top_k, const float* __restrict__ top_p,
                      const float* __restrict__ uniform, unsigned long long seed, unsigned long long step,
                      const long long* __restrict__ step_ptr, int* __restrict__ out) {
  if (step_ptr != nullptr) step += (unsigned long long)(*step_ptr);
  __shared__ ArgMax red[32];
  __shared__ float redf[96];
  __shared__ int redi[96];
  __shared__ ClusterXchg xchg;
  const int r = blockIdx.x / SAMPLE_CL;
  const int cr = (int)cluster_ctarank();
  const __nv_bfloat16* row = logits + (size_t)r * ld;
  const float temp = temperature[r];
  const bool greedy = temp <= 1e-5f;
  const float inv_t = greedy ? 1.f : 1.f / temp;
  // elements per CTA: a multiple of 2 * 512 so that pairs never straddle CTAs
  const int seg = ((V + SAMPLE_CL - 1) / SAMPLE_CL + 2 * SAMPLE_CT - 1) / (2 * SAMPLE_CT) * (2 * SAMPLE_CT);
  const int base = cr * seg + 2 * (int)threadIdx.x;
  int par = 0;
  // order-preserving 32-bit keys of the scaled logits; padding holds the key of -inf (KEY_NEG)
  uint32_t key[SAMPLE_NPT];
  const uint32_t KEY_NEG = f2key(-INFINITY);
  const bool pair_ok = ((reinterpret_cast<uintptr_t>(row) & 3) == 0);
#pragma unroll
  for (int jj = 0; jj < SAMPLE_NPT / 2; ++jj) {
    const int i = base + jj * 2 * SAMPLE_CT;
    float x0 = -INFINITY, x1 = -INFINITY;
    if (jj * 2 * SAMPLE_CT < seg && i < V) {
      if (pair_ok && i + 1 < V) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + i));
        x0 = f.x; x1 = f.y;
      } else {
        x0 = __bfloat162float(row[i]);
        if (i + 1 < V) x1 = __bfloat162float(row[i + 1]);
      }
    }
    key[2 * jj] = f2key(x0 * inv_t);
    key[2 * jj + 1] = f2key(x1 * inv_t);
  }
  auto idx = [&](int j) -> int { return base + (j >> 1) * 2 * SAMPLE_CT + (j & 1); };
  // every CTA of the cluster must be resident before the first remote read
  cluster_arrive_release();
  cluster_wait_acquire();
  if (greedy) {
    ArgMax a{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int j = 0; j < SAMPLE_NPT; ++j) {
      const float x = key2f(key[j]);
      if (x > a.v) a = ArgMax{x, idx(j)};
    }
    a = cluster_argmax(a, &xchg, red, par);
    if (cr == 0 && threadIdx.x == 0) out[r] = a.i < V ? a.i : 0;
    cluster_arrive_release();                   // nobody leaves while a peer may still read its slots
    cluster_wait_acquire();
    return;
  }
  int k = top_k[r];
  if (k <= 0 || k > V) k = V;
  const float pp = top_p[r];
  auto sat = [](unsigned long long t) -> uint32_t { return t > 0xffffffffull ? 0xffffffffu : (uint32_t)t; };

  // ---- top-k threshold: largest key with count(x >= key) >= k.  Padding (-inf) is never counted: every
  // threshold tried is above KEY_NEG once lo has passed it, and below that the real elements decide.
  uint32_t kth = 0;
  if (k < V) {
    unsigned long long lo = KEY_NEG, hi = 0xffffffffull;   // count(>= KEY_NEG + 1) is the number of finite logits
    for (int it = 0; it < 40 && lo < hi; ++it) {
      const unsigned long long q = (hi - lo) >> 2, stp = q > 0 ? q : 1;
      const unsigned long long t1 = lo + stp, t2 = t1 + stp, t3 = t2 + stp;
      const uint32_t u1 = sat(t1), u2 = sat(t2), u3 = sat(t3);
      int c1 = 0, c2 = 0, c3 = 0;
#pragma unroll
      for (int j = 0; j < SAMPLE_NPT; ++j) {
        c1 += key[j] >= u1; c2 += key[j] >= u2; c3 += key[j] >= u3;
      }
      cluster_sum3_i(c1, c2, c3, &xchg, redi, par);
      if (t3 <= hi && c3 >= k) lo = t3;
      else if (t2 <= hi && c2 >= k) { lo = t2; hi = min(hi, t3 - 1); }
      else if (t1 <= hi && c1 >= k) { lo = t1; hi = min(hi, t2 - 1); }
      else hi = min(hi, t1 - 1);
    }
    kth = (uint32_t)lo;
  }
  if (kth <= KEY_NEG) kth = KEY_NEG + 1;          // the kept set never contains padding
  // ---- softmax statistics over the kept set
  ArgMax m{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int j = 0; j < SAMPLE_NPT; ++j) {
    if (key[j] >= kth) {
      const float x = key2f(key[j]);
      if (x > m.v) m = ArgMax{x, idx(j)};
    }
  }
  const float mx = cluster_argmax(m, &xchg, red, par).v;
  uint32_t thr = kth;
  if (pp < 1.f) {
    float z = 0.f, z2 = 0.f, z3 = 0.f;
#pragma unroll
    for (int j = 0; j < SAMPLE_NPT; ++j)
      if (key[j] >= kth) z += __expf(key2f(key[j]) - mx);
    cluster_sum3_f(z, z2, z3, &xchg, redf, par);
    // largest key such that mass(x >= key) >= top_p * Z (ties at the threshold are all kept)
    unsigned long long lo = kth, hi = f2key(mx);
    const float want = pp * z;
    for (int it = 0; it < 40 && lo < hi; ++it) {
      const unsigned long long q = (hi - lo) >> 2, stp = q > 0 ? q : 1;
      const unsigned long long t1 = lo + stp, t2 = t1 + stp, t3 = t2 + stp;
      const uint32_t u1 = sat(t1), u2 = sat(t2), u3 = sat(t3);
      float m1 = 0.f, m2 = 0.f, m3 = 0.f;
#pragma unroll
      for (int j = 0; j < SAMPLE_NPT; ++j) {
        if (key[j] >= u1) {
          const float e = __expf(key2f(key[j]) - mx);
          m1 += e;
          if (key[j] >= u2) m2 += e;
          if (key[j] >= u3) m3 += e;
        }
      }
      cluster_sum3_f(m1, m2, m3, &xchg, redf, par);
      if (t3 <= hi && m3 >= want) lo = t3;
      else if (t2 <= hi && m2 >= want) { lo = t2; hi = min(hi, t3 - 1); }
      else if (t1 <= hi && m1 >= want) { lo = t1; hi = min(hi, t2 - 1); }
      else hi = min(hi, t1 - 1);
    }
    thr = (uint32_t)lo;
  }
  // ---- Gumbel-max over the kept set
  ArgMax a{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int j = 0; j < SAMPLE_NPT; ++j) {
    const int i = idx(j);
    if (key[j] >= thr) {
      float u = uniform != nullptr ? uniform[(size_t)r * V + i] : uniform_at(seed, step, r, i);
      u = fminf(fmaxf(u, 1e-20f), 1.f - 1e-7f);
      const float v = key2f(key[j]) - __logf(-__logf(u));
      if (v > a.v || (v == a.v && i < a.i)) a = ArgMax{v, i};
    }
  }
  a = cluster_argmax(a, &xchg, red, par);
  if (cr == 0 && threadIdx.x == 0) out[r] = a.i < V ? a.i : 0;
  cluster_arrive_release();
  cluster_wait_acquire();
}

// logprob of chosen token + top-k logprobs (k <= 32) with fp32 logsumexp
template <typename T>
__global__ void __launch_bounds__(SAMPLE_THREADS)
logprobs_kernel(const T* __restrict__ logits, int ld, int V, const int* __restrict__ token_ids, int k,
                float* __restrict__ tok_lp, float* __restrict__ top_lp, int* __restrict__ top_id,
                int* __restrict__ rank) {
  __shared__ ArgMax red[32];
  __shared__ float redf[32];
  __shared__ int redi[32];
  const int r = blockIdx.x;
  const T* row = logits + (size_t)r * ld;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, load_logit(row, i));
  mx = block_argmax(ArgMax{mx, 0}, red).v;
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) z += __expf(load_logit(row, i) - mx);
  z = block_sum_f(z, redf);
  const float lse = mx + __logf(z);
  const int tok = token_ids[r];
  const float tv = load_logit(row, min(max(tok, 0), V - 1));
  int c = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) c += load_logit(row, i) > tv;
  c = block_sum_i(c, redi);
  if (threadIdx.x == 0) {
    tok_lp[r] = tv - lse;
    rank[r] = c + 1;
  }
  // top-k by repeated arg-max below the previous winner (k is small)
  float prev_v = INFINITY;
  int prev_i = -1;
  for (int j = 0; j < k; ++j) {
    ArgMax a{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = load_logit(row, i);
      const bool below = v < prev_v || (v == prev_v && i > prev_i);
      if (below && (v > a.v || (v == a.v && i < a.i))) a = ArgMax{v, i};
    }
    a = block_argmax(a, red);
    if (threadIdx.x == 0) {
      top_lp[(size_t)r * k + j] = a.v - lse;
      top_id[(size_t)r * k + j] = a.i < V ? a.i : 0;
    }
    prev_v = a.v;
    prev_i = a.i;
  }
}

__global__ void philox_uniform_kernel(float* out, int R, int V, unsigned long long seed,
                                      unsigned long long step) {
  const size_t n = (size_t)R * V;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = uniform_at(seed, step, (int)(i / V), (int)(i % V));
}

// ------------------------------------------------------------------ speculative decoding
// Acceptance of drafts from a deterministic proposer (n-gram, greedy draft head).  The target's own sampler
// has drawn one token per verified row; a draft is kept while it equals that token, which is rejection
// sampling against a one-hot draft distribution (accept with p(x), else the draw from p is the replacement).
// Request r owns rows [off_r, off_r + k_r] of `target` (off_r = sum of k_i + 1 before it) and its drafts are
// the step's input tokens behind the last known one: input_ids[qsl[r+1] - k_r + i].
// out [R, kmax + 1] (unused entries -1), count [R].  One thread per request.
__global__ void spec_accept_kernel(const int* __restrict__ target, const int* __restrict__ input_ids,
                                   const int* __restrict__ qsl, const int* __restrict__ spec_k, int R, int kmax,
                                   int* __restrict__ out, int* __restrict__ count) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  int off = 0;
  for (int i = 0; i < r; ++i) off += spec_k[i] + 1;
  const int k = min(spec_k[r], kmax);
  const int* draft = input_ids + qsl[r + 1] - k;
  int n = 0;
  bool all = true;
  for (int i = 0; i < k; ++i) {
    const int t = target[off + i];
    out[r * (kmax + 1) + n++] = t;
    if (draft[i] != t) { all = false; break; }
  }
  if (all) out[r * (kmax + 1) + n++] = target[off + k];
  count[r] = n;
  for (int i = n; i <= kmax; ++i) out[r * (kmax + 1) + i] = -1;
}

__device__ __forceinline__ float block_max_f(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : -INFINITY;
  return warp_max(t);
}

// Rejection sampling against a drafter that SAMPLED its tokens from q (draft_probs [R, kmax, V], or null for
// a one-hot q).  Row i of request r: p = softmax(logits / T_r); draft x is kept when u_i * q(x) <= p(x);
// at the first rejection the replacement is drawn from normalise(max(p - q, 0)) by inverse CDF with
// u'_i, and when every draft is kept a bonus token is drawn from the last row.  T_r == 0: keep while
// x == argmax, replacement / bonus = argmax.  One CTA per request; every pass re-reads the row (L2 resident).
template <typename T>
__global__ void rejection_sample_kernel(const T* __restrict__ logits, int ld, int V, const int* __restrict__ drafts,
                                        const float* __restrict__ draft_probs, const int* __restrict__ spec_k,
                                        const float* __restrict__ temperature, const float* __restrict__ uniform,
                                        const float* __restrict__ resample_uniform, int kmax,
                                        int* __restrict__ out, int* __restrict__ count) {
  __shared__ float red[32];
  __shared__ float seg[SAMPLE_THREADS];
  __shared__ int s_pick;
  const int r = blockIdx.x;
  int off = 0;
  for (int i = 0; i < r; ++i) off += spec_k[i] + 1;
  const int k = min(spec_k[r], kmax);
  const float temp = temperature[r];
  const int per = (V + blockDim.x - 1) / blockDim.x;
  const int v0 = threadIdx.x * per, v1 = min(V, v0 + per);
  int n = 0;
  for (int i = 0; i <= k; ++i) {
    const T* row = logits + (size_t)(off + i) * ld;
    const bool bonus = i == k;
    const int x = bonus ? -1 : drafts[r * kmax + i];
    const float* q = (draft_probs != nullptr && !bonus) ? draft_probs + ((size_t)r * kmax + i) * V : nullptr;
    // row maximum (and its first index, for temperature 0)
    float m = -INFINITY;
    int mi = 0x7fffffff;
    for (int v = v0; v < v1; ++v) {
      const float l = load_logit(row, v);
      if (l > m) { m = l; mi = v; }
    }
    const float gmax = block_max_f(m, red);
    if (temp <= 0.f) {
      // greedy: smallest index that attains the maximum
      __syncthreads();
      if (threadIdx.x == 0) s_pick = 0x7fffffff;
      __syncthreads();
      if (m == gmax) atomicMin(&s_pick, mi);
      __syncthreads();
      const int am = s_pick;
      if (threadIdx.x == 0) out[r * (kmax + 1) + n] = am;
      ++n;
      if (bonus || x != am) break;
      continue;
    }
    const float inv_t = 1.f / temp;
    float z = 0.f;
    for (int v = v0; v < v1; ++v) z += __expf((load_logit(row, v) - gmax) * inv_t);
    const float Z = block_sum_f(z, red);
    bool accept = false;
    if (!bonus) {
      const float px = __expf((load_logit(row, x) - gmax) * inv_t) / Z;
      const float qx = q != nullptr ? q[x] : 1.f;
      accept = qx > 0.f && uniform[r * kmax + i] * qx <= px;
      if (accept) {
        if (threadIdx.x == 0) out[r * (kmax + 1) + n] = x;
        ++n;
        continue;
      }
    }
    // draw from the residual (or from p itself for the bonus token) by inverse CDF
    float mine = 0.f;
    for (int v = v0; v < v1; ++v) {
      const float pv = __expf((load_logit(row, v) - gmax) * inv_t) / Z;
      const float rv = bonus ? pv : fmaxf(pv - (q != nullptr ? q[v] : (v == x ? 1.f : 0.f)), 0.f);
      mine += rv;
    }
    __syncthreads();
    seg[threadIdx.x] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
      float total = 0.f;
      for (int t = 0; t < (int)blockDim.x; ++t) total += seg[t];
      const float want = resample_uniform[r * (kmax + 1) + i] * total;
      float c = 0.f;
      int pick = -1, last_nonzero = -1;
      for (int t = 0; t < (int)blockDim.x && pick < 0; ++t) {
        if (seg[t] > 0.f) last_nonzero = t;
        if (c + seg[t] >= want && seg[t] > 0.f) {
          // walk this thread's segment
          const int a = t * per, b = min(V, a + per);
          for (int v = a; v < b; ++v) {
            const float pv = __expf((load_logit(row, v) - gmax) * inv_t) / Z;
            const float rv = bonus ? pv : fmaxf(pv - (q != nullptr ? q[v] : (v == x ? 1.f : 0.f)), 0.f);
            if (rv > 0.f) {
              pick = v;
              c += rv;
              if (c >= want) break;
            }
          }
        } else {
          c += seg[t];
        }
      }
      if (pick < 0) {
        // an all-zero residual (p == q): fall back to the row's most likely token
        pick = last_nonzero >= 0 ? min(V - 1, last_nonzero * per) : 0;
        float best = -INFINITY;
        for (int v = 0; v < V; ++v) {
          const float l = load_logit(row, v);
          if (l > best) { best = l; pick = v; }
        }
      }
      out[r * (kmax + 1) + n] = pick;
    }
    ++n;
    break;
  }
  if (threadIdx.x == 0) {
    count[r] = n;
    for (int i = n; i <= kmax; ++i) out[r * (kmax + 1) + i] = -1;
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_spec_accept(const int* target, const int* input_ids, const int* qsl, const int* spec_k, int R,
                                int kmax, int* out, int* count, cudaStream_t stream) {
  if (R == 0) return 0;
  spec_accept_kernel<<<(R + 127) / 128, 128, 0, stream>>>(target, input_ids, qsl, spec_k, R, kmax, out, count);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_rejection_sample(const void* logits, int dtype, int R, int V, int ld, const int* drafts,
                                     const float* draft_probs, const int* spec_k, const float* temperature,
                                     const float* uniform, const float* resample_uniform, int kmax, int* out,
                                     int* count, cudaStream_t stream) {
  if (R == 0) return 0;
  if (dtype == 0)
    rejection_sample_kernel<__nv_bfloat16><<<R, SAMPLE_THREADS, 0, stream>>>(
        (const __nv_bfloat16*)logits, ld, V, drafts, draft_probs, spec_k, temperature, uniform, resample_uniform,
        kmax, out, count);
  else
    rejection_sample_kernel<float><<<R, SAMPLE_THREADS, 0, stream>>>(
        (const float*)logits, ld, V, drafts, draft_probs, spec_k, temperature, uniform, resample_uniform, kmax,
        out, count);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// B200_SAMPLE_CLUSTER=0 keeps the single-CTA sampler (read once)
static bool sample_cluster_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("B200_SAMPLE_CLUSTER");
    on = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

// dtype: 0 = bf16 logits, 1 = fp32 logits
extern "C" int b200_argmax(const void* logits, int dtype, int R, int V, int ld, int* out, cudaStream_t stream) {
  if (R == 0) return 0;
  if (dtype == 0)
    argmax_kernel<__nv_bfloat16><<<R, SAMPLE_THREADS, 0, stream>>>((const __nv_bfloat16*)logits, ld, V, out);
  else
    argmax_kernel<float><<<R, SAMPLE_THREADS, 0, stream>>>((const float*)logits, ld, V, out);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_sample(const void* logits, int dtype, int R, int V, int ld, const float* temperature,
                           const int* top_k, const float* top_p, const float* uniform,
                           unsigned long long seed, unsigned long long step, const long long* step_ptr,
                           int* out, cudaStream_t stream) {
  if (R == 0) return 0;
  if (dtype == 0 && V <= SAMPLE_CL * SAMPLE_CT * SAMPLE_NPT && V >= SAMPLE_CL * SAMPLE_CT * 2 &&
      sample_cluster_enabled()) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(R * SAMPLE_CL);
    cfg.blockDim = dim3(SAMPLE_CT);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = SAMPLE_CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, sample_cluster_kernel, (const __nv_bfloat16*)logits, ld, V, temperature,
                                       top_k, top_p, uniform, seed, step, step_ptr, out));
    return 0;
  }
  if (dtype == 0)
    sample_kernel<__nv_bfloat16><<<R, SAMPLE_THREADS, 0, stream>>>((const __nv_bfloat16*)logits, ld, V,
                                                                  temperature, top_k, top_p, uniform, seed,
                                                                  step, step_ptr, out);
  else
    sample_kernel<float><<<R, SAMPLE_THREADS, 0, stream>>>((const float*)logits, ld, V, temperature, top_k,
                                                          top_p, uniform, seed, step, step_ptr, out);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_logprobs(const void* logits, int dtype, int R, int V, int ld, const int* token_ids, int k,
                             float* tok_lp, float* top_lp, int* top_id, int* rank, cudaStream_t stream) {
  if (R == 0) return 0;
  if (dtype == 0)
    logprobs_kernel<__nv_bfloat16><<<R, SAMPLE_THREADS, 0, stream>>>((const __nv_bfloat16*)logits, ld, V,
                                                                    token_ids, k, tok_lp, top_lp, top_id, rank);
  else
    logprobs_kernel<float><<<R, SAMPLE_THREADS, 0, stream>>>((const float*)logits, ld, V, token_ids, k, tok_lp,
                                                            top_lp, top_id, rank);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_philox_uniform(float* out, int R, int V, unsigned long long seed, unsigned long long step,
                                   cudaStream_t stream) {
  if (R == 0) return 0;
  philox_uniform_kernel<<<148 * 4, 256, 0, stream>>>(out, R, V, seed, step);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}
