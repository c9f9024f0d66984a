// Consumer side of the "push" tensor-parallel plane: the row-parallel GEMM of every rank pushed its
// bf16 partial [T, N] into every rank's receive region (one slab per source rank) and raised one
// flag per (source rank, output tile).  The kernel here waits for the flags of a token's tiles, sums
// the slabs from local memory and, in the same pass, adds the residual stream and applies RMSNorm,
// so a decode-step all-reduce costs one NVLink store hop and no kernel of its own.
//
// Replaces the reference's all-reduce after every RowParallelLinear followed by the fused
// add + RMSNorm op (reference: src/vllm_torchtpu/layers/adapter/linear.py:25-66, ir_ops.py:63-88).
#include "common.cuh"

namespace b200 {

constexpr int RP_THREADS = 256;
constexpr int RP_MAX_VPT = 8;          // 16-byte vectors per thread: N <= 256 * 8 * 8 = 16384

struct ReducePushedParams {
  const uint8_t* recv;                 // this rank's receive region: slab of source r at r * src_stride
  unsigned long long src_stride;
  const int* flags;                    // int[world][max_tiles], raised to the producer's epoch
  const int* epoch_ptr;                // epoch of the last completed fused launch on this rank
  __nv_bfloat16* residual;             // in/out [T, N] or null
  const __nv_bfloat16* weight;         // RMSNorm weight [N] or null (then y = sum (+ residual))
  __nv_bfloat16* y;                    // [T, N]
  int* status;
  int T, N, world, max_tiles, bn, n_tiles, t_tiles;
  float eps;
  unsigned int spin_limit;
};

// index of output tile (n_tile, t_tile) in the GEMM's raster (groups of 16 weight tiles)
__device__ __forceinline__ int raster_tile(int n_tile, int t_tile, int n_tiles, int t_tiles) {
  const int g = n_tile / 16, first_n = g * 16;
  const int gsize = min(16, n_tiles - first_n);
  return g * 16 * t_tiles + t_tile * gsize + (n_tile - first_n);
}

__global__ void __launch_bounds__(RP_THREADS)
reduce_pushed_kernel(const ReducePushedParams p) {
  pdl_launch_dependents();             // the next GEMM may start prefetching its weights
  pdl_wait();                          // the producer GEMM (and its epoch bump) is complete from here on
  __shared__ float red[32];
  __shared__ int s_ok;
  const int t = blockIdx.x;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  const int epoch = *reinterpret_cast<const volatile int*>(p.epoch_ptr);
  const int t_tile = t / p.bn;
  for (int i = threadIdx.x; i < p.world * p.n_tiles; i += blockDim.x) {
    const int src = i / p.n_tiles, n_tile = i - src * p.n_tiles;
    const int tile = raster_tile(n_tile, t_tile, p.n_tiles, p.t_tiles);
    if (!wait_flag_ge(p.flags + (size_t)src * p.max_tiles + tile, epoch, p.status, p.spin_limit)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;                   // status word is set; the row is left untouched
  const int nvec = p.N >> 3;
  const size_t row_off = (size_t)t * p.N;
  float vals[RP_MAX_VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < RP_MAX_VPT; ++u) {
    const int v = threadIdx.x + u * RP_THREADS;
    if (v >= nvec) break;
    uint4 raw[8];
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < p.world)
        raw[r] = ld_relaxed_sys_v4(p.recv + (size_t)r * p.src_stride + (row_off + (size_t)v * 8) * 2);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      if (r < p.world) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[r]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
    }
    // same roundings as an all-reduce of bf16 tensors followed by the bf16 residual add
    bf16x8 a;
#pragma unroll
    for (int j = 0; j < 4; ++j) a.v[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    if (p.residual != nullptr) {
      const bf16x8 r = *reinterpret_cast<const bf16x8*>(p.residual + row_off + v * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fa = __bfloat1622float2(a.v[j]), fr = __bfloat1622float2(r.v[j]);
        a.v[j] = __floats2bfloat162_rn(fa.x + fr.x, fa.y + fr.y);
      }
      *reinterpret_cast<bf16x8*>(p.residual + row_off + v * 8) = a;
    }
    if (p.weight == nullptr) {
      *reinterpret_cast<bf16x8*>(p.y + row_off + v * 8) = a;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(a.v[j]);
        vals[u][2 * j] = f.x;
        vals[u][2 * j + 1] = f.y;
        ss += f.x * f.x + f.y * f.y;
      }
    }
  }
  if (p.weight == nullptr) return;
  const float tot = block_sum(ss, red);
  const float inv = rsqrtf(tot / (float)p.N + p.eps);
#pragma unroll
  for (int u = 0; u < RP_MAX_VPT; ++u) {
    const int v = threadIdx.x + u * RP_THREADS;
    if (v >= nvec) break;
    const bf16x8 ww = *reinterpret_cast<const bf16x8*>(p.weight + v * 8);
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = __bfloat1622float2(ww.v[j]);
      o.v[j] = __floats2bfloat162_rn(vals[u][2 * j] * inv * g.x, vals[u][2 * j + 1] * inv * g.y);
    }
    *reinterpret_cast<bf16x8*>(p.y + row_off + v * 8) = o;
  }
}

}  // namespace b200

using namespace b200;

// Sums what the ranks pushed for a [T, N] row-parallel output (GEMM launched with mode 3 and the
// same T, N) and finishes it: y = RMSNorm(sum + residual) * weight with residual updated in place
// (weight and residual given), or y = sum (+ residual) when weight is null.
// recv: this rank's heap base + the receive-region offset of that GEMM launch; flags: heap base +
// tile-flag offset; ctrl: the control words the GEMM launch used.
extern "C" int b200_reduce_pushed_rms_norm(const void* recv, unsigned long long src_stride, const int* flags,
                                           int max_tiles, const int* ctrl, void* residual, const void* weight,
                                           void* y, int T, int N, int world, float eps, int* status,
                                           unsigned int spin_limit, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (N % 8 || N > RP_THREADS * RP_MAX_VPT * 8 || world < 2 || world > 8) {
    b200_set_last_error("reduce_pushed: N % 8 == 0, N <= 16384 and 2 <= world <= 8 required", __FILE__, __LINE__);
    return -1;
  }
  ReducePushedParams p;
  p.recv = (const uint8_t*)recv;
  p.src_stride = src_stride;
  p.flags = flags;
  p.epoch_ptr = ctrl;
  p.residual = (__nv_bfloat16*)residual;
  p.weight = (const __nv_bfloat16*)weight;
  p.y = (__nv_bfloat16*)y;
  p.status = status;
  p.T = T; p.N = N; p.world = world; p.max_tiles = max_tiles;
  p.bn = T <= 32 ? 32 : (T <= 64 ? 64 : (T <= 128 ? 128 : 256));     // the GEMM's token tile for this T
  p.n_tiles = (N + 127) / 128;
  p.t_tiles = (T + p.bn - 1) / p.bn;
  p.eps = eps;
  p.spin_limit = spin_limit;
  B200_CUDA_CHECK(launch_pdl(reduce_pushed_kernel, dim3(T), dim3(RP_THREADS), 0, stream, p));
  return 0;
}
