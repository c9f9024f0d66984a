// Block-scaled fp8 (e4m3) GEMM for many tokens: tokens are the 128-row UMMA operand, weight rows are N.
//
//   Y[t, n] = sum_kb  ( sum_{k in block kb} Xq[t,k] * Wq[n,k] ) * xs[t,kb] * ws[n/128, kb]
//
// The decode-oriented kernel (gemm_fp8_tcgen05.cu) keeps weight rows on the TMEM lanes, so the
// activation scale differs per accumulator column and every K block costs one shuffle per column in
// the epilogue warps; at prefill sizes that promotion, not the tensor core, sets the pace.  Here the
// roles are swapped: a TMEM lane is a token, a 256-column tile covers two weight scale rows, so the
// scale product of a K block is ONE scalar per thread and the promotion is a plain FMA per element:
//
//   warp 0        TMA producer: X tile [128 tokens x 128 B] + W tile [256 rows x 128 B] per stage
//   warp 1        tcgen05.mma kind::f8f6f4, M128 N256 K32 x 4 per K block, into one of two 256-column
//                 partial buffers (all 512 TMEM columns)
//   warps 4..11   promotion: warp w reads lanes 32*(w%4).. and columns 128*((w-4)/4).., acc += s * partial,
//                 then bias, bf16 and 16-byte row stores while the tensor core runs the next tile
//
// The promotion is a chain of TMEM loads per K block; to keep two 32-column loads in flight next to the
// 128 fp32 accumulators the two promotion warpgroups take registers from the first warpgroup (setmaxnreg),
// whose warps 2 and 3 only take part in the barriers.
//
// Work is a static persistent schedule over (token tile, weight tile) pairs in bands of 8 token tiles, so
// the CTAs that run together share X and W tiles in L2.  Grouped mode (per-expert row ranges from a
// device array) uses the same tiles inside each group.  Every wait is bounded and reports through the
// status word.
//
// Semantics of the reference's block-wise quantised matmul
// (reference: src/vllm_torchtpu/layers/adapter/linear_common.py:69-133).
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "gemm_tcgen05.h"

namespace b200 {
namespace f8r {

constexpr int BMT = 128;          // tokens per tile (UMMA M, TMEM lanes)
constexpr int BNW = 256;          // weight rows per tile (UMMA N, TMEM columns)
constexpr int BKB = 128;          // K bytes per stage row: one scale block
constexpr int STAGES = 4;
constexpr int A_BYTES = BMT * BKB;
constexpr int B_BYTES = BNW * BKB;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 384;
constexpr int REGS_LAUNCH = 168, REGS_LEAN = 40, REGS_PROMOTE = 232;   // 128*40 + 256*232 <= 384*168
constexpr int EPI_WARPS = 8;
constexpr int MAX_GROUPS = 1024;
constexpr int BAR_BYTES = 256;
constexpr int SMEM = STAGES * STAGE_BYTES + BAR_BYTES + (MAX_GROUPS + 1) * 4 + 1024;
constexpr int BAND = 8;           // token tiles per raster band

struct Params {
  __nv_bfloat16* Y;
  const __nv_bfloat16* bias;
  const float* w_scale;
  const float* x_scale;
  int* status;
  int T, N, K, ldy;
  int n_tiles, t_tiles, kb_total;
  int ws_ld, xs_ld, ws_rows;        // scale row strides; rows of the weight scale grid (per group)
  const int* group_off;             // grouped: int[num_groups + 1]
  int num_groups, w_rows_per_group;
  int skip_promote;                 // measurement aid: partials are released unread (output undefined)
};

struct Work {
  int w_row, ws_row, t_row, t_valid, n0;
};

__device__ __forceinline__ Work get_work(int w, const Params& p, const int* s_prefix) {
  Work k;
  if (p.group_off == nullptr) {
    const int per_band = BAND * p.n_tiles;
    const int band = w / per_band, r = w - band * per_band;
    const int bt = min(BAND, p.t_tiles - band * BAND);
    const int n_tile = r / bt, t_tile = band * BAND + (r - n_tile * bt);
    k.w_row = n_tile * BNW;
    k.ws_row = n_tile * (BNW / 128);
    k.n0 = n_tile * BNW;
    k.t_row = t_tile * BMT;
    k.t_valid = min(BMT, p.T - k.t_row);
  } else {
    const int tt = w / p.n_tiles, n_tile = w - tt * p.n_tiles;
    int lo = 0, hi = p.num_groups;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_prefix[mid] <= tt) lo = mid; else hi = mid;
    }
    const int e = lo, t_tile = tt - s_prefix[e];
    const int r0 = p.group_off[e], rows = p.group_off[e + 1] - r0;
    k.w_row = e * p.w_rows_per_group + n_tile * BNW;
    k.ws_row = e * p.ws_rows + n_tile * (BNW / 128);
    k.n0 = n_tile * BNW;
    k.t_row = r0 + t_tile * BMT;
    k.t_valid = min(BMT, rows - t_tile * BMT);
  }
  return k;
}

template <int N>
__device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_rows_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                     const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* pfull = bars + 2 * STAGES;
  uint64_t* pempty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_prefix = reinterpret_cast<int*>(smem + STAGES * STAGE_BYTES + BAR_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(&pfull[0], 1);
    mbar_init(&pfull[1], 1);
    mbar_init(&pempty[0], EPI_WARPS);
    mbar_init(&pempty[1], EPI_WARPS);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  pdl_launch_dependents();
  pdl_wait();
  if (p.group_off != nullptr) {
    for (int e = threadIdx.x; e < p.num_groups; e += blockDim.x)
      s_prefix[e + 1] = (p.group_off[e + 1] - p.group_off[e] + BMT - 1) / BMT;
    __syncthreads();
    if (threadIdx.x == 0) {
      s_prefix[0] = 0;
      for (int e = 0; e < p.num_groups; ++e) s_prefix[e + 1] += s_prefix[e];
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_work = p.group_off != nullptr ? s_prefix[p.num_groups] * p.n_tiles : p.n_tiles * p.t_tiles;
  const int kb_total = p.kb_total;

  if (warp < 4) {
  setmaxnreg_dec<REGS_LEAN>();
  if (warp == 0) {
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const Work k = get_work(w, p, s_prefix);
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* a = smem + s * STAGE_BYTES;
          mbar_expect_tx(&full[s], STAGE_BYTES);
          tma_load_2d(a, &tmX, &full[s], kb * BKB, k.t_row);
          tma_load_2d(a + A_BYTES, &tmW, &full[s], kb * BKB, k.w_row);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (*abort_flag)                        // copies in flight land before the ring is released
        for (int it = 0; it < 20000; ++it) __nanosleep(100);
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_e4m3(BMT, BNW);
      int s = 0;
      uint32_t ph = 0, pc = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        for (int kb = 0; kb < kb_total; ++kb, ++pc) {
          const int pb = pc & 1;
          if (!mbar_wait(&pempty[pb], ((pc >> 1) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) {
            ok = false;
            break;
          }
          if (!mbar_wait(&full[s], ph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t adesc = umma_desc_k_sw128(a_addr);
          const uint64_t bdesc = umma_desc_k_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int q = 0; q < 4; ++q)          // 4 x (K = 32 bytes) per 128-byte row; a fresh sum per block
            umma_f8(tmem_base + pb * BNW, adesc + 2 * q, bdesc + 2 * q, idesc, q > 0 ? 1u : 0u);
          umma_commit(&empty[s]);
          umma_commit(&pfull[pb]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  }
  } else {
    setmaxnreg_inc<REGS_PROMOTE>();
    const int q = warp & 3;                    // the TMEM lane quarter this warp may read
    const int half = (warp - 4) >> 2;          // which 128 columns of the tile
    const int row = q * 32 + lane;
    const int ws_rows_total = p.group_off != nullptr ? p.ws_rows * p.num_groups : p.ws_rows;
    uint32_t pc = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      const Work k = get_work(w, p, s_prefix);
      const int t = k.t_row + row;
      const bool live = row < k.t_valid;
      const float* xs_row = p.x_scale + (size_t)(live ? t : k.t_row) * p.xs_ld;
      const float* ws_row = p.w_scale + (size_t)min(k.ws_row + half, ws_rows_total - 1) * p.ws_ld;
      float acc[128];
#pragma unroll
      for (int c = 0; c < 128; ++c) acc[c] = 0.f;
      float s_next = __ldg(xs_row) * __ldg(ws_row);
      for (int kb = 0; kb < kb_total; ++kb, ++pc) {
        const int pb = pc & 1;
        const float s = s_next;
        if (kb + 1 < kb_total) s_next = __ldg(xs_row + kb + 1) * __ldg(ws_row + kb + 1);
        if (!mbar_wait(&pfull[pb], (pc >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + pb * BNW + half * 128 + ((uint32_t)(q * 32) << 16);
        if (!p.skip_promote) {
#pragma unroll
          for (int c0 = 0; c0 < 128; c0 += 64) {
            uint32_t r0[32], r1[32];           // two loads in flight
            tmem_ld_32x32(taddr + c0, r0);
            tmem_ld_32x32(taddr + c0 + 32, r1);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[c0 + j] = fmaf(__uint_as_float(r0[j]), s, acc[c0 + j]);
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[c0 + 32 + j] = fmaf(__uint_as_float(r1[j]), s, acc[c0 + 32 + j]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pempty[pb]);
      }
      if (!ok) break;
      if (live) {
        const int n_base = k.n0 + half * 128;
        __nv_bfloat16* yrow = p.Y + (size_t)t * p.ldy + n_base;
        const bool vec = ((reinterpret_cast<uintptr_t>(yrow) & 15) == 0);
#pragma unroll
        for (int c = 0; c < 128; c += 8) {
          if (n_base + c >= p.N) break;
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            v[j] = acc[c + j];
            if (p.bias != nullptr && n_base + c + j < p.N) v[j] += __bfloat162float(__ldg(p.bias + n_base + c + j));
          }
          if (vec && n_base + c + 8 <= p.N) {
            uint4 o;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]), h1 = __floats2bfloat162_rn(v[2], v[3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]), h3 = __floats2bfloat162_rn(v[6], v[7]);
            o.x = *reinterpret_cast<uint32_t*>(&h0);
            o.y = *reinterpret_cast<uint32_t*>(&h1);
            o.z = *reinterpret_cast<uint32_t*>(&h2);
            o.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(yrow + c) = o;
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (n_base + c + j < p.N) yrow[c + j] = __float2bfloat16(v[j]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

static int launch(const CUtensorMap& tmX, const CUtensorMap& tmW, const Params& p, int grid, cudaStream_t stream) {
  static unsigned long long attr_seen = 0;
  B200_CUDA_CHECK(ensure_dynamic_smem(gemm_fp8_rows_kernel, SMEM, &attr_seen));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  B200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_fp8_rows_kernel, tmX, tmW, p));
  return 0;
}

static int fill(Params& p, const float* xs, const float* ws, void* Y, const void* bias, int T, int N, int K, int ldy,
                int* status) {
  if (K % 16) {
    b200_set_last_error("gemm_fp8_block_rows: K must be a multiple of 16", __FILE__, __LINE__);
    return -3;
  }
  memset(&p, 0, sizeof(p));
  p.Y = (__nv_bfloat16*)Y;
  p.bias = (const __nv_bfloat16*)bias;
  p.w_scale = ws;
  p.x_scale = xs;
  p.status = status;
  p.T = T; p.N = N; p.K = K; p.ldy = ldy;
  p.n_tiles = (N + BNW - 1) / BNW;
  p.t_tiles = (T + BMT - 1) / BMT;
  p.kb_total = (K + BKB - 1) / BKB;
  p.ws_ld = p.kb_total;
  p.xs_ld = p.kb_total;
  p.ws_rows = (N + 127) / 128;
  static int skip = -1;
  if (skip < 0) {
    const char* e = getenv("B200_FP8_ROWS_SKIP_PROMOTE");
    skip = (e && e[0] == '1') ? 1 : 0;
  }
  p.skip_promote = skip;
  return 0;
}

}  // namespace f8r
}  // namespace b200

using namespace b200;

// Y[T,N] bf16 = dequant(Xq, xs) * dequant(Wq, ws)^T (+bias), the many-token form: Xq [T,K], Wq [N,K]
// contiguous e4m3; xs [T, ceil(K/128)], ws [ceil(N/128), ceil(K/128)] fp32.
extern "C" int b200_gemm_fp8_block_rows(const void* Xq, const float* xs, const void* Wq, const float* ws, void* Y,
                                        const void* bias, int T, int N, int K, int ldy, int* status, int num_sms,
                                        cudaStream_t stream) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  f8r::Params p;
  int rc = f8r::fill(p, xs, ws, Y, bias, T, N, K, ldy, status);
  if (rc) return rc;
  CUtensorMap tmX, tmW;
  rc = b200_make_tmap_2d(&tmX, Xq, 1, (uint64_t)T, (uint64_t)K, (uint64_t)K, f8r::BMT, f8r::BKB);
  if (rc) return rc;
  rc = b200_make_tmap_2d(&tmW, Wq, 1, (uint64_t)N, (uint64_t)K, (uint64_t)K, f8r::BNW, f8r::BKB);
  if (rc) return rc;
  const int total = p.n_tiles * p.t_tiles;
  return f8r::launch(tmX, tmW, p, total < num_sms ? total : num_sms, stream);
}

// Grouped form: rows [group_off[e], group_off[e+1]) of Xq use expert e's Wq [N,K] and its scale grid
// ws [num_groups, ceil(N/128), ceil(K/128)]; Y [R, N].  For groups of a few hundred rows or more.
extern "C" int b200_grouped_gemm_fp8_block_rows(const void* Xq, const float* xs, const void* Wq, const float* ws,
                                                void* Y, const int* group_off, int num_groups, int R, int N, int K,
                                                int* status, int num_sms, cudaStream_t stream) {
  if (R <= 0 || N <= 0 || K <= 0 || num_groups <= 0) return 0;
  if (num_groups > f8r::MAX_GROUPS) {
    b200_set_last_error("grouped_gemm_fp8_rows: at most 1024 groups", __FILE__, __LINE__);
    return -3;
  }
  f8r::Params p;
  int rc = f8r::fill(p, xs, ws, Y, nullptr, R, N, K, N, status);
  if (rc) return rc;
  p.group_off = group_off;
  p.num_groups = num_groups;
  p.w_rows_per_group = N;
  CUtensorMap tmX, tmW;
  rc = b200_make_tmap_2d(&tmX, Xq, 1, (uint64_t)R, (uint64_t)K, (uint64_t)K, f8r::BMT, f8r::BKB);
  if (rc) return rc;
  rc = b200_make_tmap_2d(&tmW, Wq, 1, (uint64_t)num_groups * N, (uint64_t)K, (uint64_t)K, f8r::BNW, f8r::BKB);
  if (rc) return rc;
  return f8r::launch(tmX, tmW, p, num_sms, stream);
}
