// W4A16 GEMM on tcgen05: 4-bit float weights (e2m1, two per byte, low nibble = even k) with group scales,
// bf16 activations, fp32 accumulation in TMEM.
//
//   Y[t, n] = sum_k X[t, k] * e2m1(Wp[n, k]) * scale[n, k / G]          mxfp4: G = 32, scale = 2^(e8m0 - 127)
//                                                                       nvfp4: G = 16, scale = e4m3 * global
//
// The weight never exists in bf16 in global memory: a tile is expanded in shared memory, in front of the
// tensor core.  Roles of a CTA (320 threads), persistent over (weight tile, token tile) pairs:
//
//   warp 0      TMA producer: packed weight bytes [128 rows x 32 B] and the activation tile [BN x 128 B]
//   warps 2-5   expansion: thread = weight row; 64 nibbles -> e2m1 value x group scale -> bf16, written as
//               the 128-byte K-major row of the UMMA A operand at its SWIZZLE_128B position, then
//               fence.proxy.async and an arrive on the stage's "expanded" barrier
//   warp 1      tcgen05.mma kind::f16 (M 128 = weight rows, N = tokens, K 16 x 4 per stage), accumulators
//               double-buffered in TMEM
//   warps 6-9   epilogue: TMEM -> bf16 -> Y (+ bias)
//
// Same orientation as the bf16 GEMM (weights are the 128-row operand, so decode batches keep full MMA
// rows).  Grouped mode takes device-side row offsets per expert.  Every wait is bounded.
//
// Formats of the reference's 4-bit linear and MoE methods
// (reference: src/vllm_torchtpu/layers/adapter/quantization/mxfp4.py:96-761, nvfp4.py,
// layers/core/quantization.py:106-195).
#include <cstring>

#include <cuda_fp8.h>

#include "common.cuh"
#include "gemm_tcgen05.h"

namespace b200 {
namespace w4 {

constexpr int BM = 128;            // weight rows per tile (UMMA M)
constexpr int BK = 64;             // K elements per stage: one 128-byte bf16 row
constexpr int RAW_BYTES = BM * BK / 2;
constexpr int A_BYTES = BM * BK * 2;
constexpr int NUM_THREADS = 320;
constexpr int MAX_GROUPS = 1024;

template <int BN>
struct Cfg {
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = RAW_BYTES + A_BYTES + B_BYTES;      // multiples of 1024 each
  static constexpr int STAGES_RAW = 196608 / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 6 ? 6 : STAGES_RAW;
  static constexpr int BAR_BYTES = 512;
  static constexpr int PREFIX_BYTES = (MAX_GROUPS + 1) * 4 + 12;
  static constexpr int SMEM = STAGES * STAGE_BYTES + BAR_BYTES + PREFIX_BYTES + 64 + 1024;
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
};

struct Params {
  __nv_bfloat16* Y;
  const __nv_bfloat16* bias;
  const uint8_t* scales;             // mxfp4: e8m0 [rows, K / 32]; nvfp4: e4m3 [rows, K / 16]
  const float* global_scale;         // nvfp4: one fp32 per tensor (or per group of rows: see gs_per_group)
  int* status;
  int T, N, K, ldy;
  int n_tiles, t_tiles, kb_total;
  const int* group_off;              // grouped: int[num_groups + 1]
  int num_groups, w_rows_per_group, gs_per_group;
};

struct Work {
  int w_row, t_row, t_valid, n0;
};

template <int BN>
__device__ __forceinline__ Work get_work(int w, const Params& p, const int* s_prefix) {
  Work k;
  if (p.group_off == nullptr) {
    const int n_tile = w % p.n_tiles, t_tile = w / p.n_tiles;
    k.w_row = n_tile * BM;
    k.n0 = n_tile * BM;
    k.t_row = t_tile * BN;
    k.t_valid = min(BN, p.T - k.t_row);
  } else {
    const int tt = w / p.n_tiles, n_tile = w - tt * p.n_tiles;
    int lo = 0, hi = p.num_groups;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_prefix[mid] <= tt) lo = mid; else hi = mid;
    }
    const int e = lo, t_tile = tt - s_prefix[e];
    const int r0 = p.group_off[e], rows = p.group_off[e + 1] - r0;
    k.w_row = e * p.w_rows_per_group + n_tile * BM;
    k.n0 = n_tile * BM;
    k.t_row = r0 + t_tile * BN;
    k.t_valid = min(BN, rows - t_tile * BN);
  }
  return k;
}

// FMT 0: mxfp4, FMT 1: nvfp4
template <int BN, int FMT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_w4a16_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const Params p) {
  using C = Cfg<BN>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::STAGE_BYTES);
  uint64_t* full = bars;                         // TMA bytes of the stage have landed
  uint64_t* expanded = bars + STAGES;            // the A tile of the stage has been written
  uint64_t* empty = bars + 2 * STAGES;           // the MMAs that read the stage have completed
  uint64_t* tfull = bars + 3 * STAGES;
  uint64_t* tempty = bars + 3 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_prefix = reinterpret_cast<int*>(smem + STAGES * C::STAGE_BYTES + C::BAR_BYTES);
  float* s_lut = reinterpret_cast<float*>(smem + STAGES * C::STAGE_BYTES + C::BAR_BYTES + C::PREFIX_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&expanded[i], 4);
      mbar_init(&empty[i], 1);
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], 4);
    mbar_init(&tempty[1], 4);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (threadIdx.x < 16) {
    // e2m1: sign, two exponent bits, one mantissa bit
    const int c = threadIdx.x, e = (c >> 1) & 3, m = c & 1;
    const float mag = e == 0 ? 0.5f * m : (1.f + 0.5f * m) * (float)(1 << (e - 1));
    s_lut[c] = (c & 8) ? -mag : mag;
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  pdl_launch_dependents();
  pdl_wait();
  if (p.group_off != nullptr) {
    for (int e = threadIdx.x; e < p.num_groups; e += blockDim.x)
      s_prefix[e + 1] = (p.group_off[e + 1] - p.group_off[e] + BN - 1) / BN;
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

  if (warp == 0) {
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const Work k = get_work<BN>(w, p, s_prefix);
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* st = smem + s * C::STAGE_BYTES;
          mbar_expect_tx(&full[s], RAW_BYTES + C::B_BYTES);
          tma_load_2d(st, &tmW, &full[s], kb * (BK / 2), k.w_row);                  // packed bytes
          tma_load_2d(st + RAW_BYTES + A_BYTES, &tmX, &full[s], kb * BK, k.t_row);   // activations
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (*abort_flag)
        for (int it = 0; it < 20000; ++it) __nanosleep(100);
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
      int s = 0;
      uint32_t ph = 0, tile_i = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++tile_i) {
        const int acc = tile_i & 1;
        if (!mbar_wait(&tempty[acc], ((tile_i >> 1) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(&full[s], ph, abort_flag, p.status, ST_TIMEOUT_FULL) ||
              !mbar_wait(&expanded[s], ph, abort_flag, p.status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES + RAW_BYTES);
          const uint64_t adesc = umma_desc_k_sw128(a_addr);
          const uint64_t bdesc = umma_desc_k_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int q = 0; q < BK / 16; ++q)      // K = 16 per instruction: 32 bytes along the 128-byte row
            umma_f16(tmem_base + acc * BN, adesc + 2 * q, bdesc + 2 * q, idesc, (kb > 0 || q > 0) ? 1u : 0u);
          umma_commit(&empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else if (warp < 6) {
    // ---- expansion: this thread owns weight row `row` of every tile
    const int row = threadIdx.x - 64;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    constexpr int G = FMT == 0 ? 32 : 16;
    const int sc_ld = p.K / G;
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      const Work k = get_work<BN>(w, p, s_prefix);
      const bool live = k.n0 + row < p.N;
      const uint8_t* sc_row = p.scales + (size_t)(k.w_row + row) * sc_ld;
      float gs = 1.f;
      if (FMT == 1) gs = p.global_scale[p.gs_per_group ? (k.w_row / p.w_rows_per_group) : 0];
      for (int kb = 0; kb < kb_total; ++kb) {
        // group scales of this row's 64 values (2 for mxfp4, 4 for nvfp4), fetched before the wait
        float sc[BK / G];
#pragma unroll
        for (int g = 0; g < BK / G; ++g) {
          const int gi = kb * (BK / G) + g;
          float v = 0.f;
          if (live && gi < sc_ld) {
            const uint8_t b = __ldg(sc_row + gi);
            if (FMT == 0) {
              v = __uint_as_float((uint32_t)b << 23);                 // 2^(b - 127); b = 0 gives 0
            } else {
              const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
              v = __half2float(*reinterpret_cast<const __half*>(&h)) * gs;
            }
          }
          sc[g] = v;
        }
        if (!mbar_wait(&full[s], ph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
        const uint8_t* st = smem + s * C::STAGE_BYTES;
        // the packed tile was written by TMA without swizzle: dense rows of 32 bytes
        uint4 raw[2];
        raw[0] = *reinterpret_cast<const uint4*>(st + row * 32);
        raw[1] = *reinterpret_cast<const uint4*>(st + row * 32 + 16);
        uint8_t* a_row = const_cast<uint8_t*>(st) + RAW_BYTES + row * 128;
        const uint32_t* words = reinterpret_cast<const uint32_t*>(raw);
#pragma unroll
        for (int c = 0; c < 8; ++c) {            // 16-byte chunk c of the bf16 row = 8 values = one packed word
          const uint32_t wd = words[c];
          const float s8 = sc[(c * 8) / G];
          uint32_t pk[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float lo = s_lut[(wd >> (8 * j)) & 0xF] * s8;
            const float hi = s_lut[(wd >> (8 * j + 4)) & 0xF] * s8;
            __nv_bfloat162 b2 = __floats2bfloat162_rn(lo, hi);
            pk[j] = *reinterpret_cast<uint32_t*>(&b2);
          }
          *reinterpret_cast<uint4*>(a_row + ((c ^ (row & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        fence_proxy_async_smem();                // generic-proxy writes before the tensor core's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(&expanded[s]);
        if (++s == STAGES) { s = 0; ph ^= 1; }
      }
    }
  } else {
    // ---- epilogue: TMEM lane = weight row, column = token
    const int q = warp & 3;
    const int row = q * 32 + lane;
    uint32_t tile_i = 0;
    for (int w = blockIdx.x; w < total_work; w += gridDim.x, ++tile_i) {
      const Work k = get_work<BN>(w, p, s_prefix);
      const int acc = tile_i & 1;
      if (!mbar_wait(&tfull[acc], (tile_i >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const int n = k.n0 + row;
      const float bias = (p.bias != nullptr && n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        if (c0 >= k.t_valid) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        tmem_ld_wait();
        if (n < p.N) {
          __nv_bfloat16* yp = p.Y + (size_t)(k.t_row + c0) * p.ldy + n;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j < k.t_valid) yp[(size_t)j * p.ldy] = __float2bfloat16(__uint_as_float(r[j]) + bias);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

template <int BN, int FMT>
static int launch(const CUtensorMap& tmW, const CUtensorMap& tmX, const Params& p, int grid, cudaStream_t stream) {
  using C = Cfg<BN>;
  static unsigned long long attr_seen = 0;
  B200_CUDA_CHECK(ensure_dynamic_smem(gemm_w4a16_kernel<BN, FMT>, C::SMEM, &attr_seen));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = C::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  B200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_w4a16_kernel<BN, FMT>, tmW, tmX, p));
  return 0;
}

template <int FMT>
static int dispatch(int bn, const CUtensorMap& tmW, const CUtensorMap& tmX, const Params& p, int grid,
                    cudaStream_t stream) {
  switch (bn) {
    case 32: return launch<32, FMT>(tmW, tmX, p, grid, stream);
    case 64: return launch<64, FMT>(tmW, tmX, p, grid, stream);
    case 128: return launch<128, FMT>(tmW, tmX, p, grid, stream);
    default: return launch<256, FMT>(tmW, tmX, p, grid, stream);
  }
}

static int run(const void* X, const void* Wp, const void* scales, const float* global_scale, void* Y,
               const void* bias, const int* group_off, int num_groups, int gs_per_group, int T, int N, int K,
               int ldx, int ldy, int fmt, int rows_hint, int* status, int num_sms, cudaStream_t stream) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if (K % BK || (fmt != 0 && fmt != 1) || (fmt == 1 && global_scale == nullptr) || num_groups > MAX_GROUPS) {
    b200_set_last_error("gemm_w4a16: K % 64 == 0, format mxfp4 (0) or nvfp4 (1, with its global scale), "
                        "at most 1024 groups", __FILE__, __LINE__);
    return -3;
  }
  if (group_off != nullptr && N % BM) {
    b200_set_last_error("gemm_w4a16 (grouped): N % 128 == 0 required", __FILE__, __LINE__);
    return -3;
  }
  const int bn = rows_hint <= 32 ? 32 : (rows_hint <= 64 ? 64 : (rows_hint <= 128 ? 128 : 256));
  Params p;
  memset(&p, 0, sizeof(p));
  p.Y = (__nv_bfloat16*)Y;
  p.bias = (const __nv_bfloat16*)bias;
  p.scales = (const uint8_t*)scales;
  p.global_scale = global_scale;
  p.status = status;
  p.T = T; p.N = N; p.K = K; p.ldy = ldy;
  p.n_tiles = (N + BM - 1) / BM;
  p.t_tiles = (T + bn - 1) / bn;
  p.kb_total = K / BK;
  p.group_off = group_off;
  p.num_groups = num_groups;
  p.w_rows_per_group = N;
  p.gs_per_group = gs_per_group;
  const int w_rows = group_off != nullptr ? num_groups * N : N;
  CUtensorMap tmW, tmX;
  int rc = b200_make_tmap_2d_bytes_linear(&tmW, Wp, (uint64_t)w_rows, (uint64_t)(K / 2), (uint64_t)(K / 2), BM,
                                          BK / 2);
  if (rc) return rc;
  rc = b200_make_tmap_2d(&tmX, X, 2, (uint64_t)T, (uint64_t)K, (uint64_t)ldx * 2, (uint32_t)bn, BK);
  if (rc) return rc;
  const int total = group_off != nullptr ? num_sms : p.n_tiles * p.t_tiles;
  const int grid = total < num_sms ? total : num_sms;
  return fmt == 0 ? dispatch<0>(bn, tmW, tmX, p, grid, stream) : dispatch<1>(bn, tmW, tmX, p, grid, stream);
}

}  // namespace w4
}  // namespace b200

using namespace b200;

// Y[T, N] bf16 = X[T, K] bf16 x dequant(Wp [N, K / 2] packed e2m1, scales)^T (+ bias).  fmt 0: mxfp4 (scales
// e8m0 [N, K / 32]); fmt 1: nvfp4 (scales e4m3 [N, K / 16], global_scale fp32[1]).  K % 64 == 0.
extern "C" int b200_gemm_w4a16(const void* X, const void* Wp, const void* scales, const float* global_scale,
                               void* Y, const void* bias, int T, int N, int K, int ldx, int ldy, int fmt,
                               int* status, int num_sms, cudaStream_t stream) {
  return w4::run(X, Wp, scales, global_scale, Y, bias, nullptr, 0, 0, T, N, K, ldx, ldy, fmt, T, status, num_sms,
                 stream);
}

// Grouped form: rows [group_off[e], group_off[e+1]) of X use expert e's packed weights Wp [E, N, K / 2] and
// scales [E, N, K / G]; nvfp4 takes one global scale per expert (fp32[E]).  Y [R, N].
extern "C" int b200_grouped_gemm_w4a16(const void* X, const void* Wp, const void* scales, const float* global_scale,
                                       void* Y, const int* group_off, int num_groups, int R, int N, int K,
                                       int avg_rows_hint, int fmt, int* status, int num_sms, cudaStream_t stream) {
  if (num_groups <= 0) return 0;
  return w4::run(X, Wp, scales, global_scale, Y, nullptr, group_off, num_groups, 1, R, N, K, K, N, fmt,
                 avg_rows_hint, status, num_sms, stream);
}
