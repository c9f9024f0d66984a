// Prefill-sized bf16 GEMM  Y[T,N] = X[T,K] * W[N,K]^T (+ bias)  on two-SM tensor-core instructions.
//
// A cluster of two CTAs (an SM pair) computes one 256 (weight rows) x 256 (tokens) tile with
// tcgen05.mma.cta_group::2: every CTA stages its own 128 weight rows (operand A) and its own 128
// of the 256 token rows (operand B) per 64-wide K block, so a CTA moves 32 KB per K block where the
// one-SM kernel of gemm_tcgen05.cu moves 48 KB for a 128 x 256 tile.  Less shared-memory traffic per
// FLOP is what matters on a power-capped part.  The accumulator of a CTA is its own 128 rows x 256
// token columns in its own TMEM, double buffered (2 x 256 columns) so that the epilogue of a tile
// overlaps the main loop of the next one.
//
// Roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocation and (leader CTA
// only) the MMA issuer, warps 2-5 = epilogue.  Synchronisation across the pair:
//   * full[s]   lives in the leader (cluster rank 0); both producers' tensor loads complete their
//               bytes on it (the .cta_group::2 form lets a load signal the peer CTA's barrier; every
//               CTA fetches only its own operand halves, nothing is broadcast);
//   * empty[s]  lives in each CTA; the leader's tcgen05.commit arrives on both (commit multicast);
//   * tfull[a]  lives in each CTA, same commit multicast;
//   * tempty[a] lives in the leader; the four epilogue warps of both CTAs arrive on it.
// Every wait is time bounded (mbar_wait): on a timeout the CTA records a status code, leaves its
// loops, and still reaches the closing cluster barrier and the TMEM release.
//
// SwiGLU form (W = [2I, K], gate rows then up rows, Y[T, I] = silu(gate) * up): the 128 operand-A rows
// of a CTA are 64 gate rows followed by the 64 up rows of the same outputs, so the main loop and the
// double-buffered 256-column accumulator are those of the plain form.  TMEM lanes 0-63 then hold gate,
// lanes 64-127 up; the epilogue warps of a gate quarter and of the matching up quarter exchange half of
// their values through shared memory, 32 token columns at a time, and each finishes 16 of the columns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

#include "common.cuh"

extern "C" int b200_make_tmap_2d(void* out_map, const void* ptr, int elem_bytes, uint64_t rows, uint64_t cols,
                                 uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols);

namespace b200 {
namespace g2 {

constexpr int BM = 128;            // weight rows per CTA (256 per pair = UMMA M)
constexpr int BNT = 256;           // tokens per tile (UMMA N); each CTA stages BNT / 2 of them
constexpr int BK = 64;             // bf16 elements per 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = (BNT / 2) * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int BAR_BYTES = 256;
constexpr int XCHG_BYTES = 2 * 2 * 32 * 32 * 4;   // SwiGLU: two warp pairs x two buffers x [32 columns][32 rows] fp32
constexpr int SMEM = STAGES * STAGE_BYTES + BAR_BYTES + XCHG_BYTES + 1024;
constexpr int TMEM_COLS = 512;
constexpr int THREADS = 192;
constexpr int GROUP_N = 8;         // raster: 8 weight tile pairs share the activations in L2

struct Params {
  __nv_bfloat16* Y;
  const __nv_bfloat16* bias;
  int* status;
  int T, N, K, ldy;
  int n_pairs, t_tiles, kb_total;
  int up_row_off;                  // SwiGLU: first up row of W (= I)
};

__device__ __forceinline__ void tmem_alloc_2sm(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2sm() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2sm(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// 2D tiled load into this CTA's shared memory whose byte count completes on a barrier given by its
// shared::cluster address (the leader's); each CTA fetches only its own operand halves
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
// D[tmem of both CTAs] (+)= A * B with operands read from both CTAs' shared memory; one thread of the leader
__device__ __forceinline__ void umma_f16_2sm(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive (once the MMAs issued so far have completed) on the barrier at this offset in both CTAs
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__device__ __forceinline__ void decode_work(int w, const Params& p, int& n_pair, int& t_tile) {
  const int per_group = GROUP_N * p.t_tiles;
  const int g = w / per_group, rem = w - g * per_group;
  const int first = g * GROUP_N;
  const int gsize = min(GROUP_N, p.n_pairs - first);
  t_tile = rem / gsize;
  n_pair = first + rem - t_tile * gsize;
}

template <bool SWIGLU>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_bf16_2sm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                     const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                          // used in the leader only
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + 2;       // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();        // 0 = leader
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);                     // the leader's producer arms it with both CTAs' bytes
      mbar_init(&empty[s], 1);                    // one commit
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], 8);                     // four epilogue warps of each CTA
    mbar_init(&tempty[1], 8);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc_2sm(tmem_slot, TMEM_COLS);
    tmem_relinquish_2sm();
  }
  pdl_launch_dependents();
  pdl_wait();
  tc_fence_before();
  __syncthreads();
  // the peer's barriers must exist before anything of this CTA arrives on them
  cluster_arrive_release();
  cluster_wait_acquire();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_work = p.n_pairs * p.t_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int w = pair; w < total_work && ok; w += npairs) {
        int n_pair, t_tile;
        decode_work(w, p, n_pair, t_tile);
        // output rows (weight rows, or gate rows in the SwiGLU form) of this CTA's part of the tile
        const int w_row = SWIGLU ? (n_pair * 2 + (int)rank) * (BM / 2) : n_pair * (2 * BM) + (int)rank * BM;
        const int t_row = t_tile * BNT + (int)rank * (BNT / 2);
        for (int kb = 0; kb < p.kb_total; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* a = smem + s * STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
          const uint32_t bar = mapa_shared(smem_u32(&full[s]), 0);
          if (SWIGLU) {      // tmW has a 64-row box here
            tma_load_2d_pair(a, &tmW, bar, kb * BK, w_row);
            tma_load_2d_pair(a + A_BYTES / 2, &tmW, bar, kb * BK, p.up_row_off + w_row);
          } else {
            tma_load_2d_pair(a, &tmW, bar, kb * BK, w_row);
          }
          tma_load_2d_pair(a + A_BYTES, &tmX, bar, kb * BK, t_row);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (*abort_flag) {
        // give the bulk copies in flight a bounded time to land before the CTA exits
        for (int it = 0; it < 20000; ++it) __nanosleep(100);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, BNT);
      int s = 0;
      uint32_t ph = 0;
      int iter = 0;
      bool ok = true;
      for (int w = pair; w < total_work && ok; w += npairs, ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_ph = (iter >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BNT;
        for (int kb = 0; kb < p.kb_total; ++kb) {
          if (!mbar_wait(&full[s], ph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t adesc = umma_desc_k_sw128(a_addr);
          const uint64_t bdesc = umma_desc_k_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16_2sm(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty[s]);            // both CTAs may refill the stage once the MMAs have read it
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit_pair(&tfull[acc]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs)
    const int q = warp & 3;                       // TMEM lane quarter this warp may access
    const int row = q * 32 + lane;
    int iter = 0;
    for (int w = pair; w < total_work; w += npairs, ++iter) {
      int n_pair, t_tile;
      decode_work(w, p, n_pair, t_tile);
      const int acc = iter & 1;
      const uint32_t acc_ph = (iter >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_ph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const int t0 = t_tile * BNT;
      const int t_valid = min(BNT, p.T - t0);
      const uint32_t taddr = tmem_base + acc * BNT + ((uint32_t)(q * 32) << 16);
      if constexpr (SWIGLU) {
        // quarters 0, 1 hold gate rows, quarters 2, 3 the up rows of the same outputs
        const int hp = q & 1;                       // warp pair
        const int n = (n_pair * 2 + (int)rank) * (BM / 2) + hp * 32 + lane;
        float* xb = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + BAR_BYTES) + hp * (2 * 32 * 32);
        int chunk = 0;
#pragma unroll 1
        for (int c0 = 0; c0 < BNT; c0 += 32, ++chunk) {
          if (c0 >= t_valid) break;                 // uniform over the four warps
          uint32_t r[32];
          tmem_ld_32x32(taddr + c0, r);
          tmem_ld_wait();
          float* buf = xb + (chunk & 1) * (32 * 32);
          // The gate warp finishes token columns 0-15 of the chunk and the up warp columns 16-31, so
          // each hands the other the 16 values it does not finish itself.
          if (q >= 2) {
#pragma unroll
            for (int j = 0; j < 16; ++j) buf[j * 32 + lane] = __uint_as_float(r[j]);
          } else {
#pragma unroll
            for (int j = 16; j < 32; ++j) buf[j * 32 + lane] = __uint_as_float(r[j]);
          }
          // pair barrier (ids 1 and 2): this chunk's values are visible to the partner warp, and the
          // partner has finished reading the buffer written two chunks ago
          asm volatile("bar.sync %0, 64;" ::"r"(1 + hp) : "memory");
          if (n < p.N) {
            if (q >= 2) {        // up warp: columns 16-31, gate values from the partner
              __nv_bfloat16* yp = p.Y + (size_t)(t0 + c0 + 16) * p.ldy + n;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (c0 + 16 + j < t_valid) {
                  const float gv = buf[(16 + j) * 32 + lane], uv = __uint_as_float(r[16 + j]);
                  yp[(size_t)j * p.ldy] = __float2bfloat16(__fdividef(gv, 1.f + __expf(-gv)) * uv);
                }
              }
            } else {             // gate warp: columns 0-15, up values from the partner
              __nv_bfloat16* yp = p.Y + (size_t)(t0 + c0) * p.ldy + n;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (c0 + j < t_valid) {
                  const float gv = __uint_as_float(r[j]), uv = buf[j * 32 + lane];
                  yp[(size_t)j * p.ldy] = __float2bfloat16(__fdividef(gv, 1.f + __expf(-gv)) * uv);
                }
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty[acc]), 0));
        continue;
      }
      const int n = n_pair * (2 * BM) + (int)rank * BM + row;
      const float bias = (p.bias != nullptr && n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < BNT; c0 += 32) {
        if (c0 >= t_valid) break;                 // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        tmem_ld_wait();
        if (n < p.N) {
          __nv_bfloat16* yp = p.Y + (size_t)(t0 + c0) * p.ldy + n;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j < t_valid) yp[(size_t)j * p.ldy] = __float2bfloat16(__uint_as_float(r[j]) + bias);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty[acc]), 0));
    }
  }

  // Both CTAs are done with each other's shared memory, barriers and TMEM only after this point.
  tc_fence_before();
  __syncthreads();
  cluster_arrive_release();
  cluster_wait_acquire();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, TMEM_COLS);
  }
}

}  // namespace g2
}  // namespace b200

#include <mutex>
#include <unordered_map>

namespace b200 {
namespace g2 {

struct MapKey {
  const void* ptr;
  uint64_t rows, cols, stride;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && stride == o.stride;
  }
};
struct MapHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= k.rows * 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.cols * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
    h ^= k.stride * 0x165667B19E3779F9ull + (h << 6) + (h >> 2);
    return h;
  }
};

// tensor map of a row-major bf16 matrix with a box_rows x 64-column box
static int operand_map(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t stride_bytes,
                       uint32_t box_rows = BM) {
  static std::unordered_map<MapKey, CUtensorMap, MapHash> cache;
  static std::mutex mu;
  MapKey key{ptr, rows, cols | ((uint64_t)box_rows << 48), stride_bytes};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  int rc = b200_make_tmap_2d(out, ptr, 2, rows, cols, stride_bytes, box_rows, BK);
  if (rc != 0) return rc;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

// persistent grid: exactly as many SM pairs as can be resident at once (a cluster needs both SMs of a
// pair, so this can be fewer than num_sms / 2)
template <bool SWIGLU>
static int launch_pairs(const CUtensorMap& tmW, const CUtensorMap& tmX, const Params& p, int num_sms,
                        cudaStream_t stream) {
  static int max_pairs = 0;
  static unsigned long long attr_seen = 0;
  B200_CUDA_CHECK(ensure_dynamic_smem(gemm_bf16_2sm_kernel<SWIGLU>, SMEM, &attr_seen));
  if (max_pairs == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (num_sms / 2));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_bf16_2sm_kernel<SWIGLU>, &cfg) != cudaSuccess || n < 1) {
      cudaGetLastError();
      n = num_sms / 2;
    }
    max_pairs = n;
  }
  const int total = p.n_pairs * p.t_tiles;
  int pairs = max_pairs < num_sms / 2 ? max_pairs : num_sms / 2;
  if (pairs > total) pairs = total;
  if (pairs < 1) pairs = 1;
  B200_CUDA_CHECK(launch_pdl(gemm_bf16_2sm_kernel<SWIGLU>, dim3(2 * pairs), dim3(THREADS), SMEM, stream, tmW, tmX,
                             p));
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace g2
}  // namespace b200

// X [T,K] row stride ldx, W [N,K] row stride ldw, Y [T,N] row stride ldy (elements); status: device int
// that receives a time-out code (common.cuh) if a wait inside the kernel gives up.
extern "C" int b200_gemm_bf16_2sm(const void* X, const void* W, void* Y, const void* bias, int T, int N, int K,
                                  int ldx, int ldw, int ldy, int* status, int num_sms, cudaStream_t stream) {
  using namespace b200;
  using namespace b200::g2;
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 8 || ldx % 8 || ldw % 8) {
    b200_set_last_error("gemm_bf16_2sm: K and row strides must be multiples of 8 elements", __FILE__, __LINE__);
    return -3;
  }
  Params p;
  memset(&p, 0, sizeof(p));
  p.Y = reinterpret_cast<__nv_bfloat16*>(Y);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.status = status;
  p.T = T; p.N = N; p.K = K; p.ldy = ldy;
  p.n_pairs = (N + 2 * BM - 1) / (2 * BM);
  p.t_tiles = (T + BNT - 1) / BNT;
  p.kb_total = (K + BK - 1) / BK;
  CUtensorMap tmW, tmX;
  int rc = operand_map(&tmW, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw * 2);
  if (rc) return rc;
  rc = operand_map(&tmX, X, (uint64_t)T, (uint64_t)K, (uint64_t)ldx * 2);
  if (rc) return rc;
  return launch_pairs<false>(tmW, tmX, p, num_sms, stream);
}

// Y[T, I] = silu(X * W[0:I]^T) * (X * W[I:2I]^T); W [2I, K] row stride ldw.
extern "C" int b200_gemm_bf16_swiglu_2sm(const void* X, const void* W, void* Y, int T, int I, int K, int ldx,
                                         int ldw, int ldy, int* status, int num_sms, cudaStream_t stream) {
  using namespace b200;
  using namespace b200::g2;
  if (T <= 0 || I <= 0 || K <= 0) return 0;
  if (K % 8 || ldx % 8 || ldw % 8) {
    b200_set_last_error("gemm_swiglu_2sm: K and row strides must be multiples of 8 elements", __FILE__, __LINE__);
    return -3;
  }
  Params p;
  memset(&p, 0, sizeof(p));
  p.Y = reinterpret_cast<__nv_bfloat16*>(Y);
  p.status = status;
  p.T = T; p.N = I; p.K = K; p.ldy = ldy;
  p.n_pairs = (I + BM - 1) / BM;                 // a pair produces 2 x 64 output rows
  p.t_tiles = (T + BNT - 1) / BNT;
  p.kb_total = (K + BK - 1) / BK;
  p.up_row_off = I;
  CUtensorMap tmW, tmX;
  int rc = operand_map(&tmW, W, (uint64_t)2 * I, (uint64_t)K, (uint64_t)ldw * 2, BM / 2);
  if (rc) return rc;
  rc = operand_map(&tmX, X, (uint64_t)T, (uint64_t)K, (uint64_t)ldx * 2);
  if (rc) return rc;
  return launch_pairs<true>(tmW, tmX, p, num_sms, stream);
}
