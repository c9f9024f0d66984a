// fp8 (e4m3) GEMM with 128x128 weight block scales and 1x128 activation scales on tcgen05.
//
//   Y[t, n] = sum_kb  ( sum_{k in block kb} Xq[t,k] * Wq[n,k] ) * xs[t,kb] * ws[n/128, kb]
//
// tcgen05.mma (kind::f8f6f4, fp32 accumulate) cannot apply a different scale to every 128-wide
// K block inside one accumulation, so each K block is accumulated on its own in TMEM (two
// partial buffers, ping-pong) and the promotion warps (four, or eight from 64 tokens per tile on, so that
// a warp's share of a K block is at most two TMEM loads, issued together) "promote" it: tcgen05.ld the
// partial, multiply by the block's scale product and add into fp32 register accumulators while the
// tensor core already works on the next block.  A weight tile is exactly one scale row (BM = 128), so
// the weight scale is one scalar per (tile, K block); activation scales are one per column.
// Layouts: Wq [N, K] e4m3 K-major (the checkpoint layout), ws [ceil(N/128), ceil(K/128)] fp32
// (``weight_scale_inv``), Xq [T, K] e4m3, xs [T, ceil(K/128)] fp32 from the quantisation kernel
// below.  Same orientation as the bf16 kernel: weight rows are the 128-row UMMA operand, tokens
// are N (32/64/128), so decode batches keep full MMA rows.  Split-K runs as a thread-block
// cluster with a DSMEM reduction; grouped (per-expert) mode takes device-side row offsets.
//
// The same kernel, instantiated with KIND = 1, is the int8 W8A8 GEMM (per-output-channel weight
// scales, per-token activation scales): tcgen05.mma kind::i8 gives exact s32 sums per K block, the
// epilogue warps add them up in fp32 and apply ws[n] * xs[t] once at the end.
//
// Semantics of the reference's block-wise quantised matmul
// (reference: src/vllm_torchtpu/layers/adapter/linear_common.py:69-133, kernels/megablox/gmm_v2.py).
#include <cstring>

#include "common.cuh"
#include "gemm_tcgen05.h"

namespace b200 {
namespace f8 {

constexpr int BM = 128;
constexpr int BKB = 128;          // K elements (= bytes) per stage row: one scale block
constexpr int MAX_GROUPS = 1024;

template <int BN>
struct Cfg {
  // promotion warps: four cover the 128 TMEM lanes; from 64 tokens on a second set of four takes half of
  // the columns, so that a warp never has more than 64 columns (two TMEM loads) per K block
  static constexpr int EPI_WARPS = BN >= 64 ? 8 : 4;
  static constexpr int CW = BN / (EPI_WARPS / 4);
  static constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int A_BYTES = BM * BKB;
  static constexpr int B_BYTES = BN * BKB;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = 180224 / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int BAR_BYTES = 256;
  static constexpr int PREFIX_BYTES = (MAX_GROUPS + 1) * 4 + 12;      // keeps what follows 16-byte aligned
  static constexpr int SCALE_BYTES = EPI_WARPS * 2 * CW * 4;          // per promotion warp: two rows of column scales
  // routed rows: per set of four promotion warps two buffers of [32 tokens][128 rows] bf16
  static constexpr int ROUTE_BYTES = (EPI_WARPS / 4) * 2 * 32 * BM * 2;
  static constexpr int SMEM = STAGES * STAGE_BYTES + BAR_BYTES + PREFIX_BYTES + SCALE_BYTES + ROUTE_BYTES + 1024;
  static_assert(SMEM <= 232448, "shared memory budget");
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  static_assert(BM * BN * 4 <= STAGES * STAGE_BYTES, "split-K partial must fit in the stage ring");
};

struct Params {
  __nv_bfloat16* Y;
  const __nv_bfloat16* bias;
  const float* w_scale;
  const float* x_scale;
  int* status;
  int T, N, K, ldy;
  int n_tiles, t_tiles, kb_total, splits, kb_per_split;
  int ws_ld, xs_ld;                 // row strides of the scale matrices
  int cluster_splitk;
  const int* group_off;             // grouped: int[num_groups + 1]
  int num_groups, w_rows_per_group, ws_rows_per_group;
  // ---- tensor-parallel push plane (world > 1): the bf16 partial [T, N] of this rank goes into the
  // receive slab every rank keeps for it, one flag per (source rank, output tile); the consumer
  // (b200_reduce_pushed_rms_norm) sums the slabs.  Same protocol, flags and epoch word as the bf16
  // GEMM's push mode, so launches of the two kernels may alternate on one control block.
  int world, rank, max_tiles;
  uint8_t* peer[8];
  unsigned long long part_off, part_src_stride, tile_flag_off;
  int* epoch_ptr;
  int* cta_done;
  // ---- routed rows (expert-parallel combine inside a grouped launch): output row r goes to slot
  // row_route[r].y of rank row_route[r].x at heap offset route_ret_off (row length N); the last CTA
  // to exit raises int[world] flags at ret_flag_off of every rank with the epoch in *epoch_ptr
  const int2* row_route;
  unsigned long long route_ret_off, ret_flag_off;
  // dense launches may cover a sub-range of the output tiles (the ragged last wave of a persistent launch is
  // run as a second, split-K launch): tiles [tile_offset, tile_offset + launch_tiles), 0 = all
  int tile_offset, launch_tiles;
};

// index of output tile (n_tile, t_tile) in the raster the consumer uses (groups of 16 weight tiles)
__device__ __forceinline__ int raster_tile(int n_tile, int t_tile, int n_tiles, int t_tiles) {
  const int g = n_tile / 16, first_n = g * 16;
  const int gsize = min(16, n_tiles - first_n);
  return g * 16 * t_tiles + t_tile * gsize + (n_tile - first_n);
}

struct Work {
  int w_row, ws_row, t_row, t_valid, n0, kb0, kb1;
};

template <int BN>
__device__ __forceinline__ Work get_work(int w, const Params& p, const int* s_prefix) {
  Work k;
  if (p.group_off == nullptr) {
    const int local = w / p.splits, split = w - local * p.splits;
    const int tile = local + p.tile_offset;
    const int n_tile = tile % p.n_tiles, t_tile = tile / p.n_tiles;
    k.w_row = n_tile * BM;
    k.ws_row = n_tile;
    k.n0 = n_tile * BM;
    k.t_row = t_tile * BN;
    k.t_valid = min(BN, p.T - k.t_row);
    k.kb0 = split * p.kb_per_split;
    k.kb1 = min(p.kb_total, k.kb0 + p.kb_per_split);
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
    k.ws_row = e * p.ws_rows_per_group + n_tile;
    k.n0 = n_tile * BM;
    k.t_row = r0 + t_tile * BN;
    k.t_valid = min(BN, rows - t_tile * BN);
    k.kb0 = 0;
    k.kb1 = p.kb_total;
  }
  return k;
}

// MODE 0: output to Y; 1: tensor-parallel push plane; 2: routed rows (expert-parallel combine)
template <int BN, int KIND, int MODE>
__global__ void __launch_bounds__(Cfg<BN>::NUM_THREADS, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                      const Params p) {
  using C = Cfg<BN>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* pfull = bars + 2 * STAGES;
  uint64_t* pempty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_prefix = reinterpret_cast<int*>(smem + STAGES * C::STAGE_BYTES + C::BAR_BYTES);
  float* s_scale = reinterpret_cast<float*>(smem + STAGES * C::STAGE_BYTES + C::BAR_BYTES + C::PREFIX_BYTES);
  __nv_bfloat16* s_route = reinterpret_cast<__nv_bfloat16*>(smem + STAGES * C::STAGE_BYTES + C::BAR_BYTES +
                                                            C::PREFIX_BYTES + C::SCALE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&pfull[0], 1);
    mbar_init(&pfull[1], 1);
    mbar_init(&pempty[0], C::EPI_WARPS);
    mbar_init(&pempty[1], C::EPI_WARPS);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  pdl_launch_dependents();
  pdl_wait();
  // bumped by the last CTA of a push launch to exit: read by every thread before any CTA can do so
  constexpr bool PUSH = MODE == 1, ROUTED = MODE == 2;
  const int epoch = PUSH ? (*reinterpret_cast<volatile int*>(p.epoch_ptr) + 1) : 0;
  const int ndst = PUSH ? p.world : 1;
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
  const int total_work = p.group_off != nullptr
                             ? s_prefix[p.num_groups] * p.n_tiles
                             : (p.launch_tiles > 0 ? p.launch_tiles : p.n_tiles * p.t_tiles) * p.splits;

  if (warp == 0) {
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const Work k = get_work<BN>(w, p, s_prefix);
        for (int kb = k.kb0; kb < k.kb1; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* a = smem + s * C::STAGE_BYTES;
          mbar_expect_tx(&full[s], C::STAGE_BYTES);
          tma_load_2d(a, &tmW, &full[s], kb * BKB, k.w_row);
          tma_load_2d(a + C::A_BYTES, &tmX, &full[s], kb * BKB, k.t_row);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (*abort_flag)
        for (int it = 0; it < 20000; ++it) __nanosleep(100);
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = KIND == 1 ? umma_idesc_s8(BM, BN) : umma_idesc_e4m3(BM, BN);
      int s = 0;
      uint32_t ph = 0;
      uint32_t pc = 0;                         // K blocks issued by this CTA (selects the partial buffer)
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const Work k = get_work<BN>(w, p, s_prefix);
        for (int kb = k.kb0; kb < k.kb1; ++kb, ++pc) {
          const int pb = pc & 1;
          if (!mbar_wait(&pempty[pb], ((pc >> 1) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) {
            ok = false;
            break;
          }
          if (!mbar_wait(&full[s], ph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * C::STAGE_BYTES);
          const uint64_t adesc = umma_desc_k_sw128(a_addr);
          const uint64_t bdesc = umma_desc_k_sw128(a_addr + C::A_BYTES);
#pragma unroll
          for (int q = 0; q < 4; ++q) {        // 4 x (K = 32 bytes) per 128-byte row; a fresh sum per block
            if (KIND == 1) umma_i8(tmem_base + pb * BN, adesc + 2 * q, bdesc + 2 * q, idesc, q > 0 ? 1u : 0u);
            else umma_f8(tmem_base + pb * BN, adesc + 2 * q, bdesc + 2 * q, idesc, q > 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);
          umma_commit(&pfull[pb]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else {
    // promotion warps: warp w reads TMEM lanes 32 * (w % 4).. (its quarter of the weight rows) and the
    // CW columns (tokens) from col0 on; all of its TMEM loads of a K block are in flight together
    constexpr int CW = C::CW;
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int col0 = ((warp - 2) >> 2) * CW;
    uint32_t pc = 0;
    uint32_t route_count = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      const Work k = get_work<BN>(w, p, s_prefix);
      float acc[CW];
#pragma unroll
      for (int c = 0; c < CW; ++c) acc[c] = 0.f;
      for (int kb = k.kb0; kb < k.kb1; ++kb, ++pc) {
        const int pb = pc & 1;
        // the scale of column c is a warp-uniform value per accumulator register: lane j fetches the
        // scale product of column c0 + j, the warp parks the row in shared memory and reads it back four
        // columns per broadcast load (a shuffle per column would cost four times the issue slots)
        float* srow = s_scale + ((warp - 2) * 2 + pb) * CW;
        if (KIND == 0) {
          const float sw = p.w_scale[(size_t)k.ws_row * p.ws_ld + kb];
#pragma unroll
          for (int c0 = 0; c0 < CW; c0 += 32) {
            const int c = col0 + c0 + lane;
            srow[c0 + lane] = c < k.t_valid ? sw * p.x_scale[(size_t)(k.t_row + c) * p.xs_ld + kb] : 0.f;
          }
          __syncwarp();
        }
        if (!mbar_wait(&pfull[pb], (pc >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + pb * BN + col0 + ((uint32_t)(q * 32) << 16);
        uint32_t r[CW];
#pragma unroll
        for (int c0 = 0; c0 < CW; c0 += 32) tmem_ld_32x32(taddr + c0, r + c0);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < CW; j += 4) {
          if (KIND == 1) {
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[j + u] += (float)(int)r[j + u];
          } else {
            const float4 s4 = *reinterpret_cast<const float4*>(srow + j);
            acc[j] = fmaf(__uint_as_float(r[j]), s4.x, acc[j]);
            acc[j + 1] = fmaf(__uint_as_float(r[j + 1]), s4.y, acc[j + 1]);
            acc[j + 2] = fmaf(__uint_as_float(r[j + 2]), s4.z, acc[j + 2]);
            acc[j + 3] = fmaf(__uint_as_float(r[j + 3]), s4.w, acc[j + 3]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pempty[pb]);
      }
      if (!ok) break;
      const int n = k.n0 + row;
      const int cv = k.t_valid - col0;               // live columns of this warp (may be <= 0)
      if (KIND == 1) {
        // per-channel weight scale (this thread's row) times per-token activation scale (the column)
        const float wsn = n < p.N ? p.w_scale[k.ws_row * BM + row] : 0.f;
#pragma unroll
        for (int c0 = 0; c0 < CW; c0 += 32) {
          const float mine = (c0 + lane < cv) ? p.x_scale[k.t_row + col0 + c0 + lane] : 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[c0 + j] *= wsn * __shfl_sync(0xffffffffu, mine, j);
        }
      }
      if (p.cluster_splitk) {
        float* part = reinterpret_cast<float*>(smem);      // ring is idle: this CTA has one work item
#pragma unroll
        for (int c = 0; c < CW; ++c) part[(col0 + c) * BM + row] = acc[c];
      } else if (ROUTED) {
        // every output row goes to the return slot of the rank that sent the token: 32 tokens x 128 rows are
        // turned in shared memory so that a token's 256 bytes leave as sixteen 16-byte stores; the stores
        // are fenced once, before the CTA reports itself done
        const int grp = (warp - 2) >> 2;
        __nv_bfloat16* stg = s_route + grp * (2 * 32 * BM);
        const int seg = row & 15, jt = row >> 4;
#pragma unroll
        for (int c0 = 0; c0 < CW; c0 += 32) {
          if (c0 < cv) {                              // uniform over the four warps of the set
            __nv_bfloat16* st = stg + (route_count & 1) * (32 * BM);
#pragma unroll
            for (int j = 0; j < 32; ++j) st[j * BM + row] = __float2bfloat16(acc[c0 + j]);
            asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory");
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int j = jt + 8 * i;
              if (c0 + j < cv) {
                const int2 rt = __ldg(p.row_route + k.t_row + col0 + c0 + j);
                const uint4 v = *reinterpret_cast<const uint4*>(st + j * BM + seg * 8);
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.peer[rt.x] + p.route_ret_off) +
                                          (size_t)rt.y * p.N + k.n0 + seg * 8) = v;
              }
            }
            ++route_count;
          }
        }
      } else if (PUSH && (p.N & 7) == 0 && k.n0 + BM <= p.N) {
        // pushed partial (every rank receives a copy): turned in shared memory like the routed rows, sixteen
        // 16-byte stores per token and destination instead of 2-byte stores
        const float bias = p.bias != nullptr ? __bfloat162float(p.bias[n]) : 0.f;
        const int grp = (warp - 2) >> 2;
        __nv_bfloat16* stg = s_route + grp * (2 * 32 * BM);
        const int seg = row & 15, jt = row >> 4;
#pragma unroll
        for (int c0 = 0; c0 < CW; c0 += 32) {
          if (c0 < cv) {                              // uniform over the four warps of the set
            __nv_bfloat16* st = stg + (route_count & 1) * (32 * BM);
#pragma unroll
            for (int j = 0; j < 32; ++j) st[j * BM + row] = __float2bfloat16(acc[c0 + j] + bias);
            asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory");
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int j = jt + 8 * i;
              if (c0 + j < cv) {
                const uint4 v = *reinterpret_cast<const uint4*>(st + j * BM + seg * 8);
                for (int d = 0; d < ndst; ++d)
                  *reinterpret_cast<uint4*>(
                      reinterpret_cast<__nv_bfloat16*>(p.peer[d] + p.part_off + (size_t)p.rank * p.part_src_stride) +
                      (size_t)(k.t_row + col0 + c0 + j) * p.N + k.n0 + seg * 8) = v;
              }
            }
            ++route_count;
          }
        }
        {
          // the tile has been pushed: release its flag at every rank
          __threadfence_system();
          asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_WARPS * 32) : "memory");
          const int t = (int)threadIdx.x - 64;
          if (t < p.world) {
            const int tile = raster_tile(k.n0 / BM, k.t_row / BN, p.n_tiles, p.t_tiles);
            st_release_sys(reinterpret_cast<int*>(p.peer[t] + p.tile_flag_off) + (size_t)p.rank * p.max_tiles + tile,
                           epoch);
          }
        }
      } else {
        if (n < p.N) {
          const float bias = p.bias != nullptr ? __bfloat162float(p.bias[n]) : 0.f;
          for (int d = 0; d < ndst; ++d) {
            __nv_bfloat16* yp =
                PUSH ? reinterpret_cast<__nv_bfloat16*>(p.peer[d] + p.part_off + (size_t)p.rank * p.part_src_stride) +
                           (size_t)(k.t_row + col0) * p.N + n
                     : p.Y + (size_t)(k.t_row + col0) * p.ldy + n;
            const size_t ld = PUSH ? (size_t)p.N : (size_t)p.ldy;
#pragma unroll
            for (int c = 0; c < CW; ++c)
              if (c < cv) yp[(size_t)c * ld] = __float2bfloat16(acc[c] + bias);
          }
        }
        if (PUSH) {
          // the tile has been pushed: release its flag at every rank
          __threadfence_system();
          asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_WARPS * 32) : "memory");
          const int t = (int)threadIdx.x - 64;
          if (t < p.world) {
            const int tile = raster_tile(k.n0 / BM, k.t_row / BN, p.n_tiles, p.t_tiles);
            st_release_sys(reinterpret_cast<int*>(p.peer[t] + p.tile_flag_off) + (size_t)p.rank * p.max_tiles + tile,
                           epoch);
          }
        }
      }
    }
  }

  if (p.cluster_splitk) {
    __syncwarp();
    cluster_arrive_release();
    cluster_wait_acquire();
    if (warp >= 2 && !*abort_flag && (int)blockIdx.x < total_work) {
      const Work k = get_work<BN>(blockIdx.x, p, s_prefix);
      const int ew = warp - 2;
      const uint32_t rank = cluster_ctarank();
      const int S = p.splits;
      const int n4 = k.n0 + 4 * lane;
      float b4[4] = {0.f, 0.f, 0.f, 0.f};
      if (p.bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n4 + j < p.N) b4[j] = __bfloat162float(p.bias[n4 + j]);
      }
      const uint32_t part_local = smem_u32(smem);
      for (int c = (int)rank + S * ew; c < k.t_valid; c += C::EPI_WARPS * S) {
        float4 v[8];                     // all partials of the column are requested before the first is used
#pragma unroll
        for (int r2 = 0; r2 < 8; ++r2)
          if (r2 < S) v[r2] = ld_dsmem_v4(mapa_shared(part_local + (uint32_t)((c * BM + 4 * lane) * 4), r2));
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r2 = 0; r2 < 8; ++r2)
          if (r2 < S) { a.x += v[r2].x; a.y += v[r2].y; a.z += v[r2].z; a.w += v[r2].w; }
        const float vals[4] = {a.x, a.y, a.z, a.w};
        for (int d = 0; d < ndst; ++d) {
          __nv_bfloat16* yp =
              PUSH ? reinterpret_cast<__nv_bfloat16*>(p.peer[d] + p.part_off + (size_t)p.rank * p.part_src_stride) +
                         (size_t)(k.t_row + c) * p.N + n4
                   : p.Y + (size_t)(k.t_row + c) * p.ldy + n4;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (n4 + j < p.N) yp[j] = __float2bfloat16(vals[j] + b4[j]);
        }
      }
      if (PUSH) __threadfence_system();
    }
    __syncwarp();
    cluster_arrive_release();
    cluster_wait_acquire();
    if (PUSH && cluster_ctarank() == 0 && warp == 2 && (int)blockIdx.x < total_work && !*abort_flag) {
      // every CTA of the cluster has stored and fenced its columns: release the tile's flag
      const Work k = get_work<BN>(blockIdx.x, p, s_prefix);
      if (lane < p.world) {
        const int tile = raster_tile(k.n0 / BM, k.t_row / BN, p.n_tiles, p.t_tiles);
        st_release_sys(reinterpret_cast<int*>(p.peer[lane] + p.tile_flag_off) + (size_t)p.rank * p.max_tiles + tile,
                       epoch);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
  if (MODE != 0 && threadIdx.x == 64) {
    // the barrier above ordered every thread's stores before this fence (system scope for routed rows)
    if (ROUTED) __threadfence_system();
    else __threadfence();
    const int arrived = atomicAdd(p.cta_done, 1) + 1;
    if (arrived == (int)gridDim.x) {
      *p.cta_done = 0;
      if (ROUTED) {
        // every CTA fenced its routed stores before it arrived: tell all ranks their rows are back
        __threadfence_system();
        const int ep_epoch = *reinterpret_cast<volatile int*>(p.epoch_ptr);
        for (int r = 0; r < p.world; ++r)
          st_release_sys(reinterpret_cast<int*>(p.peer[r] + p.ret_flag_off) + p.rank, ep_epoch);
      } else {
        *p.epoch_ptr = epoch;        // every CTA of this launch has read the old value by now
      }
      __threadfence();
    }
  }
}

// x [T, K] bf16 -> xq [T, K] e4m3 and xs [T, ceil(K/128)] fp32: one warp per (row, 128-column group)
__global__ void quant_act_1x128_kernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_e4m3* __restrict__ xq,
                                       float* __restrict__ xs, int T, int K, int ldx, int groups) {
  pdl_launch_dependents();
  const int warps_per_block = blockDim.x >> 5;
  const long long gw = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (gw >= (long long)T * groups) return;
  const int t = (int)(gw / groups), g = (int)(gw % groups);
  const int c0 = g * 128 + lane * 4;
  float v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = (c0 + j < K) ? __bfloat162float(x[(size_t)t * ldx + c0 + j]) : 0.f;
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = warp_max(amax);
  const float scale = fmaxf(amax, 1e-12f) / 448.f;
  const float inv = 1.f / scale;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (c0 + j < K) xq[(size_t)t * K + c0 + j] = __nv_fp8_e4m3(fminf(fmaxf(v[j] * inv, -448.f), 448.f));
  if (lane == 0) xs[(size_t)t * groups + g] = scale;
}

// Same quantisation over the first *rows_ptr rows (all T when rows_ptr is null) with a grid that does not
// depend on the row count, optionally fused behind SiLU(gate) * up: with SWIGLU the input row holds
// [gate(K) | up(K)] (row stride ldx) and the product, rounded to bf16 as the stand-alone activation
// kernel would, is what gets quantised.  One warp per (row, 128-column group), grid-stride.
template <bool SWIGLU>
__global__ void quant_rows_1x128_kernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_e4m3* __restrict__ xq,
                                        float* __restrict__ xs, int T, int K, int ldx, int groups,
                                        const int* __restrict__ rows_ptr) {
  pdl_launch_dependents();
  pdl_wait();
  const int rows = rows_ptr != nullptr ? min(T, *rows_ptr) : T;
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)rows * groups;
  for (long long gw = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); gw < total;
       gw += (long long)gridDim.x * warps_per_block) {
    const int t = (int)(gw / groups), g = (int)(gw % groups);
    const int c0 = g * 128 + lane * 4;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (c0 + j >= K) { v[j] = 0.f; continue; }
      const float a = __bfloat162float(x[(size_t)t * ldx + c0 + j]);
      if (SWIGLU) {
        const float u = __bfloat162float(x[(size_t)t * ldx + K + c0 + j]);
        v[j] = __bfloat162float(__float2bfloat16(a / (1.f + __expf(-a)) * u));
      } else {
        v[j] = a;
      }
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = warp_max(amax);
    const float scale = fmaxf(amax, 1e-12f) / 448.f;
    const float inv = 1.f / scale;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (c0 + j < K) xq[(size_t)t * K + c0 + j] = __nv_fp8_e4m3(fminf(fmaxf(v[j] * inv, -448.f), 448.f));
    if (lane == 0) xs[(size_t)t * groups + g] = scale;
  }
}

// Vectorised form for K % 8 == 0 and 16-byte aligned rows: a thread owns 8 consecutive elements (one
// 16-byte load, one 8-byte store), 16 threads own a 128-column group, grid-stride over (row, group) pairs.
template <bool SWIGLU>
__global__ void quant_rows_1x128_vec_kernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_e4m3* __restrict__ xq,
                                            float* __restrict__ xs, int T, int K, int ldx, int groups,
                                            const int* __restrict__ rows_ptr) {
  pdl_launch_dependents();
  pdl_wait();
  const int rows = rows_ptr != nullptr ? min(T, *rows_ptr) : T;
  const int sub = threadIdx.x & 15;
  const long long total = (long long)rows * groups;
  const long long stride = (long long)gridDim.x * (blockDim.x >> 4);
  for (long long gi = (long long)blockIdx.x * (blockDim.x >> 4) + (threadIdx.x >> 4); gi < total; gi += stride) {
    const int t = (int)(gi / groups), g = (int)(gi % groups);
    const int c0 = g * 128 + sub * 8;
    float v[8];
    if (c0 < K) {
      const uint4 a = *reinterpret_cast<const uint4*>(x + (size_t)t * ldx + c0);
      const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
      if (SWIGLU) {
        const uint4 u = *reinterpret_cast<const uint4*>(x + (size_t)t * ldx + K + c0);
        const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 af = __bfloat1622float2(ah[j]), uf = __bfloat1622float2(uh[j]);
          v[2 * j] = __bfloat162float(__float2bfloat16(af.x / (1.f + __expf(-af.x)) * uf.x));
          v[2 * j + 1] = __bfloat162float(__float2bfloat16(af.y / (1.f + __expf(-af.y)) * uf.y));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 af = __bfloat1622float2(ah[j]);
          v[2 * j] = af.x;
          v[2 * j + 1] = af.y;
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = fmaxf(amax, 1e-12f) / 448.f;
    const float inv = 1.f / scale;
    if (c0 < K) {
      __align__(8) __nv_fp8_e4m3 o8[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o8[j] = __nv_fp8_e4m3(fminf(fmaxf(v[j] * inv, -448.f), 448.f));
      *reinterpret_cast<uint2*>(xq + (size_t)t * K + c0) = *reinterpret_cast<const uint2*>(o8);
    }
    if (sub == 0) xs[(size_t)t * groups + g] = scale;
  }
}

// x [T, K] bf16 -> xq [T, K] e4m3 with ONE scale per row (amax / 448), written `reps` times into
// xs [T, reps] so that the block-scaled GEMM can consume it as its per-(row, K block) scale: one CTA per row
__global__ void quant_act_rowwise_kernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_e4m3* __restrict__ xq,
                                         float* __restrict__ xs, int K, int ldx, int reps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  const int t = blockIdx.x;
  float amax = 0.f;
  for (int i = threadIdx.x; i < K; i += blockDim.x) amax = fmaxf(amax, fabsf(__bfloat162float(x[(size_t)t * ldx + i])));
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : 0.f;
  amax = warp_max(amax);
  const float scale = fmaxf(amax, 1e-12f) / 448.f;
  const float inv = 1.f / scale;
  for (int i = threadIdx.x; i < K; i += blockDim.x)
    xq[(size_t)t * K + i] =
        __nv_fp8_e4m3(fminf(fmaxf(__bfloat162float(x[(size_t)t * ldx + i]) * inv, -448.f), 448.f));
  for (int i = threadIdx.x; i < reps; i += blockDim.x) xs[(size_t)t * reps + i] = scale;
}

// x [T, K] bf16 -> xq [T, K] int8 and xs [T] fp32 (amax / 127): one CTA per row
__global__ void quant_act_int8_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ xq,
                                      float* __restrict__ xs, int K, int ldx) {
  __shared__ float red[32];
  pdl_launch_dependents();
  const int t = blockIdx.x;
  float amax = 0.f;
  for (int i = threadIdx.x; i < K; i += blockDim.x) amax = fmaxf(amax, fabsf(__bfloat162float(x[(size_t)t * ldx + i])));
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : 0.f;
  amax = warp_max(amax);
  const float scale = fmaxf(amax, 1e-12f) / 127.f;
  const float inv = 1.f / scale;
  for (int i = threadIdx.x; i < K; i += blockDim.x) {
    const float v = rintf(__bfloat162float(x[(size_t)t * ldx + i]) * inv);
    xq[(size_t)t * K + i] = (int8_t)fminf(fmaxf(v, -127.f), 127.f);
  }
  if (threadIdx.x == 0) xs[t] = scale;
}

template <int BN, int KIND, int MODE>
static int launch_mode(const CUtensorMap& tmW, const CUtensorMap& tmX, const Params& p, int grid,
                       cudaStream_t stream) {
  using C = Cfg<BN>;
  static unsigned long long attr_seen = 0;
  B200_CUDA_CHECK(ensure_dynamic_smem(gemm_fp8_block_kernel<BN, KIND, MODE>, C::SMEM, &attr_seen));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(C::NUM_THREADS);
  cfg.dynamicSmemBytes = C::SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (p.cluster_splitk) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = p.splits;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[na].val.programmaticStreamSerializationAllowed = 1;
  ++na;
  cfg.attrs = attr;
  cfg.numAttrs = na;
  B200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_fp8_block_kernel<BN, KIND, MODE>, tmW, tmX, p));
  return 0;
}

template <int BN, int KIND = 0>
static int launch(const CUtensorMap& tmW, const CUtensorMap& tmX, const Params& p, int grid,
                  cudaStream_t stream) {
  if (KIND == 0 && p.row_route != nullptr) return launch_mode<BN, 0, 2>(tmW, tmX, p, grid, stream);
  if (KIND == 0 && p.world > 1) return launch_mode<BN, 0, 1>(tmW, tmX, p, grid, stream);
  return launch_mode<BN, KIND, 0>(tmW, tmX, p, grid, stream);
}

template <int BN>
static int max_clusters(int splits) {
  using C = Cfg<BN>;
  cudaFuncSetAttribute(gemm_fp8_block_kernel<BN, 0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(splits * 64);
  cfg.blockDim = dim3(C::NUM_THREADS);
  cfg.dynamicSmemBytes = C::SMEM;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_fp8_block_kernel<BN, 0, 0>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

static int fit_splits(int want, int tiles, int bn) {
  static int cache[3][9];
  static bool init = false;
  if (!init) { memset(cache, -1, sizeof(cache)); init = true; }
  int s = want > 8 ? 8 : want;
  const int bi = bn == 32 ? 0 : (bn == 64 ? 1 : 2);
  while (s > 1) {
    int& c = cache[bi][s];
    if (c < 0) c = bn == 32 ? max_clusters<32>(s) : (bn == 64 ? max_clusters<64>(s) : max_clusters<128>(s));
    if (c >= tiles) break;
    --s;
  }
  return s;
}

}  // namespace f8
}  // namespace b200

using namespace b200;

extern "C" int b200_quant_act_1x128(const void* x, void* xq, float* xs, int T, int K, int ldx,
                                    cudaStream_t stream) {
  if (T == 0) return 0;
  const int groups = (K + 127) / 128;
  const long long warps = (long long)T * groups;
  const int blocks = (int)((warps + 7) / 8);
  f8::quant_act_1x128_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_fp8_e4m3*)xq, xs, T, K,
                                                         ldx, groups);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// Quantisation of at most T rows, of which the first *rows_ptr are live (device word; null = all T), with
// SiLU(gate) * up in front when swiglu != 0 (x then has 2K columns per row).
extern "C" int b200_quant_rows_1x128(const void* x, void* xq, float* xs, int T, int K, int ldx, const int* rows_ptr,
                                     int swiglu, int num_sms, cudaStream_t stream) {
  if (T == 0) return 0;
  const int groups = (K + 127) / 128;
  const long long warps = (long long)T * groups;
  long long blocks = (warps + 7) / 8;
  if (blocks > (long long)num_sms * 8) blocks = (long long)num_sms * 8;
  if (K % 8 == 0 && ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(xq) & 7) == 0) {
    long long vb = (warps + 15) / 16;                  // 16 groups per 256-thread block
    if (vb > (long long)num_sms * 8) vb = (long long)num_sms * 8;
    if (swiglu)
      f8::quant_rows_1x128_vec_kernel<true><<<(int)vb, 256, 0, stream>>>(
          (const __nv_bfloat16*)x, (__nv_fp8_e4m3*)xq, xs, T, K, ldx, groups, rows_ptr);
    else
      f8::quant_rows_1x128_vec_kernel<false><<<(int)vb, 256, 0, stream>>>(
          (const __nv_bfloat16*)x, (__nv_fp8_e4m3*)xq, xs, T, K, ldx, groups, rows_ptr);
    B200_CUDA_CHECK(cudaGetLastError());
    return 0;
  }
  if (swiglu)
    f8::quant_rows_1x128_kernel<true><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_fp8_e4m3*)xq,
                                                                       xs, T, K, ldx, groups, rows_ptr);
  else
    f8::quant_rows_1x128_kernel<false><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_fp8_e4m3*)xq,
                                                                        xs, T, K, ldx, groups, rows_ptr);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

static int fp8_common(f8::Params& p, const void* Xq, const void* Wq, int rowsW, int rowsX, int bn, int K,
                      CUtensorMap* tmW, CUtensorMap* tmX) {
  if (K % 16) {
    b200_set_last_error("gemm_fp8_block: K must be a multiple of 16", __FILE__, __LINE__);
    return -3;
  }
  int rc = b200_make_tmap_2d(tmW, Wq, 1, (uint64_t)rowsW, (uint64_t)K, (uint64_t)K, f8::BM, f8::BKB);
  if (rc) return rc;
  return b200_make_tmap_2d(tmX, Xq, 1, (uint64_t)rowsX, (uint64_t)K, (uint64_t)K, (uint32_t)bn, f8::BKB);
}

// Y[T,N] bf16 = dequant(Xq, xs) * dequant(Wq, ws)^T (+bias).  Xq [T,K], Wq [N,K] contiguous e4m3;
// xs [T, ceil(K/128)], ws [ceil(N/128), ceil(K/128)] fp32.
extern "C" int b200_gemm_fp8_block(const void* Xq, const float* xs, const void* Wq, const float* ws, void* Y,
                                   const void* bias, int T, int N, int K, int ldy, int* status, int num_sms,
                                   cudaStream_t stream) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  const int bn = T <= 32 ? 32 : (T <= 64 ? 64 : 128);
  f8::Params p;
  memset(&p, 0, sizeof(p));
  p.Y = (__nv_bfloat16*)Y;
  p.bias = (const __nv_bfloat16*)bias;
  p.w_scale = ws;
  p.x_scale = xs;
  p.status = status;
  p.T = T; p.N = N; p.K = K; p.ldy = ldy;
  p.n_tiles = (N + f8::BM - 1) / f8::BM;
  p.t_tiles = (T + bn - 1) / bn;
  p.kb_total = (K + f8::BKB - 1) / f8::BKB;
  p.ws_ld = p.kb_total;
  p.xs_ld = p.kb_total;
  const int tiles = p.n_tiles * p.t_tiles;
  int splits = 1;
  if (tiles * 2 <= num_sms) {
    splits = num_sms / tiles;
    const int by_k = p.kb_total / 4 > 0 ? p.kb_total / 4 : 1;
    if (splits > by_k) splits = by_k;
    if (splits > 1) splits = f8::fit_splits(splits, tiles, bn);
  }
  p.splits = splits;
  p.kb_per_split = (p.kb_total + splits - 1) / splits;
  while (p.splits > 1 && (p.splits - 1) * p.kb_per_split >= p.kb_total) {
    --p.splits;
    p.kb_per_split = (p.kb_total + p.splits - 1) / p.splits;
  }
  p.cluster_splitk = p.splits > 1 ? 1 : 0;
  CUtensorMap tmW, tmX;
  int rc = fp8_common(p, Xq, Wq, N, T, bn, K, &tmW, &tmX);
  if (rc) return rc;
  auto go = [&](const f8::Params& q, int grid) {
    switch (bn) {
      case 32: return f8::launch<32>(tmW, tmX, q, grid, stream);
      case 64: return f8::launch<64>(tmW, tmX, q, grid, stream);
      default: return f8::launch<128>(tmW, tmX, q, grid, stream);
    }
  };
  // A persistent launch over a few waves ends with a ragged wave: 224 tiles on 148 SMs take the time of two
  // full waves.  When the last wave fills at most half of the SMs, its tiles run as a second launch with
  // cluster split-K, so that the whole machine shares them.
  const int tail = tiles % num_sms;
  if (p.splits == 1 && tiles > num_sms && tiles <= 4 * num_sms && tail > 0 && tail * 2 <= num_sms &&
      p.kb_total >= 8) {
    int sp = num_sms / tail;
    const int by_k = p.kb_total / 4;
    if (sp > by_k) sp = by_k;
    if (sp > 1) sp = f8::fit_splits(sp, tail, bn);
    if (sp > 1) {
      f8::Params main = p, rest = p;
      main.launch_tiles = tiles - tail;
      rc = go(main, num_sms);
      if (rc) return rc;
      rest.tile_offset = tiles - tail;
      rest.launch_tiles = tail;
      rest.splits = sp;
      rest.kb_per_split = (p.kb_total + sp - 1) / sp;
      while (rest.splits > 1 && (rest.splits - 1) * rest.kb_per_split >= p.kb_total) {
        --rest.splits;
        rest.kb_per_split = (p.kb_total + rest.splits - 1) / rest.splits;
      }
      rest.cluster_splitk = rest.splits > 1 ? 1 : 0;
      const int total = tail * rest.splits;
      return go(rest, rest.cluster_splitk ? total : (total < num_sms ? total : num_sms));
    }
  }
  const int total = tiles * p.splits;
  return go(p, p.cluster_splitk ? total : (total < num_sms ? total : num_sms));
}

// Row-parallel block-scaled fp8 GEMM whose bf16 partial is pushed to every rank of the tensor-parallel
// group (decode-sized outputs): the partial lands in the receive slab at heap offset part_off that each
// rank keeps per source rank, flags int[world][max_tiles] at tile_flag_off are raised with this
// launch's epoch, and b200_reduce_pushed_rms_norm on every rank sums what it received.  ctrl is the
// control block the bf16 push GEMM uses (epoch, CTA counter).
extern "C" int b200_gemm_fp8_block_push(const void* Xq, const float* xs, const void* Wq, const float* ws, int T, int N,
                                        int K, void* const* peers, int rank, int world,
                                        unsigned long long part_off, unsigned long long part_bytes,
                                        unsigned long long tile_flag_off, int max_tiles, int* ctrl, int* status,
                                        int num_sms, cudaStream_t stream) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 2 || world > 8 || N % 8) {
    b200_set_last_error("gemm_fp8_block_push: 2 <= world <= 8 and N % 8 == 0 required", __FILE__, __LINE__);
    return -3;
  }
  const int bn = T <= 32 ? 32 : (T <= 64 ? 64 : 128);
  f8::Params p;
  memset(&p, 0, sizeof(p));
  p.w_scale = ws;
  p.x_scale = xs;
  p.status = status;
  p.T = T; p.N = N; p.K = K; p.ldy = N;
  p.n_tiles = (N + f8::BM - 1) / f8::BM;
  p.t_tiles = (T + bn - 1) / bn;
  p.kb_total = (K + f8::BKB - 1) / f8::BKB;
  p.ws_ld = p.kb_total;
  p.xs_ld = p.kb_total;
  const int tiles = p.n_tiles * p.t_tiles;
  if (tiles > max_tiles) {
    b200_set_last_error("gemm_fp8_block_push: more tiles than flag slots", __FILE__, __LINE__);
    return -4;
  }
  int splits = 1;
  if (tiles * 2 <= num_sms) {
    splits = num_sms / tiles;
    const int by_k = p.kb_total / 4 > 0 ? p.kb_total / 4 : 1;
    if (splits > by_k) splits = by_k;
    if (splits > 1) splits = f8::fit_splits(splits, tiles, bn);
  }
  p.splits = splits;
  p.kb_per_split = (p.kb_total + splits - 1) / splits;
  while (p.splits > 1 && (p.splits - 1) * p.kb_per_split >= p.kb_total) {
    --p.splits;
    p.kb_per_split = (p.kb_total + p.splits - 1) / p.splits;
  }
  p.cluster_splitk = p.splits > 1 ? 1 : 0;
  p.world = world; p.rank = rank; p.max_tiles = max_tiles;
  for (int i = 0; i < 8; ++i) p.peer[i] = i < world ? (uint8_t*)peers[i] : nullptr;
  p.part_off = part_off;
  p.part_src_stride = ((unsigned long long)T * N * 2ull + 255ull) & ~255ull;
  if (p.part_src_stride * world > part_bytes) {
    b200_set_last_error("gemm_fp8_block_push: receive region too small for this shape", __FILE__, __LINE__);
    return -5;
  }
  p.tile_flag_off = tile_flag_off;
  p.epoch_ptr = ctrl; p.cta_done = ctrl + 1;
  CUtensorMap tmW, tmX;
  int rc = fp8_common(p, Xq, Wq, N, T, bn, K, &tmW, &tmX);
  if (rc) return rc;
  const int total = tiles * p.splits;
  const int grid = p.cluster_splitk ? total : (total < num_sms ? total : num_sms);
  switch (bn) {
    case 32: return f8::launch<32>(tmW, tmX, p, grid, stream);
    case 64: return f8::launch<64>(tmW, tmX, p, grid, stream);
    default: return f8::launch<128>(tmW, tmX, p, grid, stream);
  }
}

// Grouped variant: rows [group_off[e], group_off[e+1]) of Xq use expert e's Wq [N,K] and scale grid
// [ceil(N/128), ceil(K/128)].
extern "C" int b200_grouped_gemm_fp8_block(const void* Xq, const float* xs, const void* Wq, const float* ws,
                                           void* Y, const int* group_off, int num_groups, int R, int N, int K,
                                           int avg_rows_hint, int* status, int num_sms, cudaStream_t stream) {
  if (R <= 0 || N <= 0 || K <= 0 || num_groups <= 0) return 0;
  if (N % f8::BM || num_groups > f8::MAX_GROUPS) {
    b200_set_last_error("grouped_gemm_fp8: N % 128 == 0 and <= 1024 groups required", __FILE__, __LINE__);
    return -3;
  }
  const int bn = avg_rows_hint <= 32 ? 32 : (avg_rows_hint <= 64 ? 64 : 128);
  f8::Params p;
  memset(&p, 0, sizeof(p));
  p.Y = (__nv_bfloat16*)Y;
  p.w_scale = ws;
  p.x_scale = xs;
  p.status = status;
  p.T = R; p.N = N; p.K = K; p.ldy = N;
  p.n_tiles = N / f8::BM;
  p.t_tiles = (R + bn - 1) / bn;
  p.kb_total = (K + f8::BKB - 1) / f8::BKB;
  p.ws_ld = p.kb_total;
  p.xs_ld = p.kb_total;
  p.splits = 1;
  p.kb_per_split = p.kb_total;
  p.group_off = group_off;
  p.num_groups = num_groups;
  p.w_rows_per_group = N;
  p.ws_rows_per_group = N / f8::BM;
  CUtensorMap tmW, tmX;
  int rc = fp8_common(p, Xq, Wq, num_groups * N, R, bn, K, &tmW, &tmX);
  if (rc) return rc;
  switch (bn) {
    case 32: return f8::launch<32>(tmW, tmX, p, num_sms, stream);
    case 64: return f8::launch<64>(tmW, tmX, p, num_sms, stream);
    default: return f8::launch<128>(tmW, tmX, p, num_sms, stream);
  }
}

// Grouped block-scaled fp8 GEMM whose output rows are scattered to the ranks that sent the tokens
// (expert-parallel combine inside the epilogue): same contract as b200_grouped_gemm_bf16_routed.
extern "C" int b200_grouped_gemm_fp8_block_routed(const void* Xq, const float* xs, const void* Wq, const float* ws,
                                                  const int* group_off, int num_groups, int R, int N, int K,
                                                  int avg_rows_hint, void* const* peers, int rank, int world,
                                                  const void* route, unsigned long long ret_off,
                                                  unsigned long long ret_flag_off, int* ctrl, int* status,
                                                  int num_sms, cudaStream_t stream) {
  if (R <= 0 || N <= 0 || K <= 0 || num_groups <= 0) return 0;
  if (N % f8::BM || num_groups > f8::MAX_GROUPS || world < 2 || world > 8) {
    b200_set_last_error("grouped_gemm_fp8_routed: N % 128 == 0, <= 1024 groups, 2 <= world <= 8 required",
                        __FILE__, __LINE__);
    return -3;
  }
  const int bn = avg_rows_hint <= 32 ? 32 : (avg_rows_hint <= 64 ? 64 : 128);
  f8::Params p;
  memset(&p, 0, sizeof(p));
  p.w_scale = ws;
  p.x_scale = xs;
  p.status = status;
  p.T = R; p.N = N; p.K = K; p.ldy = N;
  p.n_tiles = N / f8::BM;
  p.t_tiles = (R + bn - 1) / bn;
  p.kb_total = (K + f8::BKB - 1) / f8::BKB;
  p.ws_ld = p.kb_total;
  p.xs_ld = p.kb_total;
  p.splits = 1;
  p.kb_per_split = p.kb_total;
  p.group_off = group_off;
  p.num_groups = num_groups;
  p.w_rows_per_group = N;
  p.ws_rows_per_group = N / f8::BM;
  p.world = world; p.rank = rank;
  for (int i = 0; i < 8; ++i) p.peer[i] = i < world ? (uint8_t*)peers[i] : nullptr;
  p.row_route = reinterpret_cast<const int2*>(route);
  p.route_ret_off = ret_off;
  p.ret_flag_off = ret_flag_off;
  p.epoch_ptr = ctrl; p.cta_done = ctrl + 1;
  CUtensorMap tmW, tmX;
  int rc = fp8_common(p, Xq, Wq, num_groups * N, R, bn, K, &tmW, &tmX);
  if (rc) return rc;
  switch (bn) {
    case 32: return f8::launch<32>(tmW, tmX, p, num_sms, stream);
    case 64: return f8::launch<64>(tmW, tmX, p, num_sms, stream);
    default: return f8::launch<128>(tmW, tmX, p, num_sms, stream);
  }
}

extern "C" int b200_quant_act_rowwise(const void* x, void* xq, float* xs, int T, int K, int ldx, int reps,
                                      cudaStream_t stream) {
  if (T == 0) return 0;
  f8::quant_act_rowwise_kernel<<<T, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_fp8_e4m3*)xq, xs, K, ldx, reps);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_quant_act_int8(const void* x, void* xq, float* xs, int T, int K, int ldx, cudaStream_t stream) {
  if (T == 0) return 0;
  f8::quant_act_int8_kernel<<<T, 256, 0, stream>>>((const __nv_bfloat16*)x, (int8_t*)xq, xs, K, ldx);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// Y[T,N] bf16 = (Xq * Wq^T) * xs[t] * ws[n] (+bias): int8 operands [T,K] / [N,K] contiguous, K % 16 == 0.
extern "C" int b200_gemm_int8(const void* Xq, const float* xs, const void* Wq, const float* ws, void* Y,
                              const void* bias, int T, int N, int K, int ldy, int* status, int num_sms,
                              cudaStream_t stream) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  const int bn = T <= 32 ? 32 : (T <= 64 ? 64 : 128);
  f8::Params p;
  memset(&p, 0, sizeof(p));
  p.Y = (__nv_bfloat16*)Y;
  p.bias = (const __nv_bfloat16*)bias;
  p.w_scale = ws;
  p.x_scale = xs;
  p.status = status;
  p.T = T; p.N = N; p.K = K; p.ldy = ldy;
  p.n_tiles = (N + f8::BM - 1) / f8::BM;
  p.t_tiles = (T + bn - 1) / bn;
  p.kb_total = (K + f8::BKB - 1) / f8::BKB;
  const int tiles = p.n_tiles * p.t_tiles;
  int splits = 1;
  if (tiles * 2 <= num_sms) {
    splits = num_sms / tiles;
    const int by_k = p.kb_total / 4 > 0 ? p.kb_total / 4 : 1;
    if (splits > by_k) splits = by_k;
    if (splits > 1) splits = f8::fit_splits(splits, tiles, bn);
  }
  p.splits = splits;
  p.kb_per_split = (p.kb_total + splits - 1) / splits;
  while (p.splits > 1 && (p.splits - 1) * p.kb_per_split >= p.kb_total) {
    --p.splits;
    p.kb_per_split = (p.kb_total + p.splits - 1) / p.splits;
  }
  p.cluster_splitk = p.splits > 1 ? 1 : 0;
  CUtensorMap tmW, tmX;
  int rc = fp8_common(p, Xq, Wq, N, T, bn, K, &tmW, &tmX);
  if (rc) return rc;
  const int total = tiles * p.splits;
  const int grid = p.cluster_splitk ? total : (total < num_sms ? total : num_sms);
  switch (bn) {
    case 32: return f8::launch<32, 1>(tmW, tmX, p, grid, stream);
    case 64: return f8::launch<64, 1>(tmW, tmX, p, grid, stream);
    default: return f8::launch<128, 1>(tmW, tmX, p, grid, stream);
  }
}
