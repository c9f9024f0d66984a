// bf16 GEMM  Y[T,N] = X[T,K] * W[N,K]^T (+bias)  on tcgen05 tensor cores.
//
// Orientation: the weight is the 128-row UMMA "A" operand and the activations are
// the "B" operand, so the accumulator in TMEM is D[n (128 lanes), t (BN columns)].
// A decode step with 16..256 tokens therefore still fills the 128-row MMA with
// weight rows and only narrows N, and one kernel covers decode (BN = 32/64/128)
// and prefill (BN = 256).  Both operands are K-major in global memory
// (nn.Linear weight layout, row-major activations) and are staged by TMA with the
// 128-byte swizzle that the UMMA shared-memory descriptor expects.
//
// CTA = 6 warps, persistent over (tile, split) work items:
//   warp 0   TMA producer (one elected lane), ring of STAGES {A 128x64, B BNx64}
//   warp 1   TMEM allocation + tcgen05.mma issue (one lane), commits free stages
//   warps 2-5 epilogue: tcgen05.ld the accumulator (double buffered in TMEM so the
//            epilogue of tile i overlaps the main loop of tile i+1), bias, bf16 store
// Split-K (decode shapes with few output tiles): each split writes an fp32 partial
// to scratch; the CTA that arrives last on the tile's counter sums the partials in
// split order (deterministic), writes bf16 and re-arms the counter.
//
// No reference counterpart as CUDA: the reference's dense matmuls are XLA dots and
// Pallas quantized_matmul kernels (reference: src/vllm_torchtpu/kernels/quantized_matmul/).
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "gemm_tcgen05.h"

namespace b200 {

constexpr int BM = 128;          // weight rows per tile (UMMA M)
constexpr int BK = 64;           // bf16 elements per 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int GROUP_N = 16;      // raster group: 16 weight tiles share activations in L2

constexpr int MAX_GROUPS = 1024;  // experts per launch in grouped mode

// NACC = 2: two weight tiles (gate rows, up rows) share one activation tile and the epilogue
// writes silu(gate) * up, so a SwiGLU projection needs no separate activation kernel.
template <int BN, int NACC>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = NACC * A_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = 196608 / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int BAR_BYTES = 256;
  static constexpr int PREFIX_BYTES = (MAX_GROUPS + 1) * 4;
  // fused launches stage [32 tokens][128 rows] bf16 chunks of a partial tile here (two buffers) and
  // push each to its owner with one bulk copy
  static constexpr int PUSH_CHUNK_BYTES = 32 * BM * 2;
  static constexpr int PUSH_OFF = (STAGES * STAGE_BYTES + BAR_BYTES + PREFIX_BYTES + 127) / 128 * 128;
  static constexpr int SMEM = PUSH_OFF + 2 * PUSH_CHUNK_BYTES + 1024;                 // + alignment slack
  static_assert(SMEM <= 232448, "shared memory budget");
  static constexpr int TMEM_COLS = 2 * NACC * BN < 32 ? 32 : 2 * NACC * BN;
  static_assert(TMEM_COLS <= 512, "accumulators exceed TMEM");
};

struct GemmParams {
  __nv_bfloat16* Y;
  const __nv_bfloat16* bias;
  float* ws;
  int* counters;
  int* status;
  int T, N, K, ldy;
  int n_tiles, t_tiles, splits, kb_total, kb_per_split;
  int w_evict_first;
  // ---- SwiGLU pairs and grouped (per-expert) mode
  int cluster_splitk;                    // splits of a tile form a thread-block cluster; reduce over DSMEM
  int up_row_off;                        // NACC == 2: weight-row distance from a gate tile to its up tile
  const int* group_off;                  // grouped: int[num_groups + 1] row offsets into X / Y (null = dense)
  int num_groups, w_rows_per_group;      // grouped: weight rows of one expert
  // ---- fused cross-rank reduction over NVLink peer memory (world == 1: plain GEMM)
  int world, rank, ar_mode;              // 0: all-reduce via tile owners, 1: reduce-scatter, 2: one-shot
                                         // all-reduce, 3: push to every rank, the consumer kernel sums
  uint8_t* peer[8];                      // heap base of every rank (own heap at [rank])
  unsigned long long part_off, out_off;  // heap offsets: receive slabs (one per source rank), output [T,N] bf16
  unsigned long long part_src_stride;    // bytes between the receive slabs of two source ranks
  unsigned long long tile_flag_off;      // heap offset: int[world][max_tiles], written by producers at the owner
  unsigned long long done_flag_off;      // heap offset: int[max_tiles], written by the owner at every reader
  int max_tiles;
  // ---- routed rows (ar_mode 4, expert-parallel combine): output row r goes to the return slot
  // row_route[r] = (rank, slot) in that rank's heap at route_ret_off; done_flag_off then names the
  // int[world] "returned" flags that the last CTA raises at every rank
  const int2* row_route;
  unsigned long long route_ret_off;
  // ---- all-gather of the activations fused in front of the GEMM (ar_mode 5): the activation rows are
  // sharded over the ranks; the extra warps of every CTA push this rank's shard (ag_src, ag_rows
  // rows of ag_ld elements) into the full matrix [world * ag_rows, K] that every rank keeps at heap
  // offset ag_dst_off (the TMA operand), raising flags[src][block * ag_parts + part] per BN-row
  // block and K slice; the TMA producer waits for the flags of a block before loading from it
  const __nv_bfloat16* ag_src;
  unsigned long long ag_dst_off;
  int ag_rows, ag_ld, ag_tps, ag_parts;  // ag_tps: BN-row blocks per shard
  // back-pressure: a rank finishes reading its gather buffer `ag_flip` when its launch ends and then
  // writes the launch's epoch to ag_done[ag_flip][rank] at every rank; nobody pushes into a buffer
  // before its owner has finished the previous launch that used it (epoch kept in ctrl[2 + flip])
  unsigned long long ag_done_off;
  int ag_flip;
  unsigned long long* dbg;               // optional: per-CTA phase timestamps (ns), 16 slots per CTA
  int* epoch_ptr;                        // local: epoch of the last completed fused launch
  int* cta_done;                         // local: CTA exit counter
  unsigned int spin_limit;
};

constexpr int NUM_THREADS_FUSED = NUM_THREADS + 128;   // + 4 reducer warps

__device__ __forceinline__ void decode_tile(int tile, const GemmParams& p, int& n_tile, int& t_tile) {
  const int per_group = GROUP_N * p.t_tiles;
  const int g = tile / per_group;
  const int first_n = g * GROUP_N;
  const int gsize = min(GROUP_N, p.n_tiles - first_n);
  const int r = tile - g * per_group;
  n_tile = first_n + r % gsize;
  t_tile = r / gsize;
}

__device__ __forceinline__ void decode_work(int w, const GemmParams& p, int& n_tile, int& t_tile,
                                            int& split, int& tile) {
  tile = w / p.splits;
  split = w - tile * p.splits;
  const int per_group = GROUP_N * p.t_tiles;
  const int g = tile / per_group;
  const int first_n = g * GROUP_N;
  const int gsize = min(GROUP_N, p.n_tiles - first_n);
  const int r = tile - g * per_group;
  n_tile = first_n + r % gsize;
  t_tile = r / gsize;
}

struct Work {
  int w_row, t_row, t_valid, n0, kb0, kb1, tile, split;
};

// dense: tiles rastered in groups of GROUP_N weight tiles; grouped: work = (token tile of an expert, n tile)
template <int BN, int MODE = 2>
__device__ __forceinline__ Work get_work(int w, const GemmParams& p, const int* s_prefix) {
  constexpr bool FULL = MODE == 2;
  Work k;
  if (!FULL || p.group_off == nullptr) {
    int n_tile, t_tile;
    decode_work(w, p, n_tile, t_tile, k.split, k.tile);
    if (FULL && p.ar_mode == 5) {  // start with the token blocks of this rank's own shard
      t_tile += p.rank * p.ag_tps;
      if (t_tile >= p.t_tiles) t_tile -= p.t_tiles;
    }
    k.w_row = n_tile * BM;
    k.n0 = n_tile * BM;
    k.t_row = t_tile * BN;
    k.t_valid = min(BN, p.T - k.t_row);
    k.kb0 = k.split * p.kb_per_split;
    k.kb1 = min(p.kb_total, k.kb0 + p.kb_per_split);
  } else {
    const int tt = w / p.n_tiles, n_tile = w - tt * p.n_tiles;
    int lo = 0, hi = p.num_groups;                       // largest e with prefix[e] <= tt
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
    k.kb0 = 0;
    k.kb1 = p.kb_total;
    k.tile = w;
    k.split = 0;
  }
  return k;
}

// Where an output tile goes.  Element (column c, row) of the tile is base[c * cs + row].
//   plain GEMM                Y[t, n]
//   fused, via tile owners    the owner (tile % world) keeps, per source rank, a slab of its owned
//                             tiles, each [BN][BM] bf16; partials are PUSHED there over NVLink
//   fused, one-shot           every rank keeps a [T, N] matrix per source rank; each rank pushes its
//                             partial to all of them and sums what it received
struct TileDst {
  __nv_bfloat16* base;
  int cs;
};
template <int BN, int MODE = 2>
__device__ __forceinline__ TileDst tile_dst(const GemmParams& p, const Work& wk, int d) {
  constexpr bool FULL = MODE == 2;
  TileDst t;
  if (MODE == 1) {
    t.base = reinterpret_cast<__nv_bfloat16*>(p.peer[d] + p.part_off + (size_t)p.rank * p.part_src_stride) +
             (size_t)wk.t_row * p.N + wk.n0;
    t.cs = p.N;
  } else if (!FULL || p.world == 1 || p.ar_mode == 5) {
    t.base = p.Y + (size_t)wk.t_row * p.ldy + wk.n0;
    t.cs = p.ldy;
  } else if (p.ar_mode >= 2) {
    t.base = reinterpret_cast<__nv_bfloat16*>(p.peer[d] + p.part_off + (size_t)p.rank * p.part_src_stride) +
             (size_t)wk.t_row * p.N + wk.n0;
    t.cs = p.N;
  } else {
    t.base = reinterpret_cast<__nv_bfloat16*>(p.peer[wk.tile % p.world] + p.part_off +
                                              (size_t)p.rank * p.part_src_stride) +
             (size_t)(wk.tile / p.world) * (BM * BN);
    t.cs = BM;
  }
  return t;
}

// Tell the consumers of this rank's partial of `tile` that it has landed (t = index of the calling
// thread inside its group; the group has fenced system-wide and synchronised before the call).
template <int MODE = 2>
__device__ __forceinline__ void publish_tile(const GemmParams& p, int tile, int epoch, int t) {
  if (MODE == 1 || p.ar_mode >= 2) {
    if (t < p.world)
      st_release_sys(reinterpret_cast<int*>(p.peer[t] + p.tile_flag_off) + (size_t)p.rank * p.max_tiles + tile,
                     epoch);
  } else if (t == 0) {
    st_release_sys(reinterpret_cast<int*>(p.peer[tile % p.world] + p.tile_flag_off) +
                       (size_t)p.rank * p.max_tiles + tile, epoch);
  }
}

// Sum `world` bf16 vectors (8 elements each) that live `stride` bytes apart.
__device__ __forceinline__ uint4 sum_slabs(const uint8_t* src, size_t stride, int world) {
  uint4 raw[8];
#pragma unroll
  for (int r = 0; r < 8; ++r)
    if (r < world) raw[r] = ld_relaxed_sys_v4(src + (size_t)r * stride);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    if (r < world) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[r]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
  }
  uint4 o;
  __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
  return o;
}

// Four vectors of a [rows][BM] bf16 slab per thread (idx, idx + 128, ...), summed over `world` slabs;
// the loads of one source rank for all four are in flight together.
__device__ __forceinline__ void sum_slabs4(const uint8_t* slab, size_t stride, int world, int idx0, int total,
                                           int n_vecs, uint4 (&out)[4]) {
  float acc[4][8];
#pragma unroll
  for (int u = 0; u < 4; ++u)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
  for (int r = 0; r < world; ++r) {
    uint4 raw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int idx = idx0 + u * 128;
      raw[u] = make_uint4(0u, 0u, 0u, 0u);
      if (idx < total && (idx % (BM / 8)) < n_vecs)
        raw[u] = ld_relaxed_sys_v4(slab + (size_t)r * stride + (size_t)idx * 16);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[u][2 * j] += f.x;
        acc[u][2 * j + 1] += f.y;
      }
    }
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&out[u]);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[u][2 * j], acc[u][2 * j + 1]);
  }
}

// Split-K reduction over distributed shared memory, the share of cluster CTA `rank`, warp `q`:
// columns c = rank + S*q + 4*S*i of the fp32 partials [column][row] that every CTA of the cluster
// keeps at shared offset part_local are summed over the S CTAs in rank order and stored as bf16.
template <int BN, int SMAX, int MODE, int NACC = 1>
__device__ __forceinline__ void cluster_reduce_cols(const GemmParams& p, const Work& wk, uint32_t part_local,
                                                    int rank, int q, int lane, int ndst, const float (&b4)[4]) {
  constexpr int CPC = 16 / (SMAX * NACC) > 0 ? 16 / (SMAX * NACC) : 1;   // whole columns per batch of loads
  const int S = p.splits;
  const int n4 = wk.n0 + 4 * lane;
  for (int i0 = 0; rank + S * q + 4 * S * i0 < wk.t_valid; i0 += CPC) {
    float4 v[CPC][SMAX];
    float4 vu[NACC == 2 ? CPC : 1][NACC == 2 ? SMAX : 1];     // up-projection partials (SwiGLU)
#pragma unroll
    for (int ci = 0; ci < CPC; ++ci) {
      const int c = rank + S * q + 4 * S * (i0 + ci);
#pragma unroll
      for (int r2 = 0; r2 < SMAX; ++r2)
        if (r2 < S && c < wk.t_valid) {
          v[ci][r2] = ld_dsmem_v4(mapa_shared(part_local + (uint32_t)((c * BM + 4 * lane) * 4), r2));
          if (NACC == 2)
            vu[ci][r2] = ld_dsmem_v4(mapa_shared(part_local + (uint32_t)(((BN + c) * BM + 4 * lane) * 4), r2));
        }
    }
#pragma unroll
    for (int ci = 0; ci < CPC; ++ci) {
      const int c = rank + S * q + 4 * S * (i0 + ci);
      if (c < wk.t_valid) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r2 = 0; r2 < SMAX; ++r2)
          if (r2 < S) { a.x += v[ci][r2].x; a.y += v[ci][r2].y; a.z += v[ci][r2].z; a.w += v[ci][r2].w; }
        if (NACC == 2) {
          float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int r2 = 0; r2 < SMAX; ++r2)
            if (r2 < S) { u.x += vu[ci][r2].x; u.y += vu[ci][r2].y; u.z += vu[ci][r2].z; u.w += vu[ci][r2].w; }
          a.x = a.x / (1.f + __expf(-a.x)) * u.x;
          a.y = a.y / (1.f + __expf(-a.y)) * u.y;
          a.z = a.z / (1.f + __expf(-a.z)) * u.z;
          a.w = a.w / (1.f + __expf(-a.w)) * u.w;
        }
        for (int d = 0; d < ndst; ++d) {
          const TileDst td = tile_dst<BN, MODE>(p, wk, d);
          __nv_bfloat16* yp = td.base + (size_t)c * td.cs + 4 * lane;
          const bool vec_ok = (n4 + 3 < p.N) && ((td.cs & 3) == 0) &&
                              ((reinterpret_cast<uintptr_t>(td.base) & 7) == 0);
          if (vec_ok) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(a.x + b4[0], a.y + b4[1]);
            __nv_bfloat162 hi = __floats2bfloat162_rn(a.z + b4[2], a.w + b4[3]);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(yp) = pk;
          } else {
            const float vals[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (n4 + j < p.N) yp[j] = __float2bfloat16(vals[j] + b4[j]);
          }
        }
      }
    }
  }
}

// Phase timestamps are compiled in only with -DB200_GEMM_TIMESTAMPS (they lengthen the hot path).
__device__ __forceinline__ void dbg_stamp(const GemmParams& p, int slot) {
#ifdef B200_GEMM_TIMESTAMPS
  if (p.dbg != nullptr) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.dbg[(size_t)blockIdx.x * 16 + slot] = t;
  }
#else
  (void)p; (void)slot;
#endif
}

// MODE 0 is the compact instantiation for the common single-rank dense case (no grouped mode, no
// cross-rank roles, no global-scratch split-K): the cold paths it leaves out cost instruction-cache
// misses in the short decode GEMMs even when they are never taken.
// MODE 1 is the equally compact instantiation of the decode push plane (ar_mode 3): a dense GEMM whose
// output rows go to every rank's receive slab, flags raised per tile, nothing else.
template <int BN, int NACC, int MODE>
__global__ void __launch_bounds__(MODE == 2 ? NUM_THREADS_FUSED : NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                 const GemmParams p) {
  using Cfg = GemmCfg<BN, NACC>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int ACC_COLS = NACC * BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;
  uint64_t* tempty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);
  volatile int* red_ok = reinterpret_cast<volatile int*>(tmem_slot + 3);
  int* s_prefix = reinterpret_cast<int*>(smem + STAGES * Cfg::STAGE_BYTES + Cfg::BAR_BYTES);
  constexpr bool FULL = MODE == 2;
  constexpr bool PUSH = MODE == 1;
  const bool fused = PUSH || (FULL && p.world > 1);
  __nv_bfloat16* const dst_base = p.Y;       // SwiGLU and grouped launches (never fused)
  const bool push_out = PUSH || (fused && p.ar_mode <= 3);   // the epilogue feeds a cross-rank reduction
  const int ndst = PUSH ? p.world : ((push_out && p.ar_mode >= 2) ? p.world : 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) dbg_stamp(p, 0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], 4);
    mbar_init(&tempty[1], 4);
    *abort_flag = 0;
    *last_flag = 0;
    *red_ok = 1;
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  // Programmatic dependent launch: this grid may start while the previous kernel of the stream is
  // still running.  Everything above touched only shared memory, TMEM and kernel parameters.
  // Weights do not depend on the previous kernel, so in dense mode the producer prefetches weight
  // tiles before it waits; every other thread waits here.  Grouped mode reads the expert offsets
  // the previous kernel wrote, so all of it waits first.
  const bool dense = !FULL || p.group_off == nullptr;
  pdl_launch_dependents();
  if (!(dense && warp == 0)) pdl_wait();
  // The epoch is bumped by the last CTA of a fused launch to exit, so it must be read after the wait
  // above (the previous launch may be a fused one that is still running) and is read by every thread
  // before any CTA of this launch can bump it.  Warp 0 never uses it.
  const int epoch = (fused && warp != 0) ? (*reinterpret_cast<volatile int*>(p.epoch_ptr) + 1) : 0;
  if (FULL && p.group_off != nullptr) {
    // token tiles per expert -> exclusive prefix (serial scan: at most MAX_GROUPS short steps)
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
  const int total_work = (FULL && p.group_off != nullptr) ? s_prefix[p.num_groups] * p.n_tiles
                                                : p.n_tiles * p.t_tiles * p.splits;
  if (threadIdx.x == 0) dbg_stamp(p, 1);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      uint32_t armed = 0;       // bit s: stage s has a load whose completion nobody has consumed yet
      bool ok = true;
      int npre = 0;             // weight tiles of the first work item already in flight (dense mode)
      if (dense && (int)blockIdx.x < total_work) {
        const Work k0 = get_work<BN, MODE>(blockIdx.x, p, s_prefix);
        npre = min(STAGES, k0.kb1 - k0.kb0);
        for (int i = 0; i < npre; ++i) {
          uint8_t* a = smem + i * Cfg::STAGE_BYTES;
          mbar_expect_tx(&full[i], Cfg::STAGE_BYTES);
          tma_load_2d_hint(a, &tmW, &full[i], (k0.kb0 + i) * BK, k0.w_row,
                           p.w_evict_first ? L2_EVICT_FIRST : L2_EVICT_NORMAL);
          if (NACC == 2)
            tma_load_2d_hint(a + Cfg::A_BYTES, &tmW, &full[i], (k0.kb0 + i) * BK, k0.w_row + p.up_row_off,
                             p.w_evict_first ? L2_EVICT_FIRST : L2_EVICT_NORMAL);
        }
      }
      if (dense) pdl_wait();
      const int ag_epoch = (FULL && p.ar_mode == 5) ? *reinterpret_cast<volatile int*>(p.epoch_ptr) + 1 : 0;
      uint32_t ag_seen[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};   // blocks known to have arrived, per source
      int issued = 0;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const Work k = get_work<BN, MODE>(w, p, s_prefix);
        if (FULL && p.ar_mode == 5) {
          const int blk = k.t_row / BN, src = blk / p.ag_tps, j = blk - src * p.ag_tps;
          if (!((ag_seen[src] >> j) & 1u)) {
            const int* f = reinterpret_cast<const int*>(p.peer[p.rank] + p.tile_flag_off) +
                           (size_t)src * p.max_tiles + j * p.ag_parts;
            for (int part = 0; part < p.ag_parts && ok; ++part)
              if (!wait_flag_ge(f + part, ag_epoch, p.status, p.spin_limit)) { *abort_flag = 1; ok = false; }
            if (!ok) break;
            // the rows were written by other GPUs and are read by the async proxy (TMA) from here on
            asm volatile("fence.proxy.async;" ::: "memory");
            ag_seen[src] |= 1u << j;
          }
        }
        for (int kb = k.kb0; kb < k.kb1; ++kb, ++issued) {
          uint8_t* a = smem + s * Cfg::STAGE_BYTES;
          if (issued < npre) {
            // barrier already armed and the weight tile already requested: add the activation tile
            tma_load_2d(a + NACC * Cfg::A_BYTES, &tmX, &full[s], kb * BK, k.t_row);
            armed |= 1u << s;
            if (++s == STAGES) { s = 0; ph ^= 1; }
            continue;
          }
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(&full[s], Cfg::STAGE_BYTES);
          if (p.w_evict_first) {
            tma_load_2d_hint(a, &tmW, &full[s], kb * BK, k.w_row, L2_EVICT_FIRST);
            if (NACC == 2)
              tma_load_2d_hint(a + Cfg::A_BYTES, &tmW, &full[s], kb * BK, k.w_row + p.up_row_off, L2_EVICT_FIRST);
          } else {
            tma_load_2d(a, &tmW, &full[s], kb * BK, k.w_row);
            if (NACC == 2) tma_load_2d(a + Cfg::A_BYTES, &tmW, &full[s], kb * BK, k.w_row + p.up_row_off);
          }
          tma_load_2d(a + NACC * Cfg::A_BYTES, &tmX, &full[s], kb * BK, k.t_row);
          armed |= 1u << s;
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (*abort_flag) {
        // give this CTA's bulk copies in flight a bounded time to land before the CTA exits
        for (int it = 0; it < 20000; ++it) __nanosleep(100);
      }
      (void)armed;
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
      int s = 0;
      uint32_t ph = 0;
      int iter = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++iter) {
        const Work wk = get_work<BN, MODE>(w, p, s_prefix);
        const int kb0 = wk.kb0, kb1 = wk.kb1;
        const int acc = iter & 1;
        const uint32_t acc_ph = (iter >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[s], ph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          if (iter == 0 && kb == kb0) dbg_stamp(p, 2);
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint64_t adesc = umma_desc_k_sw128(a_addr);
          const uint64_t a2desc = umma_desc_k_sw128(a_addr + Cfg::A_BYTES);
          const uint64_t bdesc = umma_desc_k_sw128(a_addr + NACC * Cfg::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // +32 bytes per K step inside the 128-byte swizzle atom (address field is >>4)
            umma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            if (NACC == 2)
              umma_f16(d_tmem + BN, a2desc + 2 * k, bdesc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);      // stage reusable once these MMAs have read it
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) umma_commit(&tfull[acc]);
        dbg_stamp(p, 3);
      }
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;                       // TMEM lane quarter this warp may access
    const int row = q * 32 + lane;                // 0..127 inside the tile
    int iter = 0;
    uint32_t push_count = 0;                      // bulk copies issued so far (selects the staging buffer)
    for (int w = blockIdx.x; w < total_work; w += gridDim.x, ++iter) {
      const Work wk = get_work<BN, MODE>(w, p, s_prefix);
      const int tile = wk.tile, split = wk.split;
      const int acc = iter & 1;
      const uint32_t acc_ph = (iter >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_ph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) break;
      if (threadIdx.x == 64) dbg_stamp(p, 4);
      tc_fence_after();
      const int n = wk.n0 + row;
      const int t0 = wk.t_row;
      const int t_valid = wk.t_valid;
      const uint32_t taddr = tmem_base + acc * ACC_COLS + ((uint32_t)(q * 32) << 16);
      if (NACC == 2 && p.splits == 1) {
        // SwiGLU: accumulator 0 holds the gate tile, accumulator 1 the up tile of the same columns
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (c0 >= t_valid) break;               // warp-uniform
          uint32_t g[32], u[32];
          tmem_ld_32x32(taddr + c0, g);
          tmem_ld_32x32(taddr + BN + c0, u);
          tmem_ld_wait();
          if (n < p.N) {
            __nv_bfloat16* yp = dst_base + (size_t)(t0 + c0) * p.ldy + n;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (c0 + j < t_valid) {
                const float gv = __uint_as_float(g[j]), uv = __uint_as_float(u[j]);
                yp[(size_t)j * p.ldy] = __float2bfloat16(gv / (1.f + __expf(-gv)) * uv);
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
      } else if (FULL && p.row_route != nullptr) {
        // expert-parallel combine: every output row is stored into the return slot of the rank that
        // sent the token (a peer's heap or this rank's own).  32 tokens x 128 columns are turned in shared
        // memory so that a token's 256 bytes leave as sixteen 16-byte stores (NVLink packets of 2-byte
        // stores were the bottleneck); the stores are fenced once, before the CTA reports itself done.
        __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(smem + Cfg::PUSH_OFF);
        const int seg = row & 15, jt = row >> 4;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (c0 >= t_valid) break;               // uniform over the four epilogue warps
          uint32_t r[32];
          tmem_ld_32x32(taddr + c0, r);
          tmem_ld_wait();
          __nv_bfloat16* st = stg + (push_count & 1) * (32 * BM);
#pragma unroll
          for (int j = 0; j < 32; ++j) st[j * BM + row] = __float2bfloat16(__uint_as_float(r[j]));
          asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int j = jt + 8 * i;
            if (c0 + j < t_valid) {
              const int2 rt = __ldg(p.row_route + t0 + c0 + j);
              const uint4 v = *reinterpret_cast<const uint4*>(st + j * BM + seg * 8);
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.peer[rt.x] + p.route_ret_off) +
                                        (size_t)rt.y * p.N + wk.n0 + seg * 8) = v;
            }
          }
          ++push_count;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
      } else if (FULL && p.splits == 1 && fused && p.ar_mode < 2) {
        // partial tile -> the owner's slab [BN][BM] bf16, 32 columns (8 KB) per bulk copy
        uint8_t* slab = reinterpret_cast<uint8_t*>(tile_dst<BN, MODE>(p, wk, 0).base);
        __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(smem + Cfg::PUSH_OFF);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (c0 >= t_valid) break;               // uniform over the four epilogue warps
          uint32_t r[32];
          tmem_ld_32x32(taddr + c0, r);
          tmem_ld_wait();
          __nv_bfloat16* st = stg + (push_count & 1) * (32 * BM);
          // the copy that last read this buffer was issued two chunks ago
          if (threadIdx.x == 64) bulk_wait_group_read<1>();
          asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 32; ++j) st[j * BM + row] = __float2bfloat16(__uint_as_float(r[j]));
          fence_proxy_async_smem();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (threadIdx.x == 64) {
            bulk_store_s2g(slab + (size_t)c0 * BM * sizeof(__nv_bfloat16), st, Cfg::PUSH_CHUNK_BYTES);
            bulk_commit_group();
          }
          ++push_count;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
        if (threadIdx.x == 64) {
          bulk_wait_group<0>();                   // every chunk of this tile has been written
          __threadfence_system();
          publish_tile<MODE>(p, tile, epoch, 0);
        }
      } else if (p.splits == 1) {
        const float bias = (p.bias != nullptr && n < p.N) ? __bfloat162float(p.bias[n]) : 0.f;
        // pushed partials (every rank receives a copy): 32 tokens x 128 columns are turned in shared memory so
        // that a token's 256 bytes leave as sixteen 16-byte stores per destination instead of 2-byte stores
        const bool vec_push = push_out && (p.N & 7) == 0 && wk.n0 + BM <= p.N;
        if (vec_push) {
          __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(smem + Cfg::PUSH_OFF);
          const int seg = row & 15, jt = row >> 4;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            if (c0 >= t_valid) break;             // uniform over the four epilogue warps
            uint32_t r[32];
            tmem_ld_32x32(taddr + c0, r);
            tmem_ld_wait();
            __nv_bfloat16* st = stg + (push_count & 1) * (32 * BM);
#pragma unroll
            for (int j = 0; j < 32; ++j) st[j * BM + row] = __float2bfloat16(__uint_as_float(r[j]) + bias);
            asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int j = jt + 8 * i;
              if (c0 + j < t_valid) {
                const uint4 v = *reinterpret_cast<const uint4*>(st + j * BM + seg * 8);
                for (int d = 0; d < ndst; ++d) {
                  const TileDst td = tile_dst<BN, MODE>(p, wk, d);
                  *reinterpret_cast<uint4*>(td.base + (size_t)(c0 + j) * td.cs + seg * 8) = v;
                }
              }
            }
            ++push_count;
          }
        }
#pragma unroll 1
        for (int c0 = 0; c0 < BN && !vec_push; c0 += 32) {
          if (c0 >= t_valid) break;               // warp-uniform
          uint32_t r[32];
          tmem_ld_32x32(taddr + c0, r);
          tmem_ld_wait();
          if (n < p.N) {
            for (int d = 0; d < ndst; ++d) {
              const TileDst td = tile_dst<BN, MODE>(p, wk, d);
              __nv_bfloat16* yp = td.base + (size_t)c0 * td.cs + row;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                if (c0 + j < t_valid) yp[(size_t)j * td.cs] = __float2bfloat16(__uint_as_float(r[j]) + bias);
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
        if (push_out) {
          // the partial tile has been pushed; the flag stores below are release operations at system
          // scope and the barrier orders every epilogue thread's stores before them
          asm volatile("bar.sync 1, 128;" ::: "memory");
          publish_tile<MODE>(p, tile, epoch, (int)threadIdx.x - 64);
        }
      } else if (p.cluster_splitk) {
        // split-K inside a thread-block cluster: the partial stays on chip.  This CTA has exactly one
        // work item, so the stage ring is free once the accumulator is complete; it is reused as the
        // fp32 partial [column][row] that the other CTAs of the cluster read through DSMEM.
        float* part = reinterpret_cast<float*>(smem);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (c0 >= t_valid) break;
          uint32_t r[32];
          tmem_ld_32x32(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) part[(c0 + j) * BM + row] = __uint_as_float(r[j]);
          if (NACC == 2) {       // the up accumulator goes behind the gate accumulator's BN columns
            tmem_ld_32x32(taddr + BN + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) part[(BN + c0 + j) * BM + row] = __uint_as_float(r[j]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
      } else if (FULL) {
        float* wsp = p.ws + ((size_t)tile * p.splits + split) * (size_t)(BM * BN);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (c0 >= t_valid) break;
          uint32_t r[32];
          tmem_ld_32x32(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) wsp[(c0 + j) * BM + row] = __uint_as_float(r[j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[acc]);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 64) {
          const int old = atomicAdd(&p.counters[tile], 1);
          *last_flag = (old == p.splits - 1) ? 1 : 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*last_flag) {
          __threadfence();
          // partial layout is [column c][row]: lane owns rows 4*lane..4*lane+3 (one float4 per split),
          // warp q takes columns c = q, q+4, ...; four columns are in flight per iteration
          const float* base = p.ws + (size_t)tile * p.splits * (size_t)(BM * BN);
          const int n4 = wk.n0 + 4 * lane;
          float b4[4] = {0.f, 0.f, 0.f, 0.f};
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (n4 + j < p.N) b4[j] = __bfloat162float(p.bias[n4 + j]);
          }
          for (int c0 = q; c0 < t_valid; c0 += 16) {
            float4 a4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) a4[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s2 = 0; s2 < p.splits; ++s2) {
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int c = c0 + 4 * u;
                if (c < t_valid) {
                  const float4 v = __ldcg(reinterpret_cast<const float4*>(
                      base + (size_t)s2 * (BM * BN) + (size_t)c * BM + 4 * lane));
                  a4[u].x += v.x; a4[u].y += v.y; a4[u].z += v.z; a4[u].w += v.w;
                }
              }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int c = c0 + 4 * u;
              if (c >= t_valid) continue;
              for (int d = 0; d < ndst; ++d) {
                const TileDst td = tile_dst<BN, MODE>(p, wk, d);
                __nv_bfloat16* yp = td.base + (size_t)c * td.cs + 4 * lane;
                const bool vec_ok = (n4 + 3 < p.N) && ((td.cs & 3) == 0) &&
                                    ((reinterpret_cast<uintptr_t>(td.base) & 7) == 0);
                if (vec_ok) {
                  __nv_bfloat162 lo = __floats2bfloat162_rn(a4[u].x + b4[0], a4[u].y + b4[1]);
                  __nv_bfloat162 hi = __floats2bfloat162_rn(a4[u].z + b4[2], a4[u].w + b4[3]);
                  uint2 pk;
                  pk.x = *reinterpret_cast<uint32_t*>(&lo);
                  pk.y = *reinterpret_cast<uint32_t*>(&hi);
                  *reinterpret_cast<uint2*>(yp) = pk;
                } else {
                  const float vals[4] = {a4[u].x, a4[u].y, a4[u].z, a4[u].w};
#pragma unroll
                  for (int j = 0; j < 4; ++j)
                    if (n4 + j < p.N) yp[j] = __float2bfloat16(vals[j] + b4[j]);
                }
              }
            }
          }
          if (threadIdx.x == 64) p.counters[tile] = 0;
          if (push_out) {
            __threadfence_system();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            publish_tile<MODE>(p, tile, epoch, (int)threadIdx.x - 64);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // last_flag is rewritten next iteration
      }
    }
  }

  else if (FULL && fused && p.ar_mode == 5) {
    // ------------------------------------------- gather warps (threads 192..319), all-gather -> GEMM
    // unit = (destination, BN-row block of this rank's shard, K slice); destinations start with this
    // rank itself and go round, so that every link is busy and the local blocks are ready first
    const int rt = threadIdx.x - NUM_THREADS;
    const int kv = p.K >> 3;                                   // 16-byte vectors per row
    const int vpp = (kv + p.ag_parts - 1) / p.ag_parts;
    const int units = p.world * p.ag_tps * p.ag_parts;
    const int prev_use = *reinterpret_cast<volatile int*>(p.epoch_ptr + 2 + p.ag_flip);
    const int* ag_done = reinterpret_cast<const int*>(p.peer[p.rank] + p.ag_done_off) + p.ag_flip * p.world;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      const int part = u % p.ag_parts;
      const int j = (u / p.ag_parts) % p.ag_tps;
      const int d = (p.rank + u / (p.ag_parts * p.ag_tps)) % p.world;
      if (rt == 0 && !wait_flag_ge(ag_done + d, prev_use, p.status, p.spin_limit)) *red_ok = 0;
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (!*red_ok) break;
      const int row0 = j * BN, rows = min(BN, p.ag_rows - row0);
      const int v0 = part * vpp, nv = min(vpp, kv - v0);
      const uint4* src = reinterpret_cast<const uint4*>(p.ag_src + (size_t)row0 * p.ag_ld) + v0;
      uint4* dst = reinterpret_cast<uint4*>(p.peer[d] + p.ag_dst_off) +
                   ((size_t)p.rank * p.ag_rows + row0) * kv + v0;
      const int src_ldv = p.ag_ld >> 3;
      const int total = rows * nv;
      for (int base = rt; base < total; base += 128 * 4) {
        uint4 val[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int idx = base + q * 128;
          if (idx < total) val[q] = src[(size_t)(idx / nv) * src_ldv + idx % nv];
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int idx = base + q * 128;
          if (idx < total) dst[(size_t)(idx / nv) * kv + idx % nv] = val[q];
        }
      }
      __threadfence_system();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (rt == 0)
        st_release_sys(reinterpret_cast<int*>(p.peer[d] + p.tile_flag_off) + (size_t)p.rank * p.max_tiles +
                           j * p.ag_parts + part, epoch);
    }
  }

  else if (FULL && fused) {      // (absent in ar_mode 3 launches, which have no reducer warps)
    // ------------------------------------------- reducer warps (threads 192..319)
    // All cross-rank traffic is stores: partials were pushed into this rank's receive slabs, so the
    // sums below read local memory only (written by peers: L1 is bypassed).
    //   via owners (ar_mode 0/1): rank tile % world sums the slabs of a tile once every rank's flag
    //     for it is up, then pushes the bf16 result into the output buffer of every rank (all-reduce)
    //     or keeps it (reduce-scatter) and raises the tile's done flag there.
    //   one-shot (ar_mode 2): every rank received every partial; it sums all tiles for itself.
    const int rt = threadIdx.x - NUM_THREADS;        // 0..127
    if (p.cluster_splitk) {
      // take part in both cluster barriers of the split-K reduction up front: the flags this role
      // waits for are only raised after them
      cluster_arrive_release();
      cluster_wait_acquire();
      cluster_arrive_release();
      cluster_wait_acquire();
    }
    const int tiles = p.n_tiles * p.t_tiles;
    const int* my_tile_flags = reinterpret_cast<const int*>(p.peer[p.rank] + p.tile_flag_off);
    const uint8_t* recv = p.peer[p.rank] + p.part_off;
    const size_t stride = (size_t)p.part_src_stride;
    if (p.ar_mode == 2) {
      uint8_t* out = p.peer[p.rank] + p.out_off;
      for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        if (rt < p.world) {
          if (!wait_flag_ge(my_tile_flags + (size_t)rt * p.max_tiles + tile, epoch, p.status, p.spin_limit))
            *red_ok = 0;
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (!*red_ok) break;
        int n_tile, t_tile;
        decode_tile(tile, p, n_tile, t_tile);
        const int n0 = n_tile * BM, t0 = t_tile * BN;
        const int t_valid = min(BN, p.T - t0);
        const int n_vecs = min(BM, p.N - n0) >> 3;
        for (int idx = rt; idx < t_valid * (BM / 8); idx += 128) {
          const int row = idx / (BM / 8), v = idx % (BM / 8);
          if (v >= n_vecs) continue;
          const size_t off = ((size_t)(t0 + row) * p.N + n0 + v * 8) * sizeof(__nv_bfloat16);
          *reinterpret_cast<uint4*>(out + off) = sum_slabs(recv + off, stride, p.world);
        }
      }
    } else {
      int owned_idx = 0;
      for (int tile = p.rank; tile < tiles; tile += p.world, ++owned_idx) {
        if (owned_idx % (int)gridDim.x != (int)blockIdx.x) continue;
        if (rt < p.world) {
          if (!wait_flag_ge(my_tile_flags + (size_t)rt * p.max_tiles + tile, epoch, p.status, p.spin_limit))
            *red_ok = 0;
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (!*red_ok) break;
        int n_tile, t_tile;
        decode_tile(tile, p, n_tile, t_tile);
        const int n0 = n_tile * BM, t0 = t_tile * BN;
        const int t_valid = min(BN, p.T - t0);
        const int n_vecs = min(BM, p.N - n0) >> 3;             // 16-byte vectors per row (N % 8 == 0)
        const uint8_t* slab = recv + (size_t)owned_idx * (BM * BN * sizeof(__nv_bfloat16));
        const int total = t_valid * (BM / 8);
        for (int base = 0; base < total; base += 128 * 4) {
          uint4 o[4];
          sum_slabs4(slab, stride, p.world, base + rt, total, n_vecs, o);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int idx = base + rt + u * 128;
            const int row = idx / (BM / 8), v = idx % (BM / 8);
            if (idx >= total || v >= n_vecs) continue;
            const size_t off = ((size_t)(t0 + row) * p.ldy + n0 + v * 8) * sizeof(__nv_bfloat16);
            if (p.ar_mode == 0) {
              for (int r = 0; r < p.world; ++r) *reinterpret_cast<uint4*>(p.peer[r] + p.out_off + off) = o[u];
            } else {
              *reinterpret_cast<uint4*>(p.peer[p.rank] + p.out_off + off) = o[u];
            }
          }
        }
        __threadfence_system();
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (p.ar_mode == 0) {
          if (rt < p.world)
            st_release_sys(reinterpret_cast<int*>(p.peer[rt] + p.done_flag_off) + tile, epoch);
        } else if (rt == 0) {
          st_release_sys(reinterpret_cast<int*>(p.peer[p.rank] + p.done_flag_off) + tile, epoch);
        }
      }
      // this rank's output is complete once every tile it reads has its done flag
      const int* done = reinterpret_cast<const int*>(p.peer[p.rank] + p.done_flag_off);
      for (int tile = blockIdx.x * 128 + rt; tile < tiles; tile += gridDim.x * 128) {
        if (p.ar_mode == 1 && tile % p.world != p.rank) continue;
        wait_flag_ge(done + tile, epoch, p.status, p.spin_limit);
      }
    }
  }

  if (p.cluster_splitk && warp < 6) {
    // ---- cluster split-K reduction over distributed shared memory: CTA `rank` of the cluster sums
    // columns c = rank, rank + S, ... of all S partials (fixed order) and writes them as bf16.
    __syncwarp();
    cluster_arrive_release();
    cluster_wait_acquire();
    if (threadIdx.x == 64) dbg_stamp(p, 5);
    if (warp >= 2 && warp < 6 && !*abort_flag && blockIdx.x < total_work) {
      const Work wk = get_work<BN, MODE>(blockIdx.x, p, s_prefix);
      if (threadIdx.x == 64) dbg_stamp(p, 9);
      const int q = warp & 3;
      const uint32_t rank = cluster_ctarank();
      const int S = p.splits;
      const int n4 = wk.n0 + 4 * lane;
      float b4[4] = {0.f, 0.f, 0.f, 0.f};
      if (p.bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n4 + j < p.N) b4[j] = __bfloat162float(p.bias[n4 + j]);
      }
      const uint32_t part_local = smem_u32(smem);
      // Distributed-shared-memory loads have a long latency (several hundred ns each round trip): the
      // partials of as many whole columns as fit in 16 vector registers are requested together.
      if (S <= 2) cluster_reduce_cols<BN, 2, MODE, NACC>(p, wk, part_local, (int)rank, q, lane, ndst, b4);
      else if (S <= 4) cluster_reduce_cols<BN, 4, MODE, NACC>(p, wk, part_local, (int)rank, q, lane, ndst, b4);
      else cluster_reduce_cols<BN, 8, MODE, NACC>(p, wk, part_local, (int)rank, q, lane, ndst, b4);
    }
    if (threadIdx.x == 64) dbg_stamp(p, 6);
    __syncwarp();
    cluster_arrive_release();          // nobody leaves while its partial may still be read
    cluster_wait_acquire();
    if (push_out && cluster_ctarank() == 0 && warp == 2 && blockIdx.x < total_work) {
      const Work wk = get_work<BN, MODE>(blockIdx.x, p, s_prefix);
      publish_tile<MODE>(p, wk.tile, epoch, lane);
    }
  }

  if (threadIdx.x == 64) dbg_stamp(p, 7);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  if (fused && threadIdx.x == 64) {      // a thread that holds the epoch (warp 0 does not)
    // the barrier above ordered every thread's stores before this fence (system scope for the routed rows
    // that went to peers)
    if (p.ar_mode == 4) __threadfence_system();
    else __threadfence();
    const int arrived = atomicAdd(p.cta_done, 1) + 1;
    if (arrived == (int)gridDim.x) {
      *p.cta_done = 0;
      if (p.ar_mode == 4) {
        // every CTA fenced its routed stores before it arrived: tell all ranks their rows are back
        __threadfence_system();
        const int ep_epoch = *reinterpret_cast<volatile int*>(p.epoch_ptr);
        for (int r = 0; r < p.world; ++r)
          st_release_sys(reinterpret_cast<int*>(p.peer[r] + p.done_flag_off) + p.rank, ep_epoch);
      } else {
        if (p.ar_mode == 5) {
          // this rank no longer reads its gather buffer: peers may overwrite it
          for (int r = 0; r < p.world; ++r)
            st_release_sys(reinterpret_cast<int*>(p.peer[r] + p.ag_done_off) + p.ag_flip * p.world + p.rank,
                           epoch);
          p.epoch_ptr[2 + p.ag_flip] = epoch;
        }
        *p.epoch_ptr = epoch;       // every CTA of this launch has read the old value by now
      }
      __threadfence();
    }
  }
}

// --------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

}  // namespace b200

extern "C" int b200_make_tmap_2d(void* out_map, const void* ptr, int elem_bytes, uint64_t rows, uint64_t cols,
                                 uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols) {
  auto fn = b200::get_encode_fn();
  if (!fn) {
    b200_set_last_error("cuTensorMapEncodeTiled not available", __FILE__, __LINE__);
    return -1;
  }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (row_stride_bytes & 15)) {
    b200_set_last_error("TMA operand must be 16-byte aligned with a 16-byte multiple row stride", __FILE__,
                        __LINE__);
    return -2;
  }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(out_map), dt, 2, const_cast<void*>(ptr), gdim, gstride, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    b200_set_last_error("cuTensorMapEncodeTiled failed", __FILE__, __LINE__);
    return (int)r;
  }
  return 0;
}

// 2D byte tensor map without swizzle: the box lands in shared memory as dense rows of box_cols bytes
// (box_cols a multiple of 16).  For operands that threads read back themselves.
extern "C" int b200_make_tmap_2d_bytes_linear(void* out_map, const void* ptr, uint64_t rows, uint64_t cols,
                                              uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols) {
  auto fn = b200::get_encode_fn();
  if (!fn) {
    b200_set_last_error("cuTensorMapEncodeTiled not available", __FILE__, __LINE__);
    return -1;
  }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (row_stride_bytes & 15) || (box_cols & 15)) {
    b200_set_last_error("TMA operand must be 16-byte aligned with 16-byte multiple row stride and box width",
                        __FILE__, __LINE__);
    return -2;
  }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(out_map), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr),
                  gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    b200_set_last_error("cuTensorMapEncodeTiled failed", __FILE__, __LINE__);
    return (int)r;
  }
  return 0;
}

// bf16 3D tensor map: dims (x fastest, y, z), byte strides of y and z, box (bx, by, bz), SWIZZLE_128B.
extern "C" int b200_make_tmap_3d_bf16(void* out_map, const void* ptr, uint64_t dx, uint64_t dy, uint64_t dz,
                                      uint64_t stride_y_bytes, uint64_t stride_z_bytes, uint32_t bx, uint32_t by,
                                      uint32_t bz) {
  auto fn = b200::get_encode_fn();
  if (!fn) {
    b200_set_last_error("cuTensorMapEncodeTiled not available", __FILE__, __LINE__);
    return -1;
  }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (stride_y_bytes & 15) || (stride_z_bytes & 15)) {
    b200_set_last_error("TMA operand must be 16-byte aligned with 16-byte multiple strides", __FILE__, __LINE__);
    return -2;
  }
  cuuint64_t gdim[3] = {dx, dy, dz};
  cuuint64_t gstride[2] = {stride_y_bytes, stride_z_bytes};
  cuuint32_t box[3] = {bx, by, bz};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(out_map), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                  const_cast<void*>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    b200_set_last_error("cuTensorMapEncodeTiled (3D) failed", __FILE__, __LINE__);
    return (int)r;
  }
  return 0;
}

namespace b200 {

struct TmapKey {
  const void* ptr;
  uint64_t rows, cols, stride;
  uint32_t box_rows;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && stride == o.stride && box_rows == o.box_rows;
  }
};
struct TmapHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= k.rows * 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.cols * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
    h ^= (k.stride + k.box_rows) * 0x165667B19E3779F9ull + (h << 6) + (h >> 2);
    return h;
  }
};

static int cached_tmap(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t stride_bytes,
                       uint32_t box_rows, int elem_bytes = 2, uint32_t box_cols = BK) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapHash> cache;
  static std::mutex mu;
  TmapKey key{ptr, rows, cols | ((uint64_t)elem_bytes << 56), stride_bytes, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  int rc = b200_make_tmap_2d(out, ptr, elem_bytes, rows, cols, stride_bytes, box_rows, box_cols);
  if (rc != 0) return rc;
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return 0;
}


// How many clusters of `splits` CTAs of this kernel can be resident at once (GPC granularity).
template <int BN>
static int max_active_clusters_t(int splits, int threads) {
  using Cfg = GemmCfg<BN, 1>;
  auto kern = threads > NUM_THREADS ? gemm_bf16_kernel<BN, 1, 2> : gemm_bf16_kernel<BN, 1, 0>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(splits * 64);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = Cfg::SMEM;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}
static int max_active_clusters(int bn, int splits, int threads) {
  static int cache[4][9][2];
  static bool init = false;
  if (!init) { memset(cache, -1, sizeof(cache)); init = true; }
  const int bi = bn == 32 ? 0 : (bn == 64 ? 1 : (bn == 128 ? 2 : 3));
  const int ti = threads > NUM_THREADS ? 1 : 0;
  if (splits < 2 || splits > 8) return 0;
  int& c = cache[bi][splits][ti];
  if (c < 0) {
    switch (bn) {
      case 32: c = max_active_clusters_t<32>(splits, threads); break;
      case 64: c = max_active_clusters_t<64>(splits, threads); break;
      case 128: c = max_active_clusters_t<128>(splits, threads); break;
      default: c = max_active_clusters_t<256>(splits, threads); break;
    }
  }
  return c;
}
// Largest split count <= want whose clusters (one per tile) are all resident in one wave.
static int fit_cluster_splits(int want, int tiles, int bn, int threads) {
  int s = want > 8 ? 8 : want;
  while (s > 1 && max_active_clusters(bn, s, threads) < tiles) --s;
  return s;
}

// 0: compact kernel (dense single-rank launches without split-K or with cluster split-K),
// 1: compact push kernel (ar_mode 3), 2: the full kernel
static int kernel_mode(const GemmParams& p) {
  const bool simple = p.group_off == nullptr && p.row_route == nullptr && (p.splits == 1 || p.cluster_splitk);
  if (simple && p.world == 1) return 0;
  if (simple && p.world > 1 && p.ar_mode == 3) return 1;
  return 2;
}

template <int BN, int NACC, int MODE>
static int launch_gemm_v(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, int grid,
                         cudaStream_t stream);

template <int BN, int NACC = 1>
static int launch_gemm(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, int grid,
                       cudaStream_t stream) {
  const int mode = kernel_mode(p);
  if (mode == 0) return launch_gemm_v<BN, NACC, 0>(tmW, tmX, p, grid, stream);
  if (mode == 1 && NACC == 1) return launch_gemm_v<BN, 1, 1>(tmW, tmX, p, grid, stream);
  return launch_gemm_v<BN, NACC, 2>(tmW, tmX, p, grid, stream);
}

template <int BN, int NACC, int MODE>
static int launch_gemm_v(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, int grid,
                         cudaStream_t stream) {
  using Cfg = GemmCfg<BN, NACC>;
  static unsigned long long attr_seen = 0;
  B200_CUDA_CHECK(ensure_dynamic_smem(gemm_bf16_kernel<BN, NACC, MODE>, Cfg::SMEM, &attr_seen));
  const int threads = (p.world > 1 && (p.ar_mode < 3 || p.ar_mode == 5)) ? NUM_THREADS_FUSED : NUM_THREADS;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = Cfg::SMEM;
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
  if (b200_pdl_enabled()) {
    // let this grid start (and prefetch weights) while the previous kernel of the stream drains
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  B200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<BN, NACC, MODE>, tmW, tmX, p));
  return 0;
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace b200

namespace b200 { static unsigned long long* g_gemm_dbg = nullptr; }
// Debug aid (builds with -DB200_GEMM_TIMESTAMPS): plain GEMM launches record phase timestamps (ns),
// 16 slots per CTA, into `buf`
// (start, set-up done, first stage landed, last MMA issued, accumulator ready, split-K partials
// visible, reduced and stored, cluster released).
extern "C" void b200_gemm_set_debug(unsigned long long* buf) { b200::g_gemm_dbg = buf; }

extern "C" int b200_gemm_plan(int T, int N, int K, int num_sms, int* bn_out, int* splits_out,
                              size_t* ws_bytes, int* counters_needed) {
  using namespace b200;
  int bn = T <= 32 ? 32 : (T <= 64 ? 64 : (T <= 128 ? 128 : 256));
  int n_tiles = (N + BM - 1) / BM, t_tiles = (T + bn - 1) / bn;
  int tiles = n_tiles * t_tiles;
  int kb_total = (K + BK - 1) / BK;
  int splits = 1;
  if (tiles * 2 <= num_sms) {
    splits = num_sms / tiles;
    int max_by_k = kb_total / 8 > 0 ? kb_total / 8 : 1;    // at least 8 k-blocks (512 of K) per split
    if (splits > max_by_k) splits = max_by_k;
    if (splits > 8) splits = 8;       // one thread-block cluster per tile
    if (splits < 1) splits = 1;
  }
  *bn_out = bn;
  *splits_out = splits;
  *ws_bytes = splits > 1 ? (size_t)tiles * splits * BM * bn * sizeof(float) : 0;
  *counters_needed = splits > 1 ? tiles : 0;
  return 0;
}

// X [T,K] row stride ldx, W [N,K] row stride ldw, Y [T,N] row stride ldy (elements).
// ws / counters: scratch for split-K (counters must be zero on first use; the kernel re-arms them).
extern "C" int b200_gemm_bf16(const void* X, const void* W, void* Y, const void* bias, int T, int N, int K,
                              int ldx, int ldw, int ldy, void* ws, size_t ws_bytes, int* counters,
                              int counters_len, int* status, int num_sms, int force_splits,
                              cudaStream_t stream) {
  using namespace b200;
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 8 || ldx % 8 || ldw % 8) {
    b200_set_last_error("gemm_bf16: K and row strides must be multiples of 8 elements", __FILE__, __LINE__);
    return -3;
  }
  int bn, splits, cneed;
  size_t need;
  b200_gemm_plan(T, N, K, num_sms, &bn, &splits, &need, &cneed);
  if (force_splits > 0) splits = force_splits;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.world = 1;
  p.Y = reinterpret_cast<__nv_bfloat16*>(Y);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.ws = reinterpret_cast<float*>(ws);
  p.counters = counters;
  p.status = status;
  p.T = T; p.N = N; p.K = K; p.ldy = ldy;
  p.n_tiles = (N + BM - 1) / BM;
  p.t_tiles = (T + bn - 1) / bn;
  p.kb_total = (K + BK - 1) / BK;
  if (splits > p.kb_total) splits = p.kb_total;
  int tiles = p.n_tiles * p.t_tiles;
  if (splits > 1) {
    size_t req = (size_t)tiles * splits * BM * bn * sizeof(float);
    if (ws == nullptr || req > ws_bytes || counters == nullptr || tiles > counters_len) splits = 1;
  }
  if (splits > 1 && force_splits <= 0) splits = fit_cluster_splits(splits, tiles, bn, NUM_THREADS);
  p.splits = splits;
  p.kb_per_split = (p.kb_total + splits - 1) / splits;
  // every split must own at least one k-block
  while (p.splits > 1 && (p.splits - 1) * p.kb_per_split >= p.kb_total) {
    --p.splits;
    p.kb_per_split = (p.kb_total + p.splits - 1) / p.splits;
  }
  p.w_evict_first = (p.t_tiles == 1) ? 1 : 0;
  p.cluster_splitk = (p.splits > 1 && p.splits <= 8) ? 1 : 0;
  p.dbg = g_gemm_dbg;
  CUtensorMap tmW, tmX;
  int rc = cached_tmap(&tmW, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw * 2, BM);
  if (rc) return rc;
  rc = cached_tmap(&tmX, X, (uint64_t)T, (uint64_t)K, (uint64_t)ldx * 2, (uint32_t)bn);
  if (rc) return rc;
  int total = tiles * p.splits;
  int grid = p.cluster_splitk ? total : (total < num_sms ? total : num_sms);
  switch (bn) {
    case 32: return launch_gemm<32>(tmW, tmX, p, grid, stream);
    case 64: return launch_gemm<64>(tmW, tmX, p, grid, stream);
    case 128: return launch_gemm<128>(tmW, tmX, p, grid, stream);
    default: return launch_gemm<256>(tmW, tmX, p, grid, stream);
  }
}

// Row-parallel GEMM fused with the cross-rank reduction: Y = sum over ranks of X_r * W_r^T.
// Every rank of the group launches this with identical T/N (K is the local shard).  All NVLink
// traffic is stores.  mode 0 (all-reduce) and 1 (reduce-scatter by tile ownership): each rank
// pushes its partial of a tile into the receive slab the tile's owner (tile % world) keeps for it,
// the owner sums the slabs from local memory and pushes the bf16 result into the output buffer
// (heap offset out_off) of every rank (mode 0) or keeps it (mode 1).  A mode-0 call whose pushed
// bytes, T*N*2*(world-1), do not exceed one_shot_max_bytes runs one-shot instead: every rank pushes
// its partial to every rank and each sums all of it for itself, one NVLink hop in total.
// mode 3 pushes like the one-shot form but leaves the sum to the consumer
// (b200_reduce_pushed_rms_norm), which finds the partials of all ranks in its own receive region.
// part_off/part_bytes: receive region of this launch (callers alternate between two regions).
// peers: `world` heap base pointers; ctrl: local device int[4] {epoch, cta_done, -, -}.
extern "C" int b200_gemm_bf16_fused_reduce(const void* X, const void* W, int T, int N, int K, int ldx, int ldw,
                                           void* const* peers, int rank, int world, int mode,
                                           unsigned long long part_off, unsigned long long part_bytes,
                                           unsigned long long one_shot_max_bytes,
                                           unsigned long long out_off, unsigned long long tile_flag_off,
                                           unsigned long long done_flag_off, int max_tiles, int* ctrl,
                                           void* ws, size_t ws_bytes, int* counters, int counters_len,
                                           int* status, int num_sms, unsigned int spin_limit,
                                           cudaStream_t stream) {
  using namespace b200;
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 8 || ldx % 8 || ldw % 8 || N % 8 || world < 2 || world > 8) {
    b200_set_last_error("gemm_fused_reduce: K, N, strides multiples of 8 and 2 <= world <= 8 required",
                        __FILE__, __LINE__);
    return -3;
  }
  int bn, splits, cneed;
  size_t need;
  b200_gemm_plan(T, N, K, num_sms, &bn, &splits, &need, &cneed);
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.Y = nullptr;
  p.bias = nullptr;
  p.ws = reinterpret_cast<float*>(ws);
  p.counters = counters;
  p.status = status;
  p.T = T; p.N = N; p.K = K; p.ldy = N;
  p.n_tiles = (N + BM - 1) / BM;
  p.t_tiles = (T + bn - 1) / bn;
  p.kb_total = (K + BK - 1) / BK;
  int tiles = p.n_tiles * p.t_tiles;
  if (tiles > max_tiles) {
    b200_set_last_error("gemm_fused_reduce: more tiles than flag slots", __FILE__, __LINE__);
    return -4;
  }
  if (splits > p.kb_total) splits = p.kb_total;
  if (splits > 1) {
    size_t req = (size_t)tiles * splits * BM * bn * sizeof(float);
    if (ws == nullptr || req > ws_bytes || counters == nullptr || tiles > counters_len) splits = 1;
  }
  if (splits > 1) splits = fit_cluster_splits(splits, tiles, bn, mode == 3 ? NUM_THREADS : NUM_THREADS_FUSED);
  p.splits = splits;
  p.kb_per_split = (p.kb_total + splits - 1) / splits;
  while (p.splits > 1 && (p.splits - 1) * p.kb_per_split >= p.kb_total) {
    --p.splits;
    p.kb_per_split = (p.kb_total + p.splits - 1) / p.splits;
  }
  p.w_evict_first = (p.t_tiles == 1) ? 1 : 0;
  p.cluster_splitk = (p.splits > 1 && p.splits <= 8) ? 1 : 0;
  p.world = world; p.rank = rank; p.ar_mode = mode;
  if (mode == 0 && (unsigned long long)T * N * 2ull * (world - 1) <= one_shot_max_bytes) p.ar_mode = 2;
  if (p.ar_mode >= 2) {
    p.part_src_stride = ((unsigned long long)T * N * 2ull + 255ull) & ~255ull;
  } else {
    const unsigned long long owned = (unsigned long long)(tiles + world - 1) / world;
    p.part_src_stride = owned * BM * bn * 2ull;
  }
  if (p.part_src_stride * world > part_bytes) {
    b200_set_last_error("gemm_fused_reduce: receive region too small for this shape", __FILE__, __LINE__);
    return -5;
  }
  for (int i = 0; i < 8; ++i) p.peer[i] = i < world ? (uint8_t*)peers[i] : nullptr;
  p.part_off = part_off; p.out_off = out_off;
  p.tile_flag_off = tile_flag_off; p.done_flag_off = done_flag_off;
  p.max_tiles = max_tiles;
  p.epoch_ptr = ctrl; p.cta_done = ctrl + 1;
  p.spin_limit = spin_limit;
  CUtensorMap tmW, tmX;
  int rc = cached_tmap(&tmW, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw * 2, BM);
  if (rc) return rc;
  rc = cached_tmap(&tmX, X, (uint64_t)T, (uint64_t)K, (uint64_t)ldx * 2, (uint32_t)bn);
  if (rc) return rc;
  int total = tiles * p.splits;
  int grid = p.cluster_splitk ? total : (total < num_sms ? total : num_sms);
  switch (bn) {
    case 32: return launch_gemm<32>(tmW, tmX, p, grid, stream);
    case 64: return launch_gemm<64>(tmW, tmX, p, grid, stream);
    case 128: return launch_gemm<128>(tmW, tmX, p, grid, stream);
    default: return launch_gemm<256>(tmW, tmX, p, grid, stream);
  }
}

namespace b200 {
static void init_params(GemmParams& p, void* Y, int T, int N, int K, int ldy, int bn, int* status) {
  memset(&p, 0, sizeof(p));
  p.world = 1;
  p.Y = reinterpret_cast<__nv_bfloat16*>(Y);
  p.status = status;
  p.T = T; p.N = N; p.K = K; p.ldy = ldy;
  p.n_tiles = (N + BM - 1) / BM;
  p.t_tiles = (T + bn - 1) / bn;
  p.kb_total = (K + BK - 1) / BK;
  p.splits = 1;
  p.kb_per_split = p.kb_total;
}
}  // namespace b200

// Y[T, I] = silu(X * Wg^T) * (X * Wu^T) with W = [gate rows (I) ; up rows (I)] x K packed as [2I, K].
extern "C" int b200_gemm_bf16_swiglu(const void* X, const void* W, void* Y, int T, int I, int K, int ldx,
                                     int ldw, int ldy, int* status, int num_sms, cudaStream_t stream) {
  using namespace b200;
  if (T <= 0 || I <= 0 || K <= 0) return 0;
  if (K % 8 || ldx % 8 || ldw % 8) {
    b200_set_last_error("gemm_swiglu: K and row strides must be multiples of 8 elements", __FILE__, __LINE__);
    return -3;
  }
  const int bn = T <= 32 ? 32 : (T <= 64 ? 64 : 128);
  GemmParams p;
  init_params(p, Y, T, I, K, ldy, bn, status);
  p.up_row_off = I;
  p.w_evict_first = (p.t_tiles == 1) ? 1 : 0;
  {
    // few output tiles (small I per rank under tensor parallelism): split K over a cluster so that
    // every SM streams weights; the gate and up partials are reduced over DSMEM before the activation
    const int tiles = p.n_tiles * p.t_tiles;
    int splits = 1;
    if (tiles * 2 <= num_sms && bn <= 64) {
      splits = num_sms / tiles;
      const int max_by_k = p.kb_total / 8 > 0 ? p.kb_total / 8 : 1;
      if (splits > max_by_k) splits = max_by_k;
      if (splits > 8) splits = 8;
      if (splits > 1) splits = fit_cluster_splits(splits, tiles, bn, NUM_THREADS);
    }
    p.splits = splits;
    p.kb_per_split = (p.kb_total + splits - 1) / splits;
    while (p.splits > 1 && (p.splits - 1) * p.kb_per_split >= p.kb_total) {
      --p.splits;
      p.kb_per_split = (p.kb_total + p.splits - 1) / p.splits;
    }
    p.cluster_splitk = p.splits > 1 ? 1 : 0;
  }
  CUtensorMap tmW, tmX;
  int rc = cached_tmap(&tmW, W, (uint64_t)2 * I, (uint64_t)K, (uint64_t)ldw * 2, BM);
  if (rc) return rc;
  rc = cached_tmap(&tmX, X, (uint64_t)T, (uint64_t)K, (uint64_t)ldx * 2, (uint32_t)bn);
  if (rc) return rc;
  const int total = p.n_tiles * p.t_tiles * p.splits;
  const int grid = p.cluster_splitk ? total : (total < num_sms ? total : num_sms);
  switch (bn) {
    case 32: return launch_gemm<32, 2>(tmW, tmX, p, grid, stream);
    case 64: return launch_gemm<64, 2>(tmW, tmX, p, grid, stream);
    default: return launch_gemm<128, 2>(tmW, tmX, p, grid, stream);
  }
}

// Grouped (per-expert) GEMM over rows sorted by expert:
//   rows [group_off[e], group_off[e+1]) of X use weight W[e] ([N, K], or [2N, K] gate/up when swiglu).
// X: [R, K]; Y: [R, N].  group_off lives in device memory, so the launch is CUDA-graph safe; the
// grid is one persistent CTA per SM and CTAs without work exit.  avg_rows_hint picks the token tile.
extern "C" int b200_grouped_gemm_bf16(const void* X, const void* W, void* Y, const int* group_off,
                                      int num_groups, int R, int N, int K, int swiglu, int avg_rows_hint,
                                      int* status, int num_sms, cudaStream_t stream) {
  using namespace b200;
  if (R <= 0 || N <= 0 || K <= 0 || num_groups <= 0) return 0;
  if (K % 8 || N % BM || num_groups > MAX_GROUPS) {
    b200_set_last_error("grouped_gemm: K % 8 == 0, N % 128 == 0 and <= 1024 groups required", __FILE__,
                        __LINE__);
    return -3;
  }
  int bn = avg_rows_hint <= 32 ? 32 : (avg_rows_hint <= 64 ? 64 : (avg_rows_hint <= 128 || swiglu ? 128 : 256));
  GemmParams p;
  init_params(p, Y, R, N, K, N, bn, status);
  p.group_off = group_off;
  p.num_groups = num_groups;
  p.w_rows_per_group = swiglu ? 2 * N : N;
  p.up_row_off = N;
  p.w_evict_first = avg_rows_hint <= bn ? 1 : 0;
  CUtensorMap tmW, tmX;
  int rc = cached_tmap(&tmW, W, (uint64_t)num_groups * p.w_rows_per_group, (uint64_t)K, (uint64_t)K * 2, BM);
  if (rc) return rc;
  rc = cached_tmap(&tmX, X, (uint64_t)R, (uint64_t)K, (uint64_t)K * 2, (uint32_t)bn);
  if (rc) return rc;
  const int grid = num_sms;
  if (swiglu) {
    switch (bn) {
      case 32: return launch_gemm<32, 2>(tmW, tmX, p, grid, stream);
      case 64: return launch_gemm<64, 2>(tmW, tmX, p, grid, stream);
      default: return launch_gemm<128, 2>(tmW, tmX, p, grid, stream);
    }
  }
  switch (bn) {
    case 32: return launch_gemm<32>(tmW, tmX, p, grid, stream);
    case 64: return launch_gemm<64>(tmW, tmX, p, grid, stream);
    case 128: return launch_gemm<128>(tmW, tmX, p, grid, stream);
    default: return launch_gemm<256>(tmW, tmX, p, grid, stream);
  }
}

// Grouped GEMM whose output rows are scattered to the ranks that sent the tokens (expert-parallel
// combine inside the epilogue): row r of the product goes to slot route[r].y of rank route[r].x,
// at heap offset ret_off, row length N.  The last CTA raises ret_flags[rank] (heap offset
// ret_flag_off, int[world]) at every rank with the epoch in ctrl[0]; ctrl[1] is the CTA counter.
extern "C" int b200_grouped_gemm_bf16_routed(const void* X, const void* W, const int* group_off, int num_groups,
                                             int R, int N, int K, int avg_rows_hint, void* const* peers,
                                             int rank, int world, const void* route,
                                             unsigned long long ret_off, unsigned long long ret_flag_off,
                                             int* ctrl, int* status, int num_sms, cudaStream_t stream) {
  using namespace b200;
  if (R <= 0 || N <= 0 || K <= 0 || num_groups <= 0) return 0;
  if (K % 8 || N % BM || num_groups > MAX_GROUPS || world < 2 || world > 8) {
    b200_set_last_error("grouped_gemm_routed: K % 8 == 0, N % 128 == 0, <= 1024 groups, 2 <= world <= 8",
                        __FILE__, __LINE__);
    return -3;
  }
  int bn = avg_rows_hint <= 32 ? 32 : (avg_rows_hint <= 64 ? 64 : (avg_rows_hint <= 128 ? 128 : 256));
  GemmParams p;
  init_params(p, nullptr, R, N, K, N, bn, status);
  p.group_off = group_off;
  p.num_groups = num_groups;
  p.w_rows_per_group = N;
  p.w_evict_first = avg_rows_hint <= bn ? 1 : 0;
  p.world = world; p.rank = rank; p.ar_mode = 4;
  for (int i = 0; i < 8; ++i) p.peer[i] = i < world ? (uint8_t*)peers[i] : nullptr;
  p.row_route = reinterpret_cast<const int2*>(route);
  p.route_ret_off = ret_off;
  p.done_flag_off = ret_flag_off;
  p.epoch_ptr = ctrl; p.cta_done = ctrl + 1;
  CUtensorMap tmW, tmX;
  int rc = cached_tmap(&tmW, W, (uint64_t)num_groups * N, (uint64_t)K, (uint64_t)K * 2, BM);
  if (rc) return rc;
  rc = cached_tmap(&tmX, X, (uint64_t)R, (uint64_t)K, (uint64_t)K * 2, (uint32_t)bn);
  if (rc) return rc;
  switch (bn) {
    case 32: return launch_gemm<32>(tmW, tmX, p, num_sms, stream);
    case 64: return launch_gemm<64>(tmW, tmX, p, num_sms, stream);
    case 128: return launch_gemm<128>(tmW, tmX, p, num_sms, stream);
    default: return launch_gemm<256>(tmW, tmX, p, num_sms, stream);
  }
}


// All-gather fused in front of a column-parallel GEMM: the activation rows are sharded over the
// ranks (T_loc rows each, row stride ldx), Y[world * T_loc, N] = gather(X) * W^T (+bias) lands in
// local memory.  Every rank pushes its shard into the [world * T_loc, K] buffer that each rank keeps
// at heap offset xfull_off, block by block, while the tensor cores already work on the blocks that
// have arrived (this rank's own first).  T_loc must be a multiple of 32.  Callers alternate between
// two gather buffers (flip 0 / 1, each with its xfull_off); ag_done_off names int[2][world] in the heap;
// ctrl is int[4]: epoch, CTA counter, epoch of the last launch that used buffer 0 / 1.
extern "C" int b200_gemm_bf16_allgather(const void* X_loc, const void* W, void* Y, const void* bias, int T_loc,
                                        int N, int K, int ldx, int ldw, int ldy, void* const* peers, int rank,
                                        int world, unsigned long long xfull_off, unsigned long long xfull_bytes,
                                        unsigned long long tile_flag_off, int max_tiles,
                                        unsigned long long ag_done_off, int flip, int* ctrl, int* status,
                                        int num_sms, unsigned int spin_limit, cudaStream_t stream) {
  using namespace b200;
  if (T_loc <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 8 || ldx % 8 || ldw % 8 || T_loc % 32 || world < 2 || world > 8) {
    b200_set_last_error("gemm_allgather: K, strides multiples of 8, T_loc multiple of 32, 2 <= world <= 8",
                        __FILE__, __LINE__);
    return -3;
  }
  const int T = T_loc * world;
  int bn = 256;
  while (bn > 32 && (T_loc % bn || bn > T)) bn >>= 1;
  if ((unsigned long long)T * K * 2ull > xfull_bytes) {
    b200_set_last_error("gemm_allgather: gather buffer too small", __FILE__, __LINE__);
    return -5;
  }
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.Y = reinterpret_cast<__nv_bfloat16*>(Y);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.status = status;
  p.T = T; p.N = N; p.K = K; p.ldy = ldy;
  p.n_tiles = (N + BM - 1) / BM;
  p.t_tiles = T / bn;
  p.kb_total = (K + BK - 1) / BK;
  p.splits = 1;
  p.kb_per_split = p.kb_total;
  p.world = world; p.rank = rank; p.ar_mode = 5;
  for (int i = 0; i < 8; ++i) p.peer[i] = i < world ? (uint8_t*)peers[i] : nullptr;
  p.tile_flag_off = tile_flag_off;
  p.max_tiles = max_tiles;
  p.epoch_ptr = ctrl; p.cta_done = ctrl + 1;
  p.spin_limit = spin_limit;
  p.ag_src = reinterpret_cast<const __nv_bfloat16*>(X_loc);
  p.ag_dst_off = xfull_off;
  p.ag_rows = T_loc; p.ag_ld = ldx;
  p.ag_done_off = ag_done_off; p.ag_flip = flip & 1;
  p.ag_tps = T_loc / bn;
  int parts = (2 * num_sms + world * p.ag_tps - 1) / (world * p.ag_tps);
  if (parts > 8) parts = 8;
  if (parts < 1) parts = 1;
  p.ag_parts = parts;
  if (p.ag_tps > 32 || p.ag_tps * parts > max_tiles) {
    b200_set_last_error("gemm_allgather: too many row blocks per shard", __FILE__, __LINE__);
    return -4;
  }
  CUtensorMap tmW, tmX;
  int rc = cached_tmap(&tmW, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw * 2, BM);
  if (rc) return rc;
  rc = cached_tmap(&tmX, (const uint8_t*)peers[rank] + xfull_off, (uint64_t)T, (uint64_t)K, (uint64_t)K * 2,
                   (uint32_t)bn);
  if (rc) return rc;
  const int total = p.n_tiles * p.t_tiles;
  const int grid = total < num_sms ? total : num_sms;
  switch (bn) {
    case 32: return launch_gemm<32>(tmW, tmX, p, grid, stream);
    case 64: return launch_gemm<64>(tmW, tmX, p, grid, stream);
    case 128: return launch_gemm<128>(tmW, tmX, p, grid, stream);
    default: return launch_gemm<256>(tmW, tmX, p, grid, stream);
  }
}
