// Persistent decode kernel: every decoder layer of a dense (Llama-family) model for one decode step
// in ONE launch.
//
// A decode step of 8..64 requests is a chain of small, latency-bound kernels (norm, qkv GEMM, RoPE +
// KV write, attention, o_proj, norm, gate/up, SiLU*mul, down) whose pipeline fill, drain and launch
// gaps cost more than their work, most of all under tensor parallelism where every GEMM shrinks.
// Here one cooperative grid (one CTA per SM) walks the layers; phases are separated by a grid
// barrier in global memory, and inside a CTA the roles are specialised:
//
//   warp 0    producer: streams weight tiles by TMA into a ring of stages and runs AHEAD of the phases
//             (weights do not depend on activations, so the tiles of the next GEMM are already in
//             shared memory while attention or a norm is still running); the activation tile of a
//             stage is requested as soon as the phase that produces it has been released
//   warp 1    tcgen05.mma issue (weight tile = 128-row A operand, tokens = N = 64), accumulators
//             double-buffered in TMEM
//   warps 2-5 epilogue of the GEMM phases (TMEM -> fp32 partials) and all other phases
//
// GEMM phases are scheduled stream-K: the (weight tile, k-block) space of a projection is cut into
// equal contiguous ranges, one per CTA, so every SM streams the same number of weight bytes whatever
// the shape; a range that ends inside a tile leaves an fp32 partial, and the consumer of the
// projection (attention prologue, reduce + norm, SiLU*mul) sums the partials of a tile in fixed
// order.  Under tensor parallelism the row-parallel projections push their bf16 partial rows into
// every rank's receive slab over NVLink (plain stores + release flags) and the following norm phase
// sums the slabs: the all-reduce has no phase of its own.
//
// Every wait (mbarrier, grid barrier, peer flag) is bounded; on expiry the kernel records a status
// code, raises a grid-wide abort word and every role falls through to the teardown.
//
// Plays the part of the reference's decode megakernel library and its decode-fused layers
// (reference: src/vllm_torchtpu/megakernel/core/planner.py:31, runtime/contract.py:14-70,
// kernels/experimental/moe_tp_decode/all_reduce.py:174-338).
#include <cstring>

#include "attn_mma.cuh"
#include "common.cuh"
#include "decode_mega.h"

namespace b200 {
namespace mega {

constexpr int BM = 128;                 // weight rows per tile (UMMA M)
constexpr int BN = 64;                  // token columns (UMMA N); a step has at most 64 rows
constexpr int BK = 64;                  // bf16 per 128-byte swizzled row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;
constexpr int STAGES = 8;
constexpr int A_BYTES = BM * BK * 2;    // 16 KB
constexpr int B_BYTES = BN * BK * 2;    // 8 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int RING_BYTES = STAGES * STAGE_BYTES;                 // 192 KB
// The attention phase borrows the ring: streaming bandwidth is bytes in flight per SM over memory
// latency, and neither the weight ring nor the KV rings reach HBM speed on half of shared memory.
// The producer does not load weights of the projections behind an attention phase until this CTA's
// attention is done (attn_done), and attention starts only after the qkv GEMM has drained the ring.
constexpr int D = 128;                                            // head dim
constexpr int ATT_STAGES = 6;
constexpr int ATT_PAGE_BYTES = 16 * D * 2;                        // 16 tokens of K (or V)
constexpr int ATT_STAGE_BYTES = 2 * ATT_PAGE_BYTES;
constexpr int ATT_WARP_BYTES = ATT_STAGES * ATT_STAGE_BYTES;      // 48 KB per warp (also q rows + cos / sin)
constexpr int ATT_OFF = 0;
static_assert(4 * ATT_WARP_BYTES <= RING_BYTES, "attention rings alias the GEMM ring");
constexpr int BAR_OFF = RING_BYTES;
constexpr int BAR_BYTES = 1024;
constexpr int RED_OFF = BAR_OFF + BAR_BYTES;                      // block-sum scratch
constexpr int SMEM_USED = RED_OFF + 256;
constexpr int SMEM_BYTES = SMEM_USED + 1024;                      // + alignment slack
static_assert(SMEM_BYTES <= 232448, "shared memory budget");
constexpr int TMEM_COLS = 2 * BN;                                 // two accumulators
constexpr int MAXT = 64;
constexpr int MAX_SLOTS = 5;             // split-K partial slots per weight tile, at most

enum Kind : int { K_NORM_IN = 0, K_GEMM, K_ATTN, K_PUSH, K_NORM_POST, K_SWIGLU };

struct alignas(64) LayerDesc {
  CUtensorMap tm[4];                    // qkv, o, gate_up, down weights [N, K] bf16, box 128 x 64, SWIZZLE_128B
  const __nv_bfloat16* ln_in;
  const __nv_bfloat16* ln_post;
  const __nv_bfloat16* qkv_bias;        // optional [Nqkv]
  const __nv_bfloat16* q_norm;          // optional [D]
  const __nv_bfloat16* k_norm;          // optional [D]
  __nv_bfloat16* kv_cache;              // [blocks, 2, Hkv, block_size, D]
  long long pad[2];
};
static_assert(sizeof(LayerDesc) == 576, "LayerDesc layout");

struct GemmShape {
  int N, K, n_tiles, kbt, total, U;     // total = n_tiles * kbt (tile, k-block) units; U units per CTA
};

struct Params {
  const LayerDesc* layers;
  int num_layers;
  int T, H, Hq, Hkv, I, Nqkv;           // per-rank sizes; T <= 64 token rows (one per request)
  GemmShape g[4];
  const __nv_bfloat16* hidden0;         // [T, H] embedding rows
  __nv_bfloat16* residual;              // [T, H] residual stream (output: fully summed after the last layer)
  __nv_bfloat16* h;                     // [64, H] normalised activations (GEMM operand)
  __nv_bfloat16* o;                     // [64, Hq * D] attention output
  __nv_bfloat16* act;                   // [64, I] silu(gate) * up
  float* part;                          // split-K partials [seg][64][N]
  const int* positions;
  const int* slot_mapping;
  const int* block_tables;
  const int* seq_lens;
  int max_blocks, block_size;
  long long num_blocks;
  const float* inv_freq;
  int rot_pairs, interleaved;
  float eps, scale_log2;
  int kv_splits;
  float* attn_part_o;                   // [T * Hkv * splits][16][D]
  float* attn_part_ml;                  // [T * Hkv * splits][16][2]
  int* attn_counters;                   // [T * Hkv], zero between launches
  int* ctrl;                            // [0] barrier arrivals, [1] exit count, [2] launch epoch, [3] abort,
                                        // [32] number of the last completed barrier (own cache line)
  int* status;
  int world, rank;
  uint8_t* peer[8];
  unsigned long long slab_off[2];       // receive slabs [src][64][H] bf16 of o_proj / down_proj partial rows
  unsigned long long flag_off[2];       // int[world][64 * 4]
  unsigned int spin_limit;
  int dbg_layer, dbg_gi, dbg_ev_base;   // optional: rows dbg_ev_base.. of dbg get role events of one GEMM phase
  unsigned long long* dbg;              // optional: %globaltimer of every CTA when it ends a phase's work and
                                        // when it leaves the barrier after it, [2 * phase + {0, 1}][CTA]
};

__device__ __forceinline__ int phases_per_layer(const Params& p) { return p.world > 1 ? 10 : 8; }
// phase index of GEMM gi of layer l
__device__ __forceinline__ int gemm_phase(const Params& p, int l, int gi) {
  const int off1[4] = {1, 3, 5, 7}, offn[4] = {1, 3, 6, 8};
  return l * phases_per_layer(p) + (p.world > 1 ? offn[gi] : off1[gi]);
}

// ----------------------------------------------------------------- stream-K bookkeeping
struct Cursor {
  int layer, gi, u, u_end;
  bool done;
};
__device__ __forceinline__ void cur_load(Cursor& c, const Params& p) {
  const GemmShape& g = p.g[c.gi];
  c.u = min(g.total, (int)blockIdx.x * g.U);
  c.u_end = min(g.total, c.u + g.U);
}
__device__ __forceinline__ void cur_skip(Cursor& c, const Params& p) {
  while (!c.done && c.u >= c.u_end) {
    if (++c.gi == 4) {
      c.gi = 0;
      if (++c.layer == p.num_layers) {
        c.done = true;
        break;
      }
    }
    cur_load(c, p);
  }
}
__device__ __forceinline__ void cur_init(Cursor& c, const Params& p) {
  c.layer = 0; c.gi = 0; c.done = false;
  cur_load(c, p);
  cur_skip(c, p);
}
__device__ __forceinline__ void cur_next(Cursor& c, const Params& p) {
  ++c.u;
  cur_skip(c, p);
}
// partial slots of weight tile `tile`: CTAs first..last own a piece of its k range
__device__ __forceinline__ int tile_first_cta(const GemmShape& g, int tile) { return (tile * g.kbt) / g.U; }
__device__ __forceinline__ int tile_num_segs(const GemmShape& g, int tile) {
  return ((tile + 1) * g.kbt - 1) / g.U - (tile * g.kbt) / g.U + 1;
}

// ----------------------------------------------------------------- bounded waits
struct Shared {
  uint64_t* fullW;
  uint64_t* fullX;
  uint64_t* empty;
  uint64_t* tfull;
  uint64_t* tempty;
  uint32_t* tmem_slot;
  volatile int* abort_flag;
  volatile int* phase_open;
  volatile int* attn_done;              // attention phases this CTA has finished (the ring is the producer's again)
};

__device__ __forceinline__ void raise_abort(const Params& p, const Shared& sh, int code) {
  *sh.abort_flag = 1;
  atomicExch(p.ctrl + 3, 1);
  if (p.status) atomicCAS(p.status, ST_OK, code);
}

// Bounded mbarrier wait that polls: the waits of this kernel sit on the critical path of every phase
// and the waiting warps have nothing else to run.
__device__ __forceinline__ bool mbar_spin(uint64_t* bar, uint32_t parity, const Params& p, const Shared& sh,
                                          int code) {
#pragma unroll 1
  for (int it = 0; it < 256; ++it)
    if (mbar_test(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
#pragma unroll 1
  for (uint32_t it = 0;; ++it) {
    if (mbar_test(bar, parity)) return true;
    if ((it & 63u) == 63u) {
      if (*sh.abort_flag) return false;
      if (global_timer_ns() - t0 > B200_WAIT_LIMIT_NS) break;
    }
  }
  raise_abort(p, sh, code);
  return false;
}

// named barrier of the 128 compute threads (warps 2..5)
__device__ __forceinline__ void cbar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Grid barrier: arrival number `target` of the monotonic counter ctrl[0].  Called by all 128 compute
// threads; returns false when the grid aborted.
__device__ __forceinline__ bool grid_barrier(const Params& p, const Shared& sh, int target, int ct) {
  __threadfence();
  cbar();
  if (ct == 0) {
    // the last CTA to arrive publishes the barrier number in a word of its own (ctrl[32], another
    // cache line), so that the pollers do not fight the arriving atomics for the counter's line
    const int gen = target / (int)gridDim.x;
    if (atomicAdd(p.ctrl, 1) + 1 == target) st_release_gpu(p.ctrl + 32, gen);
    const unsigned long long t0 = global_timer_ns();
    bool ok = false;
#pragma unroll 1
    for (uint32_t it = 0;; ++it) {
      if (ld_acquire_gpu(p.ctrl + 32) - gen >= 0) { ok = true; break; }
      if ((it & 15u) == 15u) {
        if (*sh.abort_flag || *reinterpret_cast<volatile int*>(p.ctrl + 3)) break;
        if (global_timer_ns() - t0 > B200_WAIT_LIMIT_NS) {
          raise_abort(p, sh, ST_TIMEOUT_FLAG);
          break;
        }
      }
    }
    if (!ok) *sh.abort_flag = 1;
    __threadfence();
  }
  cbar();
  return !*sh.abort_flag;
}

__device__ __forceinline__ void stamp_ev(const Params& p, int layer, int gi, int ev) {
  if (p.dbg != nullptr && layer == p.dbg_layer && gi == p.dbg_gi)
    p.dbg[(size_t)(p.dbg_ev_base + ev) * gridDim.x + blockIdx.x] = global_timer_ns();
}

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

// Sum of the fp32 partials of 8 consecutive columns [n, n+8) of row t of a projection, in slot order.
// The loads of four slots are issued together: a consumer phase is a chain of L2 round trips otherwise.
__device__ __forceinline__ void sum_partials8(const float* part, const GemmShape& g, int t, int n, float (&acc)[8]) {
  const int tile = n / BM;
  const int ns = tile_num_segs(g, tile);
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  const size_t seg_stride = (size_t)MAXT * g.N;
  const float* base = part + (size_t)t * g.N + n;
  for (int s0 = 0; s0 < ns; s0 += 4) {
    float4 a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (s0 + i < ns) {
        const float4* src = reinterpret_cast<const float4*>(base + (size_t)(s0 + i) * seg_stride);
        a[i] = __ldcg(src);
        b[i] = __ldcg(src + 1);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (s0 + i < ns) {
        acc[0] += a[i].x; acc[1] += a[i].y; acc[2] += a[i].z; acc[3] += a[i].w;
        acc[4] += b[i].x; acc[5] += b[i].y; acc[6] += b[i].z; acc[7] += b[i].w;
      }
    }
  }
}

// ----------------------------------------------------------------- phases run by the compute warps
// residual + sum -> residual; RMSNorm -> h.  Source of the sum: nothing (layer 0: x = hidden0), the
// split-K partials of projection `src_g` (one rank), or the receive slab `slab` (tensor parallel).
__device__ __noinline__ void phase_norm(const Params& p, const Shared& sh, uint8_t* smem, int ct, int layer, bool first,
                           int src_g, int slab, int use_idx, const __nv_bfloat16* weight, bool write_h) {
  // locals: fields read through the references would be re-read after every global store
  float* const red = reinterpret_cast<float*>(smem + RED_OFF);
  const int H = p.H, T = p.T, world = p.world;
  const float eps = p.eps;
  const GemmShape g = p.g[src_g];
  const float* const part = p.part;
  const __nv_bfloat16* const hidden0 = p.hidden0;
  __nv_bfloat16* const residual = p.residual;
  __nv_bfloat16* const hbuf = p.h;
  const uint8_t* const recv = world > 1 ? p.peer[p.rank] + p.slab_off[slab] : nullptr;
  const int* const flags = world > 1 ? reinterpret_cast<const int*>(p.peer[p.rank] + p.flag_off[slab]) : nullptr;
  const unsigned int spin_limit = p.spin_limit;
  volatile int* const abort_flag = sh.abort_flag;
  const int nvec = H >> 3;
  const size_t seg_stride = (size_t)MAXT * g.N;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    if (!first && world > 1) {
      // the partial rows of every rank (this one included) arrive as quarter rows with one flag each
      if (ct < world * 4) {
        const int* f = flags + (ct >> 2) * (MAXT * 4) + t * 4 + (ct & 3);
        if (!wait_flag_ge(f, use_idx, p.status, spin_limit)) raise_abort(p, sh, ST_TIMEOUT_FLAG);
      }
      cbar();
      if (*abort_flag) return;
    }
    float ss = 0.f;
    // two vectors per pass, every load of a pass in flight together (a pass costs one L2 round trip)
#pragma unroll 1
    for (int u0 = 0; u0 < 8; u0 += 2) {
      if (ct + u0 * 128 >= nvec) break;
      bf16x8 xs[2];
      if (first) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int v = ct + (u0 + k) * 128;
          if (v < nvec) xs[k] = *reinterpret_cast<const bf16x8*>(hidden0 + (size_t)t * H + v * 8);
        }
      } else {
        float acc[2][8];
        bf16x8 res[2];
        if (world > 1) {
          uint4 raw[2][8];
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const int v = ct + (u0 + k) * 128;
            if (v >= nvec) continue;
            res[k] = *reinterpret_cast<const bf16x8*>(residual + (size_t)t * H + v * 8);
#pragma unroll
            for (int r = 0; r < 8; ++r)
              if (r < world) raw[k][r] = ld_relaxed_sys_v4(recv + (((size_t)r * MAXT + t) * H + v * 8) * 2);
          }
#pragma unroll
          for (int k = 0; k < 2; ++k) {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[k][j] = 0.f;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
              if (r < world) {
                const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw[k][r]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 f = __bfloat1622float2(hh[j]);
                  acc[k][2 * j] += f.x;
                  acc[k][2 * j + 1] += f.y;
                }
              }
            }
          }
        } else {
          float4 pa[2][MAX_SLOTS], pb[2][MAX_SLOTS];
          int ns[2] = {0, 0};
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const int v = ct + (u0 + k) * 128;
            if (v >= nvec) continue;
            res[k] = *reinterpret_cast<const bf16x8*>(residual + (size_t)t * H + v * 8);
            ns[k] = tile_num_segs(g, (v * 8) / BM);
            const float* base = part + (size_t)t * g.N + v * 8;
#pragma unroll
            for (int sl = 0; sl < MAX_SLOTS; ++sl)
              if (sl < ns[k]) {
                const float4* src = reinterpret_cast<const float4*>(base + (size_t)sl * seg_stride);
                pa[k][sl] = __ldcg(src);
                pb[k][sl] = __ldcg(src + 1);
              }
          }
#pragma unroll
          for (int k = 0; k < 2; ++k) {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[k][j] = 0.f;
#pragma unroll
            for (int sl = 0; sl < MAX_SLOTS; ++sl)
              if (sl < ns[k]) {
                acc[k][0] += pa[k][sl].x; acc[k][1] += pa[k][sl].y; acc[k][2] += pa[k][sl].z; acc[k][3] += pa[k][sl].w;
                acc[k][4] += pb[k][sl].x; acc[k][5] += pb[k][sl].y; acc[k][6] += pb[k][sl].z; acc[k][7] += pb[k][sl].w;
              }
          }
        }
        // same roundings as a bf16 projection output followed by the bf16 residual add
#pragma unroll
        for (int k = 0; k < 2; ++k) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 fa = __bfloat1622float2(__floats2bfloat162_rn(acc[k][2 * j], acc[k][2 * j + 1]));
            const float2 fr = __bfloat1622float2(res[k].v[j]);
            xs[k].v[j] = __floats2bfloat162_rn(fa.x + fr.x, fa.y + fr.y);
          }
        }
      }
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int v = ct + (u0 + k) * 128;
        if (v >= nvec) continue;
        *reinterpret_cast<bf16x8*>(residual + (size_t)t * H + v * 8) = xs[k];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(xs[k].v[j]);
          ss += f.x * f.x + f.y * f.y;
        }
      }
    }
    if (!write_h) continue;
    // block sum over the 128 compute threads
    ss = warp_sum(ss);
    if ((ct & 31) == 0) red[ct >> 5] = ss;
    cbar();
    const float tot = red[0] + red[1] + red[2] + red[3];
    cbar();
    const float inv = rsqrtf(tot / (float)H + eps);
    // second pass over the row this thread just wrote (its own stores: L1 / L2 hits, all in flight)
    bf16x8 xr[8], wr[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int v = ct + u * 128;
      if (v < nvec) {
        xr[u] = *reinterpret_cast<const bf16x8*>(residual + (size_t)t * H + v * 8);
        wr[u] = *reinterpret_cast<const bf16x8*>(weight + v * 8);
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int v = ct + u * 128;
      if (v >= nvec) break;
      bf16x8 y;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(xr[u].v[j]), g2 = __bfloat1622float2(wr[u].v[j]);
        y.v[j] = __floats2bfloat162_rn(f.x * inv * g2.x, f.y * inv * g2.y);
      }
      *reinterpret_cast<bf16x8*>(hbuf + (size_t)t * H + v * 8) = y;
    }
  }
  (void)layer;
}

// Tensor parallel: sum the split-K partials of a row-parallel projection, round to bf16 and store the
// quarter row into the receive slab of every rank, then raise that quarter's flag there.
__device__ __noinline__ void phase_push(const Params& p, const Shared& sh, int ct, int src_g, int slab, int use_idx) {
  const int H = p.H, T = p.T, world = p.world, rank = p.rank;
  const GemmShape g = p.g[src_g];
  const float* const part = p.part;
  uint8_t* peer[8];
#pragma unroll
  for (int r = 0; r < 8; ++r) peer[r] = p.peer[r];
  const unsigned long long slab_off = p.slab_off[slab], flag_off = p.flag_off[slab];
  const int qv = (H >> 3) >> 2;                       // 16-byte vectors per quarter row
  const int units = T * 4;
  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const int t = u >> 2, q = u & 3;
    for (int v = ct; v < qv; v += 128) {
      const int n = (q * qv + v) * 8;
      float acc[8];
      sum_partials8(part, g, t, n, acc);
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < world) {
          int d = rank + r;                              // start with this rank, spread the links
          if (d >= world) d -= world;
          *reinterpret_cast<uint4*>(peer[d] + slab_off + (((size_t)rank * MAXT + t) * H + n) * 2) = o;
        }
      }
    }
    __threadfence_system();
    cbar();
    if (ct < world)
      st_release_sys(reinterpret_cast<int*>(p.peer[ct] + flag_off) + rank * (MAXT * 4) + u, use_idx);
  }
  (void)sh;
}

// act = silu(gate) * up from the partials of the gate/up projection (columns [0, I) gate, [I, 2I) up)
__device__ __noinline__ void phase_swiglu(const Params& p, int ct) {
  const int I = p.I, T = p.T;
  const GemmShape g = p.g[2];
  const float* const part = p.part;
  __nv_bfloat16* const act = p.act;
  const int nvec = I >> 3;
  const int total = T * nvec;
  const int stride = (int)gridDim.x * 128;
  for (int idx = blockIdx.x * 128 + ct; idx < total; idx += stride) {
    const int t = idx / nvec, v = idx - t * nvec;
    float g8[8], u8[8];
    sum_partials8(part, g, t, v * 8, g8);
    sum_partials8(part, g, t, I + v * 8, u8);
    bf16x8 y;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      y.v[j] = __floats2bfloat162_rn(silu(g8[2 * j]) * u8[2 * j], silu(g8[2 * j + 1]) * u8[2 * j + 1]);
    *reinterpret_cast<bf16x8*>(act + (size_t)t * I + v * 8) = y;
  }
}

// The fields of Params / LayerDesc the attention phase uses, copied once per phase: the phase functions
// are separate (not inlined) to keep their registers apart, and a field read through a reference would
// be re-read from memory after every global store.
struct AttnArgs {
  const float* part;
  const int* positions;
  const int* slot_mapping;
  const int* block_tables;
  const int* seq_lens;
  const float* inv_freq;
  const __nv_bfloat16* qkv_bias;
  const __nv_bfloat16* q_norm;
  const __nv_bfloat16* k_norm;
  __nv_bfloat16* kv_cache;
  __nv_bfloat16* o;
  float* part_o;
  float* part_ml;
  int* counters;
  long long num_blocks;
  GemmShape gq;
  int Hq, Hkv, G, Z, rot_pairs, interleaved, max_blocks, block_size;
  float eps, scale_log2;
};

__device__ __forceinline__ void attn_warp_unit(const AttnArgs& p, uint8_t* smem, int lw, int lane, int r, int h,
                                               int z) {
  const int G = p.G;
  const int t = r;
  const int seq_len = p.seq_lens[r];
  if (seq_len <= 0) return;                                   // padded request (uniform for the warp)
  const int ctx = seq_len - 1;
  const int Z = p.Z;
  uint8_t* ring = smem + ATT_OFF + lw * ATT_WARP_BYTES;
  // q rows and cos / sin live in the ring until the fragments are in registers
  __nv_bfloat16* s_q = reinterpret_cast<__nv_bfloat16*>(ring);             // [16][D] bf16
  float* cs = reinterpret_cast<float*>(ring + 16 * D * 2);                  // cos | sin
  const GemmShape gq = p.gq;
  const __nv_bfloat16* const qkv_bias = p.qkv_bias;
  const __nv_bfloat16* const q_norm = p.q_norm;
  const __nv_bfloat16* const k_norm = p.k_norm;
  __nv_bfloat16* const kv_cache = p.kv_cache;
  const int C = (seq_len + 15) >> 4;
  const int per = (C + Z - 1) / Z;
  const int cb0 = min(C, z * per);
  const int cb1 = min(C, (z + 1) * per);
  const bool write_kv = (z == (C - 1) / per);               // this split reads the new token's K / V

  // ---- prologue
  {
    const float pos = (float)p.positions[t];
    for (int i = lane; i < p.rot_pairs; i += 32) {
      float sn, c;
      sincosf(pos * p.inv_freq[i], &sn, &c);
      cs[i] = c;
      cs[D / 2 + i] = sn;
    }
    for (int i = lane; i < (16 - G) * D / 2; i += 32) reinterpret_cast<uint32_t*>(s_q + G * D)[i] = 0u;
    __syncwarp();
    const long long slot = p.slot_mapping[t];
    const int nrows = write_kv ? G + 2 : G;
    constexpr int EPL = D / 32;
    int idx[EPL];
#pragma unroll
    for (int u = 0; u < EPL / 2; ++u) {
      const int i = lane * (EPL / 2) + u;
      if (p.interleaved) { idx[2 * u] = 2 * i; idx[2 * u + 1] = 2 * i + 1; }
      else { idx[2 * u] = i; idx[2 * u + 1] = i + D / 2; }
    }
    const size_t seg_stride = (size_t)MAXT * gq.N;
    constexpr int RG = 3;                      // head rows per group of loads
#pragma unroll 1
    for (int j0 = 0; j0 < nrows; j0 += RG) {
      float x[RG][EPL];
      int head_col[RG];
      {
        float v[RG][MAX_SLOTS][EPL];
        int ns[RG];
#pragma unroll
        for (int k = 0; k < RG; ++k) {
          const int j = j0 + k;
          head_col[k] = j < G ? (h * G + j) : (j == G ? p.Hq + h : p.Hq + p.Hkv + h);     // n tile index
          ns[k] = j < nrows ? tile_num_segs(gq, head_col[k]) : 0;
          const float* base = p.part + (size_t)t * gq.N + head_col[k] * D;
#pragma unroll
          for (int sl = 0; sl < MAX_SLOTS; ++sl)
            if (sl < ns[k]) {
#pragma unroll
              for (int u = 0; u < EPL; ++u) v[k][sl][u] = __ldcg(base + (size_t)sl * seg_stride + idx[u]);
            }
        }
#pragma unroll
        for (int k = 0; k < RG; ++k) {
#pragma unroll
          for (int u = 0; u < EPL; ++u) x[k][u] = 0.f;
#pragma unroll
          for (int sl = 0; sl < MAX_SLOTS; ++sl)
            if (sl < ns[k]) {
#pragma unroll
              for (int u = 0; u < EPL; ++u) x[k][u] += v[k][sl][u];
            }
        }
      }
#pragma unroll
      for (int k = 0; k < RG; ++k) {
        const int j = j0 + k;
        if (j >= nrows) break;
        const int kind = j < G ? 0 : (j == G ? 1 : 2);
#pragma unroll
        for (int u = 0; u < EPL; ++u) {
          if (qkv_bias != nullptr) x[k][u] += __bfloat162float(qkv_bias[head_col[k] * D + idx[u]]);
          x[k][u] = __bfloat162float(__float2bfloat16(x[k][u]));          // the projection's bf16 output
        }
        if (kind < 2) {
          const __nv_bfloat16* nwp = kind == 0 ? q_norm : k_norm;
          if (nwp != nullptr) {
            float ss = 0.f;
#pragma unroll
            for (int u = 0; u < EPL; ++u) ss += x[k][u] * x[k][u];
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / (float)D + p.eps);
#pragma unroll
            for (int u = 0; u < EPL; ++u)
              x[k][u] = __bfloat162float(__float2bfloat16(x[k][u] * inv * __bfloat162float(nwp[idx[u]])));
          }
#pragma unroll
          for (int u = 0; u < EPL / 2; ++u) {
            const int i = lane * (EPL / 2) + u;
            if (i < p.rot_pairs) {
              const float c = cs[i], sn = cs[D / 2 + i];
              const float a = x[k][2 * u], b = x[k][2 * u + 1];
              x[k][2 * u] = a * c - b * sn;
              x[k][2 * u + 1] = b * c + a * sn;
            }
          }
        }
        if (kind == 0) {
#pragma unroll
          for (int u = 0; u < EPL; ++u) s_q[j * D + idx[u]] = __float2bfloat16(x[k][u]);
        } else if (slot >= 0 && slot < p.num_blocks * p.block_size) {
          const long long blk = slot / p.block_size;
          const int off = (int)(slot - blk * p.block_size);
          __nv_bfloat16* dst = kv_cache + ((((size_t)blk * 2 + (kind - 1)) * p.Hkv + h) * p.block_size + off) * D;
#pragma unroll
          for (int u = 0; u < EPL; ++u) dst[idx[u]] = __float2bfloat16(x[k][u]);
        }
      }
    }
    __threadfence();                 // the new K/V row is read back through L2 by this warp's cp.async
    __syncwarp();
  }

  // ---- Q fragments: tile row g = q head g of this kv head's group
  uint32_t qf[D / 16][4];
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
    const int cb = 2 * (lane & 3);
    const __nv_bfloat16* q0 = s_q + r0 * D;
    const __nv_bfloat16* q1 = s_q + r1 * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qf[ks][0] = *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + cb);
      qf[ks][1] = *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + cb);
      qf[ks][2] = *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + cb);
      qf[ks][3] = *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + cb);
    }
  }
  __syncwarp();                      // the ring may be overwritten from here on

  const uint32_t wbase = smem_u32(ring);
  const int* bt = p.block_tables + (size_t)r * p.max_blocks;
  const size_t head_stride = (size_t)p.block_size * D;
  const int page_lo = (cb0 << 4) / p.block_size;
  const int page_hi = cb1 > cb0 ? (((cb1 << 4) - 1) / p.block_size) : page_lo - 1;
  int bt_base = page_lo;
  int bt_reg = (page_lo + lane <= page_hi) ? bt[page_lo + lane] : 0;
  const __nv_bfloat16* kv = kv_cache;
  auto issue = [&](int chunk, int stage) {
    const int tok = chunk << 4;
    const int page = tok / p.block_size, off = tok - page * p.block_size;
    if (page >= bt_base + 32) {
      bt_base = page;
      bt_reg = (page + lane <= page_hi) ? bt[page + lane] : 0;
    }
    long long blk = __shfl_sync(0xffffffffu, bt_reg, page - bt_base);
    if (blk < 0 || blk >= p.num_blocks) blk = 0;
    const size_t ko = (((size_t)blk * 2 + 0) * p.Hkv + h) * head_stride + (size_t)off * D;
    const size_t vo = (((size_t)blk * 2 + 1) * p.Hkv + h) * head_stride + (size_t)off * D;
    const uint32_t sb = wbase + stage * ATT_STAGE_BYTES;
    load_rows_async<D, 32>(sb, kv + ko, 16, lane);
    load_rows_async<D, 32>(sb + ATT_PAGE_BYTES, kv + vo, 16, lane);
  };

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const int row0 = lane >> 2, row1 = row0 + 8;
  const int lim = ctx;                                         // one query per request: last visible key

#pragma unroll
  for (int s = 0; s < ATT_STAGES - 1; ++s) {
    if (cb0 + s < cb1) issue(cb0 + s, s);
    cp_async_commit();
  }
  for (int c = cb0; c < cb1; ++c) {
    const int stage = (c - cb0) % ATT_STAGES;
    cp_async_wait<ATT_STAGES - 2>();
    __syncwarp();
    if (c + ATT_STAGES - 1 < cb1) issue(c + ATT_STAGES - 1, (c - cb0 + ATT_STAGES - 1) % ATT_STAGES);
    cp_async_commit();
    const uint32_t sb = wbase + stage * ATT_STAGE_BYTES;
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    qk_16<D>(s, qf, sb, lane);
    const int tk = (c << 4) + 2 * (lane & 3);
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = tk + nb * 8 + (e & 1);
        float v = s[nb][e] * p.scale_log2;
        v = tok <= lim ? v : -INFINITY;
        s[nb][e] = v;
        if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
    const float base0 = mn0 == -INFINITY ? 0.f : mn0, base1 = mn1 == -INFINITY ? 0.f : mn1;
    const float a0 = ex2(m[0] - base0), a1 = ex2(m[1] - base1);
    m[0] = mn0; m[1] = mn1;
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      s[nb][0] = ex2(s[nb][0] - base0); s[nb][1] = ex2(s[nb][1] - base0);
      s[nb][2] = ex2(s[nb][2] - base1); s[nb][3] = ex2(s[nb][3] - base1);
      ps0 += s[nb][0] + s[nb][1];
      ps1 += s[nb][2] + s[nb][3];
    }
    l[0] = l[0] * a0 + ps0;
    l[1] = l[1] * a1 + ps1;
    if (__any_sync(0xffffffffu, a0 != 1.f || a1 != 1.f)) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1;
      }
    }
    uint32_t pa[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]), pack_bf16(s[1][0], s[1][1]),
                      pack_bf16(s[1][2], s[1][3])};
    pv_16<D>(o, pa, sb + ATT_PAGE_BYTES, lane);
  }
  cp_async_wait<0>();
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1); l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1); l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
  __syncwarp();

  // rows of the tile held by this lane: row0 (accumulator halves 0, 1) and row0 + 8 (halves 2, 3);
  // columns i * 8 + 2 * (lane & 3) + {0, 1}
  const int cq = 2 * (lane & 3);
  if (Z == 1) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = half ? row1 : row0;
      if (row >= G) continue;
      const float inv = l[half] > 0.f ? 1.f / l[half] : 0.f;
      __nv_bfloat16* dst = p.o + ((size_t)t * p.Hq + h * G + row) * D + cq;
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][2 * half] * inv, o[i][2 * half + 1] * inv);
    }
    return;
  }
  // ---- cross-split merge by the warp that arrives last on this (request, kv head)
  const size_t unit = ((size_t)r * p.Hkv + h) * Z;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = half ? row1 : row0;
    if (row >= G) continue;
    float* po = p.part_o + ((unit + z) * 16 + row) * D + cq;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) *reinterpret_cast<float2*>(po + i * 8) = make_float2(o[i][2 * half], o[i][2 * half + 1]);
    if ((lane & 3) == 0) {
      p.part_ml[((unit + z) * 16 + row) * 2 + 0] = m[half];
      p.part_ml[((unit + z) * 16 + row) * 2 + 1] = l[half];
    }
  }
  __threadfence();
  __syncwarp();
  int last = 0;
  if (lane == 0) last = (atomicAdd(&p.counters[r * p.Hkv + h], 1) == Z - 1);
  last = __shfl_sync(0xffffffffu, last, 0);
  if (!last) return;
  __threadfence();
  // lane owns 4 columns of every row of the group
  for (int row = 0; row < G; ++row) {
    float mfin = -INFINITY;
    for (int s2 = 0; s2 < Z; ++s2) mfin = fmaxf(mfin, __ldcg(&p.part_ml[((unit + s2) * 16 + row) * 2]));
    float Lfin = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s2 = 0; s2 < Z; ++s2) {
      const float ms = __ldcg(&p.part_ml[((unit + s2) * 16 + row) * 2]);
      const float sc = (ms == -INFINITY) ? 0.f : ex2(ms - mfin);
      Lfin += __ldcg(&p.part_ml[((unit + s2) * 16 + row) * 2 + 1]) * sc;
      const float4 v = __ldcg(reinterpret_cast<const float4*>(p.part_o + ((unit + s2) * 16 + row) * D) + lane);
      acc.x += v.x * sc; acc.y += v.y * sc; acc.z += v.z * sc; acc.w += v.w * sc;
    }
    const float inv = Lfin > 0.f ? 1.f / Lfin : 0.f;
    uint2 pk;
    pk.x = pack_bf16(acc.x * inv, acc.y * inv);
    pk.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(p.o + ((size_t)t * p.Hq + h * G + row) * D + 4 * lane) = pk;
  }
  if (lane == 0) p.counters[r * p.Hkv + h] = 0;
}

__device__ __noinline__ void phase_attn(const Params& p, const Shared& sh, uint8_t* smem, const LayerDesc& L, int ct) {
  AttnArgs a;
  a.part = p.part; a.positions = p.positions; a.slot_mapping = p.slot_mapping; a.block_tables = p.block_tables;
  a.seq_lens = p.seq_lens; a.inv_freq = p.inv_freq; a.qkv_bias = L.qkv_bias; a.q_norm = L.q_norm;
  a.k_norm = L.k_norm; a.kv_cache = L.kv_cache; a.o = p.o; a.part_o = p.attn_part_o; a.part_ml = p.attn_part_ml;
  a.counters = p.attn_counters; a.num_blocks = p.num_blocks; a.gq = p.g[0]; a.Hq = p.Hq; a.Hkv = p.Hkv;
  a.G = p.Hq / p.Hkv; a.Z = p.kv_splits; a.rot_pairs = p.rot_pairs; a.interleaved = p.interleaved;
  a.max_blocks = p.max_blocks; a.block_size = p.block_size; a.eps = p.eps; a.scale_log2 = p.scale_log2;
  const int lw = ct >> 5, lane = ct & 31;
  const int total = p.T * a.Hkv * a.Z;
  const int stride = (int)gridDim.x * 4;
  volatile int* abort_flag = sh.abort_flag;
  for (int u = blockIdx.x * 4 + lw; u < total && !*abort_flag; u += stride) {
    const int z = u % a.Z, rh = u / a.Z;
    attn_warp_unit(a, smem, lw, lane, rh / a.Hkv, rh % a.Hkv, z);
    __syncwarp();
  }
}

// Epilogue of a GEMM phase: the accumulator of every segment of this CTA's range goes to its fp32
// partial slot [seg][t][n] (thread = weight row n, 32 token columns per TMEM load).
__device__ __noinline__ void phase_gemm_epilogue(const Params& p, const Shared& sh, int warp, int lane, int gi, uint32_t tmem_base,
                                    int& segcount_io, int layer) {
  // locals: fields read through the references would be re-read after every global store
  const GemmShape g = p.g[gi];
  const int T = p.T;
  float* const part = p.part;
  uint64_t* const tfull = sh.tfull;
  uint64_t* const tempty = sh.tempty;
  int segcount = segcount_io;
  const int q = warp & 3;
  const int row = q * 32 + lane;
  int u = min(g.total, (int)blockIdx.x * g.U);
  const int u_end = min(g.total, u + g.U);
  while (u < u_end) {
    const int tile = u / g.kbt;
    const int seg_end = min(u_end, (tile + 1) * g.kbt);
    const int slot = (int)blockIdx.x - tile_first_cta(g, tile);
    const int acc = segcount & 1;
    const uint32_t acc_ph = (segcount >> 1) & 1;
    if (warp == 2 && lane == 0) stamp_ev(p, layer, gi, 0);
    if (!mbar_spin(&tfull[acc], acc_ph, p, sh, ST_TIMEOUT_TMEM_FULL)) break;
    if (warp == 2 && lane == 0) stamp_ev(p, layer, gi, 4);
    tc_fence_after();
    const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
    const int n = tile * BM + row;
    float* dst = part + (size_t)slot * MAXT * g.N + n;
    const size_t ldn = (size_t)g.N;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
      if (c0 >= T) break;
      uint32_t r[32];
      tmem_ld_32x32(taddr + c0, r);
      tmem_ld_wait();
      if (n < g.N) {
        if (c0 + 32 <= T) {
#pragma unroll
          for (int j = 0; j < 32; ++j) dst[(size_t)(c0 + j) * ldn] = __uint_as_float(r[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j < T) dst[(size_t)(c0 + j) * ldn] = __uint_as_float(r[j]);
        }
      }
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&tempty[acc]);
    if (warp == 2 && lane == 0) stamp_ev(p, layer, gi, 5);
    ++segcount;
    u = seg_end;
  }
  segcount_io = segcount;
}

__global__ void __launch_bounds__(THREADS, 1)
decode_layers_kernel(const __grid_constant__ CUtensorMap tmH, const __grid_constant__ CUtensorMap tmO,
                     const __grid_constant__ CUtensorMap tmAct, const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + BAR_OFF);
  Shared sh;
  sh.fullW = bars;
  sh.fullX = bars + STAGES;
  sh.empty = bars + 2 * STAGES;
  sh.tfull = bars + 3 * STAGES;
  sh.tempty = bars + 3 * STAGES + 2;
  sh.tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * STAGES + 4);
  sh.abort_flag = reinterpret_cast<volatile int*>(sh.tmem_slot + 1);
  sh.phase_open = reinterpret_cast<volatile int*>(sh.tmem_slot + 2);
  sh.attn_done = reinterpret_cast<volatile int*>(sh.tmem_slot + 3);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sh.fullW[s], 1);
      mbar_init(&sh.fullX[s], 1);
      mbar_init(&sh.empty[s], 1);
    }
    mbar_init(&sh.tfull[0], 1);
    mbar_init(&sh.tfull[1], 1);
    mbar_init(&sh.tempty[0], 4);
    mbar_init(&sh.tempty[1], 4);
    *sh.abort_flag = 0;
    *sh.phase_open = 0;
    *sh.attn_done = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmH);
    tma_prefetch_desc(&tmO);
    tma_prefetch_desc(&tmAct);
  }
  if (warp == 1) {
    tmem_alloc(sh.tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *sh.tmem_slot;
  const int G = (int)gridDim.x;
  const int ppl = phases_per_layer(p);

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (elect_one()) {
      Cursor wc, xc;
      cur_init(wc, p);
      cur_init(xc, p);
      int wcount = 0, xcount = 0, acquired = -1;
      unsigned long long t_idle = 0;
      while (!xc.done) {
        bool progressed = false;
        // weights behind an attention phase wait until this CTA's attention has given the ring back
        if (!wc.done && wcount - xcount < STAGES && *sh.attn_done >= wc.layer + (wc.gi >= 1 ? 1 : 0)) {
          const int s = wcount % STAGES;
          const uint32_t ph = (uint32_t)(wcount / STAGES) & 1u;
          if (mbar_test(&sh.empty[s], ph ^ 1u)) {
            const GemmShape& g = p.g[wc.gi];
            const int tile = wc.u / g.kbt, kb = wc.u - tile * g.kbt;
            mbar_expect_tx(&sh.fullW[s], A_BYTES);
            tma_load_2d_hint(smem + s * STAGE_BYTES, &p.layers[wc.layer].tm[wc.gi], &sh.fullW[s], kb * BK, tile * BM,
                             L2_EVICT_FIRST);
            ++wcount;
            cur_next(wc, p);
            progressed = true;
          }
        }
        if (xcount < wcount) {
          const int ph_idx = gemm_phase(p, xc.layer, xc.gi);
          if (*sh.phase_open >= ph_idx) {
            const bool acquired_new = acquired != ph_idx;
            if (acquired != ph_idx) {
              // the operand was written by other CTAs (generic proxy; this CTA acquired the barrier
              // that follows their writes) and is read by TMA (async proxy)
              asm volatile("fence.proxy.async;" ::: "memory");
              acquired = ph_idx;
            }
            const GemmShape& g = p.g[xc.gi];
            const int tile = xc.u / g.kbt, kb = xc.u - tile * g.kbt;
            const int s = xcount % STAGES;
            const CUtensorMap* tx = xc.gi == 1 ? &tmO : (xc.gi == 3 ? &tmAct : &tmH);
            if (acquired_new) stamp_ev(p, xc.layer, xc.gi, 1);
            mbar_expect_tx(&sh.fullX[s], B_BYTES);
            tma_load_2d(smem + s * STAGE_BYTES + A_BYTES, tx, &sh.fullX[s], kb * BK, 0);
            ++xcount;
            cur_next(xc, p);
            progressed = true;
          }
        }
        if (progressed) {
          t_idle = 0;
        } else {
          if (*sh.abort_flag) break;
          __nanosleep(64);
          const unsigned long long now = global_timer_ns();
          if (t_idle == 0) t_idle = now;
          else if (now - t_idle > 2 * B200_WAIT_LIMIT_NS) {
            raise_abort(p, sh, ST_TIMEOUT_EMPTY);
            break;
          }
        }
      }
      if (*sh.abort_flag) {
        // give this CTA's bulk copies in flight a bounded time to land before the CTA exits
        for (int it = 0; it < 20000; ++it) __nanosleep(100);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
      Cursor mc;
      cur_init(mc, p);
      int count = 0, segcount = 0;
      bool ok = true;
      while (!mc.done && ok) {
        const int layer = mc.layer, gi = mc.gi;
        const int kbt = p.g[gi].kbt;
        const int tile = mc.u / kbt;
        const int acc = segcount & 1;
        const uint32_t acc_ph = (segcount >> 1) & 1;
        if (!mbar_spin(&sh.tempty[acc], acc_ph ^ 1, p, sh, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool first = true;
        do {
          const int s = count % STAGES;
          const uint32_t ph = (uint32_t)(count / STAGES) & 1u;
          if (!mbar_spin(&sh.fullW[s], ph, p, sh, ST_TIMEOUT_FULL) ||
              !mbar_spin(&sh.fullX[s], ph, p, sh, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (first) stamp_ev(p, layer, gi, 2);
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t adesc = umma_desc_k_sw128(a_addr);
          const uint64_t bdesc = umma_desc_k_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (!first || k > 0) ? 1u : 0u);
          umma_commit(&sh.empty[s]);
          first = false;
          ++count;
          cur_next(mc, p);
        } while (!mc.done && mc.layer == layer && mc.gi == gi && mc.u / kbt == tile);
        if (ok) umma_commit(&sh.tfull[acc]);
        stamp_ev(p, layer, gi, 3);
        ++segcount;
      }
    }
  } else {
    // ------------------------------------------------- compute warps: phases in program order
    const int ct = threadIdx.x - 64;
    const int epoch = *reinterpret_cast<volatile int*>(p.ctrl + 2);
    int segcount = 0;
    int pidx = 0;
    bool alive = true;
    // every phase ends with a grid barrier, except a push (the norm after it waits on peer flags);
    // the barrier count must be the same on every CTA, so `barriers` counts them
    int barriers = 0;
    auto sync_phase = [&](bool barrier) {
      if (p.dbg != nullptr && ct == 0) p.dbg[(size_t)(2 * pidx) * gridDim.x + blockIdx.x] = global_timer_ns();
      if (barrier) {
        ++barriers;
        alive = grid_barrier(p, sh, barriers * G, ct);
      } else {
        cbar();
        alive = !*sh.abort_flag;
      }
      if (p.dbg != nullptr && ct == 0) p.dbg[(size_t)(2 * pidx + 1) * gridDim.x + blockIdx.x] = global_timer_ns();
      ++pidx;
      if (ct == 0) *sh.phase_open = pidx;
      cbar();
    };
    for (int l = 0; l < p.num_layers && alive; ++l) {
      const LayerDesc& L = p.layers[l];
      const int use_idx = epoch * p.num_layers + l + 1;
      // input norm: consumes the down projection of the previous layer
      phase_norm(p, sh, smem, ct, l, l == 0, 3, 1, use_idx - 1, L.ln_in, true);
      sync_phase(true);
      if (!alive) break;
      phase_gemm_epilogue(p, sh, warp, lane, 0, tmem_base, segcount, l);
      sync_phase(true);
      if (!alive) break;
      phase_attn(p, sh, smem, L, ct);
      // generic-proxy accesses of the ring are over; the next writer is TMA (async proxy)
      fence_proxy_async_smem();
      cbar();
      if (ct == 0) *sh.attn_done = l + 1;
      sync_phase(true);
      if (!alive) break;
      phase_gemm_epilogue(p, sh, warp, lane, 1, tmem_base, segcount, l);
      sync_phase(true);
      if (!alive) break;
      if (p.world > 1) {
        phase_push(p, sh, ct, 1, 0, use_idx);
        sync_phase(false);
        if (!alive) break;
      }
      phase_norm(p, sh, smem, ct, l, false, 1, 0, use_idx, L.ln_post, true);
      sync_phase(true);
      if (!alive) break;
      phase_gemm_epilogue(p, sh, warp, lane, 2, tmem_base, segcount, l);
      sync_phase(true);
      if (!alive) break;
      phase_swiglu(p, ct);
      sync_phase(true);
      if (!alive) break;
      phase_gemm_epilogue(p, sh, warp, lane, 3, tmem_base, segcount, l);
      sync_phase(true);
      if (!alive) break;
      if (p.world > 1) {
        phase_push(p, sh, ct, 3, 1, use_idx);
        sync_phase(false);
      }
    }
    // the residual stream after the last layer (its final norm belongs to the caller)
    if (alive)
      phase_norm(p, sh, smem, ct, p.num_layers, false, 3, 1, epoch * p.num_layers + p.num_layers, nullptr, false);
    (void)ppl;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 64) {
    __threadfence();
    const int arrived = atomicAdd(p.ctrl + 1, 1) + 1;
    if (arrived == G && !*reinterpret_cast<volatile int*>(p.ctrl + 3)) {
      // every CTA is past its last barrier: re-arm the counters and open the next launch's epoch
      p.ctrl[0] = 0;
      p.ctrl[1] = 0;
      p.ctrl[32] = 0;
      p.ctrl[2] = *reinterpret_cast<volatile int*>(p.ctrl + 2) + 1;
      __threadfence();
    }
  }
}

}  // namespace mega
}  // namespace b200

using namespace b200;
using namespace b200::mega;

extern "C" int b200_make_tmap_2d(void* out_map, const void* ptr, int elem_bytes, uint64_t rows, uint64_t cols,
                                 uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols);

extern "C" int b200_mega_layer_desc_bytes(void) { return (int)sizeof(LayerDesc); }
extern "C" int b200_mega_max_tokens(void) { return MAXT; }

// Fill one LayerDesc in HOST memory (the caller copies the array to the device).  Weights are [N, K]
// bf16 with K-major rows of `ld*` elements; n_qkv = (Hq + 2 Hkv) * 128 rows, i2 = 2 * I rows.
extern "C" int b200_mega_fill_layer(void* desc_host, const void* w_qkv, int n_qkv, int ld_qkv, const void* w_o,
                                    int k_o, int ld_o, const void* w_gu, int i2, int ld_gu, const void* w_down,
                                    int k_down, int ld_down, int H, const void* ln_in, const void* ln_post,
                                    const void* qkv_bias, const void* q_norm, const void* k_norm, void* kv_cache) {
  LayerDesc* d = reinterpret_cast<LayerDesc*>(desc_host);
  memset(d, 0, sizeof(LayerDesc));
  int rc = b200_make_tmap_2d(&d->tm[0], w_qkv, 2, (uint64_t)n_qkv, (uint64_t)H, (uint64_t)ld_qkv * 2, BM, BK);
  if (rc) return rc;
  rc = b200_make_tmap_2d(&d->tm[1], w_o, 2, (uint64_t)H, (uint64_t)k_o, (uint64_t)ld_o * 2, BM, BK);
  if (rc) return rc;
  rc = b200_make_tmap_2d(&d->tm[2], w_gu, 2, (uint64_t)i2, (uint64_t)H, (uint64_t)ld_gu * 2, BM, BK);
  if (rc) return rc;
  rc = b200_make_tmap_2d(&d->tm[3], w_down, 2, (uint64_t)H, (uint64_t)k_down, (uint64_t)ld_down * 2, BM, BK);
  if (rc) return rc;
  d->ln_in = reinterpret_cast<const __nv_bfloat16*>(ln_in);
  d->ln_post = reinterpret_cast<const __nv_bfloat16*>(ln_post);
  d->qkv_bias = reinterpret_cast<const __nv_bfloat16*>(qkv_bias);
  d->q_norm = reinterpret_cast<const __nv_bfloat16*>(q_norm);
  d->k_norm = reinterpret_cast<const __nv_bfloat16*>(k_norm);
  d->kv_cache = reinterpret_cast<__nv_bfloat16*>(kv_cache);
  return 0;
}

static int mega_grid(int num_sms) {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  int& g = cached[dev & 63];
  if (g == 0) {
    if (cudaFuncSetAttribute(decode_layers_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) !=
        cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_layers_kernel, THREADS, SMEM_BYTES) !=
            cudaSuccess || per_sm < 1) {
      cudaGetLastError();
      return 0;
    }
    g = num_sms;          // one CTA per SM: all of them are resident at once (cooperative launch)
  }
  return g;
}

// Bytes of split-K partial scratch the kernel needs for these per-rank shapes on `grid` CTAs.
static size_t plan_gemm(GemmShape& g, int N, int K, int grid) {
  g.N = N; g.K = K;
  g.n_tiles = (N + BM - 1) / BM;
  g.kbt = (K + BK - 1) / BK;
  g.total = g.n_tiles * g.kbt;
  g.U = (g.total + grid - 1) / grid;
  // a consumer sums the partial slots of a tile one round trip per few slots: bound them, even if a
  // small projection then runs on fewer CTAs
  const int min_u = (g.kbt + MAX_SLOTS - 2) / (MAX_SLOTS - 1);
  if (g.U < min_u) g.U = min_u;
  int max_segs = (g.kbt + g.U - 1) / g.U + 1;
  return (size_t)max_segs * MAXT * N * sizeof(float);
}

extern "C" size_t b200_mega_partial_bytes(int H, int Hq, int Hkv, int I, int num_sms) {
  const int grid = num_sms;
  GemmShape g;
  size_t need = 0, b;
  b = plan_gemm(g, (Hq + 2 * Hkv) * D, H, grid); need = b > need ? b : need;
  b = plan_gemm(g, H, Hq * D, grid); need = b > need ? b : need;
  b = plan_gemm(g, 2 * I, H, grid); need = b > need ? b : need;
  b = plan_gemm(g, H, I, grid); need = b > need ? b : need;
  return need;
}

// One decode step through `num_layers` decoder layers.  hidden0 [T, H] (embedding rows) -> residual
// [T, H] = the residual stream after the last layer (the caller applies the final norm).  T <= 64 rows,
// one per request (padded requests: seq_len 0, slot -1).  h / o / act are [64, *] operand buffers the
// kernel owns between phases; part / attn_* are scratch; ctrl is int[64], zero before the first launch
// (the kernel re-arms it; after a launch that reported a status, zero it again).
// Tensor parallel (world > 1): peers = heap bases, slab_off / flag_off = heap offsets of the two
// receive slabs [world][64][H] bf16 and their flags int[world][256].
extern "C" int b200_mega_decode(const void* layers_dev, int num_layers, const void* hidden0, void* residual,
                                void* h, void* o, void* act, void* part, size_t part_bytes,
                                const int* positions, const int* slot_mapping, const int* block_tables,
                                const int* seq_lens, int max_blocks, int block_size, long long num_blocks, int T,
                                int H, int Hq, int Hkv, int I, const float* inv_freq, int rot_pairs,
                                int interleaved, float eps, float scale, int kv_splits, void* attn_part_o,
                                void* attn_part_ml, int* attn_counters, int* ctrl, int* status, int world,
                                int rank, void* const* peers, unsigned long long slab0_off,
                                unsigned long long slab1_off, unsigned long long flag0_off,
                                unsigned long long flag1_off, unsigned int spin_limit, int num_sms,
                                unsigned long long* dbg, int dbg_layer, int dbg_gi, int dbg_ev_base,
                                cudaStream_t stream) {
  if (T <= 0 || num_layers <= 0) return 0;
  if (T > MAXT || H % 128 || I % 128 || Hq % Hkv || (Hq / Hkv) > 16 || H > 128 * 8 * 8 || world < 1 || world > 8 ||
      kv_splits < 1 || kv_splits > 16) {
    b200_set_last_error("mega_decode: T <= 64, H and I multiples of 128, H <= 8192 and a GQA group of at most 16 heads required",
                        __FILE__, __LINE__);
    return -3;
  }
  const int grid = mega_grid(num_sms);
  if (grid <= 0) {
    b200_set_last_error("mega_decode: the kernel does not fit on an SM", __FILE__, __LINE__);
    return -4;
  }
  Params p;
  memset(&p, 0, sizeof(p));
  p.layers = reinterpret_cast<const LayerDesc*>(layers_dev);
  p.num_layers = num_layers;
  p.T = T; p.H = H; p.Hq = Hq; p.Hkv = Hkv; p.I = I; p.Nqkv = (Hq + 2 * Hkv) * D;
  size_t need = 0, b;
  b = plan_gemm(p.g[0], p.Nqkv, H, grid); need = b > need ? b : need;
  b = plan_gemm(p.g[1], H, Hq * D, grid); need = b > need ? b : need;
  b = plan_gemm(p.g[2], 2 * I, H, grid); need = b > need ? b : need;
  b = plan_gemm(p.g[3], H, I, grid); need = b > need ? b : need;
  if (need > part_bytes) {
    b200_set_last_error("mega_decode: split-K scratch too small", __FILE__, __LINE__);
    return -5;
  }
  p.hidden0 = reinterpret_cast<const __nv_bfloat16*>(hidden0);
  p.residual = reinterpret_cast<__nv_bfloat16*>(residual);
  p.h = reinterpret_cast<__nv_bfloat16*>(h);
  p.o = reinterpret_cast<__nv_bfloat16*>(o);
  p.act = reinterpret_cast<__nv_bfloat16*>(act);
  p.part = reinterpret_cast<float*>(part);
  p.positions = positions; p.slot_mapping = slot_mapping; p.block_tables = block_tables; p.seq_lens = seq_lens;
  p.max_blocks = max_blocks; p.block_size = block_size; p.num_blocks = num_blocks;
  p.inv_freq = inv_freq; p.rot_pairs = rot_pairs; p.interleaved = interleaved;
  p.eps = eps; p.scale_log2 = scale * 1.4426950408889634f;
  p.kv_splits = kv_splits;
  p.attn_part_o = reinterpret_cast<float*>(attn_part_o);
  p.attn_part_ml = reinterpret_cast<float*>(attn_part_ml);
  p.attn_counters = attn_counters;
  p.ctrl = ctrl; p.status = status;
  p.world = world; p.rank = rank;
  for (int i = 0; i < 8; ++i) p.peer[i] = (world > 1 && i < world) ? (uint8_t*)peers[i] : nullptr;
  p.slab_off[0] = slab0_off; p.slab_off[1] = slab1_off;
  p.flag_off[0] = flag0_off; p.flag_off[1] = flag1_off;
  p.spin_limit = spin_limit;
  p.dbg = dbg; p.dbg_layer = dbg_layer; p.dbg_gi = dbg_gi; p.dbg_ev_base = dbg_ev_base;
  CUtensorMap tmH, tmO, tmAct;
  int rc = b200_make_tmap_2d(&tmH, h, 2, (uint64_t)MAXT, (uint64_t)H, (uint64_t)H * 2, BN, BK);
  if (rc) return rc;
  rc = b200_make_tmap_2d(&tmO, o, 2, (uint64_t)MAXT, (uint64_t)Hq * D, (uint64_t)Hq * D * 2, BN, BK);
  if (rc) return rc;
  rc = b200_make_tmap_2d(&tmAct, act, 2, (uint64_t)MAXT, (uint64_t)I, (uint64_t)I * 2, BN, BK);
  if (rc) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  B200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, decode_layers_kernel, tmH, tmO, tmAct, p));
  return 0;
}
