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
constexpr int STAGES = 5;
constexpr int A_BYTES = BM * BK * 2;    // 16 KB
constexpr int B_BYTES = BN * BK * 2;    // 8 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int RING_BYTES = STAGES * STAGE_BYTES;                 // 120 KB
constexpr int BAR_OFF = RING_BYTES;
constexpr int BAR_BYTES = 1024;
constexpr int ATT_OFF = BAR_OFF + BAR_BYTES;                     // 1024-aligned
constexpr int D = 128;                                            // head dim
constexpr int ATT_STAGES = 3;
constexpr int ATT_PAGE_BYTES = 16 * D * 2;                        // 16 tokens of K (or V)
constexpr int ATT_STAGE_BYTES = 2 * ATT_PAGE_BYTES;
constexpr int ATT_WARP_BYTES = ATT_STAGES * ATT_STAGE_BYTES;      // 24 KB per warp (>= [16][D] fp32 merge tile)
constexpr int ATT_RING_BYTES = 4 * ATT_WARP_BYTES;                // 96 KB
constexpr int SQ_OFF = ATT_OFF + ATT_RING_BYTES;                  // q rows [16][D] bf16
constexpr int SQ_BYTES = 16 * D * 2;
constexpr int CS_OFF = SQ_OFF + SQ_BYTES;                         // cos | sin, D floats
constexpr int ML_OFF = CS_OFF + D * 4;                            // [4][16][2] floats
constexpr int RED_OFF = ML_OFF + 4 * 16 * 2 * 4;                  // 32 floats + flags
constexpr int SMEM_USED = RED_OFF + 256;
constexpr int SMEM_BYTES = SMEM_USED + 1024;                      // + alignment slack
static_assert(SMEM_BYTES <= 232448, "shared memory budget");
constexpr int TMEM_COLS = 2 * BN;                                 // two accumulators
constexpr int MAXT = 64;

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
  int* ctrl;                            // [0] grid barrier, [1] exit count, [2] launch epoch, [3] abort
  int* status;
  int world, rank;
  uint8_t* peer[8];
  unsigned long long slab_off[2];       // receive slabs [src][64][H] bf16 of o_proj / down_proj partial rows
  unsigned long long flag_off[2];       // int[world][64 * 4]
  unsigned int spin_limit;
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
  volatile int* s_last;
};

__device__ __forceinline__ void raise_abort(const Params& p, const Shared& sh, int code) {
  *sh.abort_flag = 1;
  atomicExch(p.ctrl + 3, 1);
  if (p.status) atomicCAS(p.status, ST_OK, code);
}

// named barrier of the 128 compute threads (warps 2..5)
__device__ __forceinline__ void cbar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Grid barrier: arrival number `target` of the monotonic counter ctrl[0].  Called by all 128 compute
// threads; returns false when the grid aborted.
__device__ __forceinline__ bool grid_barrier(const Params& p, const Shared& sh, int target, int ct) {
  __threadfence();
  cbar();
  if (ct == 0) {
    atomicAdd(p.ctrl, 1);
    const unsigned long long t0 = global_timer_ns();
    bool ok = false;
#pragma unroll 1
    for (uint32_t it = 0;; ++it) {
      if (ld_acquire_gpu(p.ctrl) - target >= 0) { ok = true; break; }
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

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

// Sum of the fp32 partials of 8 consecutive columns [n, n+8) of row t of a projection.
__device__ __forceinline__ void sum_partials8(const float* part, const GemmShape& g, int t, int n, float (&acc)[8]) {
  const int tile = n / BM;
  const int ns = tile_num_segs(g, tile);
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  for (int s = 0; s < ns; ++s) {
    const float4* src = reinterpret_cast<const float4*>(part + ((size_t)s * MAXT + t) * g.N + n);
    const float4 a = __ldcg(src), b = __ldcg(src + 1);
    acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
    acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
  }
}

// ----------------------------------------------------------------- phases run by the compute warps
// residual + sum -> residual; RMSNorm -> h.  Source of the sum: nothing (layer 0: x = hidden0), the
// split-K partials of projection `src_g` (one rank), or the receive slab `slab` (tensor parallel).
__device__ void phase_norm(const Params& p, const Shared& sh, uint8_t* smem, int ct, int layer, bool first,
                           int src_g, int slab, int use_idx, const __nv_bfloat16* weight, bool write_h) {
  float* red = reinterpret_cast<float*>(smem + RED_OFF);
  const int H = p.H;
  const int nvec = H >> 3;
  for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
    if (!first && p.world > 1) {
      // the partial rows of every rank (this one included) arrive as quarter rows with one flag each
      if (ct < p.world * 4) {
        const int* f = reinterpret_cast<const int*>(p.peer[p.rank] + p.flag_off[slab]) + (ct >> 2) * (MAXT * 4) +
                       t * 4 + (ct & 3);
        if (!wait_flag_ge(f, use_idx, p.status, p.spin_limit)) raise_abort(p, sh, ST_TIMEOUT_FLAG);
      }
      cbar();
      if (*sh.abort_flag) return;
    }
    float ss = 0.f;
    bf16x8 keep[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int v = ct + u * 128;
      if (v >= nvec) break;
      bf16x8 x;
      if (first) {
        x = *reinterpret_cast<const bf16x8*>(p.hidden0 + (size_t)t * H + v * 8);
      } else {
        float acc[8];
        if (p.world > 1) {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
          const uint8_t* recv = p.peer[p.rank] + p.slab_off[slab];
          for (int r = 0; r < p.world; ++r) {
            const uint4 raw = ld_relaxed_sys_v4(recv + (((size_t)r * MAXT + t) * H + v * 8) * 2);
            const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __bfloat1622float2(hh[j]);
              acc[2 * j] += f.x;
              acc[2 * j + 1] += f.y;
            }
          }
        } else {
          sum_partials8(p.part, p.g[src_g], t, v * 8, acc);
        }
        // same roundings as a bf16 projection output followed by the bf16 residual add
        const bf16x8 r = *reinterpret_cast<const bf16x8*>(p.residual + (size_t)t * H + v * 8);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fa = __bfloat1622float2(__floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]));
          const float2 fr = __bfloat1622float2(r.v[j]);
          x.v[j] = __floats2bfloat162_rn(fa.x + fr.x, fa.y + fr.y);
        }
      }
      *reinterpret_cast<bf16x8*>(p.residual + (size_t)t * H + v * 8) = x;
      keep[u] = x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(x.v[j]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
    if (!write_h) continue;
    // block sum over the 128 compute threads
    ss = warp_sum(ss);
    if ((ct & 31) == 0) red[ct >> 5] = ss;
    cbar();
    const float tot = red[0] + red[1] + red[2] + red[3];
    cbar();
    const float inv = rsqrtf(tot / (float)H + p.eps);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int v = ct + u * 128;
      if (v >= nvec) break;
      const bf16x8 ww = *reinterpret_cast<const bf16x8*>(weight + v * 8);
      bf16x8 y;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(keep[u].v[j]), g2 = __bfloat1622float2(ww.v[j]);
        y.v[j] = __floats2bfloat162_rn(f.x * inv * g2.x, f.y * inv * g2.y);
      }
      *reinterpret_cast<bf16x8*>(p.h + (size_t)t * H + v * 8) = y;
    }
  }
  (void)layer;
}

// Tensor parallel: sum the split-K partials of a row-parallel projection, round to bf16 and store the
// quarter row into the receive slab of every rank, then raise that quarter's flag there.
__device__ void phase_push(const Params& p, const Shared& sh, int ct, int src_g, int slab, int use_idx) {
  const int H = p.H;
  const int qv = (H >> 3) >> 2;                       // 16-byte vectors per quarter row
  const int units = p.T * 4;
  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const int t = u >> 2, q = u & 3;
    for (int v = ct; v < qv; v += 128) {
      const int n = (q * qv + v) * 8;
      float acc[8];
      sum_partials8(p.part, p.g[src_g], t, n, acc);
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      for (int r = 0; r < p.world; ++r) {
        const int d = (p.rank + r) % p.world;           // start with this rank, spread the links
        *reinterpret_cast<uint4*>(p.peer[d] + p.slab_off[slab] + (((size_t)p.rank * MAXT + t) * H + n) * 2) = o;
      }
    }
    __threadfence_system();
    cbar();
    if (ct < p.world)
      st_release_sys(reinterpret_cast<int*>(p.peer[ct] + p.flag_off[slab]) + p.rank * (MAXT * 4) + u, use_idx);
  }
  (void)sh;
}

// act = silu(gate) * up from the partials of the gate/up projection (columns [0, I) gate, [I, 2I) up)
__device__ void phase_swiglu(const Params& p, int ct) {
  const int I = p.I;
  const int nvec = I >> 3;
  const int total = p.T * nvec;
  for (int idx = blockIdx.x * 128 + ct; idx < total; idx += gridDim.x * 128) {
    const int t = idx / nvec, v = idx - t * nvec;
    float g8[8], u8[8];
    sum_partials8(p.part, p.g[2], t, v * 8, g8);
    sum_partials8(p.part, p.g[2], t, I + v * 8, u8);
    bf16x8 y;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      y.v[j] = __floats2bfloat162_rn(silu(g8[2 * j]) * u8[2 * j], silu(g8[2 * j + 1]) * u8[2 * j + 1]);
    *reinterpret_cast<bf16x8*>(p.act + (size_t)t * I + v * 8) = y;
  }
}

// One (request, kv head, kv split) unit of decode attention: sum the qkv partials of the request's
// token, bias, per-head q/k RMSNorm, RoPE, KV write (last split), then split-KV flash attention with
// one 16-row mma.sync tile per kv head group, as in the stand-alone decode kernel.
__device__ void attn_unit(const Params& p, const Shared& sh, uint8_t* smem, const LayerDesc& L, int ct, int r,
                          int h, int z) {
  const int lw = ct >> 5, lane = ct & 31;
  const int G = p.Hq / p.Hkv;
  const int t = r;
  const int seq_len = p.seq_lens[r];
  if (seq_len <= 0) return;                                   // padded request (uniform for the CTA)
  const int ctx = seq_len - 1;
  const int Z = p.kv_splits;
  __nv_bfloat16* s_q = reinterpret_cast<__nv_bfloat16*>(smem + SQ_OFF);
  float* cs = reinterpret_cast<float*>(smem + CS_OFF);
  float (*s_ml)[16][2] = reinterpret_cast<float (*)[16][2]>(smem + ML_OFF);
  const GemmShape& gq = p.g[0];

  // ---- prologue: q rows (and k, v of the new token on the last split)
  {
    const float pos = (float)p.positions[t];
    for (int i = ct; i < p.rot_pairs; i += 128) {
      float s, c;
      sincosf(pos * p.inv_freq[i], &s, &c);
      cs[i] = c;
      cs[D / 2 + i] = s;
    }
    for (int i = ct; i < (16 - G) * D / 2; i += 128) reinterpret_cast<uint32_t*>(s_q + G * D)[i] = 0u;
    cbar();
    const long long slot = p.slot_mapping[t];
    const bool write_kv = (z == Z - 1);
    const int nrows = write_kv ? G + 2 : G;
    constexpr int EPL = D / 32;
    for (int j = lw; j < nrows; j += 4) {
      const int kind = j < G ? 0 : (j == G ? 1 : 2);
      const int head_col = kind == 0 ? (h * G + j) : (kind == 1 ? p.Hq + h : p.Hq + p.Hkv + h);   // n tile index
      int idx[EPL];
#pragma unroll
      for (int u = 0; u < EPL / 2; ++u) {
        const int i = lane * (EPL / 2) + u;
        if (p.interleaved) { idx[2 * u] = 2 * i; idx[2 * u + 1] = 2 * i + 1; }
        else { idx[2 * u] = i; idx[2 * u + 1] = i + D / 2; }
      }
      float x[EPL];
#pragma unroll
      for (int u = 0; u < EPL; ++u) x[u] = 0.f;
      const int ns = tile_num_segs(gq, head_col);
      for (int s = 0; s < ns; ++s) {
        const float* src = p.part + ((size_t)s * MAXT + t) * gq.N + head_col * D;
#pragma unroll
        for (int u = 0; u < EPL; ++u) x[u] += __ldcg(src + idx[u]);
      }
#pragma unroll
      for (int u = 0; u < EPL; ++u) {
        if (L.qkv_bias != nullptr) x[u] += __bfloat162float(L.qkv_bias[head_col * D + idx[u]]);
        x[u] = __bfloat162float(__float2bfloat16(x[u]));          // the projection's bf16 output
      }
      if (kind < 2) {
        const __nv_bfloat16* nwp = kind == 0 ? L.q_norm : L.k_norm;
        if (nwp != nullptr) {
          float ss = 0.f;
#pragma unroll
          for (int u = 0; u < EPL; ++u) ss += x[u] * x[u];
          ss = warp_sum(ss);
          const float inv = rsqrtf(ss / (float)D + p.eps);
#pragma unroll
          for (int u = 0; u < EPL; ++u)
            x[u] = __bfloat162float(__float2bfloat16(x[u] * inv * __bfloat162float(nwp[idx[u]])));
        }
#pragma unroll
        for (int u = 0; u < EPL / 2; ++u) {
          const int i = lane * (EPL / 2) + u;
          if (i < p.rot_pairs) {
            const float c = cs[i], s = cs[D / 2 + i];
            const float a = x[2 * u], b = x[2 * u + 1];
            x[2 * u] = a * c - b * s;
            x[2 * u + 1] = b * c + a * s;
          }
        }
      }
      if (kind == 0) {
#pragma unroll
        for (int u = 0; u < EPL; ++u) s_q[j * D + idx[u]] = __float2bfloat16(x[u]);
      } else if (slot >= 0 && slot < p.num_blocks * p.block_size) {
        const long long blk = slot / p.block_size;
        const int off = (int)(slot - blk * p.block_size);
        __nv_bfloat16* dst = L.kv_cache + ((((size_t)blk * 2 + (kind - 1)) * p.Hkv + h) * p.block_size + off) * D;
#pragma unroll
        for (int u = 0; u < EPL; ++u) dst[idx[u]] = __float2bfloat16(x[u]);
      }
    }
    __threadfence();                 // the new K/V row is read back through L2 by this CTA's cp.async
    cbar();
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
  const int rows_valid = G;

  // this (split, warp) unit's range of 16-token chunks
  const int C = (seq_len + 15) >> 4;
  const int units = Z * 4;
  const int per = (C + units - 1) / units;
  const int uu = z * 4 + lw;
  const int cb0 = min(C, uu * per);
  const int cb1 = min(C, (uu + 1) * per);

  uint8_t* ring = smem + ATT_OFF;
  const uint32_t wbase = smem_u32(ring) + lw * ATT_WARP_BYTES;
  const int* bt = p.block_tables + (size_t)r * p.max_blocks;
  const size_t head_stride = (size_t)p.block_size * D;
  const int page_lo = (cb0 << 4) / p.block_size;
  const int page_hi = cb1 > cb0 ? (((cb1 << 4) - 1) / p.block_size) : page_lo - 1;
  int bt_base = page_lo;
  int bt_reg = (page_lo + lane <= page_hi) ? bt[page_lo + lane] : 0;
  const __nv_bfloat16* kv = L.kv_cache;
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

  // ---- merge the 4 warps in shared memory (each warp reuses its own ring)
  float* wo = reinterpret_cast<float*>(ring + lw * ATT_WARP_BYTES);
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    const int col = i * 8 + 2 * (lane & 3);
    *reinterpret_cast<float2*>(wo + row0 * D + col) = make_float2(o[i][0], o[i][1]);
    *reinterpret_cast<float2*>(wo + row1 * D + col) = make_float2(o[i][2], o[i][3]);
  }
  if ((lane & 3) == 0) {
    s_ml[lw][row0][0] = m[0]; s_ml[lw][row0][1] = l[0];
    s_ml[lw][row1][0] = m[1]; s_ml[lw][row1][1] = l[1];
  }
  cbar();
  const int row = ct >> 3;                          // 16 rows x 8 threads
  const int seg = ct & 7;
  constexpr int SEG = D / 8;
  float mm = -INFINITY;
#pragma unroll
  for (int w = 0; w < 4; ++w) mm = fmaxf(mm, s_ml[w][row][0]);
  float Lsum = 0.f, acc[SEG];
#pragma unroll
  for (int d = 0; d < SEG; ++d) acc[d] = 0.f;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const float mw = s_ml[w][row][0];
    const float sc = (mw == -INFINITY) ? 0.f : ex2(mw - mm);
    Lsum += s_ml[w][row][1] * sc;
    const float* src = reinterpret_cast<const float*>(ring + w * ATT_WARP_BYTES) + row * D + seg * SEG;
#pragma unroll
    for (int d = 0; d < SEG; ++d) acc[d] += src[d] * sc;
  }
  const bool row_ok = row < rows_valid;
  const int head = h * G + row;
  auto finish = [&](float Lfin, const float* a) {
    if (!row_ok) return;
    const float inv = Lfin > 0.f ? 1.f / Lfin : 0.f;
    __nv_bfloat16* dst = p.o + ((size_t)t * p.Hq + head) * D + seg * SEG;
#pragma unroll
    for (int d = 0; d < SEG; ++d) dst[d] = __float2bfloat16(a[d] * inv);
  };
  if (Z == 1) {
    finish(Lsum, acc);
    cbar();                                           // the rings and s_q are reused by the next unit
    return;
  }
  // ---- cross-split merge by the CTA that arrives last on this (request, kv head)
  const size_t unit = ((size_t)r * p.Hkv + h) * Z;
  float* po = p.attn_part_o + ((unit + z) * 16 + row) * D + seg * SEG;
#pragma unroll
  for (int d = 0; d < SEG; ++d) po[d] = acc[d];
  if (seg == 0) {
    p.attn_part_ml[((unit + z) * 16 + row) * 2 + 0] = mm;
    p.attn_part_ml[((unit + z) * 16 + row) * 2 + 1] = Lsum;
  }
  __threadfence();
  cbar();
  if (ct == 0) {
    const int old = atomicAdd(&p.attn_counters[r * p.Hkv + h], 1);
    *sh.s_last = (old == Z - 1);
  }
  cbar();
  if (*sh.s_last) {
    __threadfence();
    float mfin = -INFINITY;
    for (int s2 = 0; s2 < Z; ++s2) mfin = fmaxf(mfin, __ldcg(&p.attn_part_ml[((unit + s2) * 16 + row) * 2]));
    float Lfin = 0.f;
#pragma unroll
    for (int d = 0; d < SEG; ++d) acc[d] = 0.f;
    for (int s2 = 0; s2 < Z; ++s2) {
      const float ms = __ldcg(&p.attn_part_ml[((unit + s2) * 16 + row) * 2]);
      const float sc = (ms == -INFINITY) ? 0.f : ex2(ms - mfin);
      Lfin += __ldcg(&p.attn_part_ml[((unit + s2) * 16 + row) * 2 + 1]) * sc;
      const float* src = p.attn_part_o + ((unit + s2) * 16 + row) * D + seg * SEG;
#pragma unroll
      for (int d = 0; d < SEG; ++d) acc[d] += __ldcg(src + d) * sc;
    }
    finish(Lfin, acc);
    if (ct == 0) p.attn_counters[r * p.Hkv + h] = 0;
  }
  cbar();
}

__device__ void phase_attn(const Params& p, const Shared& sh, uint8_t* smem, const LayerDesc& L, int ct) {
  const int Z = p.kv_splits;
  const int total = p.T * p.Hkv * Z;
  for (int u = blockIdx.x; u < total && !*sh.abort_flag; u += gridDim.x) {
    const int z = u % Z, rh = u / Z;
    attn_unit(p, sh, smem, L, ct, rh / p.Hkv, rh % p.Hkv, z);
  }
}

// Epilogue of a GEMM phase: the accumulator of every segment of this CTA's range goes to its fp32
// partial slot [seg][t][n] (thread = weight row n, 32 token columns per TMEM load).
__device__ void phase_gemm_epilogue(const Params& p, const Shared& sh, int warp, int lane, int gi, uint32_t tmem_base,
                                    int& segcount) {
  const GemmShape& g = p.g[gi];
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
    if (!mbar_wait(&sh.tfull[acc], acc_ph, sh.abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) return;
    tc_fence_after();
    const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
    const int n = tile * BM + row;
    float* dst = p.part + (size_t)slot * MAXT * g.N + n;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
      if (c0 >= p.T) break;
      uint32_t r[32];
      tmem_ld_32x32(taddr + c0, r);
      tmem_ld_wait();
      if (n < g.N) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c0 + j < p.T) dst[(size_t)(c0 + j) * g.N] = __uint_as_float(r[j]);
      }
    }
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(&sh.tempty[acc]);
    ++segcount;
    u = seg_end;
  }
}

__global__ void __launch_bounds__(THREADS, 1)
decode_layers_kernel(const __grid_constant__ CUtensorMap tmH, const __grid_constant__ CUtensorMap tmO,
                     const __grid_constant__ CUtensorMap tmAct, const Params p) {
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
  sh.s_last = reinterpret_cast<volatile int*>(sh.tmem_slot + 3);
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
    *sh.s_last = 0;
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
        if (!wc.done && wcount - xcount < STAGES) {
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
            if (acquired != ph_idx) {
              // the operand was written by other CTAs (generic proxy) and is read by TMA (async proxy)
              (void)ld_acquire_gpu(p.ctrl);
              asm volatile("fence.proxy.async;" ::: "memory");
              acquired = ph_idx;
            }
            const GemmShape& g = p.g[xc.gi];
            const int tile = xc.u / g.kbt, kb = xc.u - tile * g.kbt;
            const int s = xcount % STAGES;
            const CUtensorMap* tx = xc.gi == 1 ? &tmO : (xc.gi == 3 ? &tmAct : &tmH);
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
        if (!mbar_wait(&sh.tempty[acc], acc_ph ^ 1, sh.abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool first = true;
        do {
          const int s = count % STAGES;
          const uint32_t ph = (uint32_t)(count / STAGES) & 1u;
          if (!mbar_wait(&sh.fullW[s], ph, sh.abort_flag, p.status, ST_TIMEOUT_FULL) ||
              !mbar_wait(&sh.fullX[s], ph, sh.abort_flag, p.status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
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
      if (barrier) {
        ++barriers;
        alive = grid_barrier(p, sh, barriers * G, ct);
      } else {
        cbar();
        alive = !*sh.abort_flag;
      }
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
      phase_gemm_epilogue(p, sh, warp, lane, 0, tmem_base, segcount);
      sync_phase(true);
      if (!alive) break;
      phase_attn(p, sh, smem, L, ct);
      sync_phase(true);
      if (!alive) break;
      phase_gemm_epilogue(p, sh, warp, lane, 1, tmem_base, segcount);
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
      phase_gemm_epilogue(p, sh, warp, lane, 2, tmem_base, segcount);
      sync_phase(true);
      if (!alive) break;
      phase_swiglu(p, ct);
      sync_phase(true);
      if (!alive) break;
      phase_gemm_epilogue(p, sh, warp, lane, 3, tmem_base, segcount);
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
// kernel owns between phases; part / attn_* are scratch; ctrl is int[4], zero before the first launch
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
  CUtensorMap tmH, tmO, tmAct;
  int rc = b200_make_tmap_2d(&tmH, h, 2, (uint64_t)MAXT, (uint64_t)H, (uint64_t)H * 2, BN, BK);
  if (rc) return rc;
  rc = b200_make_tmap_2d(&tmO, o, 2, (uint64_t)MAXT, (uint64_t)Hq * D, (uint64_t)Hq * D * 2, BN, BK);
  if (rc) return rc;
  rc = b200_make_tmap_2d(&tmAct, act, 2, (uint64_t)MAXT, (uint64_t)I, (uint64_t)I * 2, BN, BK);
  if (rc) return rc;
  static unsigned long long attr_seen = 0;
  B200_CUDA_CHECK(ensure_dynamic_smem(decode_layers_kernel, SMEM_BYTES, &attr_seen));
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
