// Prefill / mixed ragged paged attention on the 5th-generation tensor cores (head_dim 128, bf16).
//
// One CTA owns 128 query rows = the G q-heads of one kv head x 128/G consecutive positions of one
// request, so every K/V byte staged in shared memory serves the whole GQA group.  Per 128-key chunk:
//   S = Q K^T        tcgen05.mma (kind::f16), Q and K in shared memory (TMA, SWIZZLE_128B, K-major),
//                    S in TMEM (fp32, 128 columns, two buffers)
//   softmax          four warps, one thread per row: tcgen05.ld the row, scale / mask / running max
//                    / exp2 / sum in registers, P written as bf16 into shared memory in the K-major
//                    swizzled layout the next MMA reads
//   O_chunk = P V    tcgen05.mma with V as an MN-major operand (the cache stores V with head_dim
//                    contiguous), result in TMEM (two buffers); the softmax threads fold it into
//                    their fp32 register accumulators (acc = acc * alpha + O_chunk), so TMEM is
//                    never rescaled in place.
// Warp roles: warp 0 TMA producer (Q tile once, K and V rings, one 16-token page per copy), warp 1
// MMA issuer, warps 2-9 softmax + output (two threads per row, one per half of the key columns).  S(j+1) is issued before P V(j), so the tensor core works
// on the next scores while the softmax of the current chunk runs.  512 TMEM columns, 192 KB of
// shared memory.  Every mbarrier wait is bounded (status word + abort flag + TMEM freed on exit).
//
// Same function as the mma.sync prefill kernel in attention.cu (causal ragged batches with prefix
// context, sliding window, soft-cap, sinks, LSE); semantics of the reference's ragged paged
// attention (reference: src/vllm_torchtpu/kernels/ragged_paged_attention/v3/kernel.py:74-214).
#include <cstring>

#include "common.cuh"
#include "gemm_tcgen05.h"

namespace b200 {
namespace fa {

constexpr int D = 128;
constexpr int BM = 128;                  // query rows per CTA
constexpr int BKV = 128;                 // keys per chunk
constexpr int HALF_BYTES = 128 * 128;    // 128 rows x 64 bf16: one swizzled half of a 128 x 128 tile
constexpr int TILE_BYTES = 2 * HALF_BYTES;
constexpr int KV_STAGES = 2;
constexpr int SMEM_Q = 0;
constexpr int SMEM_K = SMEM_Q + TILE_BYTES;
constexpr int SMEM_V = SMEM_K + KV_STAGES * TILE_BYTES;
constexpr int SMEM_P = SMEM_V + KV_STAGES * TILE_BYTES;
constexpr int SMEM_BAR = SMEM_P + TILE_BYTES;
constexpr int SMEM_XCH = SMEM_BAR + 256;                // row-max and row-sum exchange between the two column halves
constexpr int SMEM_TOTAL = SMEM_XCH + 3 * 2 * 128 * 4 + 1024;     // + alignment slack
constexpr int NUM_THREADS = 64 + 256;                   // TMA warp, MMA warp, 8 softmax warps

struct Params {
  __nv_bfloat16* out;
  float* lse;
  const int* block_tables;
  const int* seq_lens;
  const int* qsl;
  const float* sinks;
  int* status;
  int max_blocks, block_size, Hq, Hkv, G, BQ, req_begin, req_end, window;
  int non_causal;                 // 1: every query row sees the whole sequence (encoders, diffusion)
  long long num_blocks;
  float scale_log2, softcap;
};

// MN-major operand whose rows (K index) are 128 bytes = 64 elements of the MN dimension, written by
// TMA with SWIZZLE_128B: 8-row groups are 1024 B apart, the next 64 MN elements are `lbo` bytes away.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// bf16 x bf16 -> fp32, A K-major, B MN-major
__host__ __device__ constexpr uint32_t umma_idesc_bf16_bmn(int M, int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKV,
                       const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_BAR);
  uint64_t* q_full = bars;                 // 1
  uint64_t* k_full = bars + 1;             // [2]
  uint64_t* k_empty = bars + 3;            // [2]
  uint64_t* v_full = bars + 5;             // [2]
  uint64_t* v_empty = bars + 7;            // [2]
  uint64_t* s_full = bars + 9;             // [2]
  uint64_t* s_empty = bars + 11;           // [2]
  uint64_t* o_full = bars + 13;            // [2]
  uint64_t* o_empty = bars + 15;           // [2]
  uint64_t* p_full = bars + 17;            // 1
  uint64_t* p_empty = bars + 18;           // 1
  uint64_t* mx_bar = bars + 19;            // [2] row-max exchange, 256 arrivals
  uint64_t* l_bar = bars + 21;             // 1   row-sum exchange, 256 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 22);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 8);
      mbar_init(&o_full[i], 1); mbar_init(&o_empty[i], 8);
      mbar_init(&mx_bar[i], 256);
    }
    mbar_init(p_full, 8);
    mbar_init(l_bar, 256);
    mbar_init(p_empty, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmKV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  pdl_launch_dependents();
  pdl_wait();

  // ---- which (request, query block) is this tile: linear scan over the ragged batch
  const int h = blockIdx.x;                       // kv head
  int r = -1, q0 = 0;
  {
    int tile = blockIdx.y;
    for (int i = p.req_begin; i < p.req_end; ++i) {
      const int ql = p.qsl[i + 1] - p.qsl[i];
      const int nt = (ql + p.BQ - 1) / p.BQ;
      if (tile < nt) { r = i; q0 = tile * p.BQ; break; }
      tile -= nt;
    }
  }
  int qs = 0, q_len = 0, seq_len = 0;
  if (r >= 0) {
    qs = p.qsl[r];
    q_len = p.qsl[r + 1] - qs;
    seq_len = p.seq_lens[r];
  }
  const bool active = r >= 0 && seq_len > 0 && q_len > 0;
  const int ctx = seq_len - q_len;
  // causal bound of the tile; the whole sequence without the mask
  const int kv_end = active ? (p.non_causal ? seq_len : min(seq_len, ctx + q0 + p.BQ)) : 0;
  int kv_begin = 0;
  if (active && p.window > 0) kv_begin = max(0, ctx + q0 - p.window + 1) / BKV * BKV;
  const int nchunks = active ? (kv_end - kv_begin + BKV - 1) / BKV : 0;

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // One chunk = 8 pages of K and 8 of V.  Lane l < 16 owns page l & 7 of K (l < 8) or V: the block
    // ids of a chunk are fetched by 16 lanes at once and every lane issues its own two copies, so no
    // copy waits behind another lane's block-table load.
    if (nchunks > 0) {
      if (lane == 0) {
        mbar_expect_tx(q_full, TILE_BYTES);
        tma_load_3d(smem + SMEM_Q, &tmQ, q_full, 0, h * p.G, qs + q0);
        tma_load_3d(smem + SMEM_Q + HALF_BYTES, &tmQ, q_full, 64, h * p.G, qs + q0);
      }
      const int* bt = p.block_tables + (size_t)r * p.max_blocks;
      const int kv = lane >> 3, pg = lane & 7;
      bool ok = true;
      for (int j = 0; j < nchunks; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int tok = kv_begin + j * BKV + pg * 16;
        long long row = 0;
        if (lane < 16) {
          long long blk = 0;
          int off = 0;
          if (tok < kv_end) {
            const int page = tok / p.block_size;
            off = tok - page * p.block_size;
            blk = page < p.max_blocks ? bt[page] : -1;
            if (blk < 0 || blk >= p.num_blocks) {
              B200_NOTE_BAD_INDEX();
              blk = 0;
            }
          }
          row = ((blk * 2 + kv) * p.Hkv + h) * p.block_size + off;     // cache as [(blocks, 2, Hkv, bs), D]
        }
        if (lane == 0) {
          ok = mbar_wait(&k_empty[st], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY) &&
               mbar_wait(&v_empty[st], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY);
          if (ok) {
            mbar_expect_tx(&k_full[st], TILE_BYTES);
            mbar_expect_tx(&v_full[st], TILE_BYTES);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        if (lane < 16) {
          uint64_t* full = kv == 0 ? &k_full[st] : &v_full[st];
          uint8_t* dst = smem + (kv == 0 ? SMEM_K : SMEM_V) + st * TILE_BYTES + pg * 16 * 128;
          tma_load_2d(dst, &tmKV, full, 0, (int)row);
          tma_load_2d(dst + HALF_BYTES, &tmKV, full, 64, (int)row);
        }
      }
      if (lane == 0 && *abort_flag)
        for (int it = 0; it < 20000; ++it) __nanosleep(100);
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer
    if (elect_one() && nchunks > 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(BM, BKV);
      constexpr uint32_t idesc_pv = umma_idesc_bf16_bmn(BM, D);
      const uint32_t q_addr = smem_u32(smem + SMEM_Q);
      const uint32_t p_addr = smem_u32(smem + SMEM_P);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, ST_TIMEOUT_FULL);
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&s_empty[st], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) return false;
        if (!mbar_wait(&k_full[st], ph, abort_flag, p.status, ST_TIMEOUT_FULL)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + SMEM_K + st * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t hoff = (ks >> 2) * HALF_BYTES;
          umma_f16(tmem_base + st * BKV, umma_desc_k_sw128(q_addr + hoff) + 2 * (ks & 3),
                   umma_desc_k_sw128(k_addr + hoff) + 2 * (ks & 3), idesc_qk, ks > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[st]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < nchunks && ok; ++j) {
        if (j + 1 < nchunks) ok = issue_qk(j + 1);
        if (!ok) break;
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&o_empty[st], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        if (!mbar_wait(&v_full[st], ph, abort_flag, p.status, ST_TIMEOUT_FULL)) break;
        if (!mbar_wait(p_full, j & 1, abort_flag, p.status, ST_TIMEOUT_FULL)) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(smem + SMEM_V + st * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < BKV / 16; ++ks) {
          const uint32_t hoff = (ks >> 2) * HALF_BYTES;
          umma_f16(tmem_base + 2 * BKV + st * D, umma_desc_k_sw128(p_addr + hoff) + 2 * (ks & 3),
                   umma_desc_mn_sw128(v_addr + ks * 16 * 128, HALF_BYTES), idesc_pv, ks > 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[st]);
        umma_commit(p_empty);
        umma_commit(&o_full[st]);
      }
    }
  } else {
    // ------------------------------------------------ softmax + output: two threads per row
    // Warps 2-5 own key columns [0, 64) of every chunk and output dims [0, 64), warps 6-9 the other
    // halves (a warp may only touch the TMEM lanes of its quarter, so the pair of a row sits in two
    // warps).  The pair agrees on the chunk's row maximum through shared memory and an mbarrier
    // (bounded wait, like every other wait here); row sums are combined once at the end.
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;                     // 0: columns 0-63, 1: columns 64-127
    const int row = qd * 32 + lane;                       // TMEM lane = tile row
    const int pos_local = row / p.G, head = h * p.G + row % p.G;
    const bool row_ok = active && (q0 + pos_local) < q_len;
    const int lim = p.non_causal ? seq_len - 1 : ctx + q0 + pos_local;    // last visible key of this row
    constexpr int HC = BKV / 2, HD = D / 2;
    float acc[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f, alpha_prev = 0.f;
    const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
    uint8_t* p_row = smem + SMEM_P + half * HALF_BYTES + row * 128;      // this thread's 64 keys of P
    float* mx_sh = reinterpret_cast<float*>(smem + SMEM_XCH);           // [2 parity][2 half][128]
    float* l_sh = mx_sh + 2 * 2 * 128;                                  // [2 half][128]
    bool ok = true;
    for (int j = 0; j < nchunks && ok; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      const int tok0 = kv_begin + j * BKV + half * HC;
      if (!mbar_wait(&s_full[st], ph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem_base + st * BKV + half * HC + lane_addr;
      // columns [c_lo, c_hi) of this thread's 64 are visible to the row (causal limit, end of the
      // sequence, sliding window); most chunks are fully visible
      const int c_hi = min(HC, min(lim, kv_end - 1) - tok0 + 1);
      const int c_lo = p.window > 0 ? max(0, lim - p.window + 1 - tok0) : 0;
      const bool full = c_lo <= 0 && c_hi >= HC;
      const bool capped = p.softcap > 0.f;
      // pass 1: row maximum (raw scores; the scale is positive, the soft-cap monotonic)
      float mx = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < HC; c0 += 32) {
        uint32_t rv[32];
        tmem_ld_32x32(s_addr + c0, rv);
        tmem_ld_wait();
        if (full) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(rv[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c0 + i >= c_lo && c0 + i < c_hi) mx = fmaxf(mx, __uint_as_float(rv[i]));
        }
      }
      mx_sh[(st * 2 + half) * 128 + row] = mx;
      mbar_arrive(&mx_bar[st]);
      if (!mbar_wait(&mx_bar[st], ph, abort_flag, p.status, ST_TIMEOUT_FLAG)) { ok = false; break; }
      mx = fmaxf(mx, mx_sh[(st * 2 + (half ^ 1)) * 128 + row]);
      if (mx != -INFINITY) {
        mx *= p.scale_log2;
        if (capped) mx = p.softcap * tanhf(mx / p.softcap);
      }
      const float m_new = fmaxf(m, mx);
      const float base = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = ex2f(m - base);
      m = m_new;
      // the P buffer is free once P V of the previous chunk has read it
      if (j > 0 && !mbar_wait(p_empty, (j - 1) & 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
      // pass 2: probabilities, row sum, P (bf16) into shared memory, K-major swizzled
      float ps = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < HC; c0 += 32) {
        uint32_t rv[32];
        tmem_ld_32x32(s_addr + c0, rv);
        tmem_ld_wait();
        float e[32];
        if (!capped) {
#pragma unroll
          for (int i = 0; i < 32; ++i) e[i] = ex2f(fmaf(__uint_as_float(rv[i]), p.scale_log2, -base));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            e[i] = ex2f(p.softcap * tanhf(__uint_as_float(rv[i]) * p.scale_log2 / p.softcap) - base);
        }
        if (!full) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c0 + i < c_lo || c0 + i >= c_hi) e[i] = 0.f;
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          ps += e[i] + e[i + 1];
          __nv_bfloat162 b2 = __floats2bfloat162_rn(e[i], e[i + 1]);
          pk[i >> 1] = *reinterpret_cast<uint32_t*>(&b2);
        }
        // 32 keys = 4 chunks of 16 bytes inside this thread's 128-byte row of the half
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const int chunk = (c0 >> 3) + cc;
          *reinterpret_cast<uint4*>(p_row + ((chunk ^ (row & 7)) << 4)) =
              make_uint4(pk[4 * cc], pk[4 * cc + 1], pk[4 * cc + 2], pk[4 * cc + 3]);
        }
      }
      l = l * alpha + ps;
      // S buffer may be overwritten; P is complete
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[st]);
        mbar_arrive(p_full);
      }
      // fold the previous chunk's P V into the accumulators while the tensor core works on this one
      if (j > 0) {
        const int so = (j - 1) & 1;
        if (!mbar_wait(&o_full[so], ((j - 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t o_addr = tmem_base + 2 * BKV + so * D + half * HD + lane_addr;
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t rv[32];
          tmem_ld_32x32(o_addr + c0, rv);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c0 + i] = acc[c0 + i] * alpha_prev + __uint_as_float(rv[i]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&o_empty[so]);
      }
      alpha_prev = alpha;
    }
    if (ok && nchunks > 0) {
      const int so = (nchunks - 1) & 1;
      if (mbar_wait(&o_full[so], ((nchunks - 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) {
        tc_fence_after();
        const uint32_t o_addr = tmem_base + 2 * BKV + so * D + half * HD + lane_addr;
#pragma unroll
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t rv[32];
          tmem_ld_32x32(o_addr + c0, rv);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c0 + i] = acc[c0 + i] * alpha_prev + __uint_as_float(rv[i]);
        }
        tc_fence_before();
      } else {
        ok = false;
      }
    }
    // row sum of the pair (each thread summed its 64 columns of every chunk)
    if (nchunks > 0) {
      l_sh[half * 128 + row] = l;
      mbar_arrive(l_bar);
      if (ok && !mbar_wait(l_bar, 0, abort_flag, p.status, ST_TIMEOUT_FLAG)) ok = false;
      if (ok) l += l_sh[(half ^ 1) * 128 + row];
    }
    if (ok && row_ok) {
      float sc = 1.f;
      if (p.sinks != nullptr) {
        const float sk = p.sinks[head] * 1.4426950408889634f;
        const float n = fmaxf(m, sk);
        sc = (m == -INFINITY) ? 0.f : ex2f(m - n);
        l = l * sc + ex2f(sk - n);
        m = n;
      }
      const float inv = l > 0.f ? sc / l : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)(qs + q0 + pos_local) * p.Hq + head) * D + half * HD;
#pragma unroll
      for (int i = 0; i < HD; i += 8) {
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int u = 0; u < 4; ++u) oh[u] = __floats2bfloat162_rn(acc[i + 2 * u] * inv, acc[i + 2 * u + 1] * inv);
        *reinterpret_cast<uint4*>(dst + i) = o;
      }
      if (p.lse != nullptr && half == 0)
        p.lse[(size_t)(qs + q0 + pos_local) * p.Hq + head] =
            l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace fa
}  // namespace b200

using namespace b200;

// Requests [req_begin, req_end) of a ragged batch; num_tiles_64 = sum over them of ceil(q_len / 64)
// (the tile count of 64-row query blocks, from which the grid for 128 / G positions per tile is bounded).
// head_dim 128, q heads per kv head in {1, 2, 4, 8}, block_size a multiple of 16.
static int attn_prefill_tc_impl(const void* q, const void* kv, void* out, float* lse, const int* block_tables,
                                const int* seq_lens, const int* qsl, int req_begin, int req_end, int num_tiles_64,
                                int total_tokens, int max_blocks, int block_size, long long num_blocks, int Hq,
                                int Hkv, int D, float scale, int window, float softcap, const float* sinks,
                                int* status, int non_causal, cudaStream_t stream) {
  if (req_end <= req_begin || num_tiles_64 <= 0) return 0;
  const int G = Hkv > 0 ? Hq / Hkv : 0;
  if (D != 128 || Hq % Hkv || (G != 1 && G != 2 && G != 4 && G != 8) || block_size % 16) {
    b200_set_last_error("attn_prefill_tc: head_dim 128, q heads per kv head in {1,2,4,8}, block_size % 16 == 0",
                        __FILE__, __LINE__);
    return -1;
  }
  fa::Params p;
  memset(&p, 0, sizeof(p));
  p.out = (__nv_bfloat16*)out; p.lse = lse; p.block_tables = block_tables; p.seq_lens = seq_lens; p.qsl = qsl;
  p.sinks = sinks; p.status = status;
  p.max_blocks = max_blocks; p.block_size = block_size; p.Hq = Hq; p.Hkv = Hkv; p.G = G; p.BQ = fa::BM / G;
  p.req_begin = req_begin; p.req_end = req_end; p.window = window; p.num_blocks = num_blocks;
  p.non_causal = non_causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.softcap = softcap > 0.f ? softcap * 1.4426950408889634f : 0.f;
  CUtensorMap tmQ, tmKV;
  // q [T, Hq, D] as (x = D, y = Hq, z = T); a tile is 64 x G x BQ elements, rows ordered (token, head)
  int rc = b200_make_tmap_3d_bf16(&tmQ, q, (uint64_t)D, (uint64_t)Hq, (uint64_t)total_tokens, (uint64_t)D * 2,
                                  (uint64_t)Hq * D * 2, 64, (uint32_t)G, (uint32_t)p.BQ);
  if (rc) return rc;
  // cache [(blocks, 2, Hkv, block_size), D]; one copy = 16 tokens x 64 elements
  rc = b200_make_tmap_2d(&tmKV, kv, 2, (uint64_t)num_blocks * 2 * Hkv * block_size, (uint64_t)D, (uint64_t)D * 2,
                         16, 64);
  if (rc) return rc;
  static unsigned long long attr_seen = 0;
  B200_CUDA_CHECK(ensure_dynamic_smem(fa::attn_prefill_tc_kernel, fa::SMEM_TOTAL, &attr_seen));
  // ceil(q_len / BQ) <= ceil(q_len / 64) * (64 / BQ) for BQ <= 64; BQ = 128 needs at most as many tiles
  const int tiles = p.BQ >= 64 ? num_tiles_64 : num_tiles_64 * (64 / p.BQ);
  dim3 grid(Hkv, tiles);
  B200_CUDA_CHECK(launch_pdl(fa::attn_prefill_tc_kernel, grid, dim3(fa::NUM_THREADS), (size_t)fa::SMEM_TOTAL, stream,
                             tmQ, tmKV, p));
  return 0;
}

extern "C" int b200_attn_prefill_tc(const void* q, const void* kv, void* out, float* lse, const int* block_tables,
                                    const int* seq_lens, const int* qsl, int req_begin, int req_end,
                                    int num_tiles_64, int total_tokens, int max_blocks, int block_size,
                                    long long num_blocks, int Hq, int Hkv, int D, float scale, int window,
                                    float softcap, const float* sinks, int* status, cudaStream_t stream) {
  return attn_prefill_tc_impl(q, kv, out, lse, block_tables, seq_lens, qsl, req_begin, req_end, num_tiles_64,
                              total_tokens, max_blocks, block_size, num_blocks, Hq, Hkv, D, scale, window, softcap,
                              sinks, status, 0, stream);
}

// Bidirectional form (vision encoders, diffusion transformers): each request's q_len equals its seq_len and
// every row sees every key.  No window, soft-cap or sinks.
extern "C" int b200_attn_encoder_tc(const void* q, const void* kv, void* out, float* lse, const int* block_tables,
                                    const int* seq_lens, const int* qsl, int req_begin, int req_end,
                                    int num_tiles_64, int total_tokens, int max_blocks, int block_size,
                                    long long num_blocks, int Hq, int Hkv, int D, float scale, int* status,
                                    cudaStream_t stream) {
  return attn_prefill_tc_impl(q, kv, out, lse, block_tables, seq_lens, qsl, req_begin, req_end, num_tiles_64,
                              total_tokens, max_blocks, block_size, num_blocks, Hq, Hkv, D, scale, 0, 0.f, nullptr,
                              status, 1, stream);
}

// see b200_bad_index_count_attention
extern "C" int b200_bad_index_count_attention_tc(unsigned int* out) {
  B200_TAKE_BAD_INDEX_COUNT(out);
  return 0;
}
