// Ragged paged attention over the block-table KV cache.
//
// Batch description (one launch covers a contiguous range of requests):
//   seq_lens[r]            KV length including this step's tokens
//   query_start_loc[r..r+1] rows of request r in the packed q tensor
//   block_tables[r, :]      pages; cache layout [blocks, 2, Hkv, block_size, D]
// Query j of request r sits at absolute position seq_len - q_len + j and attends
// keys <= that position (minus an optional sliding window).  The step's K/V were
// already written to the pages by the RoPE/cache kernel, so prefix context,
// chunked prefill and decode are one code path.  Semantics follow the reference's
// ragged paged attention (reference: src/vllm_torchtpu/kernels/ragged_paged_attention/v3/kernel.py:74-214).
//
// Two kernels, both flash-attention style with bf16 mma.sync m16n8k16 tiles, fp32
// online softmax in the log2 domain:
//  * decode / spec-verify: q_len * G <= 16 rows (G = q heads per kv head) form ONE
//    16-row MMA tile, so a kv head's group shares every K/V byte read.  Split-KV
//    over (split, warp); each warp streams 16-token pages through its own
//    3-stage cp.async ring.  Partials are merged in shared memory, then across
//    splits by the CTA that arrives last on the (request, kv head) counter.
//  * prefill / mixed: 64 query rows per CTA (4 warps x 16), KV streamed in
//    64-token chunks through a 2-stage cp.async ring shared by the CTA.
// The decode path is bound by HBM bandwidth, which mma.sync tiles already
// saturate; the tcgen05 path is reserved for the GEMMs.
#include "attn_mma.cuh"
#include "common.cuh"

namespace b200 {

struct AttnParams {
  const __nv_bfloat16* q;        // [T, Hq, D]
  const __nv_bfloat16* kv;       // [blocks, 2, Hkv, bs, D]
  __nv_bfloat16* out;            // [T, Hq, D]
  float* lse;                    // optional [T, Hq] natural-log LSE
  const int* block_tables;       // [R, max_blocks]
  const int* seq_lens;           // [R]
  const int* qsl;                // [R+1]
  float* part_o;                 // decode scratch [R, Hkv, S, 16, D] fp32
  float* part_ml;                // decode scratch [R, Hkv, S, 16, 2]
  int* counters;                 // decode scratch [R * Hkv]
  const float* sinks;            // optional [Hq]
  int max_blocks, block_size, Hq, Hkv, req_begin, req_end, num_splits, window;
  int non_causal;                // prefill kernel: every query sees all seq_len keys (encoder attention)
  long long num_blocks;
  float scale_log2, softcap;
  float v_scale;                 // fp8 cache: dequantisation factor of V (K's is folded into scale_log2)
  // decode context parallelism (prefill kernel): the cache of this rank holds the positions p with
  // (p / dcp_interleave) % dcp_size == dcp_rank, seq_lens are LOCAL lengths and global_seq_lens the true
  // ones; a query at global position g sees the first dcp_local_len(g + 1) local keys
  const int* global_seq_lens;
  int dcp_size, dcp_rank, dcp_interleave;
};

// number of positions < n that live on `rank` when positions are dealt round-robin in runs of `il`
__device__ __forceinline__ int dcp_local_len(int n, int rank, int size, int il) {
  const int period = il * size;
  const int full = n / period, rem = n - full * period;
  return full * il + min(max(rem - rank * il, 0), il);
}

// ---- fp8 (e4m3) cache path --------------------------------------------------------------------
// The raw bytes go to shared memory (16-byte chunk c of token row r at a swizzled position) and are
// widened to fp16 in registers right after ldmatrix (e4m3 is a subset of fp16, so this is exact).
// Q and P are fed as fp16 to the fp16 MMA.
//  * QK: an 8x8 b16 ldmatrix tile is 8 tokens x 16 e4m3 values, so a thread receives k = 4c..4c+3 of a
//    16-wide k block (c = lane & 3) instead of the MMA's {2c, 2c+1, 2c+8, 2c+9}; the Q fragments are
//    loaded with the same permutation of k, which leaves the dot product unchanged.
//  * PV: the transposed tile hands a thread V[tokens 2c, 2c+1][dims 2j, 2j+1] (j = lane >> 2); even and
//    odd dims go to two MMAs, so accumulator o[2 * dc + par][e] holds dim 16 * dc + 4c + par + 2 * (e & 1).
template <int D>
__device__ __forceinline__ int swz_fp8(int r, int c) {
  return D == 128 ? (c ^ (r & 7)) : (c ^ ((r >> 1) & 3));
}
template <int D, int NTHREADS>
__device__ __forceinline__ void load_rows_async_fp8(uint32_t smem_base, const uint8_t* g, int rows, int tid) {
  constexpr int CPR = D / 16;
  for (int idx = tid; idx < rows * CPR; idx += NTHREADS) {
    const int r = idx / CPR, c = idx % CPR;
    cp_async16(smem_base + (uint32_t)(r * D + (swz_fp8<D>(r, c) << 4)), g + ((size_t)idx << 4));
  }
}
// How e4m3 pairs become f16x2: bit 0 (K) / bit 1 (V) set = cvt.rn.f16x2.e4m3x2, clear = the integer
// widening below.  Measured on B200 (256 requests x 2048 context): 0.358 ms with 0, 0.334 with 1 or 2,
// 0.307 with 3; the bf16 cache takes 0.338 ms.
#ifndef B200_FP8_WIDEN
#define B200_FP8_WIDEN 3
#endif
// Two e4m3 bytes of x, picked by the byte permutation SEL = 0x{hi}4{lo}4, to f16x2 (low half first).
// Integer widening: the 7 magnitude bits of a byte placed at bit 7 of a half give exactly value / 256,
// sub-normals included, so that variant carries a factor that the host folds into the scales.
template <int HW, uint32_t SEL>
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2_scaled(uint32_t x) {
  if constexpr (HW) {
    constexpr uint32_t LO = (SEL >> 4) & 0xfu, HI = (SEL >> 12) & 0xfu;
    uint32_t h2;
    if constexpr (LO == 0 && HI == 1) {
      asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.rn.f16x2.e4m3x2 %0, lo; }" : "=r"(h2) : "r"(x));
    } else if constexpr (LO == 2 && HI == 3) {
      asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.rn.f16x2.e4m3x2 %0, hi; }" : "=r"(h2) : "r"(x));
    } else {
      uint32_t u;
      asm("prmt.b32 %0, %1, 0, %2;" : "=r"(u) : "r"(x), "n"(0x4400u | (HI << 4) | LO));
      asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.rn.f16x2.e4m3x2 %0, lo; }" : "=r"(h2) : "r"(u));
    }
    return h2;
  }
  uint32_t t;
  asm("prmt.b32 %0, %1, 0, %2;" : "=r"(t) : "r"(x), "n"(SEL));       // (b_lo << 8) | (b_hi << 24)
  return (t & 0x80008000u) | ((t >> 1) & 0x3f803f80u);
}
constexpr bool kHwK = (B200_FP8_WIDEN & 1) != 0, kHwV = (B200_FP8_WIDEN & 2) != 0;
__device__ __forceinline__ void mma_f16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_f16(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
  const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
  return pack_f16(f.x, f.y);
}
// Q fragments for the fp8 path: fp16, k permuted as described above.  q0 / q1 may be null (zero rows).
template <int D>
__device__ __forceinline__ void load_q_frags_fp8(uint32_t (*qf)[4], const __nv_bfloat16* q0,
                                                 const __nv_bfloat16* q1, int lane) {
  const int c4 = 4 * (lane & 3);
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    uint2 a = make_uint2(0u, 0u), b = make_uint2(0u, 0u);
    if (q0) a = *reinterpret_cast<const uint2*>(q0 + ks * 16 + c4);
    if (q1) b = *reinterpret_cast<const uint2*>(q1 + ks * 16 + c4);
    qf[ks][0] = bf16x2_to_f16x2(a.x); qf[ks][1] = bf16x2_to_f16x2(b.x);
    qf[ks][2] = bf16x2_to_f16x2(a.y); qf[ks][3] = bf16x2_to_f16x2(b.y);
  }
}
template <int D>
__device__ __forceinline__ void qk_16_fp8(float s[2][4], const uint32_t (*qf)[4], uint32_t kbase, int lane) {
  const int mi = lane >> 3, rr = lane & 7;
  const int tok = (mi & 1) * 8 + rr;
#pragma unroll
  for (int k2 = 0; k2 < D / 32; ++k2) {
    const int c = 2 * k2 + (mi >> 1);
    uint32_t b[4];     // (tokens 0-7, chunk 2k2) (8-15, 2k2) (0-7, 2k2+1) (8-15, 2k2+1)
    ldsm_x4(b, kbase + (uint32_t)(tok * D + (swz_fp8<D>(tok, c) << 4)));
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mma_f16_16816(s[0], qf[2 * k2 + h], e4m3x2_to_f16x2_scaled<kHwK, 0x1404u>(b[2 * h]),
                    e4m3x2_to_f16x2_scaled<kHwK, 0x3424u>(b[2 * h]));
      mma_f16_16816(s[1], qf[2 * k2 + h], e4m3x2_to_f16x2_scaled<kHwK, 0x1404u>(b[2 * h + 1]),
                    e4m3x2_to_f16x2_scaled<kHwK, 0x3424u>(b[2 * h + 1]));
    }
  }
}
template <int D>
__device__ __forceinline__ void pv_16_fp8(float (*o)[4], const uint32_t* pa, uint32_t vbase, int lane) {
  const int mi = lane >> 3, rr = lane & 7;
  const int tok = (mi & 1) * 8 + rr;
#pragma unroll
  for (int d2 = 0; d2 < D / 32; ++d2) {
    const int c = 2 * d2 + (mi >> 1);
    uint32_t b[4];     // (tokens 0-7, chunk 2d2) (8-15, 2d2) (0-7, 2d2+1) (8-15, 2d2+1)
    ldsm_x4_t(b, vbase + (uint32_t)(tok * D + (swz_fp8<D>(tok, c) << 4)));
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      // bytes of b[2h]: V[2c][2j], V[2c][2j+1], V[2c+1][2j], V[2c+1][2j+1]; b[2h+1]: tokens + 8
      const uint32_t lo = b[2 * h], hi = b[2 * h + 1];
      mma_f16_16816(o[4 * d2 + 2 * h], pa, e4m3x2_to_f16x2_scaled<kHwV, 0x2404u>(lo),
                    e4m3x2_to_f16x2_scaled<kHwV, 0x2404u>(hi));
      mma_f16_16816(o[4 * d2 + 2 * h + 1], pa, e4m3x2_to_f16x2_scaled<kHwV, 0x3414u>(lo),
                    e4m3x2_to_f16x2_scaled<kHwV, 0x3414u>(hi));
    }
  }
}

// ------------------------------------------------------------------------ decode
// FP8: the cache holds e4m3 bytes; the ring keeps the same number of bytes in flight with twice the stages.
template <int D, bool FP8>
struct DecodeSmem {
  static constexpr int STAGES = FP8 ? 6 : 3;
  static constexpr int PAGE_BYTES = 16 * D * (FP8 ? 1 : 2);           // 16 tokens of K (or V) as stored
  static constexpr int STAGE_BYTES = 2 * PAGE_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int MERGE_BYTES = 16 * D * 4;                      // [16][D] fp32 per warp at the end
  static constexpr int WARP_BYTES = RING_BYTES > MERGE_BYTES ? RING_BYTES : MERGE_BYTES;
  static constexpr int TOTAL = 4 * WARP_BYTES;
};

template <int D, bool FP8 = false>
__global__ void __launch_bounds__(128, 2) attn_decode_kernel(const AttnParams p) {
  using SM = DecodeSmem<D, FP8>;
  constexpr int STAGES = SM::STAGES;
  constexpr int PAGE_BYTES = SM::PAGE_BYTES;
  constexpr int STAGE_BYTES = SM::STAGE_BYTES;
  constexpr int WARP_BYTES = SM::WARP_BYTES;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float s_ml[4][16][2];
  __shared__ int s_last;

  pdl_launch_dependents();      // o_proj may start and prefetch its weights while this grid drains
  pdl_wait();                   // q and the new KV rows come from the kernel before this grid
  const int h = blockIdx.x, r = p.req_begin + blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  const int qs = p.qsl[r], q_len = p.qsl[r + 1] - qs, seq_len = p.seq_lens[r];
  if (q_len <= 0 || seq_len <= 0) return;       // padded request (uniform for the CTA)
  const int ctx = seq_len - q_len;
  const int rows_valid = min(q_len * G, 16);

  // Q fragments straight from global memory: tile row = j * G + g
  uint32_t qf[D / 16][4];
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
    const int cb = 2 * (lane & 3);
    const __nv_bfloat16* q0 = nullptr;
    const __nv_bfloat16* q1 = nullptr;
    if (r0 < rows_valid) q0 = p.q + ((size_t)(qs + r0 / G) * p.Hq + h * G + r0 % G) * D;
    if (r1 < rows_valid) q1 = p.q + ((size_t)(qs + r1 / G) * p.Hq + h * G + r1 % G) * D;
    if constexpr (FP8) {
      load_q_frags_fp8<D>(qf, q0, q1, lane);
    } else {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        qf[ks][0] = q0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + cb) : 0u;
        qf[ks][1] = q1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + cb) : 0u;
        qf[ks][2] = q0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + cb) : 0u;
        qf[ks][3] = q1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + cb) : 0u;
      }
    }
  }

  // this (split, warp) unit's range of 16-token chunks
  int first_tok = 0;
  if (p.window > 0) first_tok = max(0, ctx - p.window + 1);
  const int c_lo = first_tok >> 4;
  const int C = ((seq_len + 15) >> 4) - c_lo;
  const int units = p.num_splits * 4;
  const int per = (C + units - 1) / units;
  const int u = split * 4 + warp;
  const int cb0 = c_lo + min(C, u * per);
  const int cb1 = c_lo + min(C, (u + 1) * per);

  const uint32_t wbase = smem_u32(smem) + warp * WARP_BYTES;
  const int* bt = p.block_tables + (size_t)r * p.max_blocks;
  const size_t head_stride = (size_t)p.block_size * D;          // one (k|v, head) slab of a page
  // Block ids of this warp's page range are fetched 32 at a time (one per lane) and handed out by
  // shuffle, so the address of a chunk never waits on a dependent global load.
  const int page_lo = (cb0 << 4) / p.block_size;
  const int page_hi = cb1 > cb0 ? (((cb1 << 4) - 1) / p.block_size) : page_lo - 1;
  int bt_base = page_lo;
  int bt_reg = (page_lo + lane <= page_hi) ? bt[page_lo + lane] : 0;
  auto issue = [&](int chunk, int stage) {
    const int tok = chunk << 4;
    const int page = tok / p.block_size, off = tok - page * p.block_size;
    if (page >= bt_base + 32) {                       // warp-uniform
      bt_base = page;
      bt_reg = (page + lane <= page_hi) ? bt[page + lane] : 0;
    }
    long long blk = __shfl_sync(0xffffffffu, bt_reg, page - bt_base);
    if (blk < 0 || blk >= p.num_blocks || page >= p.max_blocks) {
      if (lane == 0) B200_NOTE_BAD_INDEX();
      blk = 0;
    }
    const size_t ko = (((size_t)blk * 2 + 0) * p.Hkv + h) * head_stride + (size_t)off * D;
    const size_t vo = (((size_t)blk * 2 + 1) * p.Hkv + h) * head_stride + (size_t)off * D;
    const uint32_t sb = wbase + stage * STAGE_BYTES;
    if constexpr (FP8) {
      const uint8_t* kv8 = reinterpret_cast<const uint8_t*>(p.kv);
      load_rows_async_fp8<D, 32>(sb, kv8 + ko, 16, lane);
      load_rows_async_fp8<D, 32>(sb + PAGE_BYTES, kv8 + vo, 16, lane);
    } else {
      load_rows_async<D, 32>(sb, p.kv + ko, 16, lane);
      load_rows_async<D, 32>(sb + PAGE_BYTES, p.kv + vo, 16, lane);
    }
  };

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const int row0 = lane >> 2, row1 = row0 + 8;
  const int lim0 = ctx + row0 / G, lim1 = ctx + row1 / G;       // last visible key per row

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (cb0 + s < cb1) issue(cb0 + s, s);
    cp_async_commit();
  }
  for (int c = cb0; c < cb1; ++c) {
    const int stage = (c - cb0) % STAGES;
    cp_async_wait<STAGES - 2>();
    __syncwarp();
    if (c + STAGES - 1 < cb1) issue(c + STAGES - 1, (c - cb0 + STAGES - 1) % STAGES);
    cp_async_commit();

    const uint32_t sb = wbase + stage * STAGE_BYTES;
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    if constexpr (FP8) qk_16_fp8<D>(s, qf, sb, lane);
    else qk_16<D>(s, qf, sb, lane);
    const int tk = (c << 4) + 2 * (lane & 3);
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = tk + nb * 8 + (e & 1);
        const int lim = (e < 2) ? lim0 : lim1;
        float v = s[nb][e] * p.scale_log2;
        if (p.softcap > 0.f) v = p.softcap * tanhf(v / p.softcap);
        const bool ok = tok <= lim && (p.window <= 0 || tok > lim - p.window);
        v = ok ? v : -INFINITY;
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
    if (__any_sync(0xffffffffu, a0 != 1.f || a1 != 1.f)) {     // the running max rarely moves
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1;
      }
    }
    if constexpr (FP8) {
      uint32_t pa[4] = {pack_f16(s[0][0], s[0][1]), pack_f16(s[0][2], s[0][3]), pack_f16(s[1][0], s[1][1]),
                        pack_f16(s[1][2], s[1][3])};
      pv_16_fp8<D>(o, pa, sb + PAGE_BYTES, lane);
    } else {
      uint32_t pa[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]), pack_bf16(s[1][0], s[1][1]),
                        pack_bf16(s[1][2], s[1][3])};
      pv_16<D>(o, pa, sb + PAGE_BYTES, lane);
    }
  }
  cp_async_wait<0>();
  // row sums over the 4 lanes that share a row
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1); l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1); l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
  __syncwarp();

  // ---- merge the 4 warps in shared memory (each warp reuses its own ring)
  float* wo = reinterpret_cast<float*>(smem + warp * WARP_BYTES);        // [16][D] fp32 (<= 8 KB)
  if constexpr (FP8) {
#pragma unroll
    for (int dc = 0; dc < D / 16; ++dc) {             // permuted accumulator layout of pv_16_fp8
      const int col = dc * 16 + 4 * (lane & 3);
      *reinterpret_cast<float4*>(wo + row0 * D + col) =
          make_float4(o[2 * dc][0], o[2 * dc + 1][0], o[2 * dc][1], o[2 * dc + 1][1]);
      *reinterpret_cast<float4*>(wo + row1 * D + col) =
          make_float4(o[2 * dc][2], o[2 * dc + 1][2], o[2 * dc][3], o[2 * dc + 1][3]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int col = i * 8 + 2 * (lane & 3);
      *reinterpret_cast<float2*>(wo + row0 * D + col) = make_float2(o[i][0], o[i][1]);
      *reinterpret_cast<float2*>(wo + row1 * D + col) = make_float2(o[i][2], o[i][3]);
    }
  }
  if ((lane & 3) == 0) {
    s_ml[warp][row0][0] = m[0]; s_ml[warp][row0][1] = l[0];
    s_ml[warp][row1][0] = m[1]; s_ml[warp][row1][1] = l[1];
  }
  __syncthreads();
  const int row = threadIdx.x >> 3;               // 16 rows x 8 threads
  const int seg = threadIdx.x & 7;
  constexpr int SEG = D / 8;                      // dims per thread
  float mm = -INFINITY;
#pragma unroll
  for (int w = 0; w < 4; ++w) mm = fmaxf(mm, s_ml[w][row][0]);
  float L = 0.f, acc[SEG];
#pragma unroll
  for (int d = 0; d < SEG; ++d) acc[d] = 0.f;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const float mw = s_ml[w][row][0];
    const float sc = (mw == -INFINITY) ? 0.f : ex2(mw - mm);
    L += s_ml[w][row][1] * sc;
    const float* src = reinterpret_cast<const float*>(smem + w * WARP_BYTES) + row * D + seg * SEG;
#pragma unroll
    for (int d = 0; d < SEG; ++d) acc[d] += src[d] * sc;
  }
  const bool row_ok = row < rows_valid;
  const int tok_row = qs + row / G, head = h * G + row % G;

  auto finish = [&](float mfin, float Lfin, const float* a) {
    if (!row_ok) return;
    if (p.sinks != nullptr) {
      // attention sink: one extra logit per head that only joins the normaliser
      const float sk = p.sinks[head] * 1.4426950408889634f;
      const float mnew = fmaxf(mfin, sk);
      const float sc = (mfin == -INFINITY) ? 0.f : ex2(mfin - mnew);
      Lfin = Lfin * sc + ex2(sk - mnew);
      mfin = mnew;
      const float inv = (FP8 ? p.v_scale : 1.f) / Lfin;
      __nv_bfloat16* dst = p.out + ((size_t)tok_row * p.Hq + head) * D + seg * SEG;
#pragma unroll
      for (int d = 0; d < SEG; ++d) dst[d] = __float2bfloat16(a[d] * sc * inv);
    } else {
      const float inv = Lfin > 0.f ? (FP8 ? p.v_scale : 1.f) / Lfin : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)tok_row * p.Hq + head) * D + seg * SEG;
#pragma unroll
      for (int d = 0; d < SEG; ++d) dst[d] = __float2bfloat16(a[d] * inv);
    }
    if (p.lse != nullptr && seg == 0)
      p.lse[(size_t)tok_row * p.Hq + head] =
          Lfin > 0.f ? (mfin + log2f(Lfin)) * 0.6931471805599453f : -INFINITY;
  };

  if (p.num_splits == 1) {
    finish(mm, L, acc);
    return;
  }
  // ---- cross-split merge by the last CTA of this (request, kv head)
  const size_t unit = ((size_t)blockIdx.y * p.Hkv + h) * p.num_splits;
  float* po = p.part_o + ((unit + split) * 16 + row) * D + seg * SEG;
#pragma unroll
  for (int d = 0; d < SEG; ++d) po[d] = acc[d];
  if (seg == 0) {
    p.part_ml[((unit + split) * 16 + row) * 2 + 0] = mm;
    p.part_ml[((unit + split) * 16 + row) * 2 + 1] = L;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(&p.counters[blockIdx.y * p.Hkv + h], 1);
    s_last = (old == p.num_splits - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  float mfin = -INFINITY;
  for (int s2 = 0; s2 < p.num_splits; ++s2)
    mfin = fmaxf(mfin, __ldcg(&p.part_ml[((unit + s2) * 16 + row) * 2]));
  float Lfin = 0.f;
#pragma unroll
  for (int d = 0; d < SEG; ++d) acc[d] = 0.f;
  for (int s2 = 0; s2 < p.num_splits; ++s2) {
    const float ms = __ldcg(&p.part_ml[((unit + s2) * 16 + row) * 2]);
    const float sc = (ms == -INFINITY) ? 0.f : ex2(ms - mfin);
    Lfin += __ldcg(&p.part_ml[((unit + s2) * 16 + row) * 2 + 1]) * sc;
    const float* src = p.part_o + ((unit + s2) * 16 + row) * D + seg * SEG;
#pragma unroll
    for (int d = 0; d < SEG; ++d) acc[d] += __ldcg(src + d) * sc;
  }
  finish(mfin, Lfin, acc);
  if (threadIdx.x == 0) p.counters[blockIdx.y * p.Hkv + h] = 0;
}

// ----------------------------------------------------------------------- prefill
// FP8: the stages hold raw e4m3 tiles, widened in registers (see the fp8 cache path above).
template <int D, bool FP8 = false>
__global__ void __launch_bounds__(128, 3) attn_prefill_kernel(const AttnParams p) {
  constexpr int BQ = 64, BKV = 64;
  constexpr int EB = FP8 ? 1 : 2;                  // bytes per cache element
  constexpr int TILE_BYTES = BKV * D * EB;         // K (or V) chunk as stored
  constexpr int GROUP_BYTES = 16 * D * EB;         // one 16-token group
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_launch_dependents();
  const int hq = blockIdx.x;
  const int G = p.Hq / p.Hkv;
  const int h = hq / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // find (request, q block) of this tile: linear scan over the ragged batch
  int r = -1, q0 = 0;
  {
    int tile = blockIdx.y;
    for (int i = p.req_begin; i < p.req_end; ++i) {
      const int ql = p.qsl[i + 1] - p.qsl[i];
      const int nt = (ql + BQ - 1) / BQ;
      if (tile < nt) { r = i; q0 = tile * BQ; break; }
      tile -= nt;
    }
  }
  if (r < 0) return;
  const int qs = p.qsl[r], q_len = p.qsl[r + 1] - qs, seq_len = p.seq_lens[r];
  if (seq_len <= 0) return;
  const int ctx = seq_len - q_len;
  const int row0 = q0 + warp * 16 + (lane >> 2), row1 = row0 + 8;   // rows inside the request
  // index of the last key row `row` may see: ctx + row, or under decode context parallelism the number of
  // local keys at global positions <= the row's, minus one
  const bool dcp = p.dcp_size > 1;
  const int gctx = dcp ? p.global_seq_lens[r] - q_len : ctx;
  auto last_key = [&](int row) {
    return dcp ? dcp_local_len(gctx + row + 1, p.dcp_rank, p.dcp_size, p.dcp_interleave) - 1 : ctx + row;
  };

  uint32_t qf[D / 16][4];
  {
    const int cb = 2 * (lane & 3);
    const __nv_bfloat16* qa = row0 < q_len ? p.q + ((size_t)(qs + row0) * p.Hq + hq) * D : nullptr;
    const __nv_bfloat16* qb = row1 < q_len ? p.q + ((size_t)(qs + row1) * p.Hq + hq) * D : nullptr;
    if constexpr (FP8) {
      load_q_frags_fp8<D>(qf, qa, qb, lane);
    } else {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        qf[ks][0] = qa ? *reinterpret_cast<const uint32_t*>(qa + ks * 16 + cb) : 0u;
        qf[ks][1] = qb ? *reinterpret_cast<const uint32_t*>(qb + ks * 16 + cb) : 0u;
        qf[ks][2] = qa ? *reinterpret_cast<const uint32_t*>(qa + ks * 16 + 8 + cb) : 0u;
        qf[ks][3] = qb ? *reinterpret_cast<const uint32_t*>(qb + ks * 16 + 8 + cb) : 0u;
      }
    }
  }
  const int kv_end = p.non_causal ? seq_len : min(seq_len, last_key(q0 + BQ - 1) + 1);   // causal bound of the tile
  int kv_begin = 0;
  if (p.window > 0) kv_begin = max(0, ctx + q0 - p.window + 1) / BKV * BKV;
  const int nchunks = (kv_end - kv_begin + BKV - 1) / BKV;

  const int* bt = p.block_tables + (size_t)r * p.max_blocks;
  const size_t head_stride = (size_t)p.block_size * D;
  const uint32_t sbase = smem_u32(smem);
  auto issue = [&](int chunk, int stage) {
    const int tok0 = kv_begin + chunk * BKV;
    const uint32_t sb = sbase + stage * STAGE_BYTES;
    // 64 tokens = 4 groups of 16; a group never straddles a page (block_size % 16 == 0)
#pragma unroll
    for (int g = 0; g < BKV / 16; ++g) {
      const int tok = tok0 + g * 16;
      if (tok >= kv_end) break;
      const int page = tok / p.block_size, off = tok - page * p.block_size;
      long long blk = page < p.max_blocks ? bt[page] : -1;
      if (blk < 0 || blk >= p.num_blocks) {
        if (threadIdx.x == 0) B200_NOTE_BAD_INDEX();
        blk = 0;
      }
      const size_t ko = (((size_t)blk * 2 + 0) * p.Hkv + h) * head_stride + (size_t)off * D;
      const size_t vo = (((size_t)blk * 2 + 1) * p.Hkv + h) * head_stride + (size_t)off * D;
      if constexpr (FP8) {
        const uint8_t* kv8 = reinterpret_cast<const uint8_t*>(p.kv);
        load_rows_async_fp8<D, 128>(sb + g * GROUP_BYTES, kv8 + ko, 16, threadIdx.x);
        load_rows_async_fp8<D, 128>(sb + TILE_BYTES + g * GROUP_BYTES, kv8 + vo, 16, threadIdx.x);
      } else {
        load_rows_async<D, 128>(sb + g * GROUP_BYTES, p.kv + ko, 16, threadIdx.x);
        load_rows_async<D, 128>(sb + TILE_BYTES + g * GROUP_BYTES, p.kv + vo, 16, threadIdx.x);
      }
    }
  };

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const int lim0 = p.non_causal ? 0x3fffffff : last_key(row0), lim1 = p.non_causal ? 0x3fffffff : last_key(row1);

  if (nchunks > 0) issue(0, 0);
  cp_async_commit();
  for (int c = 0; c < nchunks; ++c) {
    const int stage = c & 1;
    if (c + 1 < nchunks) issue(c + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t sb = sbase + stage * STAGE_BYTES;
    const int tok0 = kv_begin + c * BKV;
    // skip groups entirely above this warp's diagonal
    const int warp_max_key = p.non_causal ? 0x3fffffff : last_key(q0 + warp * 16 + 15);
    float s[BKV / 8][4];
#pragma unroll
    for (int i = 0; i < BKV / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int g = 0; g < BKV / 16; ++g) {
      if (tok0 + g * 16 <= warp_max_key && tok0 + g * 16 < kv_end) {
        if constexpr (FP8) qk_16_fp8<D>(reinterpret_cast<float(*)[4]>(&s[2 * g][0]), qf, sb + g * GROUP_BYTES, lane);
        else qk_16<D>(reinterpret_cast<float(*)[4]>(&s[2 * g][0]), qf, sb + g * GROUP_BYTES, lane);
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < BKV / 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = tok0 + nb * 8 + 2 * (lane & 3) + (e & 1);
        const int lim = (e < 2) ? lim0 : lim1;
        float v = s[nb][e] * p.scale_log2;
        if (p.softcap > 0.f) v = p.softcap * tanhf(v / p.softcap);
        const bool ok = tok <= lim && tok < kv_end && (p.window <= 0 || tok > lim - p.window);
        v = ok ? v : -INFINITY;
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
    for (int nb = 0; nb < BKV / 8; ++nb) {
      s[nb][0] = ex2(s[nb][0] - base0); s[nb][1] = ex2(s[nb][1] - base0);
      s[nb][2] = ex2(s[nb][2] - base1); s[nb][3] = ex2(s[nb][3] - base1);
      ps0 += s[nb][0] + s[nb][1];
      ps1 += s[nb][2] + s[nb][3];
    }
    l[0] = l[0] * a0 + ps0;
    l[1] = l[1] * a1 + ps1;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1;
    }
#pragma unroll
    for (int g = 0; g < BKV / 16; ++g) {
      if (tok0 + g * 16 <= warp_max_key && tok0 + g * 16 < kv_end) {
        if constexpr (FP8) {
          uint32_t pa[4] = {pack_f16(s[2 * g][0], s[2 * g][1]), pack_f16(s[2 * g][2], s[2 * g][3]),
                            pack_f16(s[2 * g + 1][0], s[2 * g + 1][1]),
                            pack_f16(s[2 * g + 1][2], s[2 * g + 1][3])};
          pv_16_fp8<D>(o, pa, sb + TILE_BYTES + g * GROUP_BYTES, lane);
        } else {
          uint32_t pa[4] = {pack_bf16(s[2 * g][0], s[2 * g][1]), pack_bf16(s[2 * g][2], s[2 * g][3]),
                            pack_bf16(s[2 * g + 1][0], s[2 * g + 1][1]),
                            pack_bf16(s[2 * g + 1][2], s[2 * g + 1][3])};
          pv_16<D>(o, pa, sb + TILE_BYTES + g * GROUP_BYTES, lane);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1); l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1); l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);

  float sc0 = 1.f, sc1 = 1.f;
  if (p.sinks != nullptr) {
    const float sk = p.sinks[hq] * 1.4426950408889634f;
    const float n0 = fmaxf(m[0], sk), n1 = fmaxf(m[1], sk);
    sc0 = (m[0] == -INFINITY) ? 0.f : ex2(m[0] - n0);
    sc1 = (m[1] == -INFINITY) ? 0.f : ex2(m[1] - n1);
    l[0] = l[0] * sc0 + ex2(sk - n0);
    l[1] = l[1] * sc1 + ex2(sk - n1);
    m[0] = n0; m[1] = n1;
  }
  if constexpr (FP8) { sc0 *= p.v_scale; sc1 *= p.v_scale; }
  const float inv0 = l[0] > 0.f ? sc0 / l[0] : 0.f, inv1 = l[1] > 0.f ? sc1 / l[1] : 0.f;
  if (row0 < q_len) {
    __nv_bfloat16* dst = p.out + ((size_t)(qs + row0) * p.Hq + hq) * D + (FP8 ? 4 : 2) * (lane & 3);
    if constexpr (FP8) {
#pragma unroll
      for (int dc = 0; dc < D / 16; ++dc)
        *reinterpret_cast<uint2*>(dst + dc * 16) =
            make_uint2(pack_bf16(o[2 * dc][0] * inv0, o[2 * dc + 1][0] * inv0),
                       pack_bf16(o[2 * dc][1] * inv0, o[2 * dc + 1][1] * inv0));
    } else {
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
    }
    if (p.lse != nullptr && (lane & 3) == 0)
      p.lse[(size_t)(qs + row0) * p.Hq + hq] =
          l[0] > 0.f ? (m[0] + log2f(l[0])) * 0.6931471805599453f : -INFINITY;
  }
  if (row1 < q_len) {
    __nv_bfloat16* dst = p.out + ((size_t)(qs + row1) * p.Hq + hq) * D + (FP8 ? 4 : 2) * (lane & 3);
    if constexpr (FP8) {
#pragma unroll
      for (int dc = 0; dc < D / 16; ++dc)
        *reinterpret_cast<uint2*>(dst + dc * 16) =
            make_uint2(pack_bf16(o[2 * dc][2] * inv1, o[2 * dc + 1][2] * inv1),
                       pack_bf16(o[2 * dc][3] * inv1, o[2 * dc + 1][3] * inv1));
    } else {
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
    }
    if (p.lse != nullptr && (lane & 3) == 0)
      p.lse[(size_t)(qs + row1) * p.Hq + hq] =
          l[1] > 0.f ? (m[1] + log2f(l[1])) * 0.6931471805599453f : -INFINITY;
  }
}

}  // namespace b200

using namespace b200;

static void fill_params(AttnParams& p, const void* q, const void* kv, void* out, float* lse,
                        const int* block_tables, const int* seq_lens, const int* qsl, int max_blocks,
                        int block_size, long long num_blocks, int Hq, int Hkv, int D, float scale, int window,
                        float softcap, const float* sinks) {
  p.q = (const __nv_bfloat16*)q;
  p.kv = (const __nv_bfloat16*)kv;
  p.out = (__nv_bfloat16*)out;
  p.lse = lse;
  p.block_tables = block_tables;
  p.seq_lens = seq_lens;
  p.qsl = qsl;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  p.num_blocks = num_blocks;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.softcap = softcap > 0.f ? softcap * 1.4426950408889634f : 0.f;
  p.sinks = sinks;
  p.v_scale = 1.f;
  p.non_causal = 0;
  p.global_seq_lens = nullptr;
  p.dcp_size = 1; p.dcp_rank = 0; p.dcp_interleave = 1;
  (void)D;
}

// fp8 (e4m3) cache: K's dequantisation factor joins the logit scale, V's the output normalisation.
// The integer widening variant yields value / 256 (see e4m3x2_to_f16x2_scaled), hence the factors.
static void set_fp8_scales(AttnParams& p, float k_scale, float v_scale) {
  p.scale_log2 *= k_scale * (kHwK ? 1.f : 256.f);
  p.v_scale = v_scale * (kHwV ? 1.f : 256.f);
}

template <int D, bool FP8>
static cudaError_t launch_decode(dim3 grid, cudaStream_t stream, const AttnParams& p) {
  constexpr int smem = DecodeSmem<D, FP8>::TOTAL;
  static unsigned long long seen = 0;
  cudaError_t e = ensure_dynamic_smem(attn_decode_kernel<D, FP8>, smem, &seen);
  if (e != cudaSuccess) return e;
  return launch_pdl(attn_decode_kernel<D, FP8>, grid, dim3(128), smem, stream, p);
}

template <int D, bool FP8>
static cudaError_t launch_prefill(dim3 grid, cudaStream_t stream, const AttnParams& p) {
  constexpr int smem = 2 * 2 * 64 * D * (FP8 ? 1 : 2);
  static unsigned long long seen = 0;
  cudaError_t e = ensure_dynamic_smem(attn_prefill_kernel<D, FP8>, smem, &seen);
  if (e != cudaSuccess) return e;
  attn_prefill_kernel<D, FP8><<<grid, 128, smem, stream>>>(p);
  return cudaGetLastError();
}

// Scratch sizes of the decode kernel for (num_reqs, Hkv, splits, D).
extern "C" size_t b200_attn_decode_scratch_bytes(int num_reqs, int Hkv, int splits, int D) {
  if (splits <= 1) return 0;
  return (size_t)num_reqs * Hkv * splits * 16 * (D + 2) * sizeof(float);
}

// Requests [req_begin, req_end) must have q_len * (Hq/Hkv) <= 16.  scratch holds part_o then
// part_ml; counters: [num_reqs * Hkv] ints, zero before first use (re-armed by the kernel).
static int attn_decode_impl(const void* q, const void* kv, void* out, float* lse, const int* block_tables,
                            const int* seq_lens, const int* qsl, int req_begin, int req_end,
                            int max_blocks, int block_size, long long num_blocks, int Hq, int Hkv, int D,
                            float scale, int window, float softcap, const float* sinks, int num_splits,
                            void* scratch, int* counters, int kv_fp8, float k_scale, float v_scale,
                            cudaStream_t stream) {
  const int R = req_end - req_begin;
  if (R <= 0) return 0;
  if (block_size % 16 || (Hq % Hkv) || Hq / Hkv > 16) {
    b200_set_last_error("attn_decode: block_size % 16 == 0 and q heads per kv head <= 16 required", __FILE__,
                        __LINE__);
    return -1;
  }
  AttnParams p;
  fill_params(p, q, kv, out, lse, block_tables, seq_lens, qsl, max_blocks, block_size, num_blocks, Hq, Hkv, D,
              scale, window, softcap, sinks);
  p.req_begin = req_begin;
  p.req_end = req_end;
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 1 && (scratch == nullptr || counters == nullptr)) num_splits = 1;
  p.num_splits = num_splits;
  p.part_o = (float*)scratch;
  p.part_ml = p.part_o + (size_t)R * Hkv * num_splits * 16 * D;
  p.counters = counters;
  dim3 grid(Hkv, R, num_splits);
  if (kv_fp8) set_fp8_scales(p, k_scale, v_scale);
  if (D == 128 && kv_fp8) B200_CUDA_CHECK((launch_decode<128, true>(grid, stream, p)));
  else if (D == 128) B200_CUDA_CHECK((launch_decode<128, false>(grid, stream, p)));
  else if (D == 64 && kv_fp8) B200_CUDA_CHECK((launch_decode<64, true>(grid, stream, p)));
  else if (D == 64) B200_CUDA_CHECK((launch_decode<64, false>(grid, stream, p)));
  else {
    b200_set_last_error("attn_decode: head_dim must be 64 or 128", __FILE__, __LINE__);
    return -1;
  }
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_attn_decode(const void* q, const void* kv, void* out, float* lse, const int* block_tables,
                                const int* seq_lens, const int* qsl, int req_begin, int req_end,
                                int max_blocks, int block_size, long long num_blocks, int Hq, int Hkv, int D,
                                float scale, int window, float softcap, const float* sinks, int num_splits,
                                void* scratch, int* counters, cudaStream_t stream) {
  return attn_decode_impl(q, kv, out, lse, block_tables, seq_lens, qsl, req_begin, req_end, max_blocks,
                          block_size, num_blocks, Hq, Hkv, D, scale, window, softcap, sinks, num_splits, scratch,
                          counters, 0, 1.f, 1.f, stream);
}
// The cache holds e4m3 bytes: stored value * k_scale (v_scale) is the key (value).
extern "C" int b200_attn_decode_fp8kv(const void* q, const void* kv, void* out, float* lse,
                                      const int* block_tables, const int* seq_lens, const int* qsl,
                                      int req_begin, int req_end, int max_blocks, int block_size,
                                      long long num_blocks, int Hq, int Hkv, int D, float scale, int window,
                                      float softcap, const float* sinks, int num_splits, void* scratch,
                                      int* counters, float k_scale, float v_scale, cudaStream_t stream) {
  return attn_decode_impl(q, kv, out, lse, block_tables, seq_lens, qsl, req_begin, req_end, max_blocks,
                          block_size, num_blocks, Hq, Hkv, D, scale, window, softcap, sinks, num_splits, scratch,
                          counters, 1, k_scale, v_scale, stream);
}

// num_tiles = sum over requests of ceil(q_len / 64) (computed by the caller from host metadata).
struct DcpArgs {
  const int* global_seq_lens = nullptr;
  int size = 1, rank = 0, interleave = 1;
};

static int attn_prefill_impl(const void* q, const void* kv, void* out, float* lse, const int* block_tables,
                             const int* seq_lens, const int* qsl, int req_begin, int req_end,
                             int num_tiles, int max_blocks, int block_size, long long num_blocks, int Hq,
                             int Hkv, int D, float scale, int window, float softcap, const float* sinks,
                             int kv_fp8, float k_scale, float v_scale, cudaStream_t stream,
                             const DcpArgs& dcp = DcpArgs()) {
  if (req_end <= req_begin || num_tiles <= 0) return 0;
  if (block_size % 16 || (Hq % Hkv)) {
    b200_set_last_error("attn_prefill: block_size % 16 == 0 required", __FILE__, __LINE__);
    return -1;
  }
  AttnParams p;
  fill_params(p, q, kv, out, lse, block_tables, seq_lens, qsl, max_blocks, block_size, num_blocks, Hq, Hkv, D,
              scale, window, softcap, sinks);
  p.req_begin = req_begin;
  p.req_end = req_end;
  p.num_splits = 1;
  p.part_o = nullptr; p.part_ml = nullptr; p.counters = nullptr;
  if (dcp.size > 1) {
    if (dcp.global_seq_lens == nullptr || dcp.interleave <= 0 || window > 0) {
      b200_set_last_error("attn_prefill: decode context parallelism needs the global lengths and no sliding window",
                          __FILE__, __LINE__);
      return -1;
    }
    p.global_seq_lens = dcp.global_seq_lens;
    p.dcp_size = dcp.size; p.dcp_rank = dcp.rank; p.dcp_interleave = dcp.interleave;
  }
  dim3 grid(Hq, num_tiles);
  if (kv_fp8) set_fp8_scales(p, k_scale, v_scale);
  if (D == 128 && kv_fp8) B200_CUDA_CHECK((launch_prefill<128, true>(grid, stream, p)));
  else if (D == 128) B200_CUDA_CHECK((launch_prefill<128, false>(grid, stream, p)));
  else if (D == 64 && kv_fp8) B200_CUDA_CHECK((launch_prefill<64, true>(grid, stream, p)));
  else if (D == 64) B200_CUDA_CHECK((launch_prefill<64, false>(grid, stream, p)));
  else {
    b200_set_last_error("attn_prefill: head_dim must be 64 or 128", __FILE__, __LINE__);
    return -1;
  }
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// Prefill over a cache sharded by position (decode context parallelism): seq_lens are this rank's local
// lengths, global_seq_lens the true ones; query rows see the local keys whose global position is not
// after their own.  A request without local keys gets zeros and lse = -inf from the caller's initial fill.
extern "C" int b200_attn_prefill_dcp(const void* q, const void* kv, void* out, float* lse, const int* block_tables,
                                     const int* seq_lens, const int* global_seq_lens, const int* qsl,
                                     int req_begin, int req_end, int num_tiles, int max_blocks, int block_size,
                                     long long num_blocks, int Hq, int Hkv, int D, float scale, float softcap,
                                     int dcp_size, int dcp_rank, int dcp_interleave, cudaStream_t stream) {
  DcpArgs dcp;
  dcp.global_seq_lens = global_seq_lens;
  dcp.size = dcp_size; dcp.rank = dcp_rank; dcp.interleave = dcp_interleave;
  return attn_prefill_impl(q, kv, out, lse, block_tables, seq_lens, qsl, req_begin, req_end, num_tiles, max_blocks,
                           block_size, num_blocks, Hq, Hkv, D, scale, 0, softcap, nullptr, 0, 1.f, 1.f, stream, dcp);
}

extern "C" int b200_attn_prefill(const void* q, const void* kv, void* out, float* lse, const int* block_tables,
                                 const int* seq_lens, const int* qsl, int req_begin, int req_end,
                                 int num_tiles, int max_blocks, int block_size, long long num_blocks, int Hq,
                                 int Hkv, int D, float scale, int window, float softcap, const float* sinks,
                                 cudaStream_t stream) {
  return attn_prefill_impl(q, kv, out, lse, block_tables, seq_lens, qsl, req_begin, req_end, num_tiles,
                           max_blocks, block_size, num_blocks, Hq, Hkv, D, scale, window, softcap, sinks, 0, 1.f,
                           1.f, stream);
}
// Bidirectional attention over a ragged batch whose keys and values sit in the paged layout (vision
// encoders: each request's q_len equals its seq_len).  Same arguments as b200_attn_prefill.
extern "C" int b200_attn_encoder(const void* q, const void* kv, void* out, float* lse, const int* block_tables,
                                 const int* seq_lens, const int* qsl, int req_begin, int req_end, int num_tiles,
                                 int max_blocks, int block_size, long long num_blocks, int Hq, int Hkv, int D,
                                 float scale, cudaStream_t stream) {
  if (req_end <= req_begin || num_tiles <= 0) return 0;
  if (block_size % 16 || (Hq % Hkv)) {
    b200_set_last_error("attn_encoder: block_size % 16 == 0 required", __FILE__, __LINE__);
    return -1;
  }
  AttnParams p;
  fill_params(p, q, kv, out, lse, block_tables, seq_lens, qsl, max_blocks, block_size, num_blocks, Hq, Hkv, D,
              scale, 0, 0.f, nullptr);
  p.req_begin = req_begin;
  p.req_end = req_end;
  p.num_splits = 1;
  p.part_o = nullptr; p.part_ml = nullptr; p.counters = nullptr;
  p.non_causal = 1;
  dim3 grid(Hq, num_tiles);
  if (D == 128) B200_CUDA_CHECK((launch_prefill<128, false>(grid, stream, p)));
  else if (D == 64) B200_CUDA_CHECK((launch_prefill<64, false>(grid, stream, p)));
  else {
    b200_set_last_error("attn_encoder: head_dim must be 64 or 128", __FILE__, __LINE__);
    return -1;
  }
  return 0;
}
extern "C" int b200_attn_prefill_fp8kv(const void* q, const void* kv, void* out, float* lse,
                                       const int* block_tables, const int* seq_lens, const int* qsl,
                                       int req_begin, int req_end, int num_tiles, int max_blocks,
                                       int block_size, long long num_blocks, int Hq, int Hkv, int D, float scale,
                                       int window, float softcap, const float* sinks, float k_scale,
                                       float v_scale, cudaStream_t stream) {
  return attn_prefill_impl(q, kv, out, lse, block_tables, seq_lens, qsl, req_begin, req_end, num_tiles,
                           max_blocks, block_size, num_blocks, Hq, Hkv, D, scale, window, softcap, sinks, 1,
                           k_scale, v_scale, stream);
}

// ---------------------------------------------------------------------------------------
// Decode attention with built-in scratch, for callers that cannot allocate device memory.
// The contract (limits, set-up, sharing rules) is written out in attention_no_alloc.h.
// Nothing below calls an allocator: the scratch is part of this module's device image.
// ---------------------------------------------------------------------------------------
#include "attention_no_alloc.h"

#include <cstdio>
#include <mutex>

static __device__ __align__(256) unsigned char g_attn_static_scratch[B200_ATTN_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
constexpr int kDecodeSmem128 = b200::DecodeSmem<128, false>::TOTAL;
constexpr int kDecodeSmem64 = b200::DecodeSmem<64, false>::TOTAL;
std::mutex g_static_mu;
unsigned char* g_static_ptr[kMaxDevices] = {};   // device address of the array, per device
}  // namespace

// Address of the array on the current device, looked up on the first call there.
static int attn_static_scratch(unsigned char** ptr_out) {
  int dev = -1;
  B200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    b200_set_last_error("attn_decode_static: device ordinal out of range", __FILE__, __LINE__);
    return -1;
  }
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    unsigned char* ptr = nullptr;
    B200_CUDA_CHECK(cudaGetSymbolAddress((void**)&ptr, g_attn_static_scratch));
    if (ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 255) != 0) {
      b200_set_last_error("attn_decode_static: scratch symbol has no 256-byte aligned address", __FILE__,
                          __LINE__);
      return -1;
    }
    B200_CUDA_CHECK(cudaFuncSetAttribute(attn_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kDecodeSmem128));
    B200_CUDA_CHECK(cudaFuncSetAttribute(attn_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kDecodeSmem64));
    g_static_ptr[dev] = ptr;
  }
  *ptr_out = g_static_ptr[dev];
  return 0;
}

extern "C" int b200_attn_decode_static_setup(void) {
  unsigned char* ptr = nullptr;
  return attn_static_scratch(&ptr);
}

extern "C" int b200_attn_decode_static_reset(cudaStream_t stream) {
  unsigned char* ptr = nullptr;
  if (attn_static_scratch(&ptr) != 0) return -1;
  B200_CUDA_CHECK(cudaMemsetAsync(ptr, 0, B200_ATTN_STATIC_COUNTER_BYTES, stream));
  return 0;
}

extern "C" int b200_attn_decode_static(const void* q, const void* kv, void* out, float* lse,
                                       const int* block_tables, const int* seq_lens, const int* qsl,
                                       int num_reqs, int max_blocks, int block_size, long long num_blocks,
                                       int Hq, int Hkv, int D, float scale, int window, float softcap,
                                       const float* sinks, int num_splits, cudaStream_t stream) {
  if (num_reqs <= 0) return 0;
  if (Hkv <= 0 || block_size % 16 || (Hq % Hkv) || Hq / Hkv > 16) {
    b200_set_last_error("attn_decode_static: block_size % 16 == 0 and q heads per kv head <= 16 required",
                        __FILE__, __LINE__);
    return -1;
  }
  if (D != 128 && D != 64) {
    b200_set_last_error("attn_decode_static: head_dim must be 64 or 128", __FILE__, __LINE__);
    return -1;
  }
  if (num_splits < 1) num_splits = 1;
  const size_t counters = (size_t)num_reqs * Hkv;
  const size_t part_bytes = num_splits > 1 ? counters * num_splits * 16 * (size_t)(D + 2) * sizeof(float) : 0;
  if (num_splits > 1 && (counters * sizeof(int) > B200_ATTN_STATIC_COUNTER_BYTES ||
                         part_bytes > B200_ATTN_STATIC_SCRATCH_BYTES - B200_ATTN_STATIC_COUNTER_BYTES)) {
    char msg[256];
    snprintf(msg, sizeof(msg),
             "attn_decode_static: %d requests x %d kv heads x %d splits need %zu counters and %zu scratch "
             "bytes; the built-in scratch holds %u counters and %u bytes",
             num_reqs, Hkv, num_splits, counters, part_bytes,
             (unsigned)(B200_ATTN_STATIC_COUNTER_BYTES / sizeof(int)),
             (unsigned)(B200_ATTN_STATIC_SCRATCH_BYTES - B200_ATTN_STATIC_COUNTER_BYTES));
    b200_set_last_error(msg, __FILE__, __LINE__);
    return -1;
  }
  unsigned char* base = nullptr;
  if (attn_static_scratch(&base) != 0) return -1;
  AttnParams p;
  fill_params(p, q, kv, out, lse, block_tables, seq_lens, qsl, max_blocks, block_size, num_blocks, Hq, Hkv, D,
              scale, window, softcap, sinks);
  p.req_begin = 0;
  p.req_end = num_reqs;
  p.num_splits = num_splits;
  p.counters = reinterpret_cast<int*>(base);
  p.part_o = reinterpret_cast<float*>(base + B200_ATTN_STATIC_COUNTER_BYTES);
  p.part_ml = p.part_o + counters * num_splits * 16 * D;
  dim3 grid(Hkv, num_reqs, num_splits);
  if (D == 128) attn_decode_kernel<128><<<grid, 128, kDecodeSmem128, stream>>>(p);
  else attn_decode_kernel<64><<<grid, 128, kDecodeSmem64, stream>>>(p);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// Number of out-of-range block ids / page indices the attention kernels of this file met since the last
// call (always 0 unless built with -DB200_BOUNDS_CHECK); the counter is reset.
extern "C" int b200_bad_index_count_attention(unsigned int* out) {
  B200_TAKE_BAD_INDEX_COUNT(out);
  return 0;
}
