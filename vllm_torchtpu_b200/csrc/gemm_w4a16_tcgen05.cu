// W4A16 GEMM on tcgen05: 4-bit float weights (e2m1, two per byte, low nibble = even k) with group scales,
// bf16 activations, fp32 accumulation in TMEM.
//
//   Y[t, n] = sum_k X[t, k] * e2m1(Wp[n, k]) * scale[n, k / G]          mxfp4: G = 32, scale = 2^(e8m0 - 127)
//                                                                       nvfp4: G = 16, scale = e4m3 * global
//
// The weight never exists in bf16 in global memory: a tile is expanded in shared memory, in front of the
// tensor core.  Roles of a CTA (704 threads), persistent over (weight tile, token tile) pairs:
//
//   warp 0      TMA producer: packed weight bytes [128 rows x 32 B] and the activation tile [BN x 128 B]
//   warps 2-17  expansion, four groups of four warps, K blocks dealt round-robin: thread = weight row; 64 nibbles ->
//               e2m1 value x group scale -> bf16 pairs, stored with tcgen05.st into a slot of TENSOR MEMORY (lane = weight row, 32-bit column = two
//               consecutive k): the A operand never touches shared memory, so there is no generic-to-async
//               proxy fence per K block
//   warp 1      tcgen05.mma kind::f16 with A from tensor memory and B (the activation tile) from shared
//               memory (M 128 = weight rows, N = tokens, K 16 x 4 per stage), accumulators double-buffered
//               in TMEM columns [0, 2 BN), eight A slots of 32 columns in [256, 512)
//   warps 18-21 epilogue: TMEM -> bf16 -> Y (+ bias)
//
// Few output tiles (decode-sized N): split-K as a thread-block cluster, the CTAs of a cluster take K ranges
// of one tile, leave fp32 partials in their shared memory and sum them over DSMEM.
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
constexpr int NUM_THREADS = 704;     // TMA warp, MMA warp, 16 expansion warps, 4 epilogue warps
constexpr int EXP_GROUPS = 4;        // expansion groups of four warps, K blocks dealt round-robin
constexpr int EPI_WARP0 = 2 + 4 * EXP_GROUPS;
constexpr int MAX_GROUPS = 1024;

// Two rings: load slots in shared memory (packed weight bytes + activation tile) and expanded A tiles in
// tensor memory (32 columns each).
constexpr int A_STAGES = 8;
constexpr int A_COLS = BK / 2;                  // 32-bit columns of one expanded tile
constexpr int A_TMEM_BASE = 256;                // accumulators use columns [0, 256)

template <int BN>
struct Cfg {
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = RAW_BYTES + B_BYTES;                // load ring slot (multiple of 1024)
  static constexpr int STAGES_RAW = 196608 / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 12 ? 12 : STAGES_RAW;
  static_assert(2 * BN <= A_TMEM_BASE, "accumulators and A slots share the 512 TMEM columns");
  static_assert(STAGES >= EXP_GROUPS + 2,
                "an expansion group publishes a block when it reaches its next one: the producer must run that far ahead");
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BAR_BYTES = 512;
  static constexpr int PREFIX_BYTES = (MAX_GROUPS + 1) * 4 + 12;
  static constexpr int SMEM = RING_BYTES + BAR_BYTES + PREFIX_BYTES + 64 + 1024;
  static constexpr int TMEM_COLS = 512;
};

struct Params {
  __nv_bfloat16* Y;
  const __nv_bfloat16* bias;
  const uint8_t* scales;             // mxfp4: e8m0 [rows, K / 32]; nvfp4: e4m3 [rows, K / 16]
  const float* global_scale;         // nvfp4: one fp32 per tensor (or per group of rows: see gs_per_group)
  const uint8_t* zeros;              // int4: zero point per group, uint8 [rows, K >> group_shift]; scales are fp16 there
  int group_shift;                   // int4: log2 of the group size (32 ... K)
  int* status;
  int T, N, K, ldy;
  int n_tiles, t_tiles, kb_total;
  const int* group_off;              // grouped: int[num_groups + 1]
  int num_groups, w_rows_per_group, gs_per_group;
  int splits, kb_per_split;          // cluster split-K (dense mode): work item = (tile, split)
};

struct Work {
  int w_row, t_row, t_valid, n0, kb0, kb1;
};

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp writes lane (base + i)
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// kind::f16 with the A operand in tensor memory (lane = row, column = two consecutive k), B in shared memory
__device__ __forceinline__ void umma_f16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// e2m1 -> fp32 without a table: with the two exponent bits in the low bits of the fp32 exponent field and the
// mantissa bit on top of the fraction, the fp32 value is e2m1 * 2^-126 for every code (the e = 0 codes are
// fp32 subnormals, which the multiplies below handle exactly).  The 2^126 is undone in two exact steps so
// that no realistic group scale overflows: 2^64 here, 2^62 folded into the group scale by the caller.
// Byte j of `wd` holds elements 2j (low nibble) and 2j + 1 (high nibble); returns them as a bf16 pair.
// Power-of-two group scales (mxfp4) stay in bf16: the same bit placement in a bf16 pair gives e2m1 * 2^-126
// per half (bf16 has the fp32 exponent range), and two exact bf16x2 multiplies, by 2^64 and by the group
// scale times 2^62, finish the job with a fifth of the instructions.  `s62x2` holds that scale in both halves.
template <int J>
__device__ __forceinline__ uint32_t e2m1_pair_to_bf16x2_pow2(uint32_t wd, uint32_t s62x2) {
  // low nibble of byte J -> bits [8:6] and sign bit 15; high nibble -> bits [24:22] and sign bit 31
  constexpr int LO = 6 - 8 * J, HI = 18 - 8 * J;
  const uint32_t lo_b = LO >= 0 ? (wd << (LO >= 0 ? LO : 0)) : (wd >> (LO < 0 ? -LO : 0));
  const uint32_t hi_b = HI >= 0 ? (wd << (HI >= 0 ? HI : 0)) : (wd >> (HI < 0 ? -HI : 0));
  constexpr int SL = 12 - 8 * J, SH = 24 - 8 * J;            // nibble bit 3 -> bit 15 / bit 31
  const uint32_t sl_b = SL >= 0 ? (wd << (SL >= 0 ? SL : 0)) : (wd >> (SL < 0 ? -SL : 0));
  const uint32_t sh_b = wd << SH;
  uint32_t v = (lo_b & 0x000001C0u) | (hi_b & 0x01C00000u) | (sl_b & 0x00008000u) | (sh_b & 0x80000000u);
  uint32_t out;
  asm("{\n\t"
      ".reg .b32 t;\n\t"
      "mul.bf16x2 t, %1, %2;\n\t"
      "mul.bf16x2 %0, t, %3;\n\t"
      "}"
      : "=r"(out)
      : "r"(v), "r"(0x5F805F80u), "r"(s62x2));              // 0x5F80 = 2^64 in bf16
  return out;
}

template <int J>
__device__ __forceinline__ uint32_t e2m1_pair_to_bf16x2(uint32_t wd, float scale62) {
  constexpr int LO = 22 - 8 * J, HI = 18 - 8 * J;            // nibble bit 0 -> bit 22
  const uint32_t lo_b = LO >= 0 ? (wd << (LO >= 0 ? LO : 0)) : (wd >> (LO < 0 ? -LO : 0));
  const uint32_t hi_b = HI >= 0 ? (wd << (HI >= 0 ? HI : 0)) : (wd >> (HI < 0 ? -HI : 0));
  // magnitude bits land on [24:22]; the sign bit (nibble bit 3) is 6 positions higher than bit 25
  const uint32_t lo = (lo_b & 0x01C00000u) | (((wd >> (8 * J + 3)) & 1u) << 31);
  const uint32_t hi = (hi_b & 0x01C00000u) | (((wd >> (8 * J + 7)) & 1u) << 31);
  constexpr float TWO64 = 18446744073709551616.f;
  __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(lo) * TWO64 * scale62,
                                            __uint_as_float(hi) * TWO64 * scale62);
  return *reinterpret_cast<uint32_t*>(&b2);
}

// Unsigned 4-bit integers with a group scale and zero point (AWQ / GPTQ): nibble u placed in the top fraction
// bits of 128.0f gives 128 + u exactly; (that - (128 + zero)) * scale is one exact subtraction and one rounded
// product in fp32, then one rounding to bf16: the same two roundings as dequantising in fp32 and casting.
// `zp` = 128 + zero point.
template <int J>
__device__ __forceinline__ uint32_t int4_pair_to_bf16x2(uint32_t wd, float scale, float zp) {
  constexpr int LO = 16 - 8 * J, HI = 12 - 8 * J;            // nibble bit 0 -> bit 16
  const uint32_t lo_b = LO >= 0 ? (wd << (LO >= 0 ? LO : 0)) : (wd >> (LO < 0 ? -LO : 0));
  const uint32_t hi_b = HI >= 0 ? (wd << (HI >= 0 ? HI : 0)) : (wd >> (HI < 0 ? -HI : 0));
  const float lo = __uint_as_float(0x43000000u | (lo_b & 0x000F0000u));
  const float hi = __uint_as_float(0x43000000u | (hi_b & 0x000F0000u));
  __nv_bfloat162 b2 = __floats2bfloat162_rn((lo - zp) * scale, (hi - zp) * scale);
  return *reinterpret_cast<uint32_t*>(&b2);
}

template <int BN>
__device__ __forceinline__ Work get_work(int w, const Params& p, const int* s_prefix) {
  Work k;
  if (p.group_off == nullptr) {
    const int tile = w / p.splits, split = w - tile * p.splits;
    const int n_tile = tile % p.n_tiles, t_tile = tile / p.n_tiles;
    k.w_row = n_tile * BM;
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
    k.n0 = n_tile * BM;
    k.t_row = r0 + t_tile * BN;
    k.t_valid = min(BN, rows - t_tile * BN);
    k.kb0 = 0;
    k.kb1 = p.kb_total;
  }
  return k;
}

// FMT 0: mxfp4, FMT 1: nvfp4, FMT 2: int4 with fp16 group scales and uint8 zero points
template <int BN, int FMT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_w4a16_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const Params p) {
  using C = Cfg<BN>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::RING_BYTES);
  uint64_t* full = bars;                         // load slot: TMA bytes have landed
  uint64_t* empty = bars + STAGES;               // load slot: packed bytes read (4 warps) and X consumed (1 commit)
  uint64_t* afull = bars + 2 * STAGES;           // A slot: expanded tile written (4 warps)
  uint64_t* aempty = bars + 2 * STAGES + A_STAGES;   // A slot: the MMAs that read it have completed
  uint64_t* tfull = bars + 2 * STAGES + 2 * A_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_prefix = reinterpret_cast<int*>(smem + C::RING_BYTES + C::BAR_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 5);
    }
    for (int i = 0; i < A_STAGES; ++i) {
      mbar_init(&afull[i], 4);
      mbar_init(&aempty[i], 1);
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
  const int total_work = p.group_off != nullptr ? s_prefix[p.num_groups] * p.n_tiles
                                                : p.n_tiles * p.t_tiles * p.splits;

  if (warp == 0) {
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const Work k = get_work<BN>(w, p, s_prefix);
        for (int kb = k.kb0; kb < k.kb1; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* st = smem + s * C::STAGE_BYTES;
          mbar_expect_tx(&full[s], RAW_BYTES + C::B_BYTES);
          tma_load_2d(st, &tmW, &full[s], kb * (BK / 2), k.w_row);          // packed bytes
          tma_load_2d(st + RAW_BYTES, &tmX, &full[s], kb * BK, k.t_row);     // activations
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
      if (*abort_flag)
        for (int it = 0; it < 20000; ++it) __nanosleep(100);
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
      int s = 0, as = 0;
      uint32_t ph = 0, aph = 0, tile_i = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++tile_i) {
        const Work k = get_work<BN>(w, p, s_prefix);
        const int acc = tile_i & 1;
        if (!mbar_wait(&tempty[acc], ((tile_i >> 1) & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        for (int kb = k.kb0; kb < k.kb1; ++kb) {
          if (!mbar_wait(&full[s], ph, abort_flag, p.status, ST_TIMEOUT_FULL) ||
              !mbar_wait(&afull[as], aph, abort_flag, p.status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_tmem = tmem_base + A_TMEM_BASE + as * A_COLS;
          const uint64_t bdesc = umma_desc_k_sw128(smem_u32(smem + s * C::STAGE_BYTES + RAW_BYTES));
#pragma unroll
          for (int q = 0; q < BK / 16; ++q)      // K = 16 per instruction: 32 bytes along the 128-byte row
            umma_f16_a_tmem(tmem_base + acc * BN, a_tmem + 8 * q, bdesc + 2 * q, idesc,
                            (kb > k.kb0 || q > 0) ? 1u : 0u);
          umma_commit(&empty[s]);               // the activation tile of the load slot
          umma_commit(&aempty[as]);             // the expanded tile
          if (++s == STAGES) { s = 0; ph ^= 1; }
          if (++as == A_STAGES) { as = 0; aph ^= 1; }
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else if (warp < EPI_WARP0) {
    // ---- expansion.  Four groups of four warps take the K blocks round-robin (a K block costs a warp a chain of
    // barrier waits, conversion and a TMEM store whose latencies add up, so four blocks are worked on at
    // once); inside a group a warp owns its TMEM lane quarter: weight rows 32 * (warp % 4) + lane, all 64
    // values of the row.  The completion of a block's TMEM store is awaited after the next block's values
    // have been computed.
    const int row = (warp & 3) * 32 + lane, grp = (warp - 2) >> 2;
    int s = 0, as = 0;
    uint32_t ph = 0, aph = 0;
    bool ok = true;
    constexpr int G = FMT == 1 ? 16 : 32;        // int4: the block is read as two halves of 32 (groups are >= 32)
    constexpr int SPB = BK / G;                  // scale bytes per K block
    const int sc_ld = FMT == 2 ? (p.K >> p.group_shift) : p.K / G;
    int pending = -1;                            // A slot whose store has been issued but not published
    auto publish = [&]() {
      if (pending >= 0) {
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&afull[pending]);
        pending = -1;
      }
    };
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      const Work k = get_work<BN>(w, p, s_prefix);
      const bool live = k.n0 + row < p.N;
      const uint8_t* sc_row = p.scales + (size_t)(k.w_row + row) * sc_ld * (FMT == 2 ? 2 : 1);
      const uint8_t* zp_row = FMT == 2 ? p.zeros + (size_t)(k.w_row + row) * sc_ld : nullptr;
      float gs = 1.f;
      if (FMT == 1) gs = p.global_scale[p.gs_per_group ? (k.w_row / p.w_rows_per_group) : 0];
      for (int kb = k.kb0; kb < k.kb1; ++kb) {
        if (((kb - k.kb0) % EXP_GROUPS) == grp) {
          // group scales of this block (a few bytes per row; the row's scales share cache lines over K)
          float sc[SPB], zp[SPB];
#pragma unroll
          for (int g = 0; g < SPB; ++g) {
            if (FMT == 2) {
              const int gi = (kb * BK + g * 32) >> p.group_shift;
              const bool in = live && gi < sc_ld;
              sc[g] = in ? __half2float(__ldg(reinterpret_cast<const __half*>(sc_row) + gi)) : 0.f;
              zp[g] = 128.f + (in ? (float)__ldg(zp_row + gi) : 0.f);
              continue;
            }
            zp[g] = 0.f;
            const int gi = kb * SPB + g;
            const uint8_t b = (live && gi < sc_ld) ? __ldg(sc_row + gi) : 0;
            if (FMT == 0) {
              // 2^(b - 127) * 2^62 = 2^(b - 65): exponent field b + 62 (finite for b <= 192)
              sc[g] = live ? __uint_as_float(min((uint32_t)b + 62u, 254u) << 23) : 0.f;
            } else {
              const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
              sc[g] = live ? __half2float(*reinterpret_cast<const __half*>(&h)) * gs * 4611686018427387904.f : 0.f;
            }
          }
          if (!mbar_wait(&full[s], ph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          // the packed tile was written by TMA without swizzle: dense rows of 32 bytes
          const uint8_t* st = smem + s * C::STAGE_BYTES;
          uint4 raw[2];
          raw[0] = *reinterpret_cast<const uint4*>(st + row * 32);
          raw[1] = *reinterpret_cast<const uint4*>(st + row * 32 + 16);
          const uint32_t* words = reinterpret_cast<const uint32_t*>(raw);
          uint32_t cols[32];                     // the row's 64 values as 32 bf16 pairs
#pragma unroll
          for (int c = 0; c < 8; ++c) {          // 8 values = one packed word
            const uint32_t wd = words[c];
            float s8 = sc[0], z8 = zp[0];
#pragma unroll
            for (int g = 1; g < SPB; ++g)
              if ((c * 8) / G == g) { s8 = sc[g]; z8 = zp[g]; }
            uint4 o;
            if (FMT == 2) {
              o = make_uint4(int4_pair_to_bf16x2<0>(wd, s8, z8), int4_pair_to_bf16x2<1>(wd, s8, z8),
                             int4_pair_to_bf16x2<2>(wd, s8, z8), int4_pair_to_bf16x2<3>(wd, s8, z8));
            } else if (FMT == 0) {
              // a power of two is exact in bf16: the top half of its fp32 bits, in both halves of the pair
              const uint32_t s2 = (__float_as_uint(s8) >> 16) * 0x00010001u;
              o = make_uint4(e2m1_pair_to_bf16x2_pow2<0>(wd, s2), e2m1_pair_to_bf16x2_pow2<1>(wd, s2),
                             e2m1_pair_to_bf16x2_pow2<2>(wd, s2), e2m1_pair_to_bf16x2_pow2<3>(wd, s2));
            } else {
              o = make_uint4(e2m1_pair_to_bf16x2<0>(wd, s8), e2m1_pair_to_bf16x2<1>(wd, s8),
                             e2m1_pair_to_bf16x2<2>(wd, s8), e2m1_pair_to_bf16x2<3>(wd, s8));
            }
            cols[4 * c] = o.x; cols[4 * c + 1] = o.y; cols[4 * c + 2] = o.z; cols[4 * c + 3] = o.w;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&empty[s]);   // the packed bytes of this warp's rows are in registers
          publish();                               // the previous block's store has had this long to land
          if (!mbar_wait(&aempty[as], aph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          tc_fence_after();
          const uint32_t ta = tmem_base + A_TMEM_BASE + as * A_COLS + ((uint32_t)((warp & 3) * 32) << 16);
          tmem_st_32x32b_x16(ta, cols);
          tmem_st_32x32b_x16(ta + 16, cols + 16);
          pending = as;
        }
        if (++s == STAGES) { s = 0; ph ^= 1; }
        if (++as == A_STAGES) { as = 0; aph ^= 1; }
      }
      if (!ok) break;
    }
    publish();
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
        if (p.splits > 1) {
          // fp32 partial of this K range: part[token][weight row] in the (now idle) stage ring
          float* part = reinterpret_cast<float*>(smem);
#pragma unroll
          for (int j = 0; j < 32; ++j) part[(c0 + j) * BM + row] = __uint_as_float(r[j]);
        } else if (n < p.N) {
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

  if (p.splits > 1) {
    // every CTA of the cluster has its partial in shared memory: sum them over DSMEM.  Epilogue warp e of
    // cluster rank r takes tokens r + S * e, r + S * (e + 4), ...; a lane owns four consecutive weight rows.
    __syncwarp();
    cluster_arrive_release();
    cluster_wait_acquire();
    if (warp >= EPI_WARP0 && !*abort_flag && (int)blockIdx.x < total_work) {
      const Work k = get_work<BN>(blockIdx.x, p, s_prefix);
      const int ew = warp - EPI_WARP0;
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
      for (int c = (int)rank + S * ew; c < k.t_valid; c += 4 * S) {
        float4 v[8];
#pragma unroll
        for (int r2 = 0; r2 < 8; ++r2)
          if (r2 < S) v[r2] = ld_dsmem_v4(mapa_shared(part_local + (uint32_t)((c * BM + 4 * lane) * 4), r2));
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r2 = 0; r2 < 8; ++r2)
          if (r2 < S) { a.x += v[r2].x; a.y += v[r2].y; a.z += v[r2].z; a.w += v[r2].w; }
        const float vals[4] = {a.x, a.y, a.z, a.w};
        __nv_bfloat16* yp = p.Y + (size_t)(k.t_row + c) * p.ldy + n4;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n4 + j < p.N) yp[j] = __float2bfloat16(vals[j] + b4[j]);
      }
    }
    __syncwarp();
    cluster_arrive_release();       // nobody leaves while a peer may still read its partial
    cluster_wait_acquire();
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
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (p.splits > 1) {
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
  B200_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_w4a16_kernel<BN, FMT>, tmW, tmX, p));
  return 0;
}

template <int FMT>
static int dispatch(int bn, const CUtensorMap& tmW, const CUtensorMap& tmX, const Params& p, int grid,
                    cudaStream_t stream) {
  switch (bn) {
    case 32: return launch<32, FMT>(tmW, tmX, p, grid, stream);
    case 64: return launch<64, FMT>(tmW, tmX, p, grid, stream);
    default: return launch<128, FMT>(tmW, tmX, p, grid, stream);
  }
}

static int run(const void* X, const void* Wp, const void* scales, const float* global_scale, void* Y,
               const void* bias, const int* group_off, int num_groups, int gs_per_group, int T, int N, int K,
               int ldx, int ldy, int fmt, int rows_hint, int* status, int num_sms, cudaStream_t stream,
               const void* zeros = nullptr, int group = 0) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if (K % BK || fmt < 0 || fmt > 2 || (fmt == 1 && global_scale == nullptr) || num_groups > MAX_GROUPS) {
    b200_set_last_error("gemm_w4a16: K % 64 == 0, format mxfp4 (0), nvfp4 (1, with its global scale) or int4 (2), "
                        "at most 1024 groups", __FILE__, __LINE__);
    return -3;
  }
  int group_shift = 0;
  if (fmt == 2) {
    while ((1 << group_shift) < group) ++group_shift;
    if (zeros == nullptr || group < 32 || (1 << group_shift) != group || K % group) {
      b200_set_last_error("gemm_w4a16 (int4): zero points, and a power-of-two group size >= 32 that divides K",
                          __FILE__, __LINE__);
      return -3;
    }
  }
  if (group_off != nullptr && N % BM) {
    b200_set_last_error("gemm_w4a16 (grouped): N % 128 == 0 required", __FILE__, __LINE__);
    return -3;
  }
  const int bn = rows_hint <= 32 ? 32 : (rows_hint <= 64 ? 64 : 128);
  Params p;
  memset(&p, 0, sizeof(p));
  p.Y = (__nv_bfloat16*)Y;
  p.bias = (const __nv_bfloat16*)bias;
  p.scales = (const uint8_t*)scales;
  p.global_scale = global_scale;
  p.zeros = (const uint8_t*)zeros;
  p.group_shift = group_shift;
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
  // few tiles: cluster split-K (2, 4 or 8 CTAs per tile, at least four K blocks each); the fp32 partial
  // [bn][128] of a CTA has to fit in the stage ring, which it does for every bn
  p.splits = 1;
  p.kb_per_split = p.kb_total;
  const int tiles = p.n_tiles * p.t_tiles;
  if (group_off == nullptr && tiles * 2 <= num_sms) {
    int sp = num_sms / tiles;
    sp = sp >= 8 ? 8 : (sp >= 4 ? 4 : 2);
    while (sp > 1 && p.kb_total / sp < 4) sp >>= 1;
    if (sp > 1) {
      p.splits = sp;
      p.kb_per_split = (p.kb_total + sp - 1) / sp;
      if ((sp - 1) * p.kb_per_split >= p.kb_total) { p.splits = 1; p.kb_per_split = p.kb_total; }
    }
  }
  const int total = group_off != nullptr ? num_sms : tiles * p.splits;
  const int grid = p.splits > 1 ? total : (total < num_sms ? total : num_sms);
  if (fmt == 2) return dispatch<2>(bn, tmW, tmX, p, grid, stream);
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

// Whole-tensor expansion to bf16 [rows, K] (for prefill-sized products, where expanding every tile once per
// token tile would cost more than one pass over the weight): one thread per 8 values.
namespace b200 {
namespace w4 {
template <int FMT>
__global__ void dequant_w4_kernel(const uint8_t* __restrict__ wp, const uint8_t* __restrict__ scales,
                                  const float* __restrict__ global_scale, __nv_bfloat16* __restrict__ out,
                                  long long rows, int K) {
  constexpr int G = FMT == 0 ? 32 : 16;
  const long long words = rows * (K / 8);
  const float gs = FMT == 1 ? global_scale[0] : 1.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < words;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (K / 8);
    const int c = (int)(i - r * (K / 8));
    const uint32_t wd = __ldg(reinterpret_cast<const uint32_t*>(wp) + i);
    const uint8_t b = __ldg(scales + r * (K / G) + (c * 8) / G);
    float sc;
    if (FMT == 0) {
      sc = __uint_as_float(min((uint32_t)b + 62u, 254u) << 23);
    } else {
      const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
      sc = __half2float(*reinterpret_cast<const __half*>(&h)) * gs * 4611686018427387904.f;
    }
    *reinterpret_cast<uint4*>(out + i * 8) =
        make_uint4(e2m1_pair_to_bf16x2<0>(wd, sc), e2m1_pair_to_bf16x2<1>(wd, sc),
                   e2m1_pair_to_bf16x2<2>(wd, sc), e2m1_pair_to_bf16x2<3>(wd, sc));
  }
}
}  // namespace w4
}  // namespace b200

namespace b200 {
namespace w4 {
__global__ void dequant_int4_kernel(const uint8_t* __restrict__ wp, const __half* __restrict__ scales,
                                    const uint8_t* __restrict__ zeros, __nv_bfloat16* __restrict__ out,
                                    long long rows, int K, int group_shift) {
  const long long words = rows * (K / 8);
  const int gpr = K >> group_shift;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < words;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (K / 8);
    const int c = (int)(i - r * (K / 8));
    const uint32_t wd = __ldg(reinterpret_cast<const uint32_t*>(wp) + i);
    const long long gi = r * gpr + ((c * 8) >> group_shift);
    const float sc = __half2float(__ldg(scales + gi));
    const float zp = 128.f + (float)__ldg(zeros + gi);
    *reinterpret_cast<uint4*>(out + i * 8) =
        make_uint4(int4_pair_to_bf16x2<0>(wd, sc, zp), int4_pair_to_bf16x2<1>(wd, sc, zp),
                   int4_pair_to_bf16x2<2>(wd, sc, zp), int4_pair_to_bf16x2<3>(wd, sc, zp));
  }
}
}  // namespace w4
}  // namespace b200

// int4 (AWQ / GPTQ style): Wp [N, K / 2] packed nibbles (low nibble = even k), scales fp16 [N, K / group], zero
// points uint8 [N, K / group]; value = (nibble - zero) * scale.  group a power of two >= 32 that divides K.
extern "C" int b200_gemm_w4a16_int4(const void* X, const void* Wp, const void* scales, const void* zeros, void* Y,
                                    const void* bias, int T, int N, int K, int ldx, int ldy, int group, int* status,
                                    int num_sms, cudaStream_t stream) {
  return w4::run(X, Wp, scales, nullptr, Y, bias, nullptr, 0, 0, T, N, K, ldx, ldy, 2, T, status, num_sms, stream,
                 zeros, group);
}

extern "C" int b200_dequant_int4(const void* wp, const void* scales, const void* zeros, void* out, long long rows,
                                 int K, int group, cudaStream_t stream) {
  if (rows <= 0 || K <= 0) return 0;
  int shift = 0;
  while ((1 << shift) < group) ++shift;
  if (K % 8 || group < 8 || (1 << shift) != group || K % group) {
    b200_set_last_error("dequant_int4: K % 8 == 0 and a power-of-two group size >= 8 that divides K", __FILE__,
                        __LINE__);
    return -3;
  }
  long long blocks = (rows * (K / 8) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  w4::dequant_int4_kernel<<<(int)blocks, 256, 0, stream>>>((const uint8_t*)wp, (const __half*)scales,
                                                           (const uint8_t*)zeros, (__nv_bfloat16*)out, rows, K, shift);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// out [rows, K] bf16 = dequant(wp [rows, K / 2], scales); K % 8 == 0 (mxfp4: K % 32, nvfp4: K % 16).
extern "C" int b200_dequant_w4(const void* wp, const void* scales, const float* global_scale, void* out,
                               long long rows, int K, int fmt, cudaStream_t stream) {
  if (rows <= 0 || K <= 0) return 0;
  if (K % 32 || (fmt != 0 && fmt != 1) || (fmt == 1 && global_scale == nullptr)) {
    b200_set_last_error("dequant_w4: K % 32 == 0, format mxfp4 (0) or nvfp4 (1, with its global scale)", __FILE__,
                        __LINE__);
    return -3;
  }
  const long long words = rows * (K / 8);
  long long blocks = (words + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (fmt == 0)
    w4::dequant_w4_kernel<0><<<(int)blocks, 256, 0, stream>>>((const uint8_t*)wp, (const uint8_t*)scales,
                                                              global_scale, (__nv_bfloat16*)out, rows, K);
  else
    w4::dequant_w4_kernel<1><<<(int)blocks, 256, 0, stream>>>((const uint8_t*)wp, (const uint8_t*)scales,
                                                              global_scale, (__nv_bfloat16*)out, rows, K);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
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
