// Multi-head latent attention over the paged latent cache (absorbed-query form, MQA over one latent
// "head"), dense or sparse (top-k indexed), for decode, spec-verify, chunked prefill and mixed batches.
//
//   q_latent [T, H, Dq]  Dq = kv_lora + rope (576 for DeepSeek-V3), already multiplied by W_UK
//   cache    [blocks, block_size, Dq] bf16; the value of a row is its first L = kv_lora dims
//   out      [T, H, L]
//
// One CTA per (token, group of 16 heads): all 16 rows of the MMA tile share the query position, so
// the causal limit and (sparse) the token's top-k list are uniform over the tile.  KV rows stream
// in 16-row chunks through a 2-stage cp.async ring (rows are gathered by pointer, so the dense and
// the top-k case share the loop).  The four warps split the Dq contraction of Q K^T (partials summed
// through shared memory) and each owns a quarter of the L value columns for P V, which keeps the
// 16 x 512 fp32 output in registers.  bf16 mma.sync m16n8k16, fp32 online softmax in the log2 domain.
//
// Semantics of the reference's dense / sparse MLA kernels and latent cache write
// (reference: src/vllm_torchtpu/kernels/mla/v2/, kernels/mla/sparse/, layers/adapter/attention.py:2659-2879).
#include "common.cuh"

namespace b200 {
namespace mla {

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, const uint32_t* b) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void ldsm4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp16(uint32_t smem, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

constexpr int KS_MAX = 9;             // k-steps of 16 per warp: Dq <= 4 * 9 * 16 = 576

struct Params {
  const __nv_bfloat16* q;
  const __nv_bfloat16* cache;
  __nv_bfloat16* out;
  float* lse;
  const int* block_tables;
  const int* seq_lens;
  const int* qsl;
  const int* topk;                    // optional [T, topk_k] context positions, -1 = unused
  int topk_k, T, H, Dq, L, num_reqs, max_blocks, block_size;
  long long num_blocks;
  float scale_log2;
  // split-KV: CTA (token, head group, split) covers an equal share of the token's 16-row chunks and writes a
  // normalised partial [splits, T, H, L] with its log-sum-exp [splits, T, H]; mla_merge_kernel combines them
  int splits;
  __nv_bfloat16* part_o;
  float* part_lse;
};

constexpr int NST = 3;                // cp.async stages of 16 cache rows

// LW = value columns per warp (L / 4).
template <int LW>
__global__ void __launch_bounds__(128) mla_attn_kernel(const Params p) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ const __nv_bfloat16* s_ptr[NST][16];
  __shared__ int s_valid[NST][16];
  __shared__ float s_part[4][16][17];
  pdl_launch_dependents();
  pdl_wait();
  const int groups = (p.H + 15) >> 4;
  const int sp = blockIdx.x % p.splits, tg = blockIdx.x / p.splits;
  const int t = tg / groups, g = tg - t * groups;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // request of this token: largest r with qsl[r] <= t
  int lo = 0, hi = p.num_reqs;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (p.qsl[mid] <= t) lo = mid; else hi = mid;
  }
  const int r = lo;
  const int qs = p.qsl[r], q_len = p.qsl[r + 1] - qs, kv_len = p.seq_lens[r];
  if (t >= p.qsl[p.num_reqs] || q_len <= 0 || kv_len <= 0) return;       // padded token
  const int qpos = kv_len - q_len + (t - qs);
  const int n_kv = p.topk ? p.topk_k : qpos + 1;
  const int chunks_all = (n_kv + 15) >> 4;
  const int per_split = (chunks_all + p.splits - 1) / p.splits;
  const int chunk_lo = sp * per_split;
  const int chunks = max(0, min(chunks_all, chunk_lo + per_split) - chunk_lo);     // of this split
  const int rows_valid = min(16, p.H - g * 16);
  const int ksteps = p.Dq >> 4;                    // Dq % 16 == 0
  const int nch = p.Dq >> 3;                       // 16-byte chunks per row
  const int RS = ((nch + 7) & ~7) << 4;            // row stride in shared memory (swizzle groups of 8)
  const int STAGE = 16 * RS;
  const uint32_t sbase = smem_u32(smem);

  // Q fragments of this warp's k-steps (ks = warp, warp + 4, ...)
  uint32_t qf[KS_MAX][4];
  {
    const int r0 = lane >> 2, r1 = r0 + 8, cb = 2 * (lane & 3);
    const __nv_bfloat16* q0 = r0 < rows_valid ? p.q + ((size_t)t * p.H + g * 16 + r0) * p.Dq : nullptr;
    const __nv_bfloat16* q1 = r1 < rows_valid ? p.q + ((size_t)t * p.H + g * 16 + r1) * p.Dq : nullptr;
#pragma unroll
    for (int i = 0; i < KS_MAX; ++i) {
      const int ks = warp + 4 * i;
      const bool in = ks < ksteps;
      qf[i][0] = (in && q0) ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + cb) : 0u;
      qf[i][1] = (in && q1) ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + cb) : 0u;
      qf[i][2] = (in && q0) ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + cb) : 0u;
      qf[i][3] = (in && q1) ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + cb) : 0u;
    }
  }
  const int* bt = p.block_tables + (size_t)r * p.max_blocks;

  auto prefetch = [&](int c, int stage) {
    if (threadIdx.x < 16) {
      const int i = ((chunk_lo + c) << 4) + threadIdx.x;
      int pos = -1;
      if (i < n_kv) pos = p.topk ? p.topk[(size_t)t * p.topk_k + i] : i;
      const bool ok = pos >= 0 && pos <= qpos && pos < kv_len;
      long long blk = 0;
      int off = 0;
      if (ok) {
        const int page = pos / p.block_size;
        blk = page < p.max_blocks ? bt[page] : -1;
        off = pos % p.block_size;
        if (blk < 0 || blk >= p.num_blocks) {
          B200_NOTE_BAD_INDEX();
          blk = 0;
        }
      }
      s_ptr[stage][threadIdx.x] = p.cache + ((size_t)blk * p.block_size + off) * p.Dq;
      s_valid[stage][threadIdx.x] = ok ? 1 : 0;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 16 * nch; idx += 128) {
      const int row = idx / nch, ch = idx - row * nch;
      cp16(sbase + stage * STAGE + row * RS + ((ch ^ (row & 7)) << 4), s_ptr[stage][row] + ch * 8);
    }
  };

  float o[LW / 8][4];
#pragma unroll
  for (int i = 0; i < LW / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const int mi = lane >> 3, rr = lane & 7;

#pragma unroll
  for (int c = 0; c < NST - 1; ++c) {
    if (c < chunks) prefetch(c, c);
    cp_commit();
  }
  for (int c = 0; c < chunks; ++c) {
    const int stage = c % NST;
    // the stage refilled here was consumed in the previous iteration (which ended with a barrier)
    if (c + NST - 1 < chunks) prefetch(c + NST - 1, (c + NST - 1) % NST);
    cp_commit();
    cp_wait<NST - 1>();
    __syncthreads();
    const uint32_t sb = sbase + stage * STAGE;
    // ---- partial scores over this warp's part of Dq
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      const int tok = (mi >> 1) * 8 + rr;
#pragma unroll
      for (int i = 0; i < KS_MAX; ++i) {
        const int ks = warp + 4 * i;
        if (ks < ksteps) {
          const int ch = 2 * ks + (mi & 1);
          uint32_t b[4];
          ldsm4(b, sb + (uint32_t)(tok * RS + ((ch ^ (tok & 7)) << 4)));
          mma16816(s[0], qf[i], &b[0]);
          mma16816(s[1], qf[i], &b[2]);
        }
      }
    }
    const int row0 = lane >> 2, row1 = row0 + 8, col = 2 * (lane & 3);
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      s_part[warp][row0][nb * 8 + col] = s[nb][0];
      s_part[warp][row0][nb * 8 + col + 1] = s[nb][1];
      s_part[warp][row1][nb * 8 + col] = s[nb][2];
      s_part[warp][row1][nb * 8 + col + 1] = s[nb][3];
    }
    __syncthreads();
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int rrow = (e < 2) ? row0 : row1, cc = nb * 8 + col + (e & 1);
        float v = s_part[0][rrow][cc] + s_part[1][rrow][cc] + s_part[2][rrow][cc] + s_part[3][rrow][cc];
        v = s_valid[stage][cc] ? v * p.scale_log2 : -INFINITY;
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
#pragma unroll
    for (int i = 0; i < LW / 8; ++i) {
      o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1;
    }
    const uint32_t pa[4] = {pack2(s[0][0], s[0][1]), pack2(s[0][2], s[0][3]), pack2(s[1][0], s[1][1]),
                            pack2(s[1][2], s[1][3])};
    // ---- P V on this warp's value columns [warp * LW, (warp + 1) * LW)
    {
      const int tok = (mi & 1) * 8 + rr;
#pragma unroll
      for (int np = 0; np < LW / 16; ++np) {
        const int ch = (warp * LW >> 3) + 2 * np + (mi >> 1);
        uint32_t b[4];
        ldsm4t(b, sb + (uint32_t)(tok * RS + ((ch ^ (tok & 7)) << 4)));
        mma16816(o[2 * np], pa, &b[0]);
        mma16816(o[2 * np + 1], pa, &b[2]);
      }
    }
    __syncthreads();                 // the stage and s_part are rewritten by the next iteration
  }
  cp_wait<0>();
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1); l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1); l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
  const int row0 = lane >> 2, row1 = row0 + 8;
  const float inv0 = l[0] > 0.f ? 1.f / l[0] : 0.f, inv1 = l[1] > 0.f ? 1.f / l[1] : 0.f;
  __nv_bfloat16* out = p.splits > 1 ? p.part_o + (size_t)sp * p.T * p.H * p.L : p.out;
  float* lse = p.splits > 1 ? p.part_lse + (size_t)sp * p.T * p.H : p.lse;
#pragma unroll
  for (int i = 0; i < LW / 8; ++i) {
    const int colv = warp * LW + i * 8 + 2 * (lane & 3);
    if (row0 < rows_valid)
      *reinterpret_cast<uint32_t*>(out + ((size_t)t * p.H + g * 16 + row0) * p.L + colv) =
          pack2(o[i][0] * inv0, o[i][1] * inv0);
    if (row1 < rows_valid)
      *reinterpret_cast<uint32_t*>(out + ((size_t)t * p.H + g * 16 + row1) * p.L + colv) =
          pack2(o[i][2] * inv1, o[i][3] * inv1);
  }
  if (lse != nullptr && warp == 0 && (lane & 3) == 0) {
    if (row0 < rows_valid)
      lse[(size_t)t * p.H + g * 16 + row0] = l[0] > 0.f ? (m[0] + log2f(l[0])) * 0.6931471805599453f : -INFINITY;
    if (row1 < rows_valid)
      lse[(size_t)t * p.H + g * 16 + row1] = l[1] > 0.f ? (m[1] + log2f(l[1])) * 0.6931471805599453f : -INFINITY;
  }
}

// out[t, h, :] = sum_s softmax_s(lse[s, t, h]) * part_o[s, t, h, :]; one CTA per (t, h), 8 columns per thread.
// A (token, head) whose splits all saw no key (padded rows) keeps zeros and lse = -inf.
__global__ void mla_merge_kernel(const __nv_bfloat16* __restrict__ part_o, const float* __restrict__ part_lse,
                                 __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int splits, int TH, int L) {
  pdl_launch_dependents();
  pdl_wait();
  const int th = blockIdx.x;
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, part_lse[(size_t)s * TH + th]);
  float den = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float v = part_lse[(size_t)s * TH + th];
    den += v == -INFINITY ? 0.f : __expf(v - mx);
  }
  if (lse != nullptr && threadIdx.x == 0) lse[th] = den > 0.f ? mx + __logf(den) : -INFINITY;
  for (int c = threadIdx.x * 8; c < L; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (den > 0.f) {
      for (int s = 0; s < splits; ++s) {
        const float v = part_lse[(size_t)s * TH + th];
        if (v == -INFINITY) continue;
        const float w = __expf(v - mx) / den;
        const uint4 raw = *reinterpret_cast<const uint4*>(part_o + ((size_t)s * TH + th) * L + c);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h2[j]);
          acc[2 * j] += w * f.x;
          acc[2 * j + 1] += w * f.y;
        }
      }
    }
    uint4 o;
    o.x = pack2(acc[0], acc[1]); o.y = pack2(acc[2], acc[3]); o.z = pack2(acc[4], acc[5]); o.w = pack2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + (size_t)th * L + c) = o;
  }
}

// cache row of slot s = kv_c[t] (L values) followed by k_pe[t] (R values); slot < 0: skipped
__global__ void mla_write_cache_kernel(__nv_bfloat16* __restrict__ cache, const __nv_bfloat16* __restrict__ kv_c,
                                       const __nv_bfloat16* __restrict__ k_pe, const int* __restrict__ slots,
                                       int L, int R, int ld_c, int ld_pe, long long num_slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const long long slot = slots[t];
  if (slot < 0 || slot >= num_slots) return;
  __nv_bfloat16* dst = cache + (size_t)slot * (L + R);
  for (int i = threadIdx.x; i < L + R; i += blockDim.x)
    dst[i] = i < L ? kv_c[(size_t)t * ld_c + i] : k_pe[(size_t)t * ld_pe + (i - L)];
}

}  // namespace mla
}  // namespace b200

namespace b200 {
namespace mla {

// dst[b * dst_sb + a * dst_sa + d] = src[a * src_sa + b * src_sb + d] for a < A, b < B, d < D (elements;
// D and all strides multiples of 8 so that the copy runs in 16-byte pieces).  Turns [T, H, D] slices into
// the head-major [H, T, D] rows the grouped GEMM wants (heads as groups) and back.
__global__ void permute_rows_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, int A,
                                    int B, int D8, long long src_sa, long long src_sb, long long dst_sa,
                                    long long dst_sb) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)A * B * D8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int d = (int)(i % D8);
    const long long ab = i / D8;
    const int b = (int)(ab % B);
    const int a = (int)(ab / B);
    const uint4 v = *reinterpret_cast<const uint4*>(src + a * src_sa + b * src_sb + d * 8);
    *reinterpret_cast<uint4*>(dst + a * dst_sa + b * dst_sb + d * 8) = v;
  }
}

// Rotary embedding of `pairs` dimension pairs of src[t, h, :] (strides in elements) written to dst[t, h, :]:
// interleaved pairs (2i, 2i+1) or split halves (i, i + pairs), angles position * inv_freq[i] in fp32.
__global__ void rope_rows_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                 const int* __restrict__ positions, const float* __restrict__ inv_freq, int T, int H,
                                 int pairs, int interleaved, long long src_st, long long src_sh, long long dst_st,
                                 long long dst_sh) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)T * H * pairs;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int j = (int)(i % pairs);
    const long long th = i / pairs;
    const int h = (int)(th % H);
    const int t = (int)(th / H);
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[j], &sn, &cs);
    const int i0 = interleaved ? 2 * j : j, i1 = interleaved ? 2 * j + 1 : j + pairs;
    const __nv_bfloat16* s = src + t * src_st + h * src_sh;
    __nv_bfloat16* d = dst + t * dst_st + h * dst_sh;
    const float x0 = __bfloat162float(s[i0]), x1 = __bfloat162float(s[i1]);
    d[i0] = __float2bfloat16(x0 * cs - x1 * sn);
    d[i1] = __float2bfloat16(x1 * cs + x0 * sn);
  }
}

}  // namespace mla
}  // namespace b200

using namespace b200;

extern "C" int b200_permute_rows(const void* src, void* dst, int A, int B, int D, long long src_sa, long long src_sb,
                                 long long dst_sa, long long dst_sb, cudaStream_t stream) {
  if (A <= 0 || B <= 0 || D <= 0) return 0;
  if (D % 8 || src_sa % 8 || src_sb % 8 || dst_sa % 8 || dst_sb % 8 || (reinterpret_cast<uintptr_t>(src) & 15) ||
      (reinterpret_cast<uintptr_t>(dst) & 15)) {
    b200_set_last_error("permute_rows: D, the strides and both addresses must be multiples of 8 elements",
                        __FILE__, __LINE__);
    return -1;
  }
  const long long total = (long long)A * B * (D / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  B200_CUDA_CHECK(launch_pdl(mla::permute_rows_kernel, dim3((unsigned)blocks), dim3(256), (size_t)0, stream,
                             (const __nv_bfloat16*)src, (__nv_bfloat16*)dst, A, B, D / 8, src_sa, src_sb, dst_sa,
                             dst_sb));
  return 0;
}

extern "C" int b200_rope_rows(const void* src, void* dst, const int* positions, const float* inv_freq, int T, int H,
                              int pairs, int interleaved, long long src_st, long long src_sh, long long dst_st,
                              long long dst_sh, cudaStream_t stream) {
  if (T <= 0 || H <= 0 || pairs <= 0) return 0;
  const long long total = (long long)T * H * pairs;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  B200_CUDA_CHECK(launch_pdl(mla::rope_rows_kernel, dim3((unsigned)blocks), dim3(256), (size_t)0, stream,
                             (const __nv_bfloat16*)src, (__nv_bfloat16*)dst, positions, inv_freq, T, H, pairs,
                             interleaved, src_st, src_sh, dst_st, dst_sh));
  return 0;
}

extern "C" int b200_mla_write_cache(void* cache, const void* kv_c, const void* k_pe, const int* slots, int T, int L,
                                    int R, int ld_c, int ld_pe, long long num_slots, cudaStream_t stream) {
  if (T == 0) return 0;
  B200_CUDA_CHECK(launch_pdl(mla::mla_write_cache_kernel, dim3(T), dim3(128), 0, stream, (__nv_bfloat16*)cache,
                             (const __nv_bfloat16*)kv_c, (const __nv_bfloat16*)k_pe, slots, L, R, ld_c, ld_pe,
                             num_slots));
  return 0;
}

// q [T, H, Dq], cache [num_blocks, block_size, Dq], out [T, H, L], lse [T, H] or null,
// topk [T, topk_k] or null.  Dq % 16 == 0, Dq <= 576, L in {64, 128, 256, 512}.
// splits > 1: part_o [splits, T, H, L] bf16 and part_lse [splits, T, H] fp32 are scratch of the caller.
extern "C" int b200_mla_attention(const void* q, const void* cache, void* out, float* lse, const int* block_tables,
                                  const int* seq_lens, const int* qsl, const int* topk, int topk_k, int T,
                                  int num_reqs, int H, int Dq, int L, int max_blocks, int block_size,
                                  long long num_blocks, float scale, int splits, void* part_o, float* part_lse,
                                  cudaStream_t stream) {
  if (T <= 0 || num_reqs <= 0) return 0;
  if (Dq % 16 || Dq > 4 * mla::KS_MAX * 16 || L > Dq || (L != 64 && L != 128 && L != 256 && L != 512)) {
    b200_set_last_error("mla_attention: Dq % 16 == 0, Dq <= 576 and kv_lora in {64,128,256,512} required",
                        __FILE__, __LINE__);
    return -1;
  }
  mla::Params p;
  p.q = (const __nv_bfloat16*)q; p.cache = (const __nv_bfloat16*)cache; p.out = (__nv_bfloat16*)out;
  p.lse = lse; p.block_tables = block_tables; p.seq_lens = seq_lens; p.qsl = qsl;
  p.topk = topk; p.topk_k = topk_k;
  p.T = T; p.H = H; p.Dq = Dq; p.L = L; p.num_reqs = num_reqs; p.max_blocks = max_blocks;
  p.block_size = block_size; p.num_blocks = num_blocks;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (splits < 1 || (splits > 1 && (part_o == nullptr || part_lse == nullptr))) {
    b200_set_last_error("mla_attention: split-KV needs its scratch", __FILE__, __LINE__);
    return -1;
  }
  p.splits = splits; p.part_o = (__nv_bfloat16*)part_o; p.part_lse = part_lse;
  const int nch = Dq / 8;
  const int smem = mla::NST * 16 * (((nch + 7) & ~7) << 4);
  const dim3 grid(T * ((H + 15) / 16) * splits);
#define MLA_LAUNCH(LWV)                                                                                      \
  do {                                                                                                       \
    B200_CUDA_CHECK(cudaFuncSetAttribute(mla::mla_attn_kernel<LWV>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         smem));                                                             \
    B200_CUDA_CHECK(launch_pdl(mla::mla_attn_kernel<LWV>, grid, dim3(128), (size_t)smem, stream, p));         \
  } while (0)
  if (L == 512) MLA_LAUNCH(128);
  else if (L == 256) MLA_LAUNCH(64);
  else if (L == 128) MLA_LAUNCH(32);
  else MLA_LAUNCH(16);
#undef MLA_LAUNCH
  if (splits > 1)
    B200_CUDA_CHECK(launch_pdl(mla::mla_merge_kernel, dim3(T * H), dim3(64), (size_t)0, stream,
                               (const __nv_bfloat16*)part_o, (const float*)part_lse, (__nv_bfloat16*)out, lse,
                               splits, T * H, L));
  return 0;
}

// see b200_bad_index_count_attention
extern "C" int b200_bad_index_count_attention_mla(unsigned int* out) {
  B200_TAKE_BAD_INDEX_COUNT(out);
  return 0;
}
