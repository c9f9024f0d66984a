// Gated DeltaNet kernels: causal depth-wise conv1d with a carried window, gate/normalisation
// prep, and the gated delta-rule recurrence with the per-head state held in registers.
//
// The recurrence kernel runs one CTA per (request, value head); thread j owns column j of the
// [dk, dv] state, so k^T S, the rank-1 update and q^T S are all thread-local dot products and
// the only communication per token is staging the token's k and q vectors in shared memory
// (double buffered).  The same kernel serves decode (one token) and prefill (the request's
// tokens in order); parallelism comes from requests x heads.  State lives in pools indexed by
// the request's slot; a request whose first token of the step has position 0 starts from zero.
//
// Math of the reference's fused conv1d + GDN kernels (reference: src/vllm_torchtpu/kernels/gdn/v3/),
// which use a chunked WY form for prefill; the recurrence below is the same function.
#include "common.cuh"

namespace b200 {

// grid (R, ceil(C / 128)); thread = channel.  x [T, C] bf16 -> y [T, C] bf16 (SiLU applied).
template <int K>
__global__ void gdn_conv_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                __nv_bfloat16* __restrict__ conv_pool, const __nv_bfloat16* __restrict__ w,
                                const int* __restrict__ qsl, const int* __restrict__ seq_lens,
                                const int* __restrict__ slots, int C, int ldx) {
  const int r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int qs = qsl[r], qe = qsl[r + 1];
  if (c >= C || qe <= qs) return;
  const int slot = slots[r];
  if (slot < 0) return;
  __nv_bfloat16* st = conv_pool + ((size_t)slot * C + c) * (K - 1);
  float win[K];
  const bool fresh = (seq_lens[r] - (qe - qs)) == 0;
#pragma unroll
  for (int j = 0; j < K - 1; ++j) win[j] = fresh ? 0.f : __bfloat162float(st[j]);
  float wt[K];
#pragma unroll
  for (int j = 0; j < K; ++j) wt[j] = __bfloat162float(w[(size_t)c * K + j]);
  for (int t = qs; t < qe; ++t) {
    win[K - 1] = __bfloat162float(x[(size_t)t * ldx + c]);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) acc += win[j] * wt[j];
    y[(size_t)t * C + c] = __float2bfloat16(acc / (1.f + __expf(-acc)));
#pragma unroll
    for (int j = 0; j < K - 1; ++j) win[j] = win[j + 1];
  }
#pragma unroll
  for (int j = 0; j < K - 1; ++j) st[j] = __float2bfloat16(win[j]);
}

// One warp per (token, k head): L2-normalise q and k (q also scaled by dk^-1/2) into fp32;
// one thread per (token, v head): g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b).
__global__ void gdn_prep_kernel(const __nv_bfloat16* __restrict__ conv_out, const __nv_bfloat16* __restrict__ a,
                                const __nv_bfloat16* __restrict__ b, const float* __restrict__ A_log,
                                const float* __restrict__ dt_bias, float* __restrict__ qn,
                                float* __restrict__ kn, float* __restrict__ g, float* __restrict__ beta, int T,
                                int Hk, int Hv, int dk, int C, int lda) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int total = T * Hk;
  if (warp < total) {
    const int t = warp / Hk, h = warp % Hk;
    const __nv_bfloat16* qp = conv_out + (size_t)t * C + h * dk;
    const __nv_bfloat16* kp = conv_out + (size_t)t * C + Hk * dk + h * dk;
    float sq = 0.f, sk = 0.f;
    for (int i = lane; i < dk; i += 32) {
      const float qv = __bfloat162float(qp[i]), kv = __bfloat162float(kp[i]);
      sq += qv * qv;
      sk += kv * kv;
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const float iq = rsqrtf((float)dk) / fmaxf(sqrtf(sq), 1e-12f), ik = 1.f / fmaxf(sqrtf(sk), 1e-12f);
    for (int i = lane; i < dk; i += 32) {
      qn[((size_t)t * Hk + h) * dk + i] = __bfloat162float(qp[i]) * iq;
      kn[((size_t)t * Hk + h) * dk + i] = __bfloat162float(kp[i]) * ik;
    }
  }
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < T * Hv) {
    const int t = idx / Hv, h = idx % Hv;
    const float av = __bfloat162float(a[(size_t)t * lda + h]) + dt_bias[h];
    const float sp = av > 20.f ? av : log1pf(__expf(av));
    g[idx] = -__expf(A_log[h]) * sp;
    beta[idx] = 1.f / (1.f + __expf(-__bfloat162float(b[(size_t)t * lda + h])));
  }
}

// grid (Hv, R); blockDim = dv * dk / 32; a thread owns 32 rows of column j of the state.
// KDA (Kimi Delta Attention, reference: src/vllm_torchtpu/kernels/gdn/v3/compute_kda.py:362-423): the
// log-decay g is per key channel, [T, Hv, DK], instead of one scalar per (token, head); v_base is the
// column of the first value head inside a row of conv_out (row length C).
template <int DK, bool KDA = false>
__global__ void __launch_bounds__(512)
gdn_recurrent_kernel(const float* __restrict__ qn, const float* __restrict__ kn,
                     const __nv_bfloat16* __restrict__ conv_out, const float* __restrict__ g,
                     const float* __restrict__ beta, float* __restrict__ rec_pool,
                     __nv_bfloat16* __restrict__ out, const int* __restrict__ qsl,
                     const int* __restrict__ seq_lens, const int* __restrict__ slots, int Hk, int Hv, int dv,
                     int C, int v_base) {
  // a state column is shared by SPLIT adjacent lanes (32 rows each), so that it stays in registers;
  // their partial dot products meet in one or two shuffles
  constexpr int SPLIT = DK / 32;
  constexpr int DL = DK / SPLIT;
  __shared__ float sk[2][DK], sq[2][DK];
  __shared__ float sd[2][KDA ? DK : 1];
  const int hv = blockIdx.x, r = blockIdx.y;
  const int j = threadIdx.x / SPLIT, part = threadIdx.x % SPLIT, r0 = part * DL;
  const int qs = qsl[r], qe = qsl[r + 1];
  if (qe <= qs) return;
  const int slot = slots[r];
  if (slot < 0) return;
  const int hk = hv / (Hv / Hk);
  float S[DL];
  float* sp = rec_pool + (((size_t)slot * Hv + hv) * DK + r0) * dv + j;
  const bool fresh = (seq_lens[r] - (qe - qs)) == 0;
#pragma unroll
  for (int i = 0; i < DL; ++i) S[i] = fresh ? 0.f : sp[(size_t)i * dv];
  const int v_off = v_base + hv * dv + j;
  auto stage = [&](int t, int buf) {
    for (int i = threadIdx.x; i < DK; i += blockDim.x) {
      sk[buf][i] = kn[((size_t)t * Hk + hk) * DK + i];
      sq[buf][i] = qn[((size_t)t * Hk + hk) * DK + i];
      if constexpr (KDA) sd[buf][i] = __expf(g[((size_t)t * Hv + hv) * DK + i]);
    }
  };
  stage(qs, 0);
  __syncthreads();
  for (int t = qs; t < qe; ++t) {
    const int buf = (t - qs) & 1;
    if (t + 1 < qe) stage(t + 1, buf ^ 1);
    const float decay = KDA ? 1.f : __expf(g[(size_t)t * Hv + hv]);
    const float bt = beta[(size_t)t * Hv + hv];
    const float vt = __bfloat162float(conv_out[(size_t)t * C + v_off]);
    float mem = 0.f;
#pragma unroll
    for (int i = 0; i < DL; ++i) {
      S[i] *= KDA ? sd[buf][r0 + i] : decay;
      mem += S[i] * sk[buf][r0 + i];
    }
    if constexpr (SPLIT >= 2) mem += __shfl_xor_sync(0xffffffffu, mem, 1);
    if constexpr (SPLIT == 4) mem += __shfl_xor_sync(0xffffffffu, mem, 2);
    const float u = (vt - mem) * bt;
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < DL; ++i) {
      S[i] += sk[buf][r0 + i] * u;
      o += S[i] * sq[buf][r0 + i];
    }
    if constexpr (SPLIT >= 2) o += __shfl_xor_sync(0xffffffffu, o, 1);
    if constexpr (SPLIT == 4) o += __shfl_xor_sync(0xffffffffu, o, 2);
    if (part == 0) out[((size_t)t * Hv + hv) * dv + j] = __float2bfloat16(o);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < DL; ++i) sp[(size_t)i * dv] = S[i];
}

}  // namespace b200

using namespace b200;

// mixed [T, C] (C = 2*Hk*dk + Hv*dv, row stride ldx), a/b [T, Hv] (row stride lda).
// scratch: conv_out [T, C] bf16, qn/kn [T, Hk, dk] fp32, g/beta [T, Hv] fp32 (caller allocates).
extern "C" int b200_gdn_forward(const void* mixed, int ldx, const void* a, const void* b, int lda,
                                const void* conv_w, const float* A_log, const float* dt_bias, void* conv_pool,
                                float* rec_pool, void* conv_out, float* qn, float* kn, float* g, float* beta,
                                void* out, const int* qsl, const int* seq_lens, const int* slots, int R, int T,
                                int Hk, int Hv, int dk, int dv, int conv_k, cudaStream_t stream) {
  if (R <= 0 || T <= 0) return 0;
  const int C = 2 * Hk * dk + Hv * dv;
  if (conv_k != 4 || dv * (dk / 32) > 512 || (dk != 128 && dk != 64 && dk != 32)) {
    b200_set_last_error("gdn_forward: conv kernel 4, dk in {32,64,128}, dv * dk <= 16384 required", __FILE__,
                        __LINE__);
    return -1;
  }
  dim3 cg(R, (C + 127) / 128);
  gdn_conv_kernel<4><<<cg, 128, 0, stream>>>((const __nv_bfloat16*)mixed, (__nv_bfloat16*)conv_out,
                                             (__nv_bfloat16*)conv_pool, (const __nv_bfloat16*)conv_w, qsl,
                                             seq_lens, slots, C, ldx);
  const int work = T * (Hk * 32 > Hv ? Hk * 32 : Hv);
  gdn_prep_kernel<<<(work + 255) / 256, 256, 0, stream>>>((const __nv_bfloat16*)conv_out,
                                                          (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, A_log,
                                                          dt_bias, qn, kn, g, beta, T, Hk, Hv, dk, C, lda);
  dim3 rg(Hv, R);
#define REC(DKV)                                                                                          \
  gdn_recurrent_kernel<DKV><<<rg, dv * (DKV / 32), 0, stream>>>(qn, kn, (const __nv_bfloat16*)conv_out, g, beta, rec_pool, \
                                                   (__nv_bfloat16*)out, qsl, seq_lens, slots, Hk, Hv, dv, C, \
                                                   2 * Hk * dk)
  if (dk == 128) REC(128);
  else if (dk == 64) REC(64);
  else REC(32);
#undef REC
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

namespace b200 {

// One warp per (token, k head): fp32 L2 normalisation of q (also scaled by dk^-1/2) and k.
// One thread per (token, v head, channel): per-channel log-decay, either the unbounded form
// -exp(A_log) * softplus(a + dt_bias) or, with lower_bound < 0, lower_bound * sigmoid(exp(A_log) *
// (a + dt_bias)) (reference: compute_kda.py:42-63).  One thread per (token, v head): beta = sigmoid(b).
__global__ void kda_prep_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                float lower_bound, float* __restrict__ qn, float* __restrict__ kn,
                                float* __restrict__ g, float* __restrict__ beta, int T, int Hk, int Hv, int dk) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int warp = idx >> 5, lane = threadIdx.x & 31;
  if (warp < T * Hk) {
    const __nv_bfloat16* qp = q + (size_t)warp * dk;
    const __nv_bfloat16* kp = k + (size_t)warp * dk;
    float sq = 0.f, sk = 0.f;
    for (int i = lane; i < dk; i += 32) {
      const float qv = __bfloat162float(qp[i]), kv = __bfloat162float(kp[i]);
      sq += qv * qv;
      sk += kv * kv;
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const float iq = rsqrtf((float)dk) * rsqrtf(sq + 1e-6f), ik = rsqrtf(sk + 1e-6f);
    for (int i = lane; i < dk; i += 32) {
      qn[(size_t)warp * dk + i] = __bfloat162float(qp[i]) * iq;
      kn[(size_t)warp * dk + i] = __bfloat162float(kp[i]) * ik;
    }
  }
  if (idx < T * Hv * dk) {
    const int h = (idx / dk) % Hv, c = idx % dk;
    const float av = __bfloat162float(a[idx]) + dt_bias[h * dk + c];
    const float ea = __expf(A_log[h]);
    if (lower_bound < 0.f) {
      g[idx] = lower_bound / (1.f + __expf(-ea * av));
    } else {
      const float sp = av > 20.f ? av : log1pf(__expf(av));
      g[idx] = -ea * sp;
    }
  }
  if (idx < T * Hv) beta[idx] = 1.f / (1.f + __expf(-__bfloat162float(b[idx])));
}

}  // namespace b200

// Kimi Delta Attention over a ragged batch.  q, k [T, Hk, dk] bf16 (raw; normalised here), v [T, Hv, dv]
// bf16, a [T, Hv, dk] bf16 raw gate, b [T, Hv] bf16, A_log [Hv], dt_bias [Hv, dk] fp32; lower_bound < 0
// selects the bounded gate.  rec_pool [slots, Hv, dk, dv] fp32 carries the state between steps (a request
// whose first token of the step is at position 0 starts from zero).  Scratch qn, kn [T, Hk, dk], g [T, Hv,
// dk], beta [T, Hv] fp32 from the caller.
extern "C" int b200_kda_forward(const void* q, const void* k, const void* v, const void* a, const void* b,
                                const float* A_log, const float* dt_bias, float lower_bound, float* rec_pool,
                                float* qn, float* kn, float* g, float* beta, void* out, const int* qsl,
                                const int* seq_lens, const int* slots, int R, int T, int Hk, int Hv, int dk,
                                int dv, cudaStream_t stream) {
  if (R <= 0 || T <= 0) return 0;
  if (dv * (dk / 32) > 512 || (dk != 128 && dk != 64 && dk != 32) || Hv % Hk) {
    b200_set_last_error("kda_forward: dk in {32,64,128}, dv * dk <= 16384, Hv a multiple of Hk required", __FILE__,
                        __LINE__);
    return -1;
  }
  const long long work = (long long)T * Hv * dk > (long long)T * Hk * 32 ? (long long)T * Hv * dk
                                                                         : (long long)T * Hk * 32;
  kda_prep_kernel<<<(unsigned)((work + 255) / 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b, A_log,
      dt_bias, lower_bound, qn, kn, g, beta, T, Hk, Hv, dk);
  dim3 rg(Hv, R);
#define REC(DKV)                                                                                               \
  gdn_recurrent_kernel<DKV, true><<<rg, dv * (DKV / 32), 0, stream>>>(qn, kn, (const __nv_bfloat16*)v, g, beta, rec_pool,   \
                                                         (__nv_bfloat16*)out, qsl, seq_lens, slots, Hk, Hv, dv, \
                                                         Hv * dv, 0)
  if (dk == 128) REC(128);
  else if (dk == 64) REC(64);
  else REC(32);
#undef REC
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// Causal depth-wise short convolution (kernel 4) + SiLU over a ragged batch with the window carried in
// conv_pool [slots, C, 3] bf16 — the first stage of b200_gdn_forward on its own, for layers that feed
// the convolved q, k, v to another recurrence (Kimi Delta Attention).  x [T, C] row stride ldx -> y [T, C].
extern "C" int b200_short_conv(const void* x, int ldx, const void* conv_w, void* conv_pool, void* y,
                               const int* qsl, const int* seq_lens, const int* slots, int R, int C, int conv_k,
                               cudaStream_t stream) {
  if (R <= 0 || C <= 0) return 0;
  if (conv_k != 4) {
    b200_set_last_error("short_conv: kernel width 4 required", __FILE__, __LINE__);
    return -1;
  }
  dim3 cg(R, (C + 127) / 128);
  gdn_conv_kernel<4><<<cg, 128, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, (__nv_bfloat16*)conv_pool,
                                             (const __nv_bfloat16*)conv_w, qsl, seq_lens, slots, C, ldx);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}
