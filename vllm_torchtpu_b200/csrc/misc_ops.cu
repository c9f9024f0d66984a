// Small data-movement and quantisation kernels: LoRA batched gather matrix-vector products,
// structured-decoding token bitmask, row copies between state pools, fp8 KV quantisation and the
// 4-bit TurboQuant KV encode / decode for head_dim 128.
//
// Counterparts in the reference: lora/lora_ops.py:14-101 (one-hot bgmv), structured_decoding/
// structured_decoding_manager.py (device mask op), layers/adapter/custom_ops/mamba_state_copy_op.py
// and kernels/partial_kv_update.py (pool copies), layers/core/quantization.py:91 (quantize_kv),
// layers/core/turboquant.py (Walsh-Hadamard + Lloyd-Max keys, asymmetric 4-bit values).
#include <cuda_fp8.h>

#include "common.cuh"

namespace b200 {

// ------------------------------------------------------------------------------- LoRA
// h[t, j] = sum_k x[t, k] * A[idx[t], j, k]; one warp per (t, j).  idx[t] < 0: h[t, :] = 0.
__global__ void bgmv_shrink_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ A,
                                   const int* __restrict__ idx, float* __restrict__ h, int K, int r, int ldx) {
  const int t = blockIdx.x;
  const int j = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (j >= r) return;
  const int s = idx[t];
  float acc = 0.f;
  if (s >= 0) {
    const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)t * ldx);
    const uint4* ap = reinterpret_cast<const uint4*>(A + ((size_t)s * r + j) * K);
    for (int i = lane; i < (K >> 3); i += 32) {
      const uint4 xv = xp[i], av = ap[i];
      const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv);
      const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&av);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 a = __bfloat1622float2(xh[q]), b = __bfloat1622float2(ah[q]);
        acc += a.x * b.x + a.y * b.y;
      }
    }
    acc = warp_sum(acc);
  }
  if (lane == 0) h[(size_t)t * r + j] = acc;
}

// y[t, off + n] += scale[idx[t]] * sum_j h[t, j] * B[idx[t], n, j]; thread per n.
__global__ void bgmv_expand_kernel(const float* __restrict__ h, const __nv_bfloat16* __restrict__ B,
                                   const int* __restrict__ idx, const float* __restrict__ scale,
                                   __nv_bfloat16* __restrict__ y, int N, int r, int ldy, int col_off) {
  extern __shared__ float sh[];
  const int t = blockIdx.x;
  const int s = idx[t];
  if (s < 0) return;
  for (int j = threadIdx.x; j < r; j += blockDim.x) sh[j] = h[(size_t)t * r + j];
  __syncthreads();
  const int n = blockIdx.y * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const __nv_bfloat16* bp = B + ((size_t)s * N + n) * r;
  float acc = 0.f;
  for (int j = 0; j < r; ++j) acc += sh[j] * __bfloat162float(bp[j]);
  __nv_bfloat16* yp = y + (size_t)t * ldy + col_off + n;
  *yp = __float2bfloat16(__bfloat162float(*yp) + scale[s] * acc);
}

// ------------------------------------------------------------------- structured decoding
// logits[row, v] = -inf where bit v of bitmask[m, :] is 0.  rows == null: row = m.
template <typename T>
__global__ void token_bitmask_kernel(T* __restrict__ logits, int ld, const int* __restrict__ bitmask, int words,
                                     const long long* __restrict__ rows, int V) {
  const int m = blockIdx.x;
  const long long row = rows ? rows[m] : m;
  const int v = blockIdx.y * blockDim.x + threadIdx.x;
  if (v >= V) return;
  const unsigned w = (unsigned)bitmask[(size_t)m * words + (v >> 5)];
  if (!((w >> (v & 31)) & 1u)) logits[(size_t)row * ld + v] = T(-INFINITY);
}

// --------------------------------------------------------------------------- pool copies
// dst row dst_idx[i] = src row src_idx[i]; rows of row_bytes (multiple of 16); negative index: skip.
__global__ void copy_rows_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src,
                                 const int* __restrict__ dst_idx, const int* __restrict__ src_idx, int n,
                                 size_t row_bytes) {
  const int i = blockIdx.x;
  const int d = dst_idx[i], s = src_idx[i];
  if (d < 0 || s < 0) return;
  const uint4* sp = reinterpret_cast<const uint4*>(src + (size_t)s * row_bytes);
  uint4* dp = reinterpret_cast<uint4*>(dst + (size_t)d * row_bytes);
  const size_t nv = row_bytes >> 4;
  for (size_t v = (size_t)blockIdx.y * blockDim.x + threadIdx.x; v < nv; v += (size_t)gridDim.y * blockDim.x)
    dp[v] = sp[v];
}

// ------------------------------------------------------------------------ fp8 KV (e4m3)
__global__ void kv_quant_fp8_kernel(const __nv_bfloat16* __restrict__ x, __nv_fp8_e4m3* __restrict__ q, size_t n,
                                    float inv_scale) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    q[i] = __nv_fp8_e4m3(fminf(fmaxf(__bfloat162float(x[i]) * inv_scale, -448.f), 448.f));
}
__global__ void kv_dequant_fp8_kernel(const __nv_fp8_e4m3* __restrict__ q, __nv_bfloat16* __restrict__ x, size_t n,
                                      float scale) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] = __float2bfloat16(float(q[i]) * scale);
}

// ------------------------------------------------------------------- TurboQuant, 4 bit, D = 128
// Lloyd-Max 16-level quantiser of a unit normal; a coordinate of a rotated unit vector in R^128 is
// close to N(0, 1/128), so the levels are used divided by sqrt(128).
__constant__ float TQ_LEVELS[16] = {-2.7326f, -2.0690f, -1.6181f, -1.2562f, -0.9424f, -0.6568f, -0.3881f, -0.1284f,
                                    0.1284f,  0.3881f,  0.6568f,  0.9424f,  1.2562f,  1.6181f,  2.0690f,  2.7326f};

// Orthonormal Walsh-Hadamard transform of 128 values held 4 per lane (lane l has elements 4l..4l+3).
__device__ __forceinline__ void fwht128(float (&v)[4], int lane) {
  float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
  v[0] = a + c; v[1] = b + d; v[2] = a - c; v[3] = b - d;
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float o = __shfl_xor_sync(0xffffffffu, v[j], m);
      v[j] = (lane & m) ? o - v[j] : v[j] + o;
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] *= 0.08838834764831845f;      // 1 / sqrt(128)
}

__device__ __forceinline__ int tq_nearest(float x) {             // x in units of 1/sqrt(128)
  int lo = 0;
#pragma unroll
  for (int step = 8; step > 0; step >>= 1)
    if (x > 0.5f * (TQ_LEVELS[lo + step - 1] + TQ_LEVELS[lo + step])) lo += step;
  return lo;
}

// One warp per row (one token of one head).  Key row: codes of H(k / |k|) in 64 bytes + a bf16 norm that
// already carries the correction |k| / |centroid vector|.  Value row: asymmetric uniform 4-bit codes in
// 64 bytes + bf16 (scale, zero).
__global__ void tq4_encode_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                  uint8_t* __restrict__ k_codes, __nv_bfloat16* __restrict__ k_norm,
                                  uint8_t* __restrict__ v_codes, __nv_bfloat16* __restrict__ v_meta, int rows) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  float x[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) x[j] = __bfloat162float(k[(size_t)row * 128 + 4 * lane + j]);
  float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
  const float norm = sqrtf(ss);
  const float inv = 1.f / fmaxf(norm, 1e-8f);
#pragma unroll
  for (int j = 0; j < 4; ++j) x[j] *= inv;
  fwht128(x, lane);
  int code[4];
  float cs = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    code[j] = tq_nearest(x[j] * 11.313708498984761f);            // sqrt(128)
    const float c = TQ_LEVELS[code[j]] * 0.08838834764831845f;
    cs += c * c;
  }
  cs = warp_sum(cs);
  k_codes[(size_t)row * 64 + 2 * lane] = (uint8_t)(code[0] | (code[1] << 4));
  k_codes[(size_t)row * 64 + 2 * lane + 1] = (uint8_t)(code[2] | (code[3] << 4));
  if (lane == 0) k_norm[row] = __float2bfloat16(norm * rsqrtf(cs + 1e-16f));
  // values
  float y[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) y[j] = __bfloat162float(v[(size_t)row * 128 + 4 * lane + j]);
  const float mx = warp_max(fmaxf(fmaxf(y[0], y[1]), fmaxf(y[2], y[3])));
  const float mn = -warp_max(-fminf(fminf(y[0], y[1]), fminf(y[2], y[3])));
  // the stored metadata is bf16: quantise against the rounded values so that decode matches
  const float scale = __bfloat162float(__float2bfloat16(fmaxf((mx - mn) / 15.f, 1e-8f)));
  const float zero = __bfloat162float(__float2bfloat16(mn));
  int vc[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) vc[j] = min(15, max(0, __float2int_rn((y[j] - zero) / scale)));
  v_codes[(size_t)row * 64 + 2 * lane] = (uint8_t)(vc[0] | (vc[1] << 4));
  v_codes[(size_t)row * 64 + 2 * lane + 1] = (uint8_t)(vc[2] | (vc[3] << 4));
  if (lane == 0) {
    v_meta[2 * row] = __float2bfloat16(scale);
    v_meta[2 * row + 1] = __float2bfloat16(zero);
  }
}

// Inverse: keys come back in the ORIGINAL basis (H is its own inverse), values as scale * code + zero.
__global__ void tq4_decode_kernel(const uint8_t* __restrict__ k_codes, const __nv_bfloat16* __restrict__ k_norm,
                                  const uint8_t* __restrict__ v_codes, const __nv_bfloat16* __restrict__ v_meta,
                                  __nv_bfloat16* __restrict__ k, __nv_bfloat16* __restrict__ v, int rows) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint8_t b0 = k_codes[(size_t)row * 64 + 2 * lane], b1 = k_codes[(size_t)row * 64 + 2 * lane + 1];
  float x[4] = {TQ_LEVELS[b0 & 15], TQ_LEVELS[b0 >> 4], TQ_LEVELS[b1 & 15], TQ_LEVELS[b1 >> 4]};
#pragma unroll
  for (int j = 0; j < 4; ++j) x[j] *= 0.08838834764831845f;
  fwht128(x, lane);
  const float n = __bfloat162float(k_norm[row]);
#pragma unroll
  for (int j = 0; j < 4; ++j) k[(size_t)row * 128 + 4 * lane + j] = __float2bfloat16(x[j] * n);
  const uint8_t c0 = v_codes[(size_t)row * 64 + 2 * lane], c1 = v_codes[(size_t)row * 64 + 2 * lane + 1];
  const float scale = __bfloat162float(v_meta[2 * row]), zero = __bfloat162float(v_meta[2 * row + 1]);
  const int vc[4] = {c0 & 15, c0 >> 4, c1 & 15, c1 >> 4};
#pragma unroll
  for (int j = 0; j < 4; ++j) v[(size_t)row * 128 + 4 * lane + j] = __float2bfloat16(scale * vc[j] + zero);
}

// ------------------------------------------------------------------- KV cache write
// cache[blk, 0 | 1, h, off, :] = k | v of token t, slot = slot_mapping[t] (negative: skipped), for
// callers that hand over already-rotated keys (a host framework's attention layer).  16 bytes per thread.
__global__ void kv_write_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                __nv_bfloat16* __restrict__ cache, const long long* __restrict__ slots64,
                                const int* __restrict__ slots32, int Hkv, int D, int block_size, long long num_slots,
                                long long ldk, long long ldv) {
  const int t = blockIdx.x;
  const long long slot = slots64 != nullptr ? slots64[t] : (long long)slots32[t];
  if (slot < 0 || slot >= num_slots) return;
  const long long blk = slot / block_size;
  const int off = (int)(slot - blk * block_size);
  const int vec_per_head = D >> 3;
  for (int i = threadIdx.x; i < 2 * Hkv * vec_per_head; i += blockDim.x) {
    const int kind = i / (Hkv * vec_per_head);
    const int r = i - kind * Hkv * vec_per_head;
    const int h = r / vec_per_head, c = r - h * vec_per_head;
    const __nv_bfloat16* src = (kind == 0 ? k + (size_t)t * ldk : v + (size_t)t * ldv) + h * D + c * 8;
    __nv_bfloat16* dst = cache + ((((size_t)blk * 2 + kind) * Hkv + h) * block_size + off) * D + c * 8;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_bgmv_shrink(const void* x, const void* A, const int* idx, float* h, int T, int K, int r,
                                int ldx, cudaStream_t stream) {
  if (T == 0 || r == 0) return 0;
  if (K % 8 || ldx % 8) {
    b200_set_last_error("bgmv_shrink: K and the row stride must be multiples of 8", __FILE__, __LINE__);
    return -1;
  }
  dim3 grid(T, (r + 7) / 8);
  bgmv_shrink_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)A, idx, h, K, r, ldx);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_bgmv_expand(const float* h, const void* B, const int* idx, const float* scale, void* y, int T,
                                int N, int r, int ldy, int col_off, cudaStream_t stream) {
  if (T == 0 || N == 0) return 0;
  dim3 grid(T, (N + 255) / 256);
  bgmv_expand_kernel<<<grid, 256, r * sizeof(float), stream>>>(h, (const __nv_bfloat16*)B, idx, scale,
                                                               (__nv_bfloat16*)y, N, r, ldy, col_off);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// dtype: 0 bf16 logits, 1 fp32 logits.
extern "C" int b200_apply_token_bitmask(void* logits, int dtype, int ld, const int* bitmask, int words,
                                        const long long* rows, int M, int V, cudaStream_t stream) {
  if (M == 0) return 0;
  dim3 grid(M, (V + 255) / 256);
  if (dtype == 0)
    token_bitmask_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((__nv_bfloat16*)logits, ld, bitmask, words, rows, V);
  else
    token_bitmask_kernel<float><<<grid, 256, 0, stream>>>((float*)logits, ld, bitmask, words, rows, V);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_copy_rows(void* dst, const void* src, const int* dst_idx, const int* src_idx, int n,
                              size_t row_bytes, cudaStream_t stream) {
  if (n == 0) return 0;
  if (row_bytes % 16) {
    b200_set_last_error("copy_rows: row size must be a multiple of 16 bytes", __FILE__, __LINE__);
    return -1;
  }
  int by = (int)((row_bytes / 16 + 255) / 256);
  if (by > 64) by = 64;
  if (by < 1) by = 1;
  copy_rows_kernel<<<dim3(n, by), 256, 0, stream>>>((uint8_t*)dst, (const uint8_t*)src, dst_idx, src_idx, n,
                                                    row_bytes);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

extern "C" int b200_kv_quant_fp8(const void* x, void* q, size_t n, float scale, int dequant, cudaStream_t stream) {
  if (n == 0) return 0;
  int blocks = (int)((n + 1023) / 1024);
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (dequant)
    kv_dequant_fp8_kernel<<<blocks, 256, 0, stream>>>((const __nv_fp8_e4m3*)q, (__nv_bfloat16*)x, n, scale);
  else
    kv_quant_fp8_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_fp8_e4m3*)q, n, 1.f / scale);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// rows = tokens * kv heads, head_dim 128.  k_codes / v_codes: 64 bytes per row; k_norm: bf16 per row;
// v_meta: bf16 (scale, zero) per row.
extern "C" int b200_tq4_encode(const void* k, const void* v, void* k_codes, void* k_norm, void* v_codes,
                               void* v_meta, int rows, cudaStream_t stream) {
  if (rows == 0) return 0;
  tq4_encode_kernel<<<(rows + 7) / 8, 256, 0, stream>>>((const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
                                                        (uint8_t*)k_codes, (__nv_bfloat16*)k_norm,
                                                        (uint8_t*)v_codes, (__nv_bfloat16*)v_meta, rows);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}
extern "C" int b200_tq4_decode(const void* k_codes, const void* k_norm, const void* v_codes, const void* v_meta,
                               void* k, void* v, int rows, cudaStream_t stream) {
  if (rows == 0) return 0;
  tq4_decode_kernel<<<(rows + 7) / 8, 256, 0, stream>>>((const uint8_t*)k_codes, (const __nv_bfloat16*)k_norm,
                                                        (const uint8_t*)v_codes, (const __nv_bfloat16*)v_meta,
                                                        (__nv_bfloat16*)k, (__nv_bfloat16*)v, rows);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// k, v: [T, Hkv, D] bf16 with row strides ldk / ldv (elements); cache [blocks, 2, Hkv, block_size, D] bf16;
// slot mapping as int64 (slots64) or int32 (slots32), exactly one of them non-null.
extern "C" int b200_kv_write(const void* k, const void* v, void* cache, const long long* slots64, const int* slots32,
                             int T, int Hkv, int D, int block_size, long long num_blocks, long long ldk, long long ldv,
                             cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D % 8 || ldk % 8 || ldv % 8 || (slots64 == nullptr) == (slots32 == nullptr)) {
    b200_set_last_error("kv_write: head_dim and strides multiples of 8, one slot mapping", __FILE__, __LINE__);
    return -1;
  }
  b200::kv_write_kernel<<<T, 128, 0, stream>>>((const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)cache,
                                               slots64, slots32, Hkv, D, block_size, num_blocks * block_size, ldk, ldv);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}
