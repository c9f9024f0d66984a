// mma.sync / ldmatrix / cp.async building blocks of the paged-attention kernels: 16-token K/V groups
// in swizzled shared memory, bf16 m16n8k16 tiles, fp32 online softmax in the log2 domain.  Shared by
// the stand-alone decode / prefill kernels and by the attention phase of the persistent decode kernel.
#pragma once

#include "common.cuh"

namespace b200 {

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, const uint32_t* b) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void ldsm_x4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void cp_async16(uint32_t smem, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Copy `rows` tokens x D of one K or V page region into swizzled shared memory.
// 16-byte chunk c of row r lands at chunk (c ^ (r & 7)).
template <int D, int NTHREADS>
__device__ __forceinline__ void load_rows_async(uint32_t smem_base, const __nv_bfloat16* g, int rows,
                                                int tid) {
  constexpr int CPR = D / 8;                     // chunks per row
  for (int idx = tid; idx < rows * CPR; idx += NTHREADS) {
    const int r = idx / CPR, c = idx % CPR;
    cp_async16(smem_base + (uint32_t)(r * D * 2 + ((c ^ (r & 7)) << 4)), g + (size_t)r * D + c * 8);
  }
}

// S[16 x 16 tokens] += Q(frags) * K^T for one 16-token group at shared address kbase
template <int D>
__device__ __forceinline__ void qk_16(float s[2][4], const uint32_t (*qf)[4], uint32_t kbase, int lane) {
  const int mi = lane >> 3, rr = lane & 7;
  const int tok = (mi >> 1) * 8 + rr;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int c = 2 * ks + (mi & 1);
    uint32_t b[4];
    ldsm_x4(b, kbase + (uint32_t)(tok * D * 2 + ((c ^ (tok & 7)) << 4)));
    mma_bf16_16816(s[0], qf[ks], &b[0]);
    mma_bf16_16816(s[1], qf[ks], &b[2]);
  }
}
// O[16 x D] += P[16 x 16 tokens] * V for one 16-token group at shared address vbase
template <int D>
__device__ __forceinline__ void pv_16(float (*o)[4], const uint32_t* pa, uint32_t vbase, int lane) {
  const int mi = lane >> 3, rr = lane & 7;
  const int tok = (mi & 1) * 8 + rr;
#pragma unroll
  for (int np = 0; np < D / 16; ++np) {
    const int c = 2 * np + (mi >> 1);
    uint32_t b[4];
    ldsm_x4_t(b, vbase + (uint32_t)(tok * D * 2 + ((c ^ (tok & 7)) << 4)));
    mma_bf16_16816(o[2 * np], pa, &b[0]);
    mma_bf16_16816(o[2 * np + 1], pa, &b[2]);
  }
}

}  // namespace b200
