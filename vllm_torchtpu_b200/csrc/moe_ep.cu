// Expert-parallel dispatch / combine over NVLink peer memory.
//
// Every rank of the EP group owns E / world consecutive experts.  One MoE layer call is
//   1. ep_count_kernel     per-expert histogram of this rank's (token, k) pairs, PUT into the count
//                          matrix cnt[src][E] of every rank (so every rank can lay out every
//                          owner's receive buffer by itself: one hop, no negotiation)
//   2. ep_dispatch_kernel  each (token, k) row is PUT straight into its slot of the owner's receive
//                          buffer, rows grouped by expert then by source rank, together with its
//                          return address (source rank, t * k + j); then a "landed" flag per owner
//   3. ep_wait_kernel      the owner waits for the flags of all sources
//   4. grouped SwiGLU GEMM and grouped down GEMM (tcgen05) on the received rows; the epilogue of the
//      second GEMM stores every output row directly into the return slot of its source rank and the
//      last CTA raises the "returned" flags (gemm_tcgen05.cu, routed epilogue)
//   5. ep_combine_kernel   the source waits for the flags of all owners and takes the weighted sum
//                          of its k returned rows per token.
// All cross-GPU traffic is stores; every wait is bounded and reports through the status word.
// Epochs live in device memory (ctrl[0]) so that a captured CUDA graph can be replayed.
//
// Takes the place of the reference's fused expert-parallel kernel and of its all-gather /
// reduce-scatter dispatch (reference: src/vllm_torchtpu/kernels/fused_moe/v2/layer.py:253,
// distributed/tpu_communicator.py:63-93).
#include "common.cuh"

namespace b200 {

constexpr int EP_MAX_EXPERTS = 1024;
constexpr int EP_MAX_WORLD = 8;

struct EpLayout {
  unsigned long long cnt_off;        // int[world][E]      count matrix (row s written by rank s)
  unsigned long long cnt_flag_off;   // int[world]
  unsigned long long data_flag_off;  // int[world]         "rows of rank s have landed here"
  unsigned long long ret_flag_off;   // int[world]         "owner s has returned all rows of this rank"
  unsigned long long recv_x_off;     // bf16[cap][H]       received rows, grouped by local expert
  unsigned long long recv_route_off; // int2[cap]          (source rank, return slot)
  unsigned long long ret_off;        // bf16[T_max * k][H] returned expert outputs of this rank's tokens
};

struct EpParams {
  uint8_t* peer[EP_MAX_WORLD];
  EpLayout lay;
  int* ctrl;                         // local: [0] epoch, [1] CTA counter
  int* fill;                         // local: int[E] slot cursors, zeroed by ep_count_kernel
  int* group_off;                    // local: int[E_local + 1] row offsets of the received rows
  int* status;
  const int* topk_ids;               // [T, k]
  const __nv_bfloat16* x;            // [T, H]
  int T, k, H, E, world, rank, cap;
  unsigned int spin_limit;
};

// 1 CTA.  ids outside [0, E) are ignored everywhere (they take no slot).
__global__ void __launch_bounds__(1024) ep_count_kernel(const EpParams p) {
  __shared__ int hist[EP_MAX_EXPERTS];
  const int epoch = *reinterpret_cast<volatile int*>(p.ctrl) + 1;
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
    hist[e] = 0;
    p.fill[e] = 0;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < p.T * p.k; i += blockDim.x) {
    const int e = p.topk_ids[i];
    if (e >= 0 && e < p.E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < p.world * p.E; i += blockDim.x) {
    const int r = i / p.E, e = i - r * p.E;
    reinterpret_cast<int*>(p.peer[r] + p.lay.cnt_off)[(size_t)p.rank * p.E + e] = hist[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.world)
    st_release_sys(reinterpret_cast<int*>(p.peer[threadIdx.x] + p.lay.cnt_flag_off) + p.rank, epoch);
  if (threadIdx.x == 0) {
    p.ctrl[1] = 0;
    p.ctrl[0] = epoch;               // later kernels of this layer call read the epoch from here
  }
}

// grid: any; one warp per (token, k) pair.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const EpParams p) {
  __shared__ int base[EP_MAX_EXPERTS];     // first row of (expert e, this source rank) at e's owner
  __shared__ int s_tot[EP_MAX_EXPERTS];    // rows of expert e over all source ranks
  __shared__ int s_base2[EP_MAX_EXPERTS];
  __shared__ int s_ok, s_last;
  const int epoch = *reinterpret_cast<volatile int*>(p.ctrl);
  const int e_local = p.E / p.world;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const int* f = reinterpret_cast<const int*>(p.peer[p.rank] + p.lay.cnt_flag_off) + threadIdx.x;
    if (!wait_flag_ge(f, epoch, p.status, p.spin_limit)) s_ok = 0;
  }
  __syncthreads();
  const int* cnt = reinterpret_cast<const int*>(p.peer[p.rank] + p.lay.cnt_off);   // [world][E]
  if (s_ok) {
    // per-expert totals and this rank's share in front of it, from one coalesced pass over the count
    // matrix; then an exclusive prefix over each owner's experts out of shared memory
    for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
      int tot = 0, before = 0;
      for (int s = 0; s < p.world; ++s) {
        const int c = __ldcg(cnt + (size_t)s * p.E + e);
        tot += c;
        if (s < p.rank) before += c;
      }
      s_tot[e] = tot;
      base[e] = before;
    }
  }
  __syncthreads();
  if (s_ok) {
    for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
      const int first = (e / e_local) * e_local;
      int b = base[e];
      for (int e2 = first; e2 < e; ++e2) b += s_tot[e2];
      s_base2[e] = b;
    }
    if (blockIdx.x == 0) {
      // row offsets of this rank's own experts for the grouped GEMMs
      for (int le = threadIdx.x; le <= e_local; le += blockDim.x) {
        int b = 0;
        for (int e2 = p.rank * e_local; e2 < p.rank * e_local + le; ++e2) b += s_tot[e2];
        p.group_off[le] = b < p.cap ? b : p.cap;
        if (le == e_local && b > p.cap) atomicCAS(p.status, ST_OK, ST_BAD_INDEX);
      }
    }
  }
  __syncthreads();
  if (s_ok)
    for (int e = threadIdx.x; e < p.E; e += blockDim.x) base[e] = s_base2[e];
  __syncthreads();
  if (s_ok) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    const int nvec = p.H >> 3;
    for (int pair = blockIdx.x * wpb + warp; pair < p.T * p.k; pair += gridDim.x * wpb) {
      const int e = p.topk_ids[pair];
      if (e < 0 || e >= p.E) continue;
      int slot = 0;
      if (lane == 0) slot = atomicAdd(&p.fill[e], 1);
      slot = __shfl_sync(0xffffffffu, slot, 0);
      const int owner = e / e_local;
      const int row = base[e] + slot;
      if (row >= p.cap) {
        if (lane == 0) atomicCAS(p.status, ST_OK, ST_BAD_INDEX);
        continue;
      }
      const uint4* src = reinterpret_cast<const uint4*>(p.x + (size_t)(pair / p.k) * p.H);
      uint4* dst = reinterpret_cast<uint4*>(p.peer[owner] + p.lay.recv_x_off) + (size_t)row * nvec;
      for (int i = lane; i < nvec; i += 32) dst[i] = src[i];
      if (lane == 0)
        reinterpret_cast<int2*>(p.peer[owner] + p.lay.recv_route_off)[row] = make_int2(p.rank, pair);
    }
    __threadfence_system();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = (atomicAdd(&p.ctrl[1], 1) + 1 == (int)gridDim.x) ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x < p.world)
      st_release_sys(reinterpret_cast<int*>(p.peer[threadIdx.x] + p.lay.data_flag_off) + p.rank, epoch);
    if (threadIdx.x == 0) p.ctrl[1] = 0;
  }
}

// 1 CTA: returns once flags[0..world) >= epoch (or the bounded wait gave up: status word).
__global__ void ep_wait_kernel(const int* flags, const int* ctrl, int world, int* status, unsigned int spin_limit) {
  const int epoch = *reinterpret_cast<const volatile int*>(ctrl);
  if ((int)threadIdx.x < world) wait_flag_ge(flags + threadIdx.x, epoch, status, spin_limit);
}

// grid T: out[t] = sum_j w[t, j] * ret[t * k + j] once every owner has returned its rows.
__global__ void __launch_bounds__(128) ep_combine_kernel(const uint8_t* ret, const int* ret_flags, const int* ctrl,
                                                         const int* topk_ids, const float* topk_w,
                                                         __nv_bfloat16* out, int H, int k, int E, int world,
                                                         int* status, unsigned int spin_limit) {
  __shared__ int s_ok;
  const int epoch = *reinterpret_cast<const volatile int*>(ctrl);
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < world)
    if (!wait_flag_ge(ret_flags + threadIdx.x, epoch, status, spin_limit)) s_ok = 0;
  __syncthreads();
  if (!s_ok) return;
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < k; ++j) {
      const int e = topk_ids[(size_t)t * k + j];
      if (e < 0 || e >= E) continue;
      const float wt = topk_w[(size_t)t * k + j];
      const uint4 raw = ld_relaxed_sys_v4(ret + ((size_t)(t * k + j) * H + i * 8) * 2);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h[q]);
        acc[2 * q] += wt * f.x;
        acc[2 * q + 1] += wt * f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) oh[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    *(reinterpret_cast<uint4*>(out + (size_t)t * H) + i) = o;
  }
}

}  // namespace b200

using namespace b200;

// Steps 1-3 of the header comment.  peers: `world` heap bases; layout: 7 heap offsets in the order of
// EpLayout; ctrl int[2], fill int[E], group_off int[E/world + 1] are local device arrays.
// After this call recv_x (heap, this rank) holds the rows of this rank's experts and group_off their
// per-expert row offsets; cap is the row capacity of recv_x / recv_route.
extern "C" int b200_ep_dispatch(void* const* peers, int rank, int world, const unsigned long long* layout,
                                int* ctrl, int* fill, int* group_off, const void* x, const int* topk_ids,
                                int T, int k, int H, int E, int cap, int* status, unsigned int spin_limit,
                                cudaStream_t stream) {
  if (world < 2 || world > EP_MAX_WORLD || E > EP_MAX_EXPERTS || E % world || H % 8) {
    b200_set_last_error("ep_dispatch: 2 <= world <= 8, E <= 1024, E % world == 0, H % 8 == 0 required",
                        __FILE__, __LINE__);
    return -1;
  }
  EpParams p;
  for (int i = 0; i < EP_MAX_WORLD; ++i) p.peer[i] = i < world ? (uint8_t*)peers[i] : nullptr;
  p.lay.cnt_off = layout[0]; p.lay.cnt_flag_off = layout[1]; p.lay.data_flag_off = layout[2];
  p.lay.ret_flag_off = layout[3]; p.lay.recv_x_off = layout[4]; p.lay.recv_route_off = layout[5];
  p.lay.ret_off = layout[6];
  p.ctrl = ctrl; p.fill = fill; p.group_off = group_off; p.status = status;
  p.topk_ids = topk_ids; p.x = (const __nv_bfloat16*)x;
  p.T = T; p.k = k; p.H = H; p.E = E; p.world = world; p.rank = rank; p.cap = cap;
  p.spin_limit = spin_limit;
  ep_count_kernel<<<1, 1024, 0, stream>>>(p);
  int blocks = (T * k + 7) / 8;
  if (blocks > 148 * 4) blocks = 148 * 4;
  if (blocks < 1) blocks = 1;
  ep_dispatch_kernel<<<blocks, 256, 0, stream>>>(p);
  ep_wait_kernel<<<1, 32, 0, stream>>>(reinterpret_cast<const int*>((uint8_t*)peers[rank] + p.lay.data_flag_off),
                                       ctrl, world, status, spin_limit);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}

// Step 5.  out [T, H] bf16.
extern "C" int b200_ep_combine(const void* heap_local, unsigned long long ret_off, unsigned long long ret_flag_off,
                               const int* ctrl, const int* topk_ids, const float* topk_w, void* out, int T,
                               int k, int H, int E, int world, int* status, unsigned int spin_limit,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  ep_combine_kernel<<<T, 128, 0, stream>>>((const uint8_t*)heap_local + ret_off,
                                           reinterpret_cast<const int*>((const uint8_t*)heap_local + ret_flag_off),
                                           ctrl, topk_ids, topk_w, (__nv_bfloat16*)out, H, k, E, world, status,
                                           spin_limit);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}
