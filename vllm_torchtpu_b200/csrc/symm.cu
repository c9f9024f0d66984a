// Symmetric-memory plumbing over CUDA IPC and the stand-alone peer collectives.
//
// Every rank of a group allocates one heap of the same size with cudaMalloc, exports it
// as a cudaIpcMemHandle (exchanged by the Python side over torch.distributed), and maps
// every peer's heap.  Kernels receive a table of heap base pointers indexed by group
// rank; offsets inside the heap are the same on every rank, so "peer p's copy of buffer
// B" is peers[p] + offset(B).  Reads and writes of peer memory are ordinary ld/st.global
// that travel over NVLink through NVSwitch; flags use st.release.sys / ld.acquire.sys.
// Every flag wait has an iteration limit and reports ST_TIMEOUT_FLAG in the status word.
//
// Plays the role of the reference's in-kernel remote DMA + semaphore substrate
// (reference: src/vllm_torchtpu/kernels/collectives/util.py:33-58).
#include <cuda.h>

#include "common.cuh"

using namespace b200;

extern "C" int b200_set_device(int device) {
  B200_CUDA_CHECK(cudaSetDevice(device));
  return 0;
}

extern "C" int b200_ipc_alloc(size_t bytes, void** out) {
  B200_CUDA_CHECK(cudaMalloc(out, bytes));
  B200_CUDA_CHECK(cudaMemset(*out, 0, bytes));
  B200_CUDA_CHECK(cudaDeviceSynchronize());
  return 0;
}

extern "C" int b200_ipc_free(void* p) {
  B200_CUDA_CHECK(cudaFree(p));
  return 0;
}

extern "C" int b200_ipc_get_handle(void* p, void* handle_out_64) {
  cudaIpcMemHandle_t h;
  B200_CUDA_CHECK(cudaIpcGetMemHandle(&h, p));
  memcpy(handle_out_64, &h, sizeof(h));
  return 0;
}

// Base address and size of the allocation that holds `p`: an IPC handle names the whole allocation, so
// an exporter that hands out a pointer inside a larger block (a caching allocator's segment) also
// publishes the pointer's offset from this base.
extern "C" int b200_ipc_range(const void* p, unsigned long long* base_out, unsigned long long* size_out) {
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      b200_set_last_error("cuMemGetAddressRange not available", __FILE__, __LINE__);
      return -1;
    }
    fn = reinterpret_cast<RangeFn>(ptr);
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  if (fn(&base, &size, reinterpret_cast<CUdeviceptr>(p)) != CUDA_SUCCESS) {
    b200_set_last_error("cuMemGetAddressRange failed", __FILE__, __LINE__);
    return -2;
  }
  *base_out = (unsigned long long)base;
  *size_out = (unsigned long long)size;
  return 0;
}

extern "C" int b200_ipc_open(const void* handle_64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_64, sizeof(h));
  B200_CUDA_CHECK(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}

extern "C" int b200_ipc_close(void* p) {
  B200_CUDA_CHECK(cudaIpcCloseMemHandle(p));
  return 0;
}

extern "C" int b200_enable_peer_access(int device, int peer) {
  int can = 0;
  B200_CUDA_CHECK(cudaDeviceCanAccessPeer(&can, device, peer));
  if (!can) {
    b200_set_last_error("peer access not available", __FILE__, __LINE__);
    return -1;
  }
  cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
    b200_set_last_error(cudaGetErrorString(e), __FILE__, __LINE__);
    return (int)e;
  }
  cudaGetLastError();
  return 0;
}

namespace b200 {

constexpr int MAX_RANKS = 8;

struct PeerTable {
  uint8_t* base[MAX_RANKS];
};

// ---- barrier across ranks: each rank bumps a slot in every peer, then waits for all its slots.
// flags layout at `flag_off` in every heap: int[MAX_RANKS] arrival slots (monotonic epochs).
__device__ __forceinline__ bool rank_barrier(const PeerTable& pt, size_t flag_off, int rank, int world,
                                             int epoch, int* status, uint32_t limit) {
  if (threadIdx.x < world) {
    int* remote = reinterpret_cast<int*>(pt.base[threadIdx.x] + flag_off) + rank;
    st_release_sys(remote, epoch);
  }
  bool ok = true;
  if (threadIdx.x < world) {
    const int* mine = reinterpret_cast<const int*>(pt.base[rank] + flag_off) + threadIdx.x;
    ok = wait_flag_ge(mine, epoch, status, limit);
  }
  return __syncthreads_and(ok);
}

// Two-shot all-reduce of a bf16 buffer that already sits in the symmetric heap at `buf_off`:
// rank r reduces slice r (reading every peer) and writes the sum into every peer's buffer.
// One launch per rank; grid-wide phases are separated by cross-rank barriers, the grid itself
// by an atomic counter on `grid_sync` (all CTAs are co-resident: grid <= SM count).
__global__ void p2p_all_reduce_kernel(PeerTable pt, size_t buf_off, size_t flag_off, int* epoch_ptr,
                                      int* grid_sync, int rank, int world, size_t n_elems, int* status,
                                      uint32_t limit) {
  const int epoch0 = *reinterpret_cast<volatile int*>(epoch_ptr);
  const int e1 = epoch0 + 1, e2 = epoch0 + 2;
  __shared__ int s_ok;
  // phase 0: everyone's input is in place (stream order made it visible locally; publish to peers)
  __threadfence_system();
  if (blockIdx.x == 0) {
    rank_barrier(pt, flag_off, rank, world, e1, status, limit);
    if (threadIdx.x == 0) st_release_sys(grid_sync + 1, e1);       // release the other CTAs
  }
  if (threadIdx.x == 0) s_ok = wait_flag_ge(grid_sync + 1, e1, status, limit) ? 1 : 0;
  __syncthreads();
  if (s_ok) {
    const size_t nvec = n_elems / 8;                                // 16-byte vectors
    const size_t per = (nvec + world - 1) / world;
    const size_t v0 = per * rank, v1 = min(nvec, v0 + per);
    for (size_t v = v0 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < v1;
         v += (size_t)gridDim.x * blockDim.x) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int p = 0; p < world; ++p) {
        const uint4 raw = *(reinterpret_cast<const uint4*>(pt.base[p] + buf_off) + v);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      // the sum must not land in a peer's input slice before that peer's owner has read it: slices are
      // disjoint per owner, and only the owner reads slice `rank`, so writing it everywhere is safe
      for (int p = 0; p < world; ++p) *(reinterpret_cast<uint4*>(pt.base[p] + buf_off) + v) = o;
    }
  }
  // phase 2: all my writes are out; wait until every peer has written my buffer
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int arrived = atomicAdd(grid_sync, 1) + 1;
    if (arrived == (int)gridDim.x) {
      grid_sync[0] = 0;
      __threadfence();
      st_release_sys(grid_sync + 2, e2);                            // last CTA of this rank
    }
  }
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) wait_flag_ge(grid_sync + 2, e2, status, limit);
    __syncthreads();
    rank_barrier(pt, flag_off, rank, world, e2, status, limit);
    if (threadIdx.x == 0) {
      *epoch_ptr = e2;
      __threadfence();
      st_release_sys(grid_sync + 3, e2);
    }
  }
  if (threadIdx.x == 0) wait_flag_ge(grid_sync + 3, e2, status, limit);
}

}  // namespace b200

// peers: host array of `world` heap base pointers (this rank's own base at index `rank`).
// The buffer at buf_off must hold n_elems bf16 (n_elems % 8 == 0) on every rank.
// ctrl: device int[8] in LOCAL memory: [0] epoch, [1..4] grid sync words.  flag_off: heap offset of
// int[MAX_RANKS] arrival slots.
extern "C" int b200_p2p_all_reduce(void* const* peers, int rank, int world, size_t buf_off, size_t flag_off,
                                   int* ctrl, size_t n_elems, int* status, unsigned int spin_limit,
                                   cudaStream_t stream) {
  if (world > MAX_RANKS || n_elems % 8) {
    b200_set_last_error("p2p_all_reduce: world <= 8 and n_elems % 8 == 0 required", __FILE__, __LINE__);
    return -1;
  }
  PeerTable pt;
  for (int i = 0; i < MAX_RANKS; ++i) pt.base[i] = i < world ? (uint8_t*)peers[i] : nullptr;
  size_t nvec = n_elems / 8 / world + 1;
  int blocks = (int)((nvec + 255) / 256);
  if (blocks > 64) blocks = 64;
  if (blocks < 1) blocks = 1;
  p2p_all_reduce_kernel<<<blocks, 256, 0, stream>>>(pt, buf_off, flag_off, ctrl, ctrl + 1, rank, world,
                                                    n_elems, status, spin_limit);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}
