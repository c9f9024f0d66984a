// Library-wide host helpers: last-error string, device facts, version.
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

static char g_last_error[512] = "";
static std::mutex g_err_mu;

extern "C" void b200_set_last_error(const char* msg, const char* file, int line) {
  std::lock_guard<std::mutex> lock(g_err_mu);
  snprintf(g_last_error, sizeof(g_last_error), "%s (%s:%d)", msg, file, line);
}

extern "C" const char* b200_get_last_error() { return g_last_error; }

extern "C" int b200_version() { return 1; }

// Programmatic dependent launch: kernels launched through launch_pdl() may start while the previous
// kernel of the stream drains (they call griddepcontrol.wait before touching its results).
static int g_b200_pdl = 1;
extern "C" int b200_pdl_enabled() { return g_b200_pdl; }
extern "C" void b200_set_pdl(int on) { g_b200_pdl = on ? 1 : 0; }

extern "C" int b200_device_info(int device, int* sms, int* cc_major, int* cc_minor, size_t* smem_optin) {
  cudaDeviceProp prop;
  B200_CUDA_CHECK(cudaGetDeviceProperties(&prop, device));
  *sms = prop.multiProcessorCount;
  *cc_major = prop.major;
  *cc_minor = prop.minor;
  *smem_optin = prop.sharedMemPerBlockOptin;
  return 0;
}

// Write a buffer larger than L2 so that the next timed kernel starts cold.
__global__ void b200_fill_kernel(float4* p, size_t n, float v) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    p[i] = make_float4(v, v, v, v);
}
extern "C" int b200_flush_l2(void* buf, size_t bytes, cudaStream_t stream) {
  b200_fill_kernel<<<148 * 8, 256, 0, stream>>>((float4*)buf, bytes / 16, 0.f);
  B200_CUDA_CHECK(cudaGetLastError());
  return 0;
}
