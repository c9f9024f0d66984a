// Split-KV paged decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for users of this
// library who call it from plain C or C++ without a tensor framework: a host process that
// embeds the kernels behind its own serving loop, a plug-in running inside somebody else's
// allocator or memory pool where a hidden cudaMalloc would either fail or break the pool's
// accounting, or a real-time path where an allocation (which may synchronise the device) is
// not acceptable.  The ordinary entry point, b200_attn_decode, asks its caller for a scratch
// buffer and a counter array sized by b200_attn_decode_scratch_bytes; this one brings its own.
//
// Where the scratch lives.  One array of B200_ATTN_STATIC_SCRATCH_BYTES (8 MiB) is part of
// the library's device image (a file-scope __device__ array, 256-byte aligned), so it exists
// once per device from the moment the library's module is loaded there and is never
// allocated or freed by a call.  Its first B200_ATTN_STATIC_COUNTER_BYTES (16 KiB) are the
// per-(request, kv head) arrival counters; the rest holds the per-split partial outputs.
//
// Limits.  With S = num_splits > 1 a call needs
//     num_reqs * Hkv                         <= 4096 counters, and
//     num_reqs * Hkv * S * 16 * (D + 2) * 4  <= 8 MiB - 16 KiB bytes of partials
// (for D = 128 that is num_reqs * Hkv * S <= 1006, e.g. 32 requests x 8 kv heads x 3 splits).
// A call beyond either limit is refused with -1 and a message in b200_get_last_error(); it
// is never silently run with fewer splits.  S = 1 uses no scratch and has no such limit.
//
// Set-up.  The first call on each device looks the array's address up (with that device
// current) and raises the kernel's shared-memory limit; both are one-off host-side calls
// into the CUDA runtime.  Call b200_attn_decode_static_setup() yourself, once per device
// with that device current, before any stream capture or latency-critical section; after
// it a call does nothing but check its arguments and launch the kernel.
//
// Sharing.  Every call on a device uses the same array.  Calls on one stream are ordered
// and safe.  Two calls that may overlap in time (different streams, different host threads
// on different streams) race on the partials and the counters and give wrong results:
// serialise them.  The counters must be zero when a call starts.  They are zero when the
// module is loaded and the kernel puts each one back to zero when it is done with it, so
// back-to-back calls need no clearing; only after a call that did not run to completion
// (a launch error, a device reset by the caller) call b200_attn_decode_static_reset().
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ATTN_STATIC_SCRATCH_BYTES (8u << 20)
#define B200_ATTN_STATIC_COUNTER_BYTES (16u << 10)

// One-off set-up for the current device.  Returns 0, or -1 with b200_get_last_error() set.
int b200_attn_decode_static_setup(void);

// Zeroes the arrival counters on `stream` (a memset of 16 KiB; no allocation).
int b200_attn_decode_static_reset(cudaStream_t stream);

// Same arguments and result as b200_attn_decode for requests [0, num_reqs), minus the
// scratch and counter pointers.  q [T, Hq, D] bf16, kv [num_blocks, 2, Hkv, block_size, D]
// bf16, out [T, Hq, D] bf16, lse [T, Hq] fp32 or NULL, block_tables [num_reqs, max_blocks],
// seq_lens [num_reqs], qsl [num_reqs + 1]; every request has q_len * (Hq / Hkv) <= 16.
// Returns 0 on success, -1 on a refused or failed call.
int b200_attn_decode_static(const void* q, const void* kv, void* out, float* lse, const int* block_tables,
                            const int* seq_lens, const int* qsl, int num_reqs, int max_blocks,
                            int block_size, long long num_blocks, int Hq, int Hkv, int D, float scale,
                            int window, float softcap, const float* sinks, int num_splits,
                            cudaStream_t stream);

#ifdef __cplusplus
}
#endif
