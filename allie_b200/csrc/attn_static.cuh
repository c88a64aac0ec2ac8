// Attention backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for embedders of this
// library that run where cudaMalloc is off limits - inside a host process that has handed its
// whole device memory budget to another allocator, in a plugin whose host only lends it streams
// and buffers, or in a real-time serving loop where an allocation (and the implicit device
// synchronisation it can cause) is not acceptable.  The regular entry point, ab_attn_bwd, asks its caller for a scratch buffer
// (`delta`, one float per (batch, head, position)); this variant keeps that scratch in a
// file-scope __device__ array inside the library instead, so the caller passes only inputs and
// outputs.
#pragma once
#include <cuda_runtime.h>

extern "C" {

// Largest problem the built-in scratch covers: B * H * T <= AB_ATTN_STATIC_MAX_ROWS
// (4 MiB of device memory per GPU that loads the library, held until the process exits).
#define AB_ATTN_STATIC_MAX_ROWS (1 << 20)

// Same contract as ab_attn_bwd (two-kernel backward) minus the `delta` and `dq_acc` arguments.
//
// * Allocates nothing: no cudaMalloc / cudaFree / allocating library call on any path.
// * Returns -10 when B * H * T exceeds AB_ATTN_STATIC_MAX_ROWS; nothing is launched then.
// * The first call on each device resolves the device address of the scratch array
//   (cudaGetSymbolAddress, with that device current) and caches it; make that first call
//   before any stream capture begins.  Host threads may make that first call concurrently: each
//   resolves the same address and the cache entry is an atomic.
// * Every call on a device shares the one scratch array and fully overwrites the part it uses, so
//   nothing needs clearing between calls - but two calls whose kernels overlap on the GPU (different
//   streams, no ordering between them) race on it.  Order such calls yourself.
int ab_attn_bwd_static(const void* qkv, const void* out, const float* lse, const void* dout,
                       void* dqkv, const unsigned int* drop_mask, int B, int T, int H, int hd,
                       float scale, unsigned long long seed, unsigned int stream_id,
                       unsigned int thr16, int* status, cudaStream_t stream);
}
