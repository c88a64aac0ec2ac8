// Cross-GPU synchronisation primitives shared by the NVLink kernels (gradient path, MoE
// dispatch/combine): peer pointer tables, system-scope flag stores/loads, and epoch-based phase
// flags with bounded waits.  A rank releases phase p of step `epoch` by storing `epoch` into slot
// [p][my_rank] of every peer's flag array; a kernel waits for phase p by spinning on its LOCAL
// slots until all of them reach `epoch`.  Waits give up after AB_SPIN_CYCLES and report
// ST_TIMEOUT_PEER through the status word.
#pragma once
#include "ptx.cuh"

namespace ab {

constexpr int MAX_RANKS = 8;
constexpr int FLAG_STRIDE = 32;   // uint32 slots per phase (>= MAX_RANKS, keeps phases on separate lines)

struct NvlPeers {
  void* ptr[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_relaxed_sys_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_f4(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x),
               "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void multimem_st_u2(void* mc, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)) : "memory");
}

// Block-wide bounded wait until all `world` local slots of a phase reach `epoch`.
// Returns false on time-out.  Must be called by all threads of the block.
__device__ __forceinline__ bool wait_phase(const uint32_t* local_flags, int phase, int world,
                                           uint32_t epoch, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    const uint32_t* slot = local_flags + phase * FLAG_STRIDE + threadIdx.x;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(slot) - epoch) < 0) {
      if ((++spins & 0xff) == 0 && clock64() - t0 > AB_SPIN_CYCLES) {
        s_ok = 0;
        atomicCAS(status, 0, ST_TIMEOUT_PEER);
        break;
      }
    }
  }
  __syncthreads();
  return s_ok != 0;
}

// Called by one thread per rank slot of ONE block: release `phase` to every peer.
__device__ __forceinline__ void signal_phase(const NvlPeers& flags, int phase, int rank, int world,
                                             uint32_t epoch) {
  if (threadIdx.x < world) {
    __threadfence_system();
    uint32_t* slot = static_cast<uint32_t*>(flags.ptr[threadIdx.x]) + phase * FLAG_STRIDE + rank;
    st_release_sys(slot, epoch);
  }
}


}  // namespace ab
