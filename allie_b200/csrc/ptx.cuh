// Thin inline-PTX wrappers for the Blackwell (sm_100a) execution model:
// mbarrier, TMA (cp.async.bulk.tensor, never with cluster multicast), tcgen05
// (TMEM allocation, UMMA issue, commit, TMEM loads) and the descriptor
// encodings they need.  Every wait in here is bounded: it gives up after a
// clock budget and reports failure so the caller can set a status word and
// leave the kernel cleanly instead of spinning forever.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace ab {

// A kernel attribute (dynamic shared memory limit, carve-out) belongs to one device's copy of the
// kernel, so "already set" is kept per device: one bit per device ordinal in a mask that each call
// site owns.  first_use_on_device() returns true until mark_device() was called on this device.
struct PerDeviceOnce {
  std::atomic<unsigned long long> mask{0};
  unsigned long long bit() const {
    int dev = 0;
    cudaGetDevice(&dev);
    return 1ull << (dev & 63);
  }
  bool first_use_on_device() const { return !(mask.load(std::memory_order_acquire) & bit()); }
  void mark_device() { mask.fetch_or(bit(), std::memory_order_release); }
};

// ---------------------------------------------------------------- status ---
// Kernels report trouble through a device status word owned by the host
// wrapper (never by trapping).  0 means success.
enum StatusCode : int {
  ST_OK = 0,
  ST_TIMEOUT_FULL = 1,      // consumer waited too long for a TMA stage
  ST_TIMEOUT_EMPTY = 2,     // producer waited too long for a free stage
  ST_TIMEOUT_TMEM_FULL = 3, // epilogue waited too long for an accumulator
  ST_TIMEOUT_TMEM_EMPTY = 4,// MMA warp waited too long for a drained accumulator
  ST_TIMEOUT_PEER = 5,      // wait on a flag written by another GPU ran out
  ST_TIMEOUT_MISC = 6,
  ST_BAD_ARGUMENT = 7,
};

// Spin budget in SM clock cycles (about one second at 1.9 GHz).
#ifndef AB_SPIN_CYCLES
#define AB_SPIN_CYCLES (2000000000ll)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// -------------------------------------------------------------- mbarrier ---
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok;
}
// Same test, but the thread may stay suspended for up to `hint_ns` nanoseconds waiting for the
// phase to complete before the instruction returns (it wakes as soon as the phase completes), so a
// polling loop around it issues far fewer instructions.
__device__ __forceinline__ uint32_t mbar_try_wait_suspend(uint64_t* bar, uint32_t parity,
                                                          uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok;
}
#ifndef AB_MBAR_SUSPEND_NS
#define AB_MBAR_SUSPEND_NS 2000u
#endif
// Bounded wait.  Returns false when the budget ran out (or another thread of
// the CTA has already raised `*abort_flag`).  `sleep_ns` > 0 puts the thread to sleep between
// polls: for waits with slack (an epilogue waiting for the next accumulator, a producer waiting
// for a free stage) this keeps the polling warps out of the issue slots and the power budget.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
                                          volatile int* abort_flag, uint32_t sleep_ns = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait_suspend(bar, parity, AB_MBAR_SUSPEND_NS)) {
    if (sleep_ns) __nanosleep(sleep_ns);
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > AB_SPIN_CYCLES) return false;
    }
  }
  return true;
}

// Makes generic-proxy writes to shared memory visible to the async proxy
// (TMA, tcgen05.mma operand fetch).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------- programmatic dependent launch ---
// A kernel launched with the programmatic-stream-serialization attribute may start while the
// kernel before it in the stream is still running (once that kernel has executed
// griddep_launch_dependents in every CTA, or has exited).  It must call griddep_wait before it
// touches anything the earlier kernel produces or still reads; what it does before that (barrier
// set-up, TMEM allocation, prefetch of weights) overlaps the earlier kernel.  Both instructions
// are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void griddep_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void griddep_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// First statement of a kernel that can be a link of a programmatic chain (the captured training
// micro-step): lets the kernel behind it in the stream become resident as this one drains, then
// waits for the kernel before it.  Everything the kernel reads or writes comes after this.
__device__ __forceinline__ void griddep_enter() {
  if (threadIdx.x == 0) griddep_launch_dependents();
  griddep_wait();
}

// Host side: launches made through launch_chained carry the programmatic-stream-serialization
// attribute while g_pdl_chain is set (only around the capture of a training micro-step; defined in
// embed.cu).  Every kernel launched this way starts with griddep_enter() or, for the GEMMs, does
// its set-up first and then waits.
extern int g_pdl_chain;
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  if (g_pdl_chain) {
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ------------------------------------------------------------------- TMA ---
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load global -> shared, completion counted on `bar` in bytes.
// x is the innermost (contiguous) coordinate and must be a multiple of
// 16 bytes / element size.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x),
      "r"(y)
      : "memory");
}
// 2-D tiled store shared -> global (bulk async group).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(x), "r"(y)
               : "memory");
}
// 2-D tiled reduction shared -> global: global[tile] += smem[tile] (fp32 add, bulk async group).
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* m, const void* src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// --------------------------------------------------------------- tcgen05 ---
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Whole-warp calls.  ncols: power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` once every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          smem_u32(bar))
      : "memory");
}
// Each thread of the warp reads 32 consecutive fp32 columns of its own TMEM
// lane (lane = 32 * (warp_id % 4) + lane_id, encoded in taddr bits 31..16).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ------------------------------------------------- CTA pairs (cta_group::2) ---
// Two CTAs of a cluster (ranks 0 and 1) act as one MMA unit: the leader (rank 0) issues
// tcgen05.mma for both, each CTA stages its own half of A (rows) and of B (columns) in its own
// shared memory and owns 128 lanes of the accumulator in its own TMEM.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t cta_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 2-D tiled load into this CTA's shared memory whose completion bytes are counted on a barrier
// that may live in the partner CTA (`bar_cluster_addr` from mapa_shared).  Plain unicast load.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* m,
                                                 uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x),
      "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at `bar_cluster_addr` (either CTA of the pair) once every pair MMA issued
// so far by this thread is done.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          bar_cluster_addr)
      : "memory");
}

// ----------------------------------------------------------- descriptors ---
// Shared-memory matrix descriptor for 128-byte-swizzled bf16 tiles (the layout
// a TMA load with CU_TENSOR_MAP_SWIZZLE_128B produces).  Field positions:
// start>>4 [0,14), LBO>>4 [16,30), SBO>>4 [32,46), version=1 [46,48),
// layout type [61,64) with 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t make_sdesc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                     uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// Instruction descriptor for kind::f16 with bf16 A/B and fp32 accumulator.
// a_mn / b_mn: operand is MN-major (1) rather than K-major (0).
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, int a_mn, int b_mn) {
  return (1u << 4)      // D format fp32
         | (1u << 7)    // A format bf16
         | (1u << 10)   // B format bf16
         | (static_cast<uint32_t>(a_mn) << 15) | (static_cast<uint32_t>(b_mn) << 16) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

// ------------------------------------------------------------------ misc ---
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// gelu_new (tanh form) and its derivative.
// GELU (tanh form) and its derivative, written for the fewest issue slots: the GEMM epilogues that
// use them are bound by instruction issue.  With u = k0 (x + k1 x^3) = x (k0 + k0 k1 x^2), t = tanh u:
//   gelu(x)  = 0.5 x (1 + t)                      = fma(h, t, h),  h = 0.5 x          (6 operations)
//   gelu'(x) = 0.5 (1 + t) + 0.5 x (1 - t^2) u'   with u' = k0 + 3 k0 k1 x^2          (10 operations)
constexpr float GELU_K0 = 0.7978845608028654f;
constexpr float GELU_K01 = 0.7978845608028654f * 0.044715f;
__device__ __forceinline__ float gelu_tanh(float x) {
  const float t = tanh_fast(x * fmaf(GELU_K01, x * x, GELU_K0));
  const float h = 0.5f * x;
  return fmaf(h, t, h);
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float x2 = x * x;
  const float t = tanh_fast(x * fmaf(GELU_K01, x2, GELU_K0));
  const float dt = fmaf(-t, t, 1.f) * fmaf(3.f * GELU_K01, x2, GELU_K0);
  return fmaf(0.5f * x, dt, fmaf(0.5f, t, 0.5f));
}
// both at once (they share x^2 and the tanh): returns gelu(x), stores gelu'(x)
__device__ __forceinline__ float gelu_tanh_with_grad(float x, float& grad) {
  const float x2 = x * x;
  const float t = tanh_fast(x * fmaf(GELU_K01, x2, GELU_K0));
  const float h = 0.5f * x;
  grad = fmaf(h, fmaf(-t, t, 1.f) * fmaf(3.f * GELU_K01, x2, GELU_K0), fmaf(0.5f, t, 0.5f));
  return fmaf(h, t, h);
}

// ---------------------------------------------------------------- philox ---
// Counter-based generator (Philox4x32, 7 rounds) used for every dropout mask:
// the mask of element i of stream `stream` under `seed` is a pure function of
// (seed, stream, i), so backward kernels regenerate it instead of storing it.
struct Philox4 {
  uint32_t x, y, z, w;
};
__host__ __device__ __forceinline__ uint32_t mulhi32(uint32_t a, uint32_t b) {
#ifdef __CUDA_ARCH__
  return __umulhi(a, b);
#else
  return static_cast<uint32_t>((static_cast<uint64_t>(a) * b) >> 32);
#endif
}
__host__ __device__ __forceinline__ Philox4 philox4x32_7(uint64_t seed, uint32_t stream,
                                                         uint64_t counter) {
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
  uint32_t c0 = static_cast<uint32_t>(counter), c1 = static_cast<uint32_t>(counter >> 32);
  uint32_t c2 = stream, c3 = 0x9E3779B9u;
#pragma unroll
  for (int r = 0; r < 7; ++r) {
    uint32_t hi0 = mulhi32(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    uint32_t hi1 = mulhi32(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return Philox4{c0, c1, c2, c3};
}
// The seed reaches a kernel by value, which a captured CUDA graph would freeze.  Every launcher
// therefore also hands its kernel seed_salt_ptr(): null in ordinary launches (the seed is used as
// it is), or, while a training step is being captured, the address of a device word that the
// graph's first node advances on every replay; kernels key the generator with salted(seed, salt).
extern const unsigned long long* g_seed_salt;       // host variable, defined in embed.cu
inline const unsigned long long* seed_salt_ptr() { return g_seed_salt; }
__device__ __forceinline__ unsigned long long salted(unsigned long long seed,
                                                     const unsigned long long* salt) {
  return salt ? (seed ^ __ldg(salt)) : seed;
}
// Dropout decisions come in groups of eight consecutive elements: element
// index i uses 16 bits of philox(seed, stream, i / 8).  keep iff bits >= thr16.
__host__ __device__ __forceinline__ uint32_t dropout_thr16(float p) {
  float t = p * 65536.f;
  return t <= 0.f ? 0u : (t >= 65535.f ? 65535u : static_cast<uint32_t>(t + 0.5f));
}
__host__ __device__ __forceinline__ float dropout_scale(uint32_t thr16) {
  return 65536.f / static_cast<float>(65536u - thr16);
}
// keep-mask bits (bit j set = keep element 8*group + j)
__host__ __device__ __forceinline__ uint32_t dropout_keep8(uint64_t seed, uint32_t stream,
                                                           uint64_t group, uint32_t thr16) {
  Philox4 r = philox4x32_7(seed, stream, group);
  uint32_t m = 0;
  m |= ((r.x & 0xffffu) >= thr16) << 0;
  m |= ((r.x >> 16) >= thr16) << 1;
  m |= ((r.y & 0xffffu) >= thr16) << 2;
  m |= ((r.y >> 16) >= thr16) << 3;
  m |= ((r.z & 0xffffu) >= thr16) << 4;
  m |= ((r.z >> 16) >= thr16) << 5;
  m |= ((r.w & 0xffffu) >= thr16) << 6;
  m |= ((r.w >> 16) >= thr16) << 7;
  return m;
}

// Host helper: encode a 2-D row-major tensor (rows x cols, `ld` elements
// between rows) for TMA with a (box_cols x box_rows) tile and 128B swizzle.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled();
// Returns 0 on success.
int make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows, uint32_t box_cols, int elem_bytes, bool swizzle128);
// Same with an explicit swizzle span in bytes (0, 32, 64 or 128).
int make_tmap_2d_sw(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                    uint32_t box_rows, uint32_t box_cols, int elem_bytes, int swizzle_bytes);

}  // namespace ab
