// Data-parallel gradient path over NVLink / NVSwitch, as kernels that ARE the collectives.
//
// The replicated part of the flat parameter arena is cut into buckets in the order in which the
// backward pass finishes them (last layers first, embeddings last).  Every rank owns 1/N of EACH
// bucket, so a bucket can be reduced as soon as its last weight gradient exists, while earlier
// layers are still running backward:
//
//   nvl_reduce_scatter : one launch per bucket, on a side stream behind an event recorded after the
//                        bucket's last gradient kernel.  Every rank sums its slice of the bucket
//                        across all ranks by loading the peers' arenas directly (plain peer loads,
//                        or one multimem.ld_reduce through the switch), writes the sum back into
//                        its own arena and adds the slice's sum of squares to its partial norm.
//                        128-thread blocks at <= 64 registers: one such block fits beside a
//                        resident persistent GEMM block on every SM, so the reduction shares the
//                        SMs with the backward GEMMs instead of waiting for them.
//   nvl_adamw_allgather: one launch per step, after the last bucket.  Derives the clip coefficient
//                        from all ranks' partial norms (peer loads), runs AdamW on this rank's
//                        slices of all buckets (fp32 master + moments exist only for the slices a
//                        rank owns: optimizer state is sharded N ways) and stores the updated
//                        parameters straight into every rank's arenas (peer stores or multimem.st):
//                        bf16 only for the weight-decayed region (the GEMM weights, which other
//                        ranks only ever read as bf16), fp32 + bf16 for the small rest (biases,
//                        norms, embeddings).  The all-gather is the store itself.
//   nvl_wait           : returns once every peer has delivered its slices of the new parameters.
//
// Ranks synchronise through epoch counters in a small symmetric flag array: a rank releases a
// phase by storing the step's epoch into slot [phase][my_rank] of every peer; a kernel waits for
// a phase by spinning on its LOCAL slots.  Phases: 2b = "bucket b's gradients are final",
// 2b+1 = "I have read bucket b of your gradients and published my partial norm",
// 2*MAX_BUCKETS = "my slices of the new parameters are in your memory".  Every spin is bounded;
// on time-out the kernel writes ST_TIMEOUT_PEER to the status word and returns without touching
// peer memory further, and later kernels of the step see the status and return at once.
// One process per GPU only: these kernels wait on other GPUs, never on another launch of the
// same GPU.
#include "nvl_sync.cuh"

namespace ab {

constexpr int MAX_BUCKETS = 32;
constexpr int PHASE_DELIVERED = 2 * MAX_BUCKETS;

struct RsArgs {
  NvlPeers grads;          // base of every rank's flat fp32 gradient arena
  NvlPeers flags;          // base of every rank's flag array
  const float* mc_grads;   // multicast alias of the gradient arena or null
  float* norm_part;        // local [2] partial sums of squares (symmetric memory)
  unsigned int* ticket;    // local counter, zero between launches
  long long shard_off, shard_n;   // this rank's slice of the bucket, in floats (multiples of 4)
  int rank, world;
  uint32_t epoch;
  int bucket;              // flag phases 2*bucket and 2*bucket+1
  int zero_idle;           // first bucket of a step: recycle the norm slot of the other parity
  int* status;
};

// "My gradients of this bucket are final" -> peers; wait until everyone's are.  One warp, launched
// right before the bucket's reduce-scatter kernel on the same stream: the wait for the slowest rank
// is then held by 32 threads on one SM.  (When the reduce-scatter blocks did this wait themselves,
// one block per SM sat resident for as long as the ranks were apart; with its registers taken, an
// SM holds one LayerNorm-backward block instead of two, so every bucket cost the backward pass the
// skew between the ranks.)
__global__ void __launch_bounds__(32)
nvl_bucket_sync_kernel(const NvlPeers flags, int bucket, int rank, int world, uint32_t epoch, int* status) {
  if (*reinterpret_cast<volatile int*>(status) != 0) return;     // an earlier wait of this step ran out
  signal_phase(flags, 2 * bucket, rank, world, epoch);
  wait_phase(static_cast<const uint32_t*>(flags.ptr[rank]), 2 * bucket, world, epoch, status);
}

__global__ void __launch_bounds__(128, 8)
nvl_reduce_scatter_kernel(const RsArgs a) {
  // the bucket's sync kernel ran before this one; if its wait (or an earlier one) ran out, stop here
  if (*reinterpret_cast<volatile int*>(a.status) != 0) return;
  if (blockIdx.x == 0 && threadIdx.x == 0 && a.zero_idle) a.norm_part[(a.epoch + 1) & 1] = 0.f;
  float ss = 0.f;
  float* mine = static_cast<float*>(a.grads.ptr[a.rank]) + a.shard_off;
  const long long n4 = a.shard_n >> 2;
  // four independent 16-byte reductions in flight per thread: one NVLink round trip is several
  // microseconds, so a single outstanding load per thread leaves the links half idle
  constexpr int RS_UNROLL = 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < n4; i0 += stride * RS_UNROLL) {
    float4 s[RS_UNROLL];
    if (a.mc_grads) {
#pragma unroll
      for (int u = 0; u < RS_UNROLL; ++u) {
        const long long i = i0 + u * stride;
        s[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) s[u] = multimem_ld_reduce_f4(a.mc_grads + a.shard_off + i * 4);
      }
    } else {
#pragma unroll
      for (int u = 0; u < RS_UNROLL; ++u) s[u] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int p = 0; p < MAX_RANKS; ++p)
        if (p < a.world) {
          // start with the next rank so the peers' links are loaded evenly
          const int src = (a.rank + 1 + p) % a.world;
          const float* base = static_cast<const float*>(a.grads.ptr[src]) + a.shard_off;
#pragma unroll
          for (int u = 0; u < RS_UNROLL; ++u) {
            const long long i = i0 + u * stride;
            if (i >= n4) continue;
            const float4 v = ld_relaxed_sys_f4(base + i * 4);
            s[u].x += v.x; s[u].y += v.y; s[u].z += v.z; s[u].w += v.w;
          }
        }
    }
#pragma unroll
    for (int u = 0; u < RS_UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i >= n4) continue;
      reinterpret_cast<float4*>(mine)[i] = s[u];
      ss += s[u].x * s[u].x + s[u].y * s[u].y + s[u].z * s[u].z + s[u].w * s[u].w;
    }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  __shared__ float red[32];
  __shared__ unsigned int s_last;
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
    atomicAdd(&a.norm_part[a.epoch & 1], t);
    __threadfence();
    s_last = (atomicAdd(a.ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  // "I have read this bucket of your gradients and my partial norm includes it"
  if (s_last) {
    if (threadIdx.x == 0) *a.ticket = 0;
    signal_phase(a.flags, 2 * a.bucket + 1, a.rank, a.world, a.epoch);
  }
}

struct AgArgs {
  NvlPeers master;         // every rank's flat fp32 master arena
  NvlPeers shadow;         // every rank's flat bf16 shadow arena
  NvlPeers flags;
  NvlPeers norm_parts;     // every rank's norm_part[2]
  float* mc_master;        // multicast aliases or null
  void* mc_shadow;
  const float* grad;       // local gradient arena (summed slices inside)
  float* exp_avg;          // local, all of this rank's slices back to back
  float* exp_avg_sq;
  unsigned int* ticket;
  int nb;                               // buckets
  long long s_off[MAX_BUCKETS];         // arena offset of this rank's slice of bucket b
  long long s_n[MAX_BUCKETS];           // its length (multiple of 4, may be 0)
  long long hend[MAX_BUCKETS];          // arena offset where bucket b's bf16-only part ends (<= dend)
  long long dend[MAX_BUCKETS];          // arena offset where bucket b's weight-decayed part ends
  long long m_off[MAX_BUCKETS];         // offset of the slice inside exp_avg / exp_avg_sq
  int rank, world;
  uint32_t epoch;
  float lr, beta1, beta2, eps, wd, bc1, bc2_sqrt, max_norm, grad_scale;
  float* total_norm_sq;    // optional out: the global sum of squares (for rank-local parameters)
  int* status;
};

__global__ void __launch_bounds__(512)
nvl_adamw_allgather_kernel(const AgArgs a) {
  if (*reinterpret_cast<volatile int*>(a.status) != 0) return;
  // side-stream launches of a rank run in bucket order, so the last bucket's "read" flag covers all
  if (!wait_phase(static_cast<const uint32_t*>(a.flags.ptr[a.rank]), 2 * (a.nb - 1) + 1, a.world,
                  a.epoch, a.status))
    return;
  __shared__ float s_clip;
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int p = 0; p < a.world; ++p) {
      float v;
      const float* src = static_cast<const float*>(a.norm_parts.ptr[p]) + (a.epoch & 1);
      asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(src) : "memory");
      tot += v;
    }
    if (a.total_norm_sq && blockIdx.x == 0) *a.total_norm_sq = tot;
    float clip = a.grad_scale;
    if (a.max_norm > 0.f) {
      const float norm = sqrtf(tot) * a.grad_scale;
      const float c = a.max_norm / (norm + 1e-6f);
      if (c < 1.f) clip *= c;
    }
    s_clip = clip;
  }
  __syncthreads();
  const float clip = s_clip;
  const float step = a.lr / a.bc1;
  float* my_master = static_cast<float*>(a.master.ptr[a.rank]);
  for (int b = 0; b < a.nb; ++b) {
    const long long n4 = a.s_n[b] >> 2;
    float* mom1 = a.exp_avg + a.m_off[b];
    float* mom2 = a.exp_avg_sq + a.m_off[b];
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
      const long long gi = a.s_off[b] + i * 4;     // index in the flat arena
      const bool decayed = gi < a.dend[b];
      const bool half_only = gi < a.hend[b];   // other ranks read this parameter only as bf16
      const float decay = decayed ? 1.f - a.lr * a.wd : 1.f;
      const float4 p4 = *reinterpret_cast<const float4*>(my_master + gi);
      const float4 g4 = *reinterpret_cast<const float4*>(a.grad + gi);
      const float4 m4 = reinterpret_cast<const float4*>(mom1)[i];
      const float4 v4 = reinterpret_cast<const float4*>(mom2)[i];
      float pe[4] = {p4.x, p4.y, p4.z, p4.w}, ge[4] = {g4.x, g4.y, g4.z, g4.w};
      float me[4] = {m4.x, m4.y, m4.z, m4.w}, ve[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float g = ge[j] * clip;
        pe[j] *= decay;
        me[j] = a.beta1 * me[j] + (1.f - a.beta1) * g;
        ve[j] = a.beta2 * ve[j] + (1.f - a.beta2) * g * g;
        pe[j] -= step * me[j] / (sqrtf(ve[j]) / a.bc2_sqrt + a.eps);
      }
      reinterpret_cast<float4*>(mom1)[i] = make_float4(me[0], me[1], me[2], me[3]);
      reinterpret_cast<float4*>(mom2)[i] = make_float4(ve[0], ve[1], ve[2], ve[3]);
      const float4 pn = make_float4(pe[0], pe[1], pe[2], pe[3]);
      uint2 pb;
      pb.x = pack_bf16x2(pe[0], pe[1]);
      pb.y = pack_bf16x2(pe[2], pe[3]);
      // GEMM weights: the other ranks only read their bf16 copy, so the fp32 master stays with
      // its owner (gathered on demand for checkpoints)
      if (half_only) *reinterpret_cast<float4*>(my_master + gi) = pn;
      if (a.mc_master) {
        if (!half_only) multimem_st_f4(a.mc_master + gi, pn);
        multimem_st_u2(static_cast<__nv_bfloat16*>(a.mc_shadow) + gi, pb);
      } else {
#pragma unroll
        for (int p = 0; p < MAX_RANKS; ++p)
          if (p < a.world) {
            const int dst = (a.rank + p) % a.world;
            if (!half_only) *reinterpret_cast<float4*>(static_cast<float*>(a.master.ptr[dst]) + gi) = pn;
            *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(a.shadow.ptr[dst]) + gi) = pb;
          }
      }
    }
  }
  __shared__ unsigned int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = (atomicAdd(a.ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  // "my slices of the new parameters are in your memory"
  if (s_last) {
    if (threadIdx.x == 0) *a.ticket = 0;
    signal_phase(a.flags, PHASE_DELIVERED, a.rank, a.world, a.epoch);
  }
}

__global__ void nvl_wait_kernel(const uint32_t* local_flags, int phase, int world, uint32_t epoch,
                                int* status) {
  wait_phase(local_flags, phase, world, epoch, status);
}

}  // namespace ab

extern "C" {

int ab_nvl_max_buckets() { return ab::MAX_BUCKETS; }
int ab_nvl_flag_words() { return (ab::PHASE_DELIVERED + 1) * ab::FLAG_STRIDE; }
int ab_nvl_phase_delivered() { return ab::PHASE_DELIVERED; }

// One bucket: `shard_off` / `shard_n` are this rank's slice of it.  `grid` blocks of 128 threads
// (148 = one per SM shares the SMs with a running persistent GEMM; more when nothing else runs).
int ab_nvl_reduce_scatter(void* const* grad_ptrs, void* const* flag_ptrs, const float* mc_grads,
                          float* norm_part, unsigned int* ticket, long long shard_off,
                          long long shard_n, int rank, int world, unsigned int epoch, int bucket,
                          int zero_idle, int grid, int* status, cudaStream_t stream) {
  using namespace ab;
  if (world < 1 || world > MAX_RANKS || (shard_off & 3) || (shard_n & 3) || bucket < 0 ||
      bucket >= MAX_BUCKETS || grid < 1)
    return -1;
  RsArgs a;
  for (int i = 0; i < MAX_RANKS; ++i) {
    a.grads.ptr[i] = i < world ? grad_ptrs[i] : nullptr;
    a.flags.ptr[i] = i < world ? flag_ptrs[i] : nullptr;
  }
  a.mc_grads = mc_grads; a.norm_part = norm_part; a.ticket = ticket; a.shard_off = shard_off;
  a.shard_n = shard_n; a.rank = rank; a.world = world; a.epoch = epoch; a.bucket = bucket;
  a.zero_idle = zero_idle; a.status = status;
  nvl_bucket_sync_kernel<<<1, 32, 0, stream>>>(a.flags, bucket, rank, world, epoch, status);
  nvl_reduce_scatter_kernel<<<grid, 128, 0, stream>>>(a);
  return (int)cudaGetLastError();
}

int ab_nvl_adamw_allgather(void* const* master_ptrs, void* const* shadow_ptrs,
                           void* const* flag_ptrs, void* const* norm_ptrs, float* mc_master,
                           void* mc_shadow, const float* grad, float* exp_avg, float* exp_avg_sq,
                           unsigned int* ticket, int nb, const long long* s_off,
                           const long long* s_n, const long long* hend, const long long* dend,
                           const long long* m_off,
                           int rank, int world, unsigned int epoch, float lr,
                           float beta1, float beta2, float eps, float wd, int step, float max_norm,
                           float grad_scale, float* total_norm_sq, int* status, cudaStream_t stream) {
  using namespace ab;
  if (world < 1 || world > MAX_RANKS || nb < 1 || nb > MAX_BUCKETS) return -1;
  AgArgs a;
  for (int i = 0; i < MAX_RANKS; ++i) {
    a.master.ptr[i] = i < world ? master_ptrs[i] : nullptr;
    a.shadow.ptr[i] = i < world ? shadow_ptrs[i] : nullptr;
    a.flags.ptr[i] = i < world ? flag_ptrs[i] : nullptr;
    a.norm_parts.ptr[i] = i < world ? norm_ptrs[i] : nullptr;
  }
  a.nb = nb;
  for (int b = 0; b < MAX_BUCKETS; ++b) {
    a.s_off[b] = b < nb ? s_off[b] : 0; a.s_n[b] = b < nb ? s_n[b] : 0;
    a.hend[b] = b < nb ? hend[b] : 0;
    a.dend[b] = b < nb ? dend[b] : 0; a.m_off[b] = b < nb ? m_off[b] : 0;
    if ((a.s_off[b] & 3) || (a.s_n[b] & 3) || (a.m_off[b] & 3) || (a.dend[b] & 3) || (a.hend[b] & 3)) return -1;
  }
  a.mc_master = mc_master; a.mc_shadow = mc_shadow; a.grad = grad; a.exp_avg = exp_avg;
  a.exp_avg_sq = exp_avg_sq; a.ticket = ticket;
  a.rank = rank; a.world = world; a.epoch = epoch; a.lr = lr;
  a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2_sqrt = sqrtf(1.f - powf(beta2, (float)step));
  a.max_norm = max_norm; a.grad_scale = grad_scale; a.total_norm_sq = total_norm_sq; a.status = status;
  nvl_adamw_allgather_kernel<<<148 * 2, 512, 0, stream>>>(a);
  return (int)cudaGetLastError();
}

int ab_nvl_wait(const void* local_flags, int phase, int world, unsigned int epoch, int* status,
                cudaStream_t stream) {
  ab::nvl_wait_kernel<<<1, 32, 0, stream>>>((const uint32_t*)local_flags, phase, world, epoch,
                                            status);
  return (int)cudaGetLastError();
}
}
