// Expert-parallel mixture-of-experts: routing, dispatch and combine as kernels that write peer
// memory directly (no all-to-all library call).  The expert projections themselves are the grouped
// tcgen05 GEMM of gemm_grouped.cu, which waits for arriving rows tile by tile and scatters the
// down projection's rows back to their source ranks from its epilogue.
//
// Layout on the rank that owns local expert `le`: rows [le*cap_e, (le+1)*cap_e) of the receive
// buffers, filled densely from the bottom, one contiguous segment per source rank in rank order.
//
//   moe_route_plan_dispatch   ONE kernel behind the router GEMM: (a) softmax over experts, top-2,
//                      normalised gates, per-expert counts and probability sums; (b) the last block
//                      to finish routing adds the layer's load-balance loss, publishes this rank's
//                      counts into every peer's count matrix, waits for everybody's, and derives
//                      where this rank's rows go in each destination (send_off) and how many rows
//                      each local expert receives; (c) one warp per (token, choice) claims the next
//                      free row of its segment, stores the token's activation row straight into the
//                      destination rank's receive buffer together with a return address, and
//                      increments that rank's arrival counter of the 128-row block (release).
//   moe_combine        waits for every rank's scattered expert outputs, then
//                      out = residual + dropout(sum_k gate_k * y_k)   (un-permute is implicit)
//   backward mirrors   moe_combine_bwd_dispatch (gate gradients + gate-weighted rows to the
//                      experts, again with arrival counters; also clears the padding rows of the
//                      local gradient buffer), moe_router_bwd (gate / load-balance gradients ->
//                      d logits) and moe_dx_sum (waits for the scattered input gradients).
// Every cross-GPU wait is an epoch flag or an arrival counter with a bounded spin (nvl_sync.cuh).
#include "nvl_sync.cuh"

namespace ab {

constexpr int MOE_K = 2;

// --------------------------------------------------------------- route + plan + dispatch
__device__ __forceinline__ void red_release_sys_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct RpdArgs {
  // routing
  const float* logits;   // [M, E] fp32
  int* topi;             // [M*2]
  float* gates;          // [M*2]
  float* probs;          // [M, E]
  int* counts;           // [E]  zero on entry
  float* psum;           // [E]  zero on entry
  float* aux_total;      // += E * sum_e (counts_e / (2 M)) * (psum_e / M)
  // plan
  NvlPeers all_counts;   // every rank's [R][E] int matrix (row s = counts sent by rank s)
  NvlPeers flags;
  int* send_off;         // [E]  offset of my segment inside expert e's region on its owner
  int* rows_local;       // [El] rows received per local expert (clipped to cap_e)
  int* rows_pad;         // [El] the same rounded up to 128
  int* cursor;           // [E]  zeroed here (dispatch claims rows through it)
  int* overflow;         // set to 1 when some expert received more than cap_e rows
  unsigned int* ready_fwd_local;   // my arrival counters, zeroed here: El*cap_e/128 each
  unsigned int* ready_bwd_local;
  unsigned int* ticket;  // zero between launches
  unsigned int* go;      // local: set to `epoch` once the plan is ready
  // dispatch
  NvlPeers xr;           // every rank's receive buffer [El*cap_e, d] bf16
  NvlPeers ret;          // every rank's return-address buffer [El*cap_e] int
  NvlPeers ready_fwd;    // every rank's forward arrival counters
  const __nv_bfloat16* x;   // my tokens [M, d]
  int* dest;             // [M*2] out: (rank << 24) | row, or -1 when dropped
  int M, E, El, R, rank, cap_e, d, phase;
  uint32_t epoch;
  int* status;
};

// one warp per token; E <= 128
__device__ __forceinline__ void route_token(const RpdArgs& a, int t, int lane, int* s_cnt, float* s_ps) {
  const int E = a.E;
  float v[4], mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? a.logits[static_cast<long long>(t) * E + e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) { v[i] = (lane + 32 * i) < E ? __expf(v[i] - mx) : 0.f; s += v[i]; }
#pragma unroll
  for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const float inv = 1.f / s;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[i] *= inv;
    const int e = lane + 32 * i;
    if (e < E) {
      a.probs[static_cast<long long>(t) * E + e] = v[i];
      atomicAdd(&s_ps[e], v[i]);
    }
  }
  // top-2: lowest index wins ties (torch.topk order on equal values is unspecified; ties do not
  // occur with real-valued logits)
  int best[MOE_K];
  float bestv[MOE_K];
  float w[4] = {v[0], v[1], v[2], v[3]};
#pragma unroll
  for (int k = 0; k < MOE_K; ++k) {
    float bv = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = lane + 32 * i;
      if (e < E && (w[i] > bv || (w[i] == bv && e < bi))) { bv = w[i]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    best[k] = bi;
    bestv[k] = bv;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (lane + 32 * i == bi) w[i] = -2.f;
  }
  if (lane == 0) {
    const float den = bestv[0] + bestv[1];
    a.topi[t * 2] = best[0];
    a.topi[t * 2 + 1] = best[1];
    a.gates[t * 2] = bestv[0] / den;
    a.gates[t * 2 + 1] = bestv[1] / den;
    atomicAdd(&s_cnt[best[0]], 1);
    atomicAdd(&s_cnt[best[1]], 1);
  }
}

__global__ void __launch_bounds__(256) moe_route_plan_dispatch_kernel(const RpdArgs a) {
  __shared__ int s_cnt[128];
  __shared__ float s_ps[128];
  __shared__ unsigned int s_last;
  __shared__ int s_go;
  const int lane = threadIdx.x & 31;
  const int warp_g = blockIdx.x * 8 + (threadIdx.x >> 5), n_warps = gridDim.x * 8;
  // ---- (a) routing
  if (threadIdx.x < 128) { s_cnt[threadIdx.x] = 0; s_ps[threadIdx.x] = 0.f; }
  __syncthreads();
  for (int t = warp_g; t < a.M; t += n_warps) route_token(a, t, lane, s_cnt, s_ps);
  __syncthreads();
  if (threadIdx.x < a.E) {
    if (s_cnt[threadIdx.x]) atomicAdd(&a.counts[threadIdx.x], s_cnt[threadIdx.x]);
    atomicAdd(&a.psum[threadIdx.x], s_ps[threadIdx.x]);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = (atomicAdd(a.ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  // ---- (b) the last block to finish routing exchanges counts and makes the plan
  if (s_last) {
    __threadfence();
    const int blocks = a.El * a.cap_e / 128;
    for (int i = threadIdx.x; i < blocks; i += blockDim.x) { a.ready_fwd_local[i] = 0u; a.ready_bwd_local[i] = 0u; }
    // load-balance loss of this layer: E * sum_e f_e * P_e
    float part = 0.f;
    if (threadIdx.x < a.E)
      part = (static_cast<float>(__ldcg(a.counts + threadIdx.x)) / (static_cast<float>(a.M) * MOE_K)) *
             (__ldcg(a.psum + threadIdx.x) / static_cast<float>(a.M));
#pragma unroll
    for (int o = 16; o; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0 && threadIdx.x < 128) s_ps[threadIdx.x >> 5] = part;      // routing sums are no longer needed
    __syncthreads();
    if (threadIdx.x == 0) atomicAdd(a.aux_total, a.E * (s_ps[0] + s_ps[1] + s_ps[2] + s_ps[3]));
    // publish my counts row into every peer's matrix
    for (int i = threadIdx.x; i < a.R * a.E; i += blockDim.x) {
      const int r = i / a.E, e = i % a.E;
      int* dst = static_cast<int*>(a.all_counts.ptr[r]) + a.rank * a.E + e;
      asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(__ldcg(a.counts + e)) : "memory");
    }
    __syncthreads();
    signal_phase(a.flags, a.phase, a.rank, a.R, a.epoch);
    const bool ok = wait_phase(static_cast<const uint32_t*>(a.flags.ptr[a.rank]), a.phase, a.R, a.epoch, a.status);
    if (ok) {
      const int* mat = static_cast<const int*>(a.all_counts.ptr[a.rank]);
      for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
        int off = 0;
        for (int sr = 0; sr < a.rank; ++sr) off += __ldcg(mat + sr * a.E + e);
        a.send_off[e] = off;
        a.cursor[e] = 0;
      }
      for (int le = threadIdx.x; le < a.El; le += blockDim.x) {
        int tot = 0;
        for (int sr = 0; sr < a.R; ++sr) tot += __ldcg(mat + sr * a.E + a.rank * a.El + le);
        if (tot > a.cap_e) { tot = a.cap_e; *a.overflow = 1; }
        a.rows_local[le] = tot;
        a.rows_pad[le] = (tot + 127) & ~127;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      *a.ticket = 0;
      __threadfence();
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(a.go), "r"(a.epoch) : "memory");
    }
  }
  // ---- every block waits for the plan (the block that makes it is running by construction)
  if (threadIdx.x == 0) {
    int okg = 1;
    const long long t0 = clock64();
    uint32_t spins = 0, v;
    for (;;) {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a.go) : "memory");
      if (v == a.epoch) break;
      if ((++spins & 0xff) == 0 && clock64() - t0 > 2 * AB_SPIN_CYCLES) {
        okg = 0;
        atomicCAS(a.status, 0, ST_TIMEOUT_MISC);
        break;
      }
    }
    if (*reinterpret_cast<volatile int*>(a.status) != 0) okg = 0;     // the exchange itself ran out
    s_go = okg;
  }
  __syncthreads();
  if (!s_go) return;
  // ---- (c) dispatch: one warp per (token, choice).  A warp first stores all of its rows (lane i
  // remembers the arrival counter of the i-th), then ONE system-scope fence per thread orders every
  // store of the warp before the counter increments that follow: a fence per row would cost more
  // than the row itself.
  unsigned int* my_ctr = nullptr;
  int n_mine = 0;
  for (int slot = warp_g; slot < a.M * MOE_K; slot += n_warps) {
    const int e = a.topi[slot];
    const int r = e / a.El, le = e % a.El;
    int p = 0;
    if (lane == 0) p = atomicAdd(&a.cursor[e], 1);
    p = __shfl_sync(0xffffffffu, p, 0);
    const int off = a.send_off[e] + p;
    if (off >= a.cap_e) {
      if (lane == 0) a.dest[slot] = -1;
      continue;
    }
    const int row = le * a.cap_e + off;
    const uint4* src = reinterpret_cast<const uint4*>(a.x + static_cast<long long>(slot / MOE_K) * a.d);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.xr.ptr[r]) +
                                          static_cast<long long>(row) * a.d);
    for (int c = lane; c < a.d / 8; c += 32) dst[c] = src[c];
    if (lane == 0) {
      static_cast<int*>(a.ret.ptr[r])[row] = (a.rank << 24) | slot;
      a.dest[slot] = (r << 24) | row;
    }
    unsigned int* ctr = static_cast<unsigned int*>(a.ready_fwd.ptr[r]) + row / 128;
    if (n_mine == 32) {              // more than 32 rows per warp: flush what has been collected
      __threadfence_system();
      __syncwarp();
      red_release_sys_add(my_ctr, 1u);
      n_mine = 0;
    }
    if (lane == n_mine) my_ctr = ctr;
    ++n_mine;
  }
  __threadfence_system();
  __syncwarp();
  if (lane < n_mine) red_release_sys_add(my_ctr, 1u);
}

// out[t] = resid[t] + dropout(sum_k gate_k * comb[2t+k]); one warp per token
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ comb, const float* __restrict__ gates,
                   const int* __restrict__ dest, const float* __restrict__ resid,
                   float* __restrict__ out, int M, int d, unsigned long long seed,
                   unsigned int stream_id, unsigned int thr16, const uint32_t* local_flags, int phase,
                   int world, uint32_t epoch, int* status) {
  // every rank's expert GEMM has released `phase` once its rows are in my combine buffer
  if (local_flags && !wait_phase(local_flags, phase, world, epoch, status)) return;
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= M) return;
  const float g0 = dest[2 * t] >= 0 ? gates[2 * t] : 0.f;
  const float g1 = dest[2 * t + 1] >= 0 ? gates[2 * t + 1] : 0.f;
  const uint4* y0 = reinterpret_cast<const uint4*>(comb + static_cast<long long>(2 * t) * d);
  const uint4* y1 = reinterpret_cast<const uint4*>(comb + static_cast<long long>(2 * t + 1) * d);
  const float scale = dropout_scale(thr16);
  for (int c = lane; c < d / 8; c += 32) {
    const uint4 a = g0 != 0.f ? y0[c] : make_uint4(0, 0, 0, 0);
    const uint4 b = g1 != 0.f ? y1[c] : make_uint4(0, 0, 0, 0);
    float v[8] = {g0 * bf16_lo(a.x) + g1 * bf16_lo(b.x), g0 * bf16_hi(a.x) + g1 * bf16_hi(b.x),
                  g0 * bf16_lo(a.y) + g1 * bf16_lo(b.y), g0 * bf16_hi(a.y) + g1 * bf16_hi(b.y),
                  g0 * bf16_lo(a.z) + g1 * bf16_lo(b.z), g0 * bf16_hi(a.z) + g1 * bf16_hi(b.z),
                  g0 * bf16_lo(a.w) + g1 * bf16_lo(b.w), g0 * bf16_hi(a.w) + g1 * bf16_hi(b.w)};
    if (thr16) {
      const uint64_t e0 = static_cast<uint64_t>(t) * d + c * 8;
      const uint32_t keep = dropout_keep8(seed, stream_id, e0 >> 3, thr16);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = ((keep >> j) & 1u) ? v[j] * scale : 0.f;
    }
    const float4 r0 = *reinterpret_cast<const float4*>(resid + static_cast<long long>(t) * d + c * 8);
    const float4 r1 = *reinterpret_cast<const float4*>(resid + static_cast<long long>(t) * d + c * 8 + 4);
    *reinterpret_cast<float4*>(out + static_cast<long long>(t) * d + c * 8) =
        make_float4(v[0] + r0.x, v[1] + r0.y, v[2] + r0.z, v[3] + r0.w);
    *reinterpret_cast<float4*>(out + static_cast<long long>(t) * d + c * 8 + 4) =
        make_float4(v[4] + r1.x, v[5] + r1.y, v[6] + r1.z, v[7] + r1.w);
  }
}

// ------------------------------------------------------------------------------- backward
// per (token, choice): dgate = <dy[t], comb[slot]>, and the row gate*dy[t] goes to the expert's
// gradient buffer at the same row the forward pass used
struct BwdDispatchArgs {
  NvlPeers dyr;          // every rank's [El*cap_e, d] bf16 output-gradient buffer
  NvlPeers ready_bwd;    // every rank's backward arrival counters (one per 128 rows)
  __nv_bfloat16* dyr_local;    // my own gradient buffer: its padding rows are cleared here
  const int* rows_local;       // [El]
  const int* rows_pad;         // [El]
  int El, cap_e;
  const __nv_bfloat16* dy;     // [M, d] gradient of the layer output (dropout mask already applied)
  const __nv_bfloat16* comb;   // [M*2, d] forward expert outputs
  const float* gates;
  const int* dest;
  float* dgate;          // [M*2]
  int M, d, rank, R;
};

__global__ void __launch_bounds__(256) moe_combine_bwd_dispatch_kernel(const BwdDispatchArgs a) {
  const int lane = threadIdx.x & 31;
  // rows [rows_local, rows_pad) of every local expert take part in the weight-gradient
  // contraction (it runs over whole 128-row blocks): they must be zero.  Nobody else writes them.
  for (int le = 0; le < a.El; ++le) {
    const int r0 = a.rows_local[le], r1 = min(a.rows_pad[le], a.cap_e);
    const long long n8 = static_cast<long long>(r1 - r0) * (a.d / 8);
    uint4* base = reinterpret_cast<uint4*>(a.dyr_local + (static_cast<long long>(le) * a.cap_e + r0) * a.d);
    for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n8; i += gridDim.x * 256ll)
      base[i] = make_uint4(0, 0, 0, 0);
  }
  // one warp per (token, choice), warp-stride; the arrival counters are incremented after ONE
  // system-scope fence per thread at the end (see the forward dispatch)
  const int warp_g = blockIdx.x * 8 + (threadIdx.x >> 5), n_warps = gridDim.x * 8;
  unsigned int* my_ctr = nullptr;
  int n_mine = 0;
  for (int slot = warp_g; slot < a.M * MOE_K; slot += n_warps) {
    const int de = a.dest[slot];
    float dot = 0.f;
    if (de >= 0) {
      const int r = de >> 24, row = de & 0xffffff;
      const float g = a.gates[slot];
      const uint4* dyv = reinterpret_cast<const uint4*>(a.dy + static_cast<long long>(slot / MOE_K) * a.d);
      const uint4* yv = reinterpret_cast<const uint4*>(a.comb + static_cast<long long>(slot) * a.d);
      uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.dyr.ptr[r]) +
                                            static_cast<long long>(row) * a.d);
      for (int c = lane; c < a.d / 8; c += 32) {
        const uint4 u = dyv[c], y = yv[c];
        const float f[8] = {bf16_lo(u.x), bf16_hi(u.x), bf16_lo(u.y), bf16_hi(u.y),
                            bf16_lo(u.z), bf16_hi(u.z), bf16_lo(u.w), bf16_hi(u.w)};
        dot += f[0] * bf16_lo(y.x) + f[1] * bf16_hi(y.x) + f[2] * bf16_lo(y.y) + f[3] * bf16_hi(y.y) +
               f[4] * bf16_lo(y.z) + f[5] * bf16_hi(y.z) + f[6] * bf16_lo(y.w) + f[7] * bf16_hi(y.w);
        uint4 o;
        o.x = pack_bf16x2(g * f[0], g * f[1]); o.y = pack_bf16x2(g * f[2], g * f[3]);
        o.z = pack_bf16x2(g * f[4], g * f[5]); o.w = pack_bf16x2(g * f[6], g * f[7]);
        dst[c] = o;
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) a.dgate[slot] = dot;
    if (de >= 0) {
      if (n_mine == 32) {
        __threadfence_system();
        __syncwarp();
        red_release_sys_add(my_ctr, 1u);
        n_mine = 0;
      }
      if (lane == n_mine) my_ctr = static_cast<unsigned int*>(a.ready_bwd.ptr[de >> 24]) + (de & 0xffffff) / 128;
      ++n_mine;
    }
  }
  __threadfence_system();
  __syncwarp();
  if (lane < n_mine) red_release_sys_add(my_ctr, 1u);
}

// d logits of the router from the gate gradients and the load-balance term; one warp per token.
//   gates g_k = p_k / (p_a + p_b)  ->  dp_k = (dg_k - sum_j dg_j g_j) / (p_a + p_b)
//   aux = coef * E * sum_e f_e * mean_t p_te   ->  dp_te += coef * E * f_e / M
//   dlogits = p * (dp - sum_e p_e dp_e)
__global__ void __launch_bounds__(256)
moe_router_bwd_kernel(const float* __restrict__ probs, const int* __restrict__ topi,
                      const float* __restrict__ gates, const float* __restrict__ dgate,
                      const int* __restrict__ counts, float aux_scale, float grad_scale, int M, int E,
                      __nv_bfloat16* __restrict__ dlogits) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= M) return;
  const int ia = topi[2 * t], ib = topi[2 * t + 1];
  const float ga = gates[2 * t], gb = gates[2 * t + 1];
  const float dga = dgate[2 * t], dgb = dgate[2 * t + 1];
  const float pa = probs[static_cast<long long>(t) * E + ia], pb = probs[static_cast<long long>(t) * E + ib];
  const float den = pa + pb;
  const float mix = dga * ga + dgb * gb;
  float p[4], dp[4], dotp = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int e = lane + 32 * i;
    p[i] = e < E ? probs[static_cast<long long>(t) * E + e] : 0.f;
    dp[i] = 0.f;
    if (e < E) {
      dp[i] = aux_scale * static_cast<float>(counts[e]);      // load-balance term
      if (e == ia) dp[i] += grad_scale * (dga - mix) / den;
      if (e == ib) dp[i] += grad_scale * (dgb - mix) / den;
    }
    dotp += p[i] * dp[i];
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) dotp += __shfl_xor_sync(0xffffffffu, dotp, o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int e = lane + 32 * i;
    if (e < E) dlogits[static_cast<long long>(t) * E + e] = __float2bfloat16(p[i] * (dp[i] - dotp));
  }
}

// dx[t] += sum_k comb[2t+k] (dropped choices contribute nothing); bf16 in place
__global__ void __launch_bounds__(256)
moe_dx_sum_kernel(__nv_bfloat16* __restrict__ dx, const __nv_bfloat16* __restrict__ comb,
                  const int* __restrict__ dest, int M, int d, const uint32_t* local_flags, int phase,
                  int world, uint32_t epoch, int* status) {
  if (local_flags && !wait_phase(local_flags, phase, world, epoch, status)) return;
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= M) return;
  const bool k0 = dest[2 * t] >= 0, k1 = dest[2 * t + 1] >= 0;
  uint4* o = reinterpret_cast<uint4*>(dx + static_cast<long long>(t) * d);
  const uint4* a = reinterpret_cast<const uint4*>(comb + static_cast<long long>(2 * t) * d);
  const uint4* b = reinterpret_cast<const uint4*>(comb + static_cast<long long>(2 * t + 1) * d);
  for (int c = lane; c < d / 8; c += 32) {
    uint4 x = o[c];
    const uint4 u = k0 ? a[c] : make_uint4(0, 0, 0, 0), w = k1 ? b[c] : make_uint4(0, 0, 0, 0);
    x.x = pack_bf16x2(bf16_lo(x.x) + bf16_lo(u.x) + bf16_lo(w.x), bf16_hi(x.x) + bf16_hi(u.x) + bf16_hi(w.x));
    x.y = pack_bf16x2(bf16_lo(x.y) + bf16_lo(u.y) + bf16_lo(w.y), bf16_hi(x.y) + bf16_hi(u.y) + bf16_hi(w.y));
    x.z = pack_bf16x2(bf16_lo(x.z) + bf16_lo(u.z) + bf16_lo(w.z), bf16_hi(x.z) + bf16_hi(u.z) + bf16_hi(w.z));
    x.w = pack_bf16x2(bf16_lo(x.w) + bf16_lo(u.w) + bf16_lo(w.w), bf16_hi(x.w) + bf16_hi(u.w) + bf16_hi(w.w));
    o[c] = x;
  }
}

}  // namespace ab

// ------------------------------------------------------------------------------------ host side
extern "C" {

using ab::NvlPeers;
static void fill_peers(NvlPeers& p, void* const* ptrs, int R) {
  for (int i = 0; i < ab::MAX_RANKS; ++i) p.ptr[i] = i < R ? ptrs[i] : nullptr;
}

int ab_moe_route_plan_dispatch(const float* logits, int* topi, float* gates, float* probs, int* counts,
                               float* psum, float* aux_total, void* const* all_counts, void* const* flags,
                               int* send_off, int* rows_local, int* rows_pad, int* cursor, int* overflow,
                               unsigned int* ready_fwd_local, unsigned int* ready_bwd_local,
                               unsigned int* ticket, unsigned int* go, void* const* xr, void* const* ret,
                               void* const* ready_fwd, const void* x, int* dest, int M, int E, int El, int R,
                               int rank, int cap_e, int d, int phase, unsigned int epoch, int* status,
                               cudaStream_t stream) {
  if (E > 128 || E < 2 || d % 8 || R < 1 || R > ab::MAX_RANKS || E != R * El || cap_e % 128) return -1;
  ab::RpdArgs a;
  a.logits = logits; a.topi = topi; a.gates = gates; a.probs = probs; a.counts = counts; a.psum = psum;
  a.aux_total = aux_total;
  fill_peers(a.all_counts, all_counts, R); fill_peers(a.flags, flags, R);
  a.send_off = send_off; a.rows_local = rows_local; a.rows_pad = rows_pad; a.cursor = cursor;
  a.overflow = overflow; a.ready_fwd_local = ready_fwd_local; a.ready_bwd_local = ready_bwd_local;
  a.ticket = ticket; a.go = go;
  fill_peers(a.xr, xr, R); fill_peers(a.ret, ret, R); fill_peers(a.ready_fwd, ready_fwd, R);
  a.x = (const __nv_bfloat16*)x; a.dest = dest; a.M = M; a.E = E; a.El = El; a.R = R; a.rank = rank;
  a.cap_e = cap_e; a.d = d; a.phase = phase; a.epoch = epoch; a.status = status;
  // every block has to be resident while it waits for the plan: two blocks per SM at most
  int grid = (M * 2 + 7) / 8;
  if (grid > 148 * 2) grid = 148 * 2;
  ab::moe_route_plan_dispatch_kernel<<<grid, 256, 0, stream>>>(a);
  return (int)cudaGetLastError();
}

// `local_flags` (optional): wait until every rank has released `phase` with `epoch` first.
int ab_moe_combine(const void* comb, const float* gates, const int* dest, const float* resid, float* out, int M,
                   int d, unsigned long long seed, unsigned int stream_id, unsigned int thr16,
                   const void* local_flags, int phase, int world, unsigned int epoch, int* status,
                   cudaStream_t stream) {
  if (d % 8) return -1;
  ab::moe_combine_kernel<<<(M + 7) / 8, 256, 0, stream>>>((const __nv_bfloat16*)comb, gates, dest, resid, out, M,
                                                          d, seed, stream_id, thr16,
                                                          (const uint32_t*)local_flags, phase, world, epoch, status);
  return (int)cudaGetLastError();
}

int ab_moe_combine_bwd_dispatch(void* const* dyr, void* const* ready_bwd, void* dyr_local,
                                const int* rows_local, const int* rows_pad, int El, int cap_e,
                                const void* dy, const void* comb, const float* gates, const int* dest,
                                float* dgate, int M, int d, int rank, int R, cudaStream_t stream) {
  if (d % 8 || R < 1 || R > ab::MAX_RANKS) return -1;
  ab::BwdDispatchArgs a;
  fill_peers(a.dyr, dyr, R); fill_peers(a.ready_bwd, ready_bwd, R);
  a.dyr_local = (__nv_bfloat16*)dyr_local; a.rows_local = rows_local; a.rows_pad = rows_pad; a.El = El;
  a.cap_e = cap_e;
  a.dy = (const __nv_bfloat16*)dy; a.comb = (const __nv_bfloat16*)comb; a.gates = gates; a.dest = dest;
  a.dgate = dgate; a.M = M; a.d = d; a.rank = rank; a.R = R;
  int grid = (M * 2 + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  ab::moe_combine_bwd_dispatch_kernel<<<grid, 256, 0, stream>>>(a);
  return (int)cudaGetLastError();
}

int ab_moe_router_bwd(const float* probs, const int* topi, const float* gates, const float* dgate,
                      const int* counts, float aux_scale, float grad_scale, int M, int E, void* dlogits,
                      cudaStream_t stream) {
  if (E > 128) return -1;
  ab::moe_router_bwd_kernel<<<(M + 7) / 8, 256, 0, stream>>>(probs, topi, gates, dgate, counts, aux_scale,
                                                             grad_scale, M, E, (__nv_bfloat16*)dlogits);
  return (int)cudaGetLastError();
}

int ab_moe_dx_sum(void* dx, const void* comb, const int* dest, int M, int d, const void* local_flags, int phase,
                  int world, unsigned int epoch, int* status, cudaStream_t stream) {
  if (d % 8) return -1;
  ab::moe_dx_sum_kernel<<<(M + 7) / 8, 256, 0, stream>>>((__nv_bfloat16*)dx, (const __nv_bfloat16*)comb, dest, M, d,
                                                         (const uint32_t*)local_flags, phase, world, epoch, status);
  return (int)cudaGetLastError();
}
}
