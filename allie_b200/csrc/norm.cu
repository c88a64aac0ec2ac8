// LayerNorm / RMSNorm forward and backward for the fp32 residual stream.
//
// forward : x fp32 [M,d] -> y bf16 [M,d] (the A operand of the next GEMM), mean/rstd fp32 [M]
// backward: dy bf16 (+ optional rank-2 term from the scalar heads) -> dx fp32, added to the
//           incoming residual gradient; optionally also emits the bf16, dropout-masked copy of
//           dx that the previous branch's projection GEMMs consume, and accumulates
//           dgamma/dbeta into the fp32 gradient buffers with one atomic per column per block.
// One warp owns one row; a lane owns float4 columns lane*4 + 128*i.
#include "ptx.cuh"

namespace ab {

constexpr int LN_WARPS = 8;

template <int NV_MAX>
__global__ void __launch_bounds__(LN_WARPS * 32)
ln_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
              const float* __restrict__ beta, __nv_bfloat16* __restrict__ y,
              float* __restrict__ mean_out, float* __restrict__ rstd_out, int M, int d, float eps,
              int rms) {
  if (threadIdx.x == 0) griddep_launch_dependents();   // a dependent GEMM may start fetching its weights
  griddep_wait();       // launched as a dependent itself: x comes from the kernel before (no-op otherwise)

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nv = d >> 7;  // float4 per lane
  for (int row = blockIdx.x * LN_WARPS + warp; row < M; row += gridDim.x * LN_WARPS) {
    const float4* xr = reinterpret_cast<const float4*>(x + (long long)row * d);
    float4 v[NV_MAX];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV_MAX; ++i)
      if (i < nv) {
        v[i] = xr[lane + 32 * i];
        s += v[i].x + v[i].y + v[i].z + v[i].w;
      }
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = rms ? 0.f : s / d;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV_MAX; ++i)
      if (i < nv) {
        float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, e = v[i].w - mean;
        q += a * a + b * b + c * c + e * e;
      }
#pragma unroll
    for (int o = 16; o; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    const float rstd = rsqrtf(q / d + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    uint2* yr = reinterpret_cast<uint2*>(y + (long long)row * d);
#pragma unroll
    for (int i = 0; i < NV_MAX; ++i)
      if (i < nv) {
        const float4 g = __ldg(reinterpret_cast<const float4*>(gamma) + lane + 32 * i);
        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
        if (beta) b = __ldg(reinterpret_cast<const float4*>(beta) + lane + 32 * i);
        uint2 o;
        o.x = pack_bf16x2((v[i].x - mean) * rstd * g.x + b.x, (v[i].y - mean) * rstd * g.y + b.y);
        o.y = pack_bf16x2((v[i].z - mean) * rstd * g.z + b.z, (v[i].w - mean) * rstd * g.w + b.w);
        yr[lane + 32 * i] = o;
      }
  }
}

struct LnBwdArgs {
  const __nv_bfloat16* dy;   // [M,d] grad wrt normalised output (may be null if only heads feed)
  const float* x;            // [M,d] forward input
  const float* mean;         // [M]
  const float* rstd;         // [M]
  const float* gamma;        // [d]
  const float* dres_in;      // [M,d] incoming residual gradient or null
  float* dx;                 // [M,d] out (may alias dres_in)
  __nv_bfloat16* dbranch;    // [M,d] out or null: bf16(dropout_mask * dx)
  float* dgamma;             // [d] accumulated
  float* dbeta;              // [d] accumulated or null
  float* dbias;              // [d] accumulated or null: column sums of the masked copy (the bias
                             // gradient of the projection whose output that copy is the gradient of)
  // optional rank-2 term: dy_eff[m,c] = dy[m,c] + s0[m]*w0[c] + s1[m]*w1[c]
  const float* s0; const float* w0; const float* s1; const float* w1;
  int M, d, rms;
  unsigned long long drop_seed; unsigned int drop_stream, drop_thr16;
  const unsigned long long* salt;   // seed_salt_ptr() at launch: folded into drop_seed when not null
};

// dy (+ rank-2 term) of lane-owned float4 column c4 of one row
__device__ __forceinline__ float4 ln_dy_eff(const LnBwdArgs& a, uint2 p, bool has_dy, int c4,
                                            float sc0, float sc1) {
  float4 dyv = make_float4(0.f, 0.f, 0.f, 0.f);
  if (has_dy) dyv = make_float4(bf16_lo(p.x), bf16_hi(p.x), bf16_lo(p.y), bf16_hi(p.y));
  if (a.s0) {
    const float4 w = __ldg(reinterpret_cast<const float4*>(a.w0) + c4);
    dyv.x += sc0 * w.x; dyv.y += sc0 * w.y; dyv.z += sc0 * w.z; dyv.w += sc0 * w.w;
  }
  if (a.s1) {
    const float4 w = __ldg(reinterpret_cast<const float4*>(a.w1) + c4);
    dyv.x += sc1 * w.x; dyv.y += sc1 * w.y; dyv.z += sc1 * w.z; dyv.w += sc1 * w.w;
  }
  return dyv;
}

// Row kernel: every global load of a row (x, dy, incoming residual gradient) is issued up front,
// so a row costs one memory round trip; dy stays packed in registers and gamma*dy is recomputed.
//
// PARAMS: the warp also accumulates dgamma / dbeta of its rows in a private shared-memory row
// (3 x d floats per warp: dgamma, dbeta and the column sums of the masked copy; plain
// read-add-write, no atomics); the block folds its eight rows and
// issues one vector atomic per four columns at the end.  This saves the second pass over x and dy
// that a separate column kernel needs.
template <int NV_MAX, bool PARAMS>
__global__ void __launch_bounds__(LN_WARPS * 32, NV_MAX <= 8 ? 2 : 1)
ln_bwd_kernel(const LnBwdArgs a) {
  griddep_enter();
  extern __shared__ __align__(16) float ln_acc[];     // [LN_WARPS][3][d] when PARAMS
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int d = a.d, nv = d >> 7;
  float4* acc_g = reinterpret_cast<float4*>(ln_acc + (warp * 3 + 0) * d);
  float4* acc_b = reinterpret_cast<float4*>(ln_acc + (warp * 3 + 1) * d);
  float4* acc_c = reinterpret_cast<float4*>(ln_acc + (warp * 3 + 2) * d);
  const bool want_bias = PARAMS && a.dbias != nullptr && a.dbranch != nullptr;
  if (PARAMS) {
    for (int c4 = lane; c4 < (d >> 2); c4 += 32) {
      acc_g[c4] = make_float4(0.f, 0.f, 0.f, 0.f);
      acc_b[c4] = make_float4(0.f, 0.f, 0.f, 0.f);
      acc_c[c4] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncwarp();
  }
  const float dscale = dropout_scale(a.drop_thr16);
  const bool has_dy = a.dy != nullptr, has_r = a.dres_in != nullptr;
  for (int row = blockIdx.x * LN_WARPS + warp; row < a.M; row += gridDim.x * LN_WARPS) {
    const float4* xr = reinterpret_cast<const float4*>(a.x + (long long)row * d);
    const uint2* dyr = reinterpret_cast<const uint2*>(a.dy + (long long)row * d);
    const float4* rr = reinterpret_cast<const float4*>(a.dres_in + (long long)row * d);
    float4 xh[NV_MAX], rv[NV_MAX];
    uint2 dyp[NV_MAX];
#pragma unroll
    for (int i = 0; i < NV_MAX; ++i)
      if (i < nv) {
        const int c4 = lane + 32 * i;
        xh[i] = xr[c4];
        dyp[i] = has_dy ? dyr[c4] : make_uint2(0u, 0u);
        rv[i] = has_r ? rr[c4] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    const float mean = a.rms ? 0.f : a.mean[row];
    const float rstd = a.rstd[row];
    const float sc0 = a.s0 ? a.s0[row] : 0.f, sc1 = a.s1 ? a.s1[row] : 0.f;
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV_MAX; ++i)
      if (i < nv) {
        const int c4 = lane + 32 * i;
        const float4 dyv = ln_dy_eff(a, dyp[i], has_dy, c4, sc0, sc1);
        const float4 g = __ldg(reinterpret_cast<const float4*>(a.gamma) + c4);
        xh[i] = make_float4((xh[i].x - mean) * rstd, (xh[i].y - mean) * rstd,
                            (xh[i].z - mean) * rstd, (xh[i].w - mean) * rstd);
        const float4 gy = make_float4(dyv.x * g.x, dyv.y * g.y, dyv.z * g.z, dyv.w * g.w);
        s1 += gy.x + gy.y + gy.z + gy.w;
        s2 += gy.x * xh[i].x + gy.y * xh[i].y + gy.z * xh[i].z + gy.w * xh[i].w;
      }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      s1 += __shfl_xor_sync(0xffffffffu, s1, o);
      s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    const float m1 = a.rms ? 0.f : s1 / d, m2 = s2 / d;
    float4* dxr = reinterpret_cast<float4*>(a.dx + (long long)row * d);
    uint2* dbr = a.dbranch ? reinterpret_cast<uint2*>(a.dbranch + (long long)row * d) : nullptr;
#pragma unroll
    for (int i = 0; i < NV_MAX; ++i)
      if (i < nv) {
        const int c4 = lane + 32 * i;
        const float4 dyv = ln_dy_eff(a, dyp[i], has_dy, c4, sc0, sc1);
        const float4 g = __ldg(reinterpret_cast<const float4*>(a.gamma) + c4);
        if (PARAMS) {
          float4 t = acc_g[c4];
          t.x += dyv.x * xh[i].x; t.y += dyv.y * xh[i].y; t.z += dyv.z * xh[i].z; t.w += dyv.w * xh[i].w;
          acc_g[c4] = t;
          float4 u = acc_b[c4];
          u.x += dyv.x; u.y += dyv.y; u.z += dyv.z; u.w += dyv.w;
          acc_b[c4] = u;
        }
        float4 o;
        o.x = (dyv.x * g.x - m1 - xh[i].x * m2) * rstd + rv[i].x;
        o.y = (dyv.y * g.y - m1 - xh[i].y * m2) * rstd + rv[i].y;
        o.z = (dyv.z * g.z - m1 - xh[i].z * m2) * rstd + rv[i].z;
        o.w = (dyv.w * g.w - m1 - xh[i].w * m2) * rstd + rv[i].w;
        dxr[c4] = o;
        if (dbr) {
          float4 m = o;
          if (a.drop_thr16) {
            const uint64_t e0 = static_cast<uint64_t>(row) * d + c4 * 4;
            const uint32_t keep =
                dropout_keep8(salted(a.drop_seed, a.salt), a.drop_stream, e0 >> 3, a.drop_thr16) >> (e0 & 7);
            m.x = (keep & 1u) ? m.x * dscale : 0.f;
            m.y = (keep & 2u) ? m.y * dscale : 0.f;
            m.z = (keep & 4u) ? m.z * dscale : 0.f;
            m.w = (keep & 8u) ? m.w * dscale : 0.f;
          }
          uint2 p;
          p.x = pack_bf16x2(m.x, m.y);
          p.y = pack_bf16x2(m.z, m.w);
          dbr[c4] = p;
          if (want_bias) {
            float4 t = acc_c[c4];
            t.x += m.x; t.y += m.y; t.z += m.z; t.w += m.w;
            acc_c[c4] = t;
          }
        }
      }
  }
  if (PARAMS) {
    __syncthreads();
    for (int c4 = threadIdx.x; c4 < (d >> 2); c4 += LN_WARPS * 32) {
      float4 sg = make_float4(0.f, 0.f, 0.f, 0.f), sb = sg, sc = sg;
#pragma unroll
      for (int w = 0; w < LN_WARPS; ++w) {
        const float4 tg = reinterpret_cast<const float4*>(ln_acc + (w * 3 + 0) * d)[c4];
        const float4 tb = reinterpret_cast<const float4*>(ln_acc + (w * 3 + 1) * d)[c4];
        const float4 tc = reinterpret_cast<const float4*>(ln_acc + (w * 3 + 2) * d)[c4];
        sg.x += tg.x; sg.y += tg.y; sg.z += tg.z; sg.w += tg.w;
        sb.x += tb.x; sb.y += tb.y; sb.z += tb.z; sb.w += tb.w;
        sc.x += tc.x; sc.y += tc.y; sc.z += tc.z; sc.w += tc.w;
      }
      if (want_bias)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(a.dbias + c4 * 4),
                     "f"(sc.x), "f"(sc.y), "f"(sc.z), "f"(sc.w) : "memory");
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(a.dgamma + c4 * 4),
                   "f"(sg.x), "f"(sg.y), "f"(sg.z), "f"(sg.w) : "memory");
      if (a.dbeta)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(a.dbeta + c4 * 4),
                     "f"(sb.x), "f"(sb.y), "f"(sb.z), "f"(sb.w) : "memory");
    }
  }
}

}  // namespace ab

template <int NV>
static int launch_ln_dependent(int grid, const float* x, const float* gamma, const float* beta, void* y,
                               float* mean, float* rstd, int M, int d, float eps, int rms,
                               cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(ab::LN_WARPS * 32);
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, ab::ln_fwd_kernel<NV>, x, gamma, beta, (__nv_bfloat16*)y, mean, rstd, M, d,
                                 eps, rms);
}

extern "C" {

// d must be a multiple of 128 and at most 2048.
// Same as ab_layernorm_fwd, launched as a programmatic dependent of the kernel before it in the
// stream (its launch overlaps that kernel's tail; it waits for it before reading x).
int ab_layernorm_fwd_dependent(const float* x, const float* gamma, const float* beta, void* y, float* mean,
                               float* rstd, int M, int d, float eps, int rms, cudaStream_t stream) {
  using namespace ab;
  if (d % 128 != 0 || d > 2048 || M <= 0) return -1;
  int grid = (M + LN_WARPS - 1) / LN_WARPS;
  if (grid > 148 * 8) grid = 148 * 8;
  if (d <= 1024) return launch_ln_dependent<8>(grid, x, gamma, beta, y, mean, rstd, M, d, eps, rms, stream);
  return launch_ln_dependent<16>(grid, x, gamma, beta, y, mean, rstd, M, d, eps, rms, stream);
}

int ab_layernorm_fwd(const float* x, const float* gamma, const float* beta, void* y, float* mean,
                     float* rstd, int M, int d, float eps, int rms, cudaStream_t stream) {
  using namespace ab;
  if (d % 128 != 0 || d > 2048 || M <= 0) return -1;
  int grid = (M + LN_WARPS - 1) / LN_WARPS;
  if (grid > 148 * 8) grid = 148 * 8;
  if (d <= 1024)
    launch_chained(ln_fwd_kernel<8>, dim3(grid), dim3(LN_WARPS * 32), 0, stream, x, gamma, beta, (__nv_bfloat16*)y, mean,
                                                         rstd, M, d, eps, rms);
  else
    launch_chained(ln_fwd_kernel<16>, dim3(grid), dim3(LN_WARPS * 32), 0, stream, x, gamma, beta, (__nv_bfloat16*)y, mean,
                                                          rstd, M, d, eps, rms);
  return (int)cudaGetLastError();
}

int ab_layernorm_bwd(const void* dy, const float* x, const float* mean, const float* rstd,
                     const float* gamma, const float* dres_in, float* dx, void* dbranch,
                     float* dgamma, float* dbeta, float* dbias, const float* s0, const float* w0,
                     const float* s1, const float* w1, int M, int d, int rms,
                     unsigned long long drop_seed, unsigned int drop_stream,
                     unsigned int drop_thr16, cudaStream_t stream) {
  using namespace ab;
  if (d % 128 != 0 || d > 2048 || M <= 0) return -1;
  LnBwdArgs a;
  a.dy = (const __nv_bfloat16*)dy; a.x = x; a.mean = mean; a.rstd = rstd; a.gamma = gamma;
  a.dres_in = dres_in; a.dx = dx; a.dbranch = (__nv_bfloat16*)dbranch; a.dgamma = dgamma;
  a.dbeta = dbeta; a.dbias = dbias; a.s0 = s0; a.w0 = w0; a.s1 = s1; a.w1 = w1; a.M = M; a.d = d; a.rms = rms;
  a.drop_seed = drop_seed; a.drop_stream = drop_stream; a.drop_thr16 = drop_thr16; a.salt = seed_salt_ptr();
  int grid = (M + LN_WARPS - 1) / LN_WARPS;
  if (!dgamma) {
    if (grid > 148 * 16) grid = 148 * 16;
    if (d <= 1024) launch_chained(ln_bwd_kernel<8, false>, dim3(grid), dim3(LN_WARPS * 32), 0, stream, a);
    else           launch_chained(ln_bwd_kernel<16, false>, dim3(grid), dim3(LN_WARPS * 32), 0, stream, a);
    return (int)cudaGetLastError();
  }
  // with parameter gradients: exactly the resident blocks, each warp keeps its column sums
  const int smem = LN_WARPS * 3 * d * (int)sizeof(float);
  static PerDeviceOnce attr_set;
  if (attr_set.first_use_on_device()) {
    cudaError_t e = cudaFuncSetAttribute(ln_bwd_kernel<8, true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, LN_WARPS * 3 * 1024 * 4);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(ln_bwd_kernel<16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               LN_WARPS * 3 * 2048 * 4);
    if (e != cudaSuccess) return (int)e;
    attr_set.mark_device();
  }
  const int resident = d <= 1024 ? 148 * 2 : 148;
  if (grid > resident) grid = resident;
  if (d <= 1024) launch_chained(ln_bwd_kernel<8, true>, dim3(grid), dim3(LN_WARPS * 32), smem, stream, a);
  else           launch_chained(ln_bwd_kernel<16, true>, dim3(grid), dim3(LN_WARPS * 32), smem, stream, a);
  return (int)cudaGetLastError();
}
}
