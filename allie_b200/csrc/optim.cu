// Optimizer-side kernels over flat fp32 buffers.
//
// sumsq      : sum of squares of a flat gradient buffer into a device scalar (for the global
//              L2-norm clip) - two-level: per-block partial then one atomic.
// adamw      : decoupled-weight-decay Adam on fp32 master weights.  The clip coefficient is
//              derived on the device from the squared norm (no host round trip), and the kernel
//              also refreshes the bf16 shadow copy that the GEMMs read.
#include "ptx.cuh"

namespace ab {

__global__ void __launch_bounds__(256)
sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ out) {
  float s = 0.f;
  const long long n4 = n >> 2;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 v = g4[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const float v = g[(n4 << 2) + threadIdx.x];
    s += v * v;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __shared__ float red[8];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    atomicAdd(out, t);
  }
}

struct AdamArgs {
  float* p; const float* g; float* m; float* v; __nv_bfloat16* p_bf16;
  long long n;
  float lr, beta1, beta2, eps, wd;
  float bc1, bc2_sqrt;           // 1 - beta1^t, sqrt(1 - beta2^t)
  const float* gnorm_sq;         // device scalar or null
  float max_norm;                // <= 0: no clipping
  float grad_scale;              // extra multiplier on g (e.g. 1/world for a summed gradient)
};

__global__ void __launch_bounds__(256) adamw_kernel(const AdamArgs a) {
  float clip = a.grad_scale;
  if (a.gnorm_sq && a.max_norm > 0.f) {
    const float norm = sqrtf(*a.gnorm_sq) * a.grad_scale;
    const float c = a.max_norm / (norm + 1e-6f);
    if (c < 1.f) clip *= c;
  }
  const long long n4 = a.n >> 2;
  const float decay = 1.f - a.lr * a.wd;
  const float step = a.lr / a.bc1;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 p = reinterpret_cast<float4*>(a.p)[i];
    const float4 g0 = reinterpret_cast<const float4*>(a.g)[i];
    float4 m = reinterpret_cast<float4*>(a.m)[i];
    float4 v = reinterpret_cast<float4*>(a.v)[i];
    float pe[4] = {p.x, p.y, p.z, p.w}, ge[4] = {g0.x, g0.y, g0.z, g0.w};
    float me[4] = {m.x, m.y, m.z, m.w}, ve[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float g = ge[j] * clip;
      pe[j] *= decay;
      me[j] = a.beta1 * me[j] + (1.f - a.beta1) * g;
      ve[j] = a.beta2 * ve[j] + (1.f - a.beta2) * g * g;
      const float denom = sqrtf(ve[j]) / a.bc2_sqrt + a.eps;
      pe[j] -= step * me[j] / denom;
    }
    reinterpret_cast<float4*>(a.p)[i] = make_float4(pe[0], pe[1], pe[2], pe[3]);
    reinterpret_cast<float4*>(a.m)[i] = make_float4(me[0], me[1], me[2], me[3]);
    reinterpret_cast<float4*>(a.v)[i] = make_float4(ve[0], ve[1], ve[2], ve[3]);
    if (a.p_bf16) {
      uint2 o;
      o.x = pack_bf16x2(pe[0], pe[1]);
      o.y = pack_bf16x2(pe[2], pe[3]);
      reinterpret_cast<uint2*>(a.p_bf16)[i] = o;
    }
  }
}

__global__ void __launch_bounds__(256)
cast_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n4) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(src)[i];
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    reinterpret_cast<uint2*>(dst)[i] = o;
  }
}

}  // namespace ab

extern "C" {

int ab_sumsq(const float* g, long long n, float* out, cudaStream_t stream) {
  if (reinterpret_cast<uintptr_t>(g) & 15) return -1;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  ab::sumsq_kernel<<<(int)blocks, 256, 0, stream>>>(g, n, out);
  return (int)cudaGetLastError();
}

// n must be a multiple of 4 and all buffers 16-byte aligned.
int ab_adamw(float* p, const float* g, float* m, float* v, void* p_bf16, long long n, float lr,
             float beta1, float beta2, float eps, float wd, int step, const float* gnorm_sq,
             float max_norm, float grad_scale, cudaStream_t stream) {
  if (n & 3) return -1;
  ab::AdamArgs a;
  a.p = p; a.g = g; a.m = m; a.v = v; a.p_bf16 = (__nv_bfloat16*)p_bf16; a.n = n;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2_sqrt = sqrtf(1.f - powf(beta2, (float)step));
  a.gnorm_sq = gnorm_sq; a.max_norm = max_norm; a.grad_scale = grad_scale;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  ab::adamw_kernel<<<(int)blocks, 256, 0, stream>>>(a);
  return (int)cudaGetLastError();
}

int ab_cast_bf16(const float* src, void* dst, long long n, cudaStream_t stream) {
  if (n & 3) return -1;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  ab::cast_bf16_kernel<<<(int)blocks, 256, 0, stream>>>(src, (__nv_bfloat16*)dst, n / 4);
  return (int)cudaGetLastError();
}
}

// ---------------------------------------------------------------------------------------------
// colsum: out[n] += sum_m x[m][n] for a bf16 matrix (bias gradients).  A block covers
// 128 rows and 1024 columns: 128 column threads (8 adjacent columns each) times two row
// phases, eight independent 16-byte loads in flight per thread.
namespace ab {
constexpr int CS_ROWS = 128;
__global__ void __launch_bounds__(256)
colsum_bf16_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int M, int N,
                   float* __restrict__ out, const int* __restrict__ m_limit) {
  griddep_enter();
  __shared__ float part[128][9];
  const int tx = threadIdx.x & 127, ty = threadIdx.x >> 7;
  const int c = (blockIdx.x * 128 + tx) * 8;
  // grouped form (blockIdx.z = group): group g owns rows [g*M, (g+1)*M) of x, row g of `out` and
  // entry g of `m_limit`
  x += static_cast<long long>(blockIdx.z) * M * ld;
  out += static_cast<long long>(blockIdx.z) * N;
  if (m_limit) M = min(M, __ldg(m_limit + blockIdx.z));
  const int r0 = blockIdx.y * CS_ROWS;
  const int r1 = min(M, r0 + CS_ROWS);
  float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c < N) {
    const __nv_bfloat16* base = x + c;
    for (int r = r0 + ty; r < r1; r += 16) {
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int rr = r + 2 * j;
        v[j] = rr < r1 ? __ldcs(reinterpret_cast<const uint4*>(base + (long long)rr * ld))
                       : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        s[0] += bf16_lo(v[j].x); s[1] += bf16_hi(v[j].x); s[2] += bf16_lo(v[j].y); s[3] += bf16_hi(v[j].y);
        s[4] += bf16_lo(v[j].z); s[5] += bf16_hi(v[j].z); s[6] += bf16_lo(v[j].w); s[7] += bf16_hi(v[j].w);
      }
    }
  }
  if (ty == 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) part[tx][j] = s[j];
  }
  __syncthreads();
  if (ty == 0 && c < N && r0 < r1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j] += part[tx][j];
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + c), "f"(s[0]),
                 "f"(s[1]), "f"(s[2]), "f"(s[3]) : "memory");
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + c + 4), "f"(s[4]),
                 "f"(s[5]), "f"(s[6]), "f"(s[7]) : "memory");
  }
}
}  // namespace ab

// out[g][n] += sum over the first min(cap, m_limit[g]) rows of group g of x ([groups*cap, N] bf16)
extern "C" int ab_colsum_grouped_bf16(const void* x, long long ld, int groups, int cap, int N, float* out,
                                      const int* m_limit, cudaStream_t stream) {
  if ((N & 7) || (ld & 7) || groups < 1 || groups > 65535 || !m_limit) return -1;
  dim3 grid((N / 8 + 127) / 128, (cap + ab::CS_ROWS - 1) / ab::CS_ROWS, groups);
  ab::launch_chained(ab::colsum_bf16_kernel, dim3(grid), dim3(256), 0, stream, (const __nv_bfloat16*)x, ld, cap, N, out, m_limit);
  return (int)cudaGetLastError();
}

extern "C" int ab_colsum_bf16(const void* x, long long ld, int M, int N, float* out,
                              const int* m_limit, cudaStream_t stream) {
  if ((N & 7) || (ld & 7)) return -1;
  dim3 grid((N / 8 + 127) / 128, (M + ab::CS_ROWS - 1) / ab::CS_ROWS);
  ab::launch_chained(ab::colsum_bf16_kernel, dim3(grid), dim3(256), 0, stream, (const __nv_bfloat16*)x, ld, M, N, out, m_limit);
  return (int)cudaGetLastError();
}
