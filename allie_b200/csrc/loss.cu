// Loss heads.
//
// ce_fwd_bwd   : cross entropy over bf16 logits [M,V] with ignore index -100, mean over the valid
//                rows; one pass computes the loss sum and overwrites the logits with
//                d(loss)/d(logits) = (softmax - onehot) * coef / n_valid, ready to be the operand
//                of the lm_head dgrad / wgrad GEMMs.  One warp per row, row cached in registers.
// heads_fwd    : value = tanh(h.w_v + b_v), time = h.w_t + b_t on the final hidden state, masked
//                MSE sums against labels (-100 = ignore) and the per-row upstream scalars
//                dv[m], dt[m] that the final LayerNorm backward folds in as a rank-2 term.
// heads_bwd_w  : gradients of the two head weight vectors and biases.
// finalize     : combines the three sums into [loss, lm, value, time].
#include "ptx.cuh"

namespace ab {

constexpr int CE_WARPS = 8;

// loss_acc[0] += sum over valid rows of -log p(label)
template <int MAXV8>  // capacity in uint4 (8 bf16) per lane
__global__ void __launch_bounds__(CE_WARPS * 32)
ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const int* __restrict__ labels,
                  const int* __restrict__ n_valid, float coef, int M, int V, long long ld,
                  float* __restrict__ loss_acc, int write_grad) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nv = V >> 8;  // uint4 per lane
  const int nval = *n_valid;
  const float gscale = nval > 0 ? coef / static_cast<float>(nval) : 0.f;
  float local_loss = 0.f;
  for (int row = blockIdx.x * CE_WARPS + warp; row < M; row += gridDim.x * CE_WARPS) {
    uint4* lr = reinterpret_cast<uint4*>(logits + (long long)row * ld);
    const int label = labels[row];
    if (label < 0) {
      if (write_grad) {
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < MAXV8; ++i)
          if (i < nv) lr[lane + 32 * i] = z;
      }
      continue;
    }
    uint4 v[MAXV8];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < MAXV8; ++i)
      if (i < nv) {
        v[i] = lr[lane + 32 * i];
        mx = fmaxf(mx, fmaxf(fmaxf(bf16_lo(v[i].x), bf16_hi(v[i].x)),
                             fmaxf(bf16_lo(v[i].y), bf16_hi(v[i].y))));
        mx = fmaxf(mx, fmaxf(fmaxf(bf16_lo(v[i].z), bf16_hi(v[i].z)),
                             fmaxf(bf16_lo(v[i].w), bf16_hi(v[i].w))));
      }
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float s = 0.f;
    const float L2E = 1.4426950408889634f;
#pragma unroll
    for (int i = 0; i < MAXV8; ++i)
      if (i < nv) {
        s += ex2_fast((bf16_lo(v[i].x) - mx) * L2E) + ex2_fast((bf16_hi(v[i].x) - mx) * L2E);
        s += ex2_fast((bf16_lo(v[i].y) - mx) * L2E) + ex2_fast((bf16_hi(v[i].y) - mx) * L2E);
        s += ex2_fast((bf16_lo(v[i].z) - mx) * L2E) + ex2_fast((bf16_hi(v[i].z) - mx) * L2E);
        s += ex2_fast((bf16_lo(v[i].w) - mx) * L2E) + ex2_fast((bf16_hi(v[i].w) - mx) * L2E);
      }
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    // logit of the label: it lives in lane (label/8)%32, slot (label/8)/32, element label%8
    const float lab_logit = __bfloat162float(logits[(long long)row * ld + label]);
    __syncwarp();  // every lane has read the label logit before any lane overwrites the row
    if (lane == 0) local_loss += (logf(s) + mx) - lab_logit;
    if (write_grad) {
      const float inv = gscale / s;
#pragma unroll
      for (int i = 0; i < MAXV8; ++i)
        if (i < nv) {
          const int col0 = (lane + 32 * i) * 8;
          float p[8];
          p[0] = ex2_fast((bf16_lo(v[i].x) - mx) * L2E) * inv;
          p[1] = ex2_fast((bf16_hi(v[i].x) - mx) * L2E) * inv;
          p[2] = ex2_fast((bf16_lo(v[i].y) - mx) * L2E) * inv;
          p[3] = ex2_fast((bf16_hi(v[i].y) - mx) * L2E) * inv;
          p[4] = ex2_fast((bf16_lo(v[i].z) - mx) * L2E) * inv;
          p[5] = ex2_fast((bf16_hi(v[i].z) - mx) * L2E) * inv;
          p[6] = ex2_fast((bf16_lo(v[i].w) - mx) * L2E) * inv;
          p[7] = ex2_fast((bf16_hi(v[i].w) - mx) * L2E) * inv;
          const int rel = label - col0;
          if (rel >= 0 && rel < 8) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (j == rel) p[j] -= gscale;
          }
          uint4 o;
          o.x = pack_bf16x2(p[0], p[1]); o.y = pack_bf16x2(p[2], p[3]);
          o.z = pack_bf16x2(p[4], p[5]); o.w = pack_bf16x2(p[6], p[7]);
          lr[lane + 32 * i] = o;
        }
    }
  }
  __shared__ float red[CE_WARPS];
  if (lane == 0) red[warp] = local_loss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < CE_WARPS; ++w) t += red[w];
    if (t != 0.f) atomicAdd(loss_acc, t);
  }
}

// One warp per row.  acc[1] += sum (v-y)^2 over valid value labels, acc[2] likewise for time.
__global__ void __launch_bounds__(256)
heads_fwd_kernel(const __nv_bfloat16* __restrict__ h, const float* __restrict__ wv,
                 const float* __restrict__ bv, const float* __restrict__ wt,
                 const float* __restrict__ bt, const float* __restrict__ value_labels,
                 const float* __restrict__ time_labels, const int* __restrict__ counts,
                 float value_coef, float time_coef, float* __restrict__ value_out,
                 float* __restrict__ time_out, float* __restrict__ dv, float* __restrict__ dt,
                 float* __restrict__ acc, int M, int d) {
  griddep_enter();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x * 8 + warp;
  float lv = 0.f, lt = 0.f;
  if (row < M) {
    const uint2* hr = reinterpret_cast<const uint2*>(h + (long long)row * d);
    float sv = 0.f, st = 0.f;
    for (int c4 = lane; c4 < d / 4; c4 += 32) {
      const uint2 p = hr[c4];
      const float4 a = __ldg(reinterpret_cast<const float4*>(wv) + c4);
      const float4 b = __ldg(reinterpret_cast<const float4*>(wt) + c4);
      const float x0 = bf16_lo(p.x), x1 = bf16_hi(p.x), x2 = bf16_lo(p.y), x3 = bf16_hi(p.y);
      sv += x0 * a.x + x1 * a.y + x2 * a.z + x3 * a.w;
      st += x0 * b.x + x1 * b.y + x2 * b.z + x3 * b.w;
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      sv += __shfl_xor_sync(0xffffffffu, sv, o);
      st += __shfl_xor_sync(0xffffffffu, st, o);
    }
    if (lane == 0) {
      const float v = tanhf(sv + bv[0]);
      const float t = st + bt[0];
      value_out[row] = v;
      time_out[row] = t;
      float gv = 0.f, gt = 0.f;
      if (value_labels) {
        const float y = value_labels[row];
        if (y != -100.f) {
          const float e = v - y;
          lv = e * e;
          const int n = counts[1];
          gv = 2.f * e * (1.f - v * v) * value_coef / static_cast<float>(n > 0 ? n : 1);
        }
      }
      if (time_labels) {
        const float y = time_labels[row];
        if (y != -100.f) {
          const float e = t - y;
          lt = e * e;
          const int n = counts[2];
          gt = 2.f * e * time_coef / static_cast<float>(n > 0 ? n : 1);
        }
      }
      if (dv) dv[row] = gv;
      if (dt) dt[row] = gt;
    }
  }
  __shared__ float red[2][8];
  if (lane == 0) { red[0][warp] = lv; red[1][warp] = lt; }
  __syncthreads();
  if (threadIdx.x == 0 && acc) {
    float a = 0.f, b = 0.f;
    for (int w = 0; w < 8; ++w) { a += red[0][w]; b += red[1][w]; }
    if (a != 0.f) atomicAdd(&acc[1], a);
    if (b != 0.f) atomicAdd(&acc[2], b);
  }
}

// dwv[c] += sum_m dv[m] h[m,c]; dwt likewise; dbv += sum dv; dbt += sum dt.
__global__ void __launch_bounds__(256)
heads_bwd_w_kernel(const __nv_bfloat16* __restrict__ h, const float* __restrict__ dv,
                   const float* __restrict__ dt, float* __restrict__ dwv, float* __restrict__ dbv,
                   float* __restrict__ dwt, float* __restrict__ dbt, int M, int d, int rows_per_blk) {
  griddep_enter();
  // block covers rows [r0, r1) and all columns; thread covers columns tid*4 + 1024*i
  const int r0 = blockIdx.x * rows_per_blk;
  const int r1 = min(M, r0 + rows_per_blk);
  for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
    float4 av = make_float4(0.f, 0.f, 0.f, 0.f), at = av;
    for (int r = r0; r < r1; ++r) {
      const uint2 p = *reinterpret_cast<const uint2*>(h + (long long)r * d + c);
      const float gv = dv[r], gt = dt[r];
      const float x0 = bf16_lo(p.x), x1 = bf16_hi(p.x), x2 = bf16_lo(p.y), x3 = bf16_hi(p.y);
      av.x += gv * x0; av.y += gv * x1; av.z += gv * x2; av.w += gv * x3;
      at.x += gt * x0; at.y += gt * x1; at.z += gt * x2; at.w += gt * x3;
    }
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dwv + c), "f"(av.x),
                 "f"(av.y), "f"(av.z), "f"(av.w) : "memory");
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dwt + c), "f"(at.x),
                 "f"(at.y), "f"(at.z), "f"(at.w) : "memory");
  }
  if (threadIdx.x == 0) {
    float sv = 0.f, st = 0.f;
    for (int r = r0; r < r1; ++r) { sv += dv[r]; st += dt[r]; }
    atomicAdd(dbv, sv);
    atomicAdd(dbt, st);
  }
}

// acc: [0]=sum nll, [1]=sum value se, [2]=sum time se.  out: [loss, lm, value, time]
__global__ void loss_finalize_kernel(const float* __restrict__ acc, const int* __restrict__ counts,
                                     float lm_coef, float value_coef, float time_coef,
                                     float* __restrict__ out) {
  griddep_enter();
  const float lm = counts[0] > 0 ? acc[0] / counts[0] : 0.f;
  const float vl = counts[1] > 0 ? acc[1] / counts[1] : 0.f;
  const float tl = counts[2] > 0 ? acc[2] / counts[2] : 0.f;
  out[0] = lm * lm_coef + vl * value_coef + tl * time_coef;
  out[1] = lm; out[2] = vl; out[3] = tl;
}

}  // namespace ab

extern "C" {

// V must be a multiple of 256 and at most 8192.  logits are overwritten by their gradient when
// write_grad != 0.
int ab_ce_fwd_bwd(void* logits, const int* labels, const int* n_valid, float coef, int M, int V,
                  long long ld, float* loss_acc, int write_grad, cudaStream_t stream) {
  using namespace ab;
  if (V % 256 != 0 || V > 8192 || (ld & 7)) return -1;
  int grid = (M + CE_WARPS - 1) / CE_WARPS;
  if (grid > 148 * 8) grid = 148 * 8;
  auto lg = (__nv_bfloat16*)logits;
  if (V <= 2048)
    ce_fwd_bwd_kernel<8><<<grid, CE_WARPS * 32, 0, stream>>>(lg, labels, n_valid, coef, M, V, ld,
                                                            loss_acc, write_grad);
  else
    ce_fwd_bwd_kernel<32><<<grid, CE_WARPS * 32, 0, stream>>>(lg, labels, n_valid, coef, M, V, ld,
                                                             loss_acc, write_grad);
  return (int)cudaGetLastError();
}

int ab_heads_fwd(const void* h, const float* wv, const float* bv, const float* wt, const float* bt,
                 const float* value_labels, const float* time_labels, const int* counts,
                 float value_coef, float time_coef, float* value_out, float* time_out, float* dv,
                 float* dt, float* acc, int M, int d, cudaStream_t stream) {
  if (d % 4) return -1;
  ab::launch_chained(ab::heads_fwd_kernel, dim3((M + 7) / 8), dim3(256), 0, stream, 
      (const __nv_bfloat16*)h, wv, bv, wt, bt, value_labels, time_labels, counts, value_coef,
      time_coef, value_out, time_out, dv, dt, acc, M, d);
  return (int)cudaGetLastError();
}

int ab_heads_bwd_w(const void* h, const float* dv, const float* dt, float* dwv, float* dbv,
                   float* dwt, float* dbt, int M, int d, cudaStream_t stream) {
  if (d % 4) return -1;
  const int rows_per_blk = 64;
  ab::launch_chained(ab::heads_bwd_w_kernel, dim3((M + rows_per_blk - 1) / rows_per_blk), dim3(256), 0, stream, 
      (const __nv_bfloat16*)h, dv, dt, dwv, dbv, dwt, dbt, M, d, rows_per_blk);
  return (int)cudaGetLastError();
}

int ab_loss_finalize(const float* acc, const int* counts, float lm_coef, float value_coef,
                     float time_coef, float* out, cudaStream_t stream) {
  ab::launch_chained(ab::loss_finalize_kernel, dim3(1), dim3(1), 0, stream, acc, counts, lm_coef, value_coef, time_coef, out);
  return (int)cudaGetLastError();
}
}
