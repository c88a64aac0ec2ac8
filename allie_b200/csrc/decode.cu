// Kernels of the KV-cached MCTS leaf evaluator (one new token per search tree and step).
//
//   kv_store        : copies the keys/values of a prefilled prompt (rows of the packed QKV
//                     activation) into the per-tree cache
//   decode_attn     : q_len = 1 attention of every tree's new token over that tree's prompt slots
//                     [0, prefix_len) plus the cache slots of the leaf's ancestors (an index list);
//                     also appends the new token's key/value to the cache
//   policy_epilogue : per tree, softmax over the logits of the leaf's legal moves only, plus value,
//                     think time and the resign logit, packed into one row for a single
//                     device-to-host copy
// Cache layout per layer: K and V as [tree][slot][H*hd] bf16.
#include "ptx.cuh"

namespace ab {

// grid (n_trees, H), block 128.  Lane owns hd/32 consecutive dims of the head.
template <int HD>
__global__ void __launch_bounds__(128)
decode_attn_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ kc,
                   __nv_bfloat16* __restrict__ vc, const int* __restrict__ active,
                   const int* __restrict__ slot, const int* __restrict__ prefix_len,
                   const int* __restrict__ anc, int anc_stride, const int* __restrict__ n_anc,
                   __nv_bfloat16* __restrict__ out, int H, int S, float scale) {
  constexpr int E = HD / 32;             // dims per lane
  const int t = blockIdx.x, h = blockIdx.y;
  if (!active[t]) return;
  const int d = H * HD;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const __nv_bfloat16* row = qkv + static_cast<long long>(t) * 3 * d;
  const long long cache_base = static_cast<long long>(t) * S * d + h * HD;
  // append this token's key / value (self is the last entry of the ancestor list)
  if (warp == 0) {
    const long long dst = cache_base + static_cast<long long>(slot[t]) * d + lane * E;
#pragma unroll
    for (int e = 0; e < E; ++e) {
      kc[dst + e] = row[d + h * HD + lane * E + e];
      vc[dst + e] = row[2 * d + h * HD + lane * E + e];
    }
  }
  float q[E];
#pragma unroll
  for (int e = 0; e < E; ++e) q[e] = __bfloat162float(row[h * HD + lane * E + e]) * scale;
  __syncthreads();
  const int P = prefix_len[t], A = n_anc[t];
  float m = -INFINITY, l = 0.f, acc[E];
#pragma unroll
  for (int e = 0; e < E; ++e) acc[e] = 0.f;
  for (int i = warp; i < P + A; i += 4) {
    const int s = i < P ? i : anc[t * anc_stride + (i - P)];
    const long long off = cache_base + static_cast<long long>(s) * d + lane * E;
    float kv[E], dot = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) { kv[e] = __bfloat162float(kc[off + e]); dot += q[e] * kv[e]; }
#pragma unroll
    for (int o = 16; o; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float m_new = fmaxf(m, dot);
    const float a = __expf(m - m_new), p = __expf(dot - m_new);
    l = l * a + p;
#pragma unroll
    for (int e = 0; e < E; ++e) acc[e] = acc[e] * a + p * __bfloat162float(vc[off + e]);
    m = m_new;
  }
  __shared__ float sm[4], sl[4], sacc[4][HD];
  if (lane == 0) { sm[warp] = m; sl[warp] = l; }
#pragma unroll
  for (int e = 0; e < E; ++e) sacc[warp][lane * E + e] = acc[e];
  __syncthreads();
  if (warp == 0) {
    float M = fmaxf(fmaxf(sm[0], sm[1]), fmaxf(sm[2], sm[3]));
    float L = 0.f, o[E];
#pragma unroll
    for (int e = 0; e < E; ++e) o[e] = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = sm[w] == -INFINITY ? 0.f : __expf(sm[w] - M);
      L += sl[w] * f;
#pragma unroll
      for (int e = 0; e < E; ++e) o[e] += sacc[w][lane * E + e] * f;
    }
    const float inv = 1.f / L;
#pragma unroll
    for (int e = 0; e < E; ++e)
      out[static_cast<long long>(t) * d + h * HD + lane * E + e] = __float2bfloat16(o[e] * inv);
  }
}

// rows of qkv [n_trees * Lp, 3d] -> cache slots [tree][pos] for pos < len[tree]
__global__ void __launch_bounds__(256)
kv_store_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ kc,
                __nv_bfloat16* __restrict__ vc, const int* __restrict__ len, int Lp, int S, int d) {
  const int t = blockIdx.y, p = blockIdx.x;
  if (p >= len[t]) return;
  const uint4* src = reinterpret_cast<const uint4*>(qkv + (static_cast<long long>(t) * Lp + p) * 3 * d);
  uint4* dk = reinterpret_cast<uint4*>(kc + (static_cast<long long>(t) * S + p) * d);
  uint4* dv = reinterpret_cast<uint4*>(vc + (static_cast<long long>(t) * S + p) * d);
  const int n8 = d / 8;
  for (int i = threadIdx.x; i < n8; i += 256) {
    dk[i] = src[n8 + i];
    dv[i] = src[2 * n8 + i];
  }
}

// out row: [0, max_legal) priors over the legal moves in list order, then value, time, resign logit,
// best legal logit.  One warp per tree.
__global__ void __launch_bounds__(32)
policy_epilogue_kernel(const __nv_bfloat16* __restrict__ logits, long long ld,
                       const int* __restrict__ active, const int* __restrict__ legal, int legal_stride,
                       const int* __restrict__ n_legal, const float* __restrict__ value,
                       const float* __restrict__ time, int resign_id, float inv_temperature,
                       float* __restrict__ out, int out_stride) {
  const int t = blockIdx.x, lane = threadIdx.x;
  if (!active[t]) return;
  const int n = min(n_legal[t], legal_stride);
  const __nv_bfloat16* lr = logits + static_cast<long long>(t) * ld;
  float mx = -INFINITY;
  for (int i = lane; i < n; i += 32) mx = fmaxf(mx, __bfloat162float(lr[legal[t * legal_stride + i]]));
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float s = 0.f;
  for (int i = lane; i < n; i += 32)
    s += __expf((__bfloat162float(lr[legal[t * legal_stride + i]]) - mx) * inv_temperature);
#pragma unroll
  for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  float* orow = out + static_cast<long long>(t) * out_stride;
  for (int i = lane; i < n; i += 32)
    orow[i] = __expf((__bfloat162float(lr[legal[t * legal_stride + i]]) - mx) * inv_temperature) / s;
  if (lane == 0) {
    orow[legal_stride] = value ? value[t] : 0.f;
    orow[legal_stride + 1] = time ? time[t] : 0.f;
    orow[legal_stride + 2] = __bfloat162float(lr[resign_id]);
    orow[legal_stride + 3] = mx;
  }
}

}  // namespace ab

extern "C" {

int ab_decode_attn(const void* qkv, void* kc, void* vc, const int* active, const int* slot,
                   const int* prefix_len, const int* anc, int anc_stride, const int* n_anc, void* out,
                   int n_trees, int H, int hd, int S, float scale, cudaStream_t stream) {
  using namespace ab;
  dim3 grid(n_trees, H);
  if (hd == 64)
    decode_attn_kernel<64><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)qkv, (__nv_bfloat16*)kc,
        (__nv_bfloat16*)vc, active, slot, prefix_len, anc, anc_stride, n_anc, (__nv_bfloat16*)out, H, S, scale);
  else if (hd == 128)
    decode_attn_kernel<128><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)qkv, (__nv_bfloat16*)kc,
        (__nv_bfloat16*)vc, active, slot, prefix_len, anc, anc_stride, n_anc, (__nv_bfloat16*)out, H, S, scale);
  else
    return -1;
  return (int)cudaGetLastError();
}

int ab_kv_store(const void* qkv, void* kc, void* vc, const int* len, int n_trees, int Lp, int S, int d,
                cudaStream_t stream) {
  if (d % 8) return -1;
  dim3 grid(Lp, n_trees);
  ab::kv_store_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)qkv, (__nv_bfloat16*)kc,
                                                (__nv_bfloat16*)vc, len, Lp, S, d);
  return (int)cudaGetLastError();
}

int ab_policy_epilogue(const void* logits, long long ld, const int* active, const int* legal,
                       int legal_stride, const int* n_legal, const float* value, const float* time,
                       int resign_id, float inv_temperature, float* out, int out_stride, int n_trees,
                       cudaStream_t stream) {
  ab::policy_epilogue_kernel<<<n_trees, 32, 0, stream>>>((const __nv_bfloat16*)logits, ld, active, legal,
                                                         legal_stride, n_legal, value, time, resign_id,
                                                         inv_temperature, out, out_stride);
  return (int)cudaGetLastError();
}
}
