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
// Cache layout per layer: K and V as [tree][head][slot][hd] bf16, so the rows one (tree, head)
// attention block streams are contiguous in memory.
#include "ptx.cuh"

namespace ab {

// grid (n_trees, H), block 128.  A key's row for one head is HD/8 chunks of 16 bytes; the block is
// 128 / (HD/8) key groups times HD/8 chunk lanes, so the lanes of a group read one contiguous row
// and the groups walk the keys in parallel.  One pass with a running maximum per group: the K and V
// chunks of a key are fetched together and every load is independent of the arithmetic, so the
// kernel streams the tree's K/V rows at memory speed; the groups' partial results are merged at
// the end.
template <int HD>
__global__ void __launch_bounds__(128)
decode_attn_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ kc,
                   __nv_bfloat16* __restrict__ vc, const int* __restrict__ active,
                   const int* __restrict__ slot, const int* __restrict__ prefix_len,
                   const int* __restrict__ anc, int anc_stride, const int* __restrict__ n_anc,
                   __nv_bfloat16* __restrict__ out, int H, int S, float scale) {
  constexpr int CH = HD / 8;             // 16-byte chunks per row = lanes per key group
  constexpr int KG = 128 / CH;           // key groups per block
  constexpr int UNROLL = 4;
  const int t = blockIdx.x, h = blockIdx.y;
  if (!active[t]) return;
  __shared__ float s_m[KG], s_l[KG];
  __shared__ float s_acc[KG][HD];
  const int d = H * HD;
  const int tid = threadIdx.x;
  const int c = tid % CH, kg = tid / CH;
  const __nv_bfloat16* row = qkv + static_cast<long long>(t) * 3 * d;
  const long long cache_base = (static_cast<long long>(t) * H + h) * S * HD;
  // append this token's key / value (self is the last entry of the ancestor list)
  if (tid < CH) {
    const long long dst = cache_base + static_cast<long long>(slot[t]) * HD + tid * 8;
    *reinterpret_cast<uint4*>(kc + dst) = *reinterpret_cast<const uint4*>(row + d + h * HD + tid * 8);
    *reinterpret_cast<uint4*>(vc + dst) = *reinterpret_cast<const uint4*>(row + 2 * d + h * HD + tid * 8);
  }
  float q[8];
  {
    const uint4 qv = *reinterpret_cast<const uint4*>(row + h * HD + c * 8);
    q[0] = bf16_lo(qv.x) * scale; q[1] = bf16_hi(qv.x) * scale; q[2] = bf16_lo(qv.y) * scale;
    q[3] = bf16_hi(qv.y) * scale; q[4] = bf16_lo(qv.z) * scale; q[5] = bf16_hi(qv.z) * scale;
    q[6] = bf16_lo(qv.w) * scale; q[7] = bf16_hi(qv.w) * scale;
  }
  // No barrier: the token's own key (the last entry of the ancestor list) is read from the
  // packed QKV row it was just copied from, never back from the cache.
  const int P = prefix_len[t];
  const int n = P + n_anc[t];
  const int* anc_t = anc + static_cast<long long>(t) * anc_stride;
  const __nv_bfloat16* kbase = kc + cache_base + c * 8;
  const __nv_bfloat16* vbase = vc + cache_base + c * 8;
  const __nv_bfloat16* kself = row + d + h * HD + c * 8;
  const __nv_bfloat16* vself = row + 2 * d + h * HD + c * 8;
  float m = -INFINITY, l = 0.f;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  // uniform trip count over the block: the group shuffles below need every lane of the warp
  for (int i0 = 0; i0 < n; i0 += KG * UNROLL) {
    uint4 kv[UNROLL], vv[UNROLL];
    bool live[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int i = i0 + u * KG + kg;
      live[u] = i < n;
      kv[u] = make_uint4(0, 0, 0, 0);
      vv[u] = kv[u];
      if (live[u]) {
        if (i == n - 1) {
          kv[u] = *reinterpret_cast<const uint4*>(kself);
          vv[u] = *reinterpret_cast<const uint4*>(vself);
        } else {
          const long long off = static_cast<long long>(i < P ? i : anc_t[i - P]) * HD;
          kv[u] = *reinterpret_cast<const uint4*>(kbase + off);
          vv[u] = *reinterpret_cast<const uint4*>(vbase + off);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      float dot = q[0] * bf16_lo(kv[u].x) + q[1] * bf16_hi(kv[u].x) + q[2] * bf16_lo(kv[u].y) +
                  q[3] * bf16_hi(kv[u].y) + q[4] * bf16_lo(kv[u].z) + q[5] * bf16_hi(kv[u].z) +
                  q[6] * bf16_lo(kv[u].w) + q[7] * bf16_hi(kv[u].w);
#pragma unroll
      for (int o = CH / 2; o; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      if (live[u]) {                      // uniform within the key group
        const float m_new = fmaxf(m, dot);
        const float a = __expf(m - m_new), p = __expf(dot - m_new);
        l = l * a + p;
        acc[0] = acc[0] * a + p * bf16_lo(vv[u].x); acc[1] = acc[1] * a + p * bf16_hi(vv[u].x);
        acc[2] = acc[2] * a + p * bf16_lo(vv[u].y); acc[3] = acc[3] * a + p * bf16_hi(vv[u].y);
        acc[4] = acc[4] * a + p * bf16_lo(vv[u].z); acc[5] = acc[5] * a + p * bf16_hi(vv[u].z);
        acc[6] = acc[6] * a + p * bf16_lo(vv[u].w); acc[7] = acc[7] * a + p * bf16_hi(vv[u].w);
        m = m_new;
      }
    }
  }
  if (c == 0) { s_m[kg] = m; s_l[kg] = l; }
#pragma unroll
  for (int e = 0; e < 8; ++e) s_acc[kg][c * 8 + e] = acc[e];
  __syncthreads();
  if (tid < HD) {
    float M = -INFINITY;
#pragma unroll
    for (int g = 0; g < KG; ++g) M = fmaxf(M, s_m[g]);
    float L = 0.f, o = 0.f;
#pragma unroll
    for (int g = 0; g < KG; ++g) {
      const float f = s_m[g] == -INFINITY ? 0.f : __expf(s_m[g] - M);
      L += s_l[g] * f;
      o += s_acc[g][tid] * f;
    }
    out[static_cast<long long>(t) * d + h * HD + tid] = __float2bfloat16(o / L);
  }
}

// rows of qkv [n_trees * Lp, 3d] -> cache slots [tree][pos] for pos < len[tree]
__global__ void __launch_bounds__(256)
kv_store_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ kc,
                __nv_bfloat16* __restrict__ vc, const int* __restrict__ len, int Lp, int S, int d,
                int hd) {
  const int t = blockIdx.y, p = blockIdx.x;
  if (p >= len[t]) return;
  const uint4* src = reinterpret_cast<const uint4*>(qkv + (static_cast<long long>(t) * Lp + p) * 3 * d);
  const int n8 = d / 8, hd8 = hd / 8, H = d / hd;
  for (int i = threadIdx.x; i < n8; i += 256) {
    const int h = i / hd8, c = i - h * hd8;
    const long long dst = (((static_cast<long long>(t) * H + h) * S + p) * hd) / 8 + c;
    reinterpret_cast<uint4*>(kc)[dst] = src[n8 + i];
    reinterpret_cast<uint4*>(vc)[dst] = src[2 * n8 + i];
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
                int hd, cudaStream_t stream) {
  if (d % 8 || hd % 8 || d % hd) return -1;
  dim3 grid(Lp, n_trees);
  ab::kv_store_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)qkv, (__nv_bfloat16*)kc,
                                                (__nv_bfloat16*)vc, len, Lp, S, d, hd);
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
