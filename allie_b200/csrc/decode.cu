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

// grid (n_trees, H), block 128.  A key's row for one head is HD/8 chunks of 16 bytes; the block is
// 128 / (HD/8) key groups times HD/8 chunk lanes, so the lanes of a group read one contiguous row
// and the groups walk the keys in parallel with every load independent of the others (the kernel
// is a stream over the tree's K/V rows and has to run at memory speed).  Two passes: scores into
// shared memory and the block maximum, then probabilities times V.
constexpr int DEC_MAX_KEYS = 1024;     // prompt slots + ancestor list per tree

template <int HD>
__global__ void __launch_bounds__(128)
decode_attn_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ kc,
                   __nv_bfloat16* __restrict__ vc, const int* __restrict__ active,
                   const int* __restrict__ slot, const int* __restrict__ prefix_len,
                   const int* __restrict__ anc, int anc_stride, const int* __restrict__ n_anc,
                   __nv_bfloat16* __restrict__ out, int H, int S, float scale) {
  constexpr int CH = HD / 8;             // 16-byte chunks per row = lanes per key group
  constexpr int KG = 128 / CH;           // key groups per block
  const int t = blockIdx.x, h = blockIdx.y;
  if (!active[t]) return;
  __shared__ float s_score[DEC_MAX_KEYS];
  __shared__ float s_red[4];
  __shared__ float s_acc[KG][HD];
  const int d = H * HD;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = tid % CH, kg = tid / CH;
  const __nv_bfloat16* row = qkv + static_cast<long long>(t) * 3 * d;
  const long long cache_base = static_cast<long long>(t) * S * d + h * HD;
  // append this token's key / value (self is the last entry of the ancestor list)
  if (tid < CH) {
    const long long dst = cache_base + static_cast<long long>(slot[t]) * d + tid * 8;
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
  __syncthreads();                        // the appended row is visible to the whole block
  const int P = prefix_len[t];
  const int n = min(P + n_anc[t], DEC_MAX_KEYS);
  const int* anc_t = anc + static_cast<long long>(t) * anc_stride;
  // ---- pass 1: scores
  float mx = -INFINITY;
#pragma unroll 4
  for (int i0 = 0; i0 < n; i0 += KG) {     // uniform trip count: the shuffles below need every lane
    const int i = i0 + kg;
    const bool live = i < n;
    uint4 kv = make_uint4(0, 0, 0, 0);
    if (live) {
      const int sl = i < P ? i : anc_t[i - P];
      kv = *reinterpret_cast<const uint4*>(kc + cache_base + static_cast<long long>(sl) * d + c * 8);
    }
    float dot = q[0] * bf16_lo(kv.x) + q[1] * bf16_hi(kv.x) + q[2] * bf16_lo(kv.y) + q[3] * bf16_hi(kv.y) +
                q[4] * bf16_lo(kv.z) + q[5] * bf16_hi(kv.z) + q[6] * bf16_lo(kv.w) + q[7] * bf16_hi(kv.w);
#pragma unroll
    for (int o = CH / 2; o; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (live) {
      if (c == 0) s_score[i] = dot;
      mx = fmaxf(mx, dot);
    }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) s_red[warp] = mx;
  __syncthreads();
  const float M = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
  // ---- pass 2: probabilities x V (this thread: 8 dims of the keys of its group)
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float l = 0.f;
#pragma unroll 4
  for (int i = kg; i < n; i += KG) {
    const int sl = i < P ? i : anc_t[i - P];
    const uint4 vv = *reinterpret_cast<const uint4*>(vc + cache_base + static_cast<long long>(sl) * d + c * 8);
    const float p = __expf(s_score[i] - M);
    l += p;
    acc[0] += p * bf16_lo(vv.x); acc[1] += p * bf16_hi(vv.x); acc[2] += p * bf16_lo(vv.y); acc[3] += p * bf16_hi(vv.y);
    acc[4] += p * bf16_lo(vv.z); acc[5] += p * bf16_hi(vv.z); acc[6] += p * bf16_lo(vv.w); acc[7] += p * bf16_hi(vv.w);
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) s_acc[kg][c * 8 + e] = acc[e];
  // every lane of a key group carries the same l; count each group once
  if (c != 0) l = 0.f;
#pragma unroll
  for (int o = 16; o; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
  __syncthreads();                        // also orders the s_red reads above before the writes below
  if (lane == 0) s_red[warp] = l;
  __syncthreads();
  if (tid < HD) {
    const float L = s_red[0] + s_red[1] + s_red[2] + s_red[3];
    float o = 0.f;
#pragma unroll
    for (int g = 0; g < KG; ++g) o += s_acc[g][tid];
    out[static_cast<long long>(t) * d + h * HD + tid] = __float2bfloat16(o / L);
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
