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

// One CTA per (tree, group of DA_HEADS heads): warp 0 produces, warp 1 + i consumes head i.
//
// Producer: it walks the tree's keys in chunks of DA_CHUNK, head by head inside a chunk, and brings
// each (chunk, head)'s K and V rows into a shared-memory ring with bulk asynchronous copies
// (cp.async.bulk global -> shared, completion counted on the stage's mbarrier): the prompt slots
// [0, prefix_len) of a (tree, head) are contiguous in the cache, so a chunk of them is ONE copy of
// up to 8 KB for K and one for V; ancestor slots are scattered single rows (one 128/256-byte copy
// each, issued by the producer warp's lanes in parallel), and the token's own key / value come from
// the packed QKV row they are appended from.  Up to DA_STAGES stages per CTA are in flight, with no
// registers or load instructions of the consumers tied up, which is what lets a kernel whose CTAs
// each touch only a few tens of KB stream at memory speed.
// Consumers: a warp owns one head, so there is nothing to merge between warps.  Four lanes share a
// key (each a quarter of the head dimension), eight keys per round, one online-softmax state per
// key group, merged across the groups with shuffles at the end.
// Every wait is bounded; on expiry the CTA records ST_TIMEOUT_MISC and leaves.
constexpr int DA_HEADS = 4;
constexpr int DA_CHUNK = 64;
constexpr int DA_STAGES = 6;

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

template <int HD>
__global__ void __launch_bounds__(32 * (1 + DA_HEADS))
decode_attn_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ kc,
                   __nv_bfloat16* __restrict__ vc, const int* __restrict__ active,
                   const int* __restrict__ slot, const int* __restrict__ prefix_len,
                   const int* __restrict__ anc, int anc_stride, const int* __restrict__ n_anc,
                   __nv_bfloat16* __restrict__ out, int H, int S, float scale, int* status) {
  constexpr int DPL = HD / 4;            // head dimensions per lane (four lanes share a key)
  constexpr int ROW = HD * 2;            // bytes per key row
  constexpr int STAGE = 2 * DA_CHUNK * ROW;
  const int t = blockIdx.x, hg = blockIdx.y;
  if (threadIdx.x == 0) griddep_launch_dependents();   // the output projection may start fetching its weights
  if (!active[t]) return;
  extern __shared__ __align__(128) uint8_t da_smem[];
  uint8_t* ring = da_smem;
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + DA_STAGES * STAGE);
  uint64_t* empty = full + DA_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + DA_STAGES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < DA_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const int d = H * HD;
  const int P = prefix_len[t];
  const int n = P + n_anc[t];
  const int n_chunks = (n + DA_CHUNK - 1) / DA_CHUNK;
  const int* anc_t = anc + static_cast<long long>(t) * anc_stride;
  const __nv_bfloat16* row = qkv + static_cast<long long>(t) * 3 * d;
  const int h0 = hg * DA_HEADS;
  const int nh = min(H - h0, DA_HEADS);          // heads of this CTA; item (chunk c, head i) = c * nh + i

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    // Launched as a programmatic dependent, the chunks that hold prompt slots only are fetched while
    // the kernel before (the QKV projection) is still running: the cache rows of earlier positions
    // do not depend on it.  The first chunk that needs the token's own row waits for it.
    int item = 0;
    bool waited = false;
    for (int c = 0; c < n_chunks; ++c) {
      const int i0 = c * DA_CHUNK, i1 = min(n, i0 + DA_CHUNK);
      const int pre = max(0, min(P, i1) - i0);         // keys of this chunk that are prompt slots
      if (!waited && pre < i1 - i0) { griddep_wait(); waited = true; }
      for (int hi = 0; hi < nh; ++hi, ++item) {
        const int h = h0 + hi;
        const int stage = item % DA_STAGES;
        const uint32_t parity = ((item / DA_STAGES) & 1) ^ 1;
        const long long cache_base = (static_cast<long long>(t) * H + h) * S * HD;
        int okw = 1;
        if (lane == 0) okw = mbar_wait(&empty[stage], parity, abort_flag) ? 1 : 0;
        okw = __shfl_sync(0xffffffffu, okw, 0);
        if (!okw) {
          if (lane == 0) { *abort_flag = 1; atomicCAS(status, 0, ST_TIMEOUT_MISC); }
          return;
        }
        uint8_t* sk = ring + stage * STAGE;
        uint8_t* sv = sk + DA_CHUNK * ROW;
        if (lane == 0) mbar_expect_tx(&full[stage], static_cast<uint32_t>(2 * (i1 - i0) * ROW));
        __syncwarp();
        if (lane == 0 && pre > 0) {
          bulk_load(sk, kc + cache_base + static_cast<long long>(i0) * HD, pre * ROW, &full[stage]);
          bulk_load(sv, vc + cache_base + static_cast<long long>(i0) * HD, pre * ROW, &full[stage]);
        }
        // ancestor rows (and the token's own row, the last entry): one lane each
        for (int i = i0 + pre + lane; i < i1; i += 32) {
          const void *ks, *vs;
          if (i == n - 1) {
            ks = row + d + h * HD;
            vs = row + 2 * d + h * HD;
          } else {
            const long long off = cache_base + static_cast<long long>(anc_t[i - P]) * HD;
            ks = kc + off;
            vs = vc + off;
          }
          bulk_load(sk + (i - i0) * ROW, ks, ROW, &full[stage]);
          bulk_load(sv + (i - i0) * ROW, vs, ROW, &full[stage]);
        }
      }
    }
    return;
  }
  // -------------------------------------------------------------------- consumers
  griddep_wait();                        // q and the token's key / value come from the kernel before
  const int hi = warp - 1;
  if (hi >= nh) return;
  const int h = h0 + hi;
  const int c4 = lane & 3, kg = lane >> 2;             // quarter of the row, key group 0..7
  const long long cache_base = (static_cast<long long>(t) * H + h) * S * HD;
  // append this token's key / value to the cache
  if (lane < HD / 8) {
    const long long dst = cache_base + static_cast<long long>(slot[t]) * HD + lane * 8;
    *reinterpret_cast<uint4*>(kc + dst) = *reinterpret_cast<const uint4*>(row + d + h * HD + lane * 8);
    *reinterpret_cast<uint4*>(vc + dst) = *reinterpret_cast<const uint4*>(row + 2 * d + h * HD + lane * 8);
  }
  float q[DPL];
#pragma unroll
  for (int u = 0; u < DPL / 8; ++u) {
    const uint4 qv = *reinterpret_cast<const uint4*>(row + h * HD + c4 * DPL + u * 8);
    q[u * 8 + 0] = bf16_lo(qv.x) * scale; q[u * 8 + 1] = bf16_hi(qv.x) * scale;
    q[u * 8 + 2] = bf16_lo(qv.y) * scale; q[u * 8 + 3] = bf16_hi(qv.y) * scale;
    q[u * 8 + 4] = bf16_lo(qv.z) * scale; q[u * 8 + 5] = bf16_hi(qv.z) * scale;
    q[u * 8 + 6] = bf16_lo(qv.w) * scale; q[u * 8 + 7] = bf16_hi(qv.w) * scale;
  }
  float m = -INFINITY, l = 0.f;
  float acc[DPL];
#pragma unroll
  for (int e = 0; e < DPL; ++e) acc[e] = 0.f;
  for (int ch = 0; ch < n_chunks; ++ch) {
    const int item = ch * nh + hi;
    const int stage = item % DA_STAGES;
    const uint32_t parity = (item / DA_STAGES) & 1;
    const int cnt = min(n, (ch + 1) * DA_CHUNK) - ch * DA_CHUNK;
    if (!mbar_wait(&full[stage], parity, abort_flag)) {
      *abort_flag = 1;
      atomicCAS(status, 0, ST_TIMEOUT_MISC);
      return;
    }
    const uint8_t* sk = ring + stage * STAGE + c4 * (DPL * 2);
    const uint8_t* sv = sk + DA_CHUNK * ROW;
    // eight keys per round; uniform trip count over the warp (the shuffles need every lane)
#pragma unroll 2
    for (int j0 = 0; j0 < DA_CHUNK; j0 += 8) {
      if (j0 >= cnt) break;
      const int j = j0 + kg;
      const bool live = j < cnt;
      uint4 kv[DPL / 8], vv[DPL / 8];
#pragma unroll
      for (int u = 0; u < DPL / 8; ++u) {
        kv[u] = make_uint4(0, 0, 0, 0);
        vv[u] = kv[u];
        if (live) {
          kv[u] = *reinterpret_cast<const uint4*>(sk + j * ROW + u * 16);
          vv[u] = *reinterpret_cast<const uint4*>(sv + j * ROW + u * 16);
        }
      }
      float dot = 0.f;
#pragma unroll
      for (int u = 0; u < DPL / 8; ++u)
        dot += q[u * 8 + 0] * bf16_lo(kv[u].x) + q[u * 8 + 1] * bf16_hi(kv[u].x) + q[u * 8 + 2] * bf16_lo(kv[u].y) +
               q[u * 8 + 3] * bf16_hi(kv[u].y) + q[u * 8 + 4] * bf16_lo(kv[u].z) + q[u * 8 + 5] * bf16_hi(kv[u].z) +
               q[u * 8 + 6] * bf16_lo(kv[u].w) + q[u * 8 + 7] * bf16_hi(kv[u].w);
      dot += __shfl_xor_sync(0xffffffffu, dot, 1);
      dot += __shfl_xor_sync(0xffffffffu, dot, 2);
      if (live) {                       // uniform within the key group
        const float m_new = fmaxf(m, dot);
        const float a = __expf(m - m_new), p = __expf(dot - m_new);
        l = l * a + p;
#pragma unroll
        for (int u = 0; u < DPL / 8; ++u) {
          acc[u * 8 + 0] = acc[u * 8 + 0] * a + p * bf16_lo(vv[u].x); acc[u * 8 + 1] = acc[u * 8 + 1] * a + p * bf16_hi(vv[u].x);
          acc[u * 8 + 2] = acc[u * 8 + 2] * a + p * bf16_lo(vv[u].y); acc[u * 8 + 3] = acc[u * 8 + 3] * a + p * bf16_hi(vv[u].y);
          acc[u * 8 + 4] = acc[u * 8 + 4] * a + p * bf16_lo(vv[u].z); acc[u * 8 + 5] = acc[u * 8 + 5] * a + p * bf16_hi(vv[u].z);
          acc[u * 8 + 6] = acc[u * 8 + 6] * a + p * bf16_lo(vv[u].w); acc[u * 8 + 7] = acc[u * 8 + 7] * a + p * bf16_hi(vv[u].w);
        }
        m = m_new;
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[stage]);
  }
  // merge the eight key groups (lanes with equal lane & 3 hold the same quarter of the row)
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    const float m_o = __shfl_xor_sync(0xffffffffu, m, o);
    const float l_o = __shfl_xor_sync(0xffffffffu, l, o);
    const float m_new = fmaxf(m, m_o);
    const float fa = m == -INFINITY ? 0.f : __expf(m - m_new);
    const float fb = m_o == -INFINITY ? 0.f : __expf(m_o - m_new);
    l = l * fa + l_o * fb;
#pragma unroll
    for (int e = 0; e < DPL; ++e) {
      const float a_o = __shfl_xor_sync(0xffffffffu, acc[e], o);
      acc[e] = acc[e] * fa + a_o * fb;
    }
    m = m_new;
  }
  if (kg == 0) {
    const float inv = 1.f / l;
    __nv_bfloat16* dst = out + static_cast<long long>(t) * d + h * HD + c4 * DPL;
#pragma unroll
    for (int u = 0; u < DPL / 8; ++u) {
      uint4 o;
      o.x = pack_bf16x2(acc[u * 8 + 0] * inv, acc[u * 8 + 1] * inv);
      o.y = pack_bf16x2(acc[u * 8 + 2] * inv, acc[u * 8 + 3] * inv);
      o.z = pack_bf16x2(acc[u * 8 + 4] * inv, acc[u * 8 + 5] * inv);
      o.w = pack_bf16x2(acc[u * 8 + 6] * inv, acc[u * 8 + 7] * inv);
      *reinterpret_cast<uint4*>(dst + u * 8) = o;
    }
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
                   int n_trees, int H, int hd, int S, float scale, int dependent, int* status,
                   cudaStream_t stream) {
  using namespace ab;
  if (!status || (H * hd) % 8 || (hd != 64 && hd != 128)) return -1;
  const int smem = DA_STAGES * 2 * DA_CHUNK * hd * 2 + 2 * DA_STAGES * 8 + 64;
  auto kern = hd == 64 ? decode_attn_kernel<64> : decode_attn_kernel<128>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_trees, (H + DA_HEADS - 1) / DA_HEADS);
  cfg.blockDim = dim3(32 * (1 + DA_HEADS));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  // `dependent`: programmatic dependent of the kernel before it in the stream (see the producer)
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = dependent ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, kern, (const __nv_bfloat16*)qkv, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc,
                                 active, slot, prefix_len, anc, anc_stride, n_anc, (__nv_bfloat16*)out, H, S, scale,
                                 status);
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
