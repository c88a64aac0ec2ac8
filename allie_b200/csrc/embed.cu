// Input side of the model.
//
// unpack_window : raw uint32 training words (token id in the low 14 bits, game outcome in bits
//                 14-15, seconds+1 of the next move in the high 16 bits) -> input ids, shifted LM
//                 labels, value labels, normalised time labels and the three valid-label counts.
//                 This is the collate arithmetic of the data pipeline done on the GPU, so only the
//                 raw window crosses PCIe.
// embed_fwd     : x = dropout(where(id >= V, [e, 1-e] @ W_ctrl, wte[id]) + wpe[pos]) in fp32,
//                 e = (clamp(id - V, 500, 3000) - 500) / 2500  (soft ELO conditioning).
// embed_bwd     : scatter-add of the (dropout-masked) gradient into wte / wpe / W_ctrl.
#include "ptx.cuh"

namespace ab {

__global__ void unpack_window_kernel(const uint32_t* __restrict__ words, int B, int T, int vocab,
                                     int pad_id, float time_mean, float time_std,
                                     int* __restrict__ ids, int* __restrict__ pos,
                                     int* __restrict__ lm_labels, float* __restrict__ value_labels,
                                     float* __restrict__ time_labels, int* __restrict__ counts) {
  griddep_enter();
  // counts[0] = #valid shifted LM labels, counts[1] = #valid value labels, counts[2] = #valid time
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  int c0 = 0, c1 = 0, c2 = 0;
  if (i < B * T) {
    const int t = i % T;
    const uint32_t w = words[i];
    const int id = w & 0x3FFF;
    const int enc = w >> 16;
    const int outcome = (w & 0xFFFF) >> 14;
    ids[i] = id;
    pos[i] = t;  // training windows carry no padding, so position = offset
    const bool real = id != pad_id;
    float tl = -100.f;
    if (enc != 0) {
      float s = static_cast<float>(enc - 1);
      s = fminf(fmaxf(s, 0.f), 60.f);
      tl = (s - time_mean) / time_std;
      c2 = 1;
    }
    time_labels[i] = tl;
    float vl = -100.f;
    if (real) { vl = 1.f - static_cast<float>(outcome); c1 = 1; }
    value_labels[i] = vl;
    // label for position t is the token at t+1 (causal LM shift); ELO ids and pad are ignored
    int lab = -100;
    if (t + 1 < T) {
      const int nid = words[i + 1] & 0x3FFF;
      if (nid != pad_id && nid < vocab) { lab = nid; c0 = 1; }
    }
    lm_labels[i] = lab;
  }
  c0 = __reduce_add_sync(0xffffffffu, c0);
  c1 = __reduce_add_sync(0xffffffffu, c1);
  c2 = __reduce_add_sync(0xffffffffu, c2);
  if ((threadIdx.x & 31) == 0) {
    if (c0) atomicAdd(&counts[0], c0);
    if (c1) atomicAdd(&counts[1], c1);
    if (c2) atomicAdd(&counts[2], c2);
  }
}

__device__ __forceinline__ float elo_frac(int id, int vocab) {
  int e = id - vocab;
  e = e < 500 ? 500 : (e > 3000 ? 3000 : e);
  return static_cast<float>(e - 500) / 2500.f;
}

// One warp per token row; lane covers float4 columns lane + 32*i.
__global__ void __launch_bounds__(256)
embed_fwd_kernel(const int* __restrict__ ids, const int* __restrict__ pos,
                 const float* __restrict__ wte, const float* __restrict__ wpe,
                 const float* __restrict__ ctrl, float* __restrict__ x, int M, int d, int vocab,
                 unsigned long long seed, unsigned int stream_id, unsigned int thr16,
                 const unsigned long long* __restrict__ salt) {
  griddep_enter();
  seed = salted(seed, salt);
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= M) return;
  const int id = ids[row];
  const int p = pos[row];
  const bool is_elo = ctrl != nullptr && id >= vocab;
  const float e = is_elo ? elo_frac(id, vocab) : 0.f;
  const int tid = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const float4* te = reinterpret_cast<const float4*>(wte + (long long)tid * d);
  const float4* pe = reinterpret_cast<const float4*>(wpe + (long long)p * d);
  const float4* c0 = reinterpret_cast<const float4*>(ctrl);
  const float4* c1 = reinterpret_cast<const float4*>(ctrl + d);
  float4* xr = reinterpret_cast<float4*>(x + (long long)row * d);
  const float scale = dropout_scale(thr16);
  for (int c4 = lane; c4 < d / 4; c4 += 32) {
    float4 v;
    if (is_elo) {
      const float4 a = __ldg(c0 + c4), b = __ldg(c1 + c4);
      v = make_float4(e * a.x + (1.f - e) * b.x, e * a.y + (1.f - e) * b.y,
                      e * a.z + (1.f - e) * b.z, e * a.w + (1.f - e) * b.w);
    } else {
      v = __ldg(te + c4);
    }
    const float4 q = __ldg(pe + c4);
    v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
    if (thr16) {
      const uint64_t e0 = static_cast<uint64_t>(row) * d + c4 * 4;
      const uint32_t keep = dropout_keep8(seed, stream_id, e0 >> 3, thr16) >> (e0 & 7);
      v.x = (keep & 1u) ? v.x * scale : 0.f;
      v.y = (keep & 2u) ? v.y * scale : 0.f;
      v.z = (keep & 4u) ? v.z * scale : 0.f;
      v.w = (keep & 8u) ? v.w * scale : 0.f;
    }
    xr[c4] = v;
  }
}

__device__ __forceinline__ void red_add4(float* p, float4 v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

__global__ void __launch_bounds__(256)
embed_bwd_kernel(const int* __restrict__ ids, const int* __restrict__ pos,
                 const float* __restrict__ dx, float* __restrict__ dwte, float* __restrict__ dwpe,
                 float* __restrict__ dctrl, int M, int d, int vocab, unsigned long long seed,
                 unsigned int stream_id, unsigned int thr16, const unsigned long long* __restrict__ salt) {
  griddep_enter();
  seed = salted(seed, salt);
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= M) return;
  const int id = ids[row];
  const int p = pos[row];
  const bool is_elo = dctrl != nullptr && id >= vocab;
  const float e = is_elo ? elo_frac(id, vocab) : 0.f;
  const int tid = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const float4* dxr = reinterpret_cast<const float4*>(dx + (long long)row * d);
  const float scale = dropout_scale(thr16);
  for (int c4 = lane; c4 < d / 4; c4 += 32) {
    float4 v = dxr[c4];
    if (thr16) {
      const uint64_t e0 = static_cast<uint64_t>(row) * d + c4 * 4;
      const uint32_t keep = dropout_keep8(seed, stream_id, e0 >> 3, thr16) >> (e0 & 7);
      v.x = (keep & 1u) ? v.x * scale : 0.f;
      v.y = (keep & 2u) ? v.y * scale : 0.f;
      v.z = (keep & 4u) ? v.z * scale : 0.f;
      v.w = (keep & 8u) ? v.w * scale : 0.f;
    }
    red_add4(dwpe + (long long)p * d + c4 * 4, v);
    if (is_elo) {
      red_add4(dctrl + c4 * 4, make_float4(e * v.x, e * v.y, e * v.z, e * v.w));
      const float f = 1.f - e;
      red_add4(dctrl + d + c4 * 4, make_float4(f * v.x, f * v.y, f * v.z, f * v.w));
    } else {
      red_add4(dwte + (long long)tid * d + c4 * 4, v);
    }
  }
}

const unsigned long long* g_seed_salt = nullptr;
int g_pdl_chain = 0;

// *salt = next value of a 64-bit linear congruential sequence: the first node of a captured step
__global__ void seed_salt_advance_kernel(unsigned long long* salt) {
  *salt = *salt * 6364136223846793005ull + 1442695040888963407ull;
}

}  // namespace ab

extern "C" {
// Registers (or, with null, clears) the device word that kernels launched from now on fold into
// their dropout seeds.  Meant to be set only around the capture of a CUDA graph.
int ab_set_seed_salt(const void* salt) {
  ab::g_seed_salt = static_cast<const unsigned long long*>(salt);
  return 0;
}
// Nonzero: launches of the training kernels from now on are links of a programmatic chain (each
// may become resident while the one before it drains).  Meant to be set only around the capture of
// a training micro-step.
int ab_set_pdl_chain(int on) {
  ab::g_pdl_chain = on;
  return 0;
}
int ab_seed_salt_advance(void* salt, cudaStream_t stream) {
  ab::seed_salt_advance_kernel<<<1, 1, 0, stream>>>(static_cast<unsigned long long*>(salt));
  return (int)cudaGetLastError();
}


int ab_unpack_window(const void* words, int B, int T, int vocab, int pad_id, float time_mean,
                     float time_std, int* ids, int* pos, int* lm_labels, float* value_labels,
                     float* time_labels, int* counts, cudaStream_t stream) {
  cudaError_t e = cudaMemsetAsync(counts, 0, 3 * sizeof(int), stream);
  if (e != cudaSuccess) return (int)e;
  const int n = B * T;
  ab::launch_chained(ab::unpack_window_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, 
      (const uint32_t*)words, B, T, vocab, pad_id, time_mean, time_std, ids, pos, lm_labels,
      value_labels, time_labels, counts);
  return (int)cudaGetLastError();
}

int ab_embed_fwd(const int* ids, const int* pos, const float* wte, const float* wpe,
                 const float* ctrl, float* x, int M, int d, int vocab, unsigned long long seed,
                 unsigned int stream_id, unsigned int thr16, cudaStream_t stream) {
  if (d % 4) return -1;
  ab::launch_chained(ab::embed_fwd_kernel, dim3((M + 7) / 8), dim3(256), 0, stream, ids, pos, wte, wpe, ctrl, x, M, d, vocab,
                                                        seed, stream_id, thr16, ab::seed_salt_ptr());
  return (int)cudaGetLastError();
}

int ab_embed_bwd(const int* ids, const int* pos, const float* dx, float* dwte, float* dwpe,
                 float* dctrl, int M, int d, int vocab, unsigned long long seed,
                 unsigned int stream_id, unsigned int thr16, cudaStream_t stream) {
  if (d % 4) return -1;
  ab::launch_chained(ab::embed_bwd_kernel, dim3((M + 7) / 8), dim3(256), 0, stream, ids, pos, dx, dwte, dwpe, dctrl, M, d,
                                                        vocab, seed, stream_id, thr16, ab::seed_salt_ptr());
  return (int)cudaGetLastError();
}
}

// Host-side statement of the dropout keep decisions (the same Philox function the kernels call,
// compiled for the CPU): out[i] = 1 when element i of stream `stream` under `seed` is kept.
// For tests that rebuild a kernel's mask outside the kernel.  n: multiple of 8.
extern "C" int ab_dropout_mask_host(unsigned long long seed, unsigned int stream, long long n,
                                    unsigned int thr16, unsigned char* out) {
  if (n & 7) return -1;
  for (long long g = 0; g < n / 8; ++g) {
    const uint32_t keep = ab::dropout_keep8(seed, stream, static_cast<uint64_t>(g), thr16);
    for (int j = 0; j < 8; ++j) out[g * 8 + j] = (keep >> j) & 1u;
  }
  return 0;
}
